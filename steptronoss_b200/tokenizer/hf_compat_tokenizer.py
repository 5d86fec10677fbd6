"""Wrapper around Hugging Face tokenizers that keeps the contract the data pipeline and the RL code rely on
(reference ``steptronoss/tokenizer/hf_compat_tokenizer.py:10-175``):

* ``apply_chat_template(..., tokenize=True)`` always returns a flat ``list[int]`` (newer ``transformers``
  return a ``BatchEncoding``, tensors or nested lists depending on arguments);
* local byte-level BPE tokenizers that declare ``LlamaTokenizerFast`` but ship only ``tokenizer.json`` are
  loaded through ``PreTrainedTokenizerFast`` so that the pre-tokenizer / decoder pipeline of the file is
  used unchanged;
* the wrapper pickles (worker processes) and forwards every other attribute to the wrapped tokenizer.
"""
from __future__ import annotations

import json
import os
from typing import Any


class BaseTokenizer:
    """Minimal interface expected by the data pipeline."""

    def encode(self, text: str, add_special_tokens: bool = True, split_special_tokens: bool = False, **kw) -> list:
        raise NotImplementedError

    def decode(self, token_ids, skip_special_tokens: bool = False, **kw) -> str:
        raise NotImplementedError

    def apply_chat_template(self, *args, **kwargs):
        raise NotImplementedError


def _flat_ids(tokenized: Any) -> list:
    ids = getattr(tokenized, "input_ids", None)
    if ids is None and isinstance(tokenized, dict):
        ids = tokenized.get("input_ids")
    if ids is None:
        ids = tokenized
    if hasattr(ids, "tolist"):
        ids = ids.tolist()
    if isinstance(ids, tuple):
        ids = list(ids)
    if isinstance(ids, list) and ids and isinstance(ids[0], list):
        ids = ids[0]
    if not isinstance(ids, list):
        raise TypeError(f"Unsupported tokenized output type: {type(tokenized).__name__}")
    return ids


def _is_tokenizer_json_only_llama_fast(path: str) -> bool:
    if not os.path.isdir(path):
        return False
    has = lambda name: os.path.isfile(os.path.join(path, name))  # noqa: E731
    if not has("tokenizer.json") or has("tokenizer.model") or not has("tokenizer_config.json"):
        return False
    try:
        with open(os.path.join(path, "tokenizer_config.json"), encoding="utf-8") as f:
            return json.load(f).get("tokenizer_class") == "LlamaTokenizerFast"
    except (OSError, json.JSONDecodeError):
        return False


def _load_raw(path: str, **kw):
    from transformers import AutoTokenizer, PreTrainedTokenizerFast

    if _is_tokenizer_json_only_llama_fast(path):
        return PreTrainedTokenizerFast.from_pretrained(path, **kw)
    return AutoTokenizer.from_pretrained(path, **kw)


class HFCompatTokenizer(BaseTokenizer):
    def __init__(self, hf_path: str | None = None, hf_tokenizer=None, **kw):
        os.environ["TOKENIZERS_PARALLELISM"] = "false"
        if hf_path is not None:
            self.hf_path = hf_path
        self.hf_tokenizer = hf_tokenizer if hf_tokenizer is not None else _load_raw(hf_path, **kw)

    def encode(self, text, add_special_tokens=True, split_special_tokens=False, **kw):
        return self.hf_tokenizer.encode(text=text, add_special_tokens=add_special_tokens,
                                        split_special_tokens=split_special_tokens, **kw)

    def decode(self, token_ids, skip_special_tokens=False, **kw):
        return self.hf_tokenizer.decode(token_ids, skip_special_tokens=skip_special_tokens, **kw)

    def apply_chat_template(self, *args, **kwargs):
        out = self.hf_tokenizer.apply_chat_template(*args, **kwargs)
        return _flat_ids(out) if kwargs.get("tokenize", True) else out

    def __getattr__(self, key: str):
        if key == "hf_tokenizer":  # not set yet (unpickling): do not recurse
            raise AttributeError(key)
        return getattr(self.hf_tokenizer, key)

    def __dir__(self):
        return dir(self.hf_tokenizer)

    def __len__(self):
        return len(self.hf_tokenizer)

    def __getstate__(self):
        return {"hf_tokenizer": self.hf_tokenizer, "hf_path": self.__dict__.get("hf_path")}

    def __setstate__(self, state):
        self.hf_tokenizer = state["hf_tokenizer"]
        if state.get("hf_path") is not None:
            self.hf_path = state["hf_path"]


def load_hf_tokenizer(hf_path: str, **kw) -> HFCompatTokenizer:
    return HFCompatTokenizer(hf_path=hf_path, **kw)
