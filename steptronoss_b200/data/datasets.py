"""Datasets (reference ``steptronoss/data/datasets/*.py``): raw StepChat JSON conversations, and compiled
datasets (templated samples pickled into indexed-bin shards: sample ``i`` lives in shard ``i % n_shards`` at
local index ``i // n_shards``; ``compiled_dataset.pkl`` holds ``length``, ``shards`` and ``sample_meta``)."""
from __future__ import annotations

import json
import os
import pickle
import random
from typing import Any, Literal, TypedDict

from ..utils.logger import logger
from .indexed_bin import IndexedBinReader, IndexedBinWriter
from .recipe import DataSourceFile
from .types import VALID_MESSAGE_CONTENT_TYPES


class Dataset:
    def __len__(self) -> int:
        raise NotImplementedError

    def __getitem__(self, i: int) -> dict:
        raise NotImplementedError

    def sample_length(self, i: int) -> int:
        return len(self[i]["tokens"])


class JSONMessage(TypedDict, total=False):
    """One message of a raw StepChat sample."""

    role: str
    content: Any                 # text, or a list of {"type", "value", "loss_mask"} parts
    name: str
    loss_mask: Literal[0, 1] | None
    ground_truth: Any | None


class JSONSample(TypedDict, total=False):
    conversations: list
    images: list | None


class StepChatSampleFormatError(TypeError, ValueError):
    """A sample is not a mapping with a ``conversations`` list."""


class StepChatJsonDataset(Dataset):
    """StepChat JSON files: each a top-level list of ``{"conversations": [...], "images": [...]}``
    (reference: data/datasets/stepchat_dataset.py:44-272).

    ``files``: paths or ``DataSourceFile``s; a ``subsample_rate`` below 1 keeps that share of a file's samples, drawn
    with a fixed seed.  Every sample is normalised (``convert_dialog``: lower-case roles, content as a list of typed
    parts, ``value`` accepted for ``content``, defaults for ``name`` / ``loss_mask``, ``tools`` accepted for
    ``tool_schemas``) and checked (``check_error``); samples that fail the check are dropped with a warning and
    ``valid_dialog_nums_per_file`` says how many each file kept.  Files are parsed with ``ijson`` when it is
    installed (streaming), with ``json`` otherwise."""

    def __init__(self, files, template=None):
        self.filelist = [files] if isinstance(files, (str, DataSourceFile)) else list(files)
        self.template = template
        self.data: list = []
        self.valid_dialog_nums_per_file: dict = {}
        for f in self.filelist:
            path, dialogs = self._load_dialog(f if isinstance(f, DataSourceFile) else DataSourceFile(str(f)))
            self.data.extend(dialogs)
            self.valid_dialog_nums_per_file[path] = len(dialogs)

    @property
    def records(self) -> list:
        return self.data

    # ---- reading ----------------------------------------------------------------------------------------------
    @staticmethod
    def _peek_json_root_token(path: str) -> str:
        with open(path, "rb") as f:
            while True:
                ch = f.read(1)
                if not ch:
                    raise ValueError(f"empty json file: {path}")
                if not ch.isspace():
                    return ch.decode("utf-8", "replace")

    @classmethod
    def _read(cls, path: str) -> list:
        if cls._peek_json_root_token(path) != "[":
            raise ValueError(f"StepChat json file must be a top-level list of samples: {path}")
        try:
            import ijson

            with open(path, "rb") as f:
                return list(ijson.items(f, "item", use_float=True))
        except ImportError:
            with open(path) as f:
                return json.load(f)

    @classmethod
    def _load_dialog(cls, src: DataSourceFile):
        raw = cls._read(src.path)
        picked = list(range(len(raw)))
        if 0.0 < src.subsample_rate < 1.0:
            picked = random.Random(1234).sample(picked, int(len(raw) * src.subsample_rate))
            logger.info(f"Downsampled {len(raw)} dialogs to {len(picked)} dialogs from {src.path}", at=None)
        dialogs = []
        for idx in picked:
            dialog = cls.convert_dialog(raw[idx], src.path)
            err = cls.check_error(dialog)
            if err is None:
                dialogs.append(dialog)
            else:
                logger.warning(f"Invalid dialog ({err}) from {src.path}: {idx}", at=None)
        return src.path, dialogs

    @classmethod
    def read_from_file(cls, filelist: list):
        """``(dialogs of all files, {path: valid dialogs})``."""
        data, counts = [], {}
        for f in filelist:
            path, dialogs = cls._load_dialog(f if isinstance(f, DataSourceFile) else DataSourceFile(str(f)))
            data.extend(dialogs)
            counts[path] = len(dialogs)
        return data, counts

    # ---- normalisation ----------------------------------------------------------------------------------------
    @classmethod
    def convert_content_part(cls, p) -> dict:
        if isinstance(p, str):
            return {"type": "text", "value": p}
        try:
            if not (isinstance(p["type"], str) and isinstance(p["value"], str)) or p["type"] not in VALID_MESSAGE_CONTENT_TYPES:
                raise ValueError("type / value must be text and the type a known one")
            part = {"type": p["type"], "value": p["value"]}
            if "loss_mask" in p:
                if not isinstance(p["loss_mask"], (int, float)) or int(p["loss_mask"]) not in (0, 1):
                    raise ValueError("loss_mask must be 0 or 1")
                part["loss_mask"] = int(p["loss_mask"])
            return part
        except Exception as e:
            raise ValueError(f"Invalid content message part: {p}, {e}") from None

    @classmethod
    def convert_message_item(cls, item: dict) -> list:
        if "content" in item:
            content = item["content"]
        elif "value" in item:                                # files written before the key was renamed
            content = item["value"]
        else:
            raise ValueError(f"message without content: {item}")
        parts = content if isinstance(content, list) else [content]
        return [cls.convert_content_part(c) for c in parts if c is not None]

    @classmethod
    def convert_dialog(cls, raw_dialog, f_path: str = "") -> dict:
        if not isinstance(raw_dialog, dict):
            raise StepChatSampleFormatError(f"StepChat sample must be a dict with 'conversations' list: {type(raw_dialog)}")
        if not isinstance(raw_dialog.get("conversations"), list):
            raise ValueError(f"StepChat sample must contain a 'conversations' list: {f_path}")
        return {"conversations": [{"role": item["role"].lower(),
                                   "content": cls.convert_message_item(item),
                                   "name": (item.get("name", "") or "").strip(),
                                   "loss_mask": item.get("loss_mask", 1),
                                   "ground_truth": item.get("ground_truth"),
                                   "tool_calls": item.get("tool_calls"),
                                   "reasoning_content": item.get("reasoning_content"),
                                   "tool_schemas": item.get("tools") or item.get("tool_schemas"),
                                   "data_path": f_path} for item in raw_dialog["conversations"]],
                "images": raw_dialog.get("images")}

    @classmethod
    def check_error(cls, dialog: dict) -> str | None:
        """Why a normalised dialog cannot be trained on, or None."""
        conv = dialog["conversations"]
        if len(conv) < 2:
            return "less than 2 msgs"
        for msg in conv:
            if msg["name"] and "\n" in msg["name"]:
                return "name contains newline"
            if msg["role"] == "assistant" and not msg["content"] and not msg["tool_calls"]:
                return "empty or invalid content and toolcall"
        if conv[-1]["role"] != "assistant":
            return "the last message is not assistant"
        return None

    # ---- access -----------------------------------------------------------------------------------------------
    def __len__(self) -> int:
        return len(self.data)

    def __getitem__(self, i: int) -> dict:
        rec = self.data[i]
        if self.template is None:
            return rec
        out = self.template(rec)
        out["raw_index"] = i
        return out

    def get_sample_sizes(self, size_func) -> list:
        return [size_func(self[i]) for i in range(len(self))]


def compile_dataset(dataset: Dataset, save_path: str, n_shards: int = 1, cfg: dict | None = None) -> dict:
    os.makedirs(save_path, exist_ok=True)
    writers = [IndexedBinWriter(os.path.join(save_path, f"shard_{s:05d}"), cfg=cfg) for s in range(n_shards)]
    meta = []
    for i in range(len(dataset)):
        sample = dataset[i]
        writers[i % n_shards].append(sample)
        meta.append(len(sample["tokens"]))
    for w in writers:
        w.close()
    manifest = {"length": len(dataset), "shards": [{"path": f"shard_{s:05d}", "size": len(range(s, len(dataset), n_shards))}
                                                    for s in range(n_shards)], "sample_meta": meta}
    with open(os.path.join(save_path, "compiled_dataset.pkl"), "wb") as f:
        pickle.dump(manifest, f)
    return manifest


class CompiledDataset(Dataset):
    def __init__(self, path: str):
        mf = os.path.join(path, "compiled_dataset.pkl")
        if not os.path.exists(mf):
            raise FileNotFoundError(f"manifest file not found: is '{path}' a compiled dataset?")
        with open(mf, "rb") as f:
            self.manifest = pickle.load(f)
        self.readers = [IndexedBinReader(os.path.join(path, s["path"])) for s in self.manifest["shards"]]

    def __len__(self) -> int:
        return self.manifest["length"]

    def __getitem__(self, i: int) -> dict:
        n = len(self.readers)
        return self.readers[i % n][i // n]

    def sample_length(self, i: int) -> int:
        return self.manifest["sample_meta"][i]
