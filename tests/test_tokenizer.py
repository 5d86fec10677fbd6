"""HFCompatTokenizer on a tokenizer.json built in the test (no downloads)."""
import json
import pickle

import pytest


@pytest.fixture()
def tok_dir(tmp_path):
    from tokenizers import Tokenizer, models, pre_tokenizers

    vocab = {"<unk>": 0, "<|im_start|>": 1, "<|im_end|>": 2, "hello": 3, "world": 4, "user": 5, "assistant": 6, "\n": 7}
    t = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    t.pre_tokenizer = pre_tokenizers.Whitespace()
    t.add_special_tokens(["<|im_start|>", "<|im_end|>"])
    t.save(str(tmp_path / "tokenizer.json"))
    cfg = {"tokenizer_class": "LlamaTokenizerFast", "unk_token": "<unk>",
           "chat_template": "{% for m in messages %}<|im_start|> {{ m['role'] }} {{ m['content'] }} <|im_end|> {% endfor %}"
                            "{% if add_generation_prompt %}<|im_start|> assistant{% endif %}"}
    (tmp_path / "tokenizer_config.json").write_text(json.dumps(cfg))
    return str(tmp_path)


def test_compat_tokenizer_contract(tok_dir):
    from steptronoss_b200.tokenizer import load_hf_tokenizer
    from steptronoss_b200.tokenizer.hf_compat_tokenizer import _is_tokenizer_json_only_llama_fast

    assert _is_tokenizer_json_only_llama_fast(tok_dir)
    tok = load_hf_tokenizer(tok_dir)
    assert tok.encode("hello world", add_special_tokens=False) == [3, 4]
    assert tok.decode([3, 4]).replace(" ", "") == "helloworld"
    ids = tok.apply_chat_template([{"role": "user", "content": "hello"}], add_generation_prompt=True)
    assert isinstance(ids, list) and all(isinstance(i, int) for i in ids) and ids[:3] == [1, 5, 3]
    text = tok.apply_chat_template([{"role": "user", "content": "hello"}], tokenize=False)
    assert isinstance(text, str) and "hello" in text
    clone = pickle.loads(pickle.dumps(tok))
    assert clone.encode("world", add_special_tokens=False) == [4] and clone.vocab_size == tok.vocab_size
