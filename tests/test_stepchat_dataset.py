"""StepChat JSON files: normalisation, validation, sub-sampling; and what the chat template trains on."""
import json

import numpy as np
import pytest

from steptronoss_b200.data.chat_template import HuggingFaceTemplate
from steptronoss_b200.data.datasets import StepChatJsonDataset, StepChatSampleFormatError
from steptronoss_b200.data.recipe import DataSourceFile


class CharTok:
    """One token per character; no template of its own, so the ChatML fallback renders."""

    chat_template = None

    def encode(self, text, add_special_tokens=False):
        return [ord(c) for c in text]


def _text(tokens, mask=None):
    return "".join(chr(t) for t, m in zip(tokens, mask if mask is not None else [1] * len(tokens)) if m)


def test_only_the_answers_after_the_last_user_turn_are_trained_without_their_headers():
    conv = [{"role": "user", "content": "q1"}, {"role": "assistant", "content": "early"},
            {"role": "user", "content": "q2"}, {"role": "assistant", "content": "call", "tool_calls": [{"name": "f"}]},
            {"role": "tool", "content": "result"}, {"role": "assistant", "content": [{"type": "text", "value": "final"}]}]
    out = HuggingFaceTemplate(CharTok())({"conversations": conv})
    assert out["tokens"].dtype == np.int32 and out["loss_mask"].dtype == np.float16
    full = _text(out["tokens"])
    assert full.count("<|im_start|>assistant\n") == 3 and full.endswith("final<|im_end|>\n")
    # the generation prompt belongs to the prefix: answers are trained from their first own token to the turn's end
    assert _text(out["tokens"], out["loss_mask"]) == "call<|im_end|>\nfinal<|im_end|>\n"
    conv[3]["loss_mask"] = 0
    assert _text(*HuggingFaceTemplate(CharTok())(conv).values()) == "final<|im_end|>\n"
    with pytest.raises(ValueError, match="ends with an assistant"):
        HuggingFaceTemplate(CharTok())(conv[:-1])
    with pytest.raises(ValueError, match="no user turn"):
        HuggingFaceTemplate(CharTok())([{"role": "system", "content": "s"}, {"role": "assistant", "content": "a"}])
    sys = HuggingFaceTemplate(CharTok(), system_prompt="be brief")(conv)
    assert _text(sys["tokens"]).startswith("<|im_start|>system\nbe brief<|im_end|>\n")


def test_tools_and_message_fields_reach_the_tokenizer_template():
    seen = []

    class TemplTok(CharTok):
        chat_template = "{{ x }}"

        def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=False, tools=None):
            seen.append((len(messages), add_generation_prompt, tools, [sorted(m) for m in messages]))
            text = "".join(f"[{m['role']}:{m['content']}]" for m in messages) + ("[assistant:" if add_generation_prompt else "")
            return {"input_ids": self.encode(text)} if tokenize else text

    conv = [{"role": "user", "content": "q", "tool_schemas": [{"name": "f"}]},
            {"role": "assistant", "content": "a", "reasoning_content": "hm", "name": "bot"}]
    out = HuggingFaceTemplate(TemplTok())(conv)
    assert seen[0][:3] == (2, False, [{"name": "f"}]) and seen[1][:3] == (1, True, [{"name": "f"}])
    assert seen[0][3][1] == ["content", "name", "reasoning_content", "role"]
    assert _text(out["tokens"], out["loss_mask"]) == "a]"


def test_files_are_normalised_checked_and_subsampled(tmp_path):
    good = {"conversations": [{"role": "USER", "value": "hi", "tools": [{"name": "t"}]},
                              {"role": "assistant", "content": ["a", None, {"type": "text", "value": "b", "loss_mask": 0}],
                               "name": " bot "}], "images": ["x.png"]}
    bad = [{"conversations": [{"role": "user", "content": "only one"}]},
           {"conversations": [{"role": "user", "content": "q"}, {"role": "assistant", "content": []}]},
           {"conversations": [{"role": "assistant", "content": "a"}, {"role": "user", "content": "last is user"}]},
           {"conversations": [{"role": "user", "content": "q", "name": "a\nb"}, {"role": "assistant", "content": "a"}]}]
    (tmp_path / "a.json").write_text(json.dumps([good] + bad))
    ds = StepChatJsonDataset(str(tmp_path / "a.json"))
    assert len(ds) == 1 and ds.valid_dialog_nums_per_file == {str(tmp_path / "a.json"): 1}
    d = ds[0]
    first, second = d["conversations"]
    assert first["role"] == "user" and first["content"] == [{"type": "text", "value": "hi"}] and first["tool_schemas"] == [{"name": "t"}]
    assert second["name"] == "bot" and second["loss_mask"] == 1 and d["images"] == ["x.png"]
    assert second["content"] == [{"type": "text", "value": "a"}, {"type": "text", "value": "b", "loss_mask": 0}]
    assert second["data_path"].endswith("a.json") and StepChatJsonDataset.check_error(d) is None
    templ = StepChatJsonDataset(str(tmp_path / "a.json"), template=HuggingFaceTemplate(CharTok()))
    assert _text(templ[0]["tokens"], templ[0]["loss_mask"]) == "ab<|im_end|>\n" and templ.get_sample_sizes(lambda s: len(s["tokens"])) == [len(templ[0]["tokens"])]
    # malformed files and samples
    (tmp_path / "obj.json").write_text(json.dumps({"conversations": []}))
    with pytest.raises(ValueError, match="top-level list"):
        StepChatJsonDataset(str(tmp_path / "obj.json"))
    (tmp_path / "empty.json").write_text("  \n")
    with pytest.raises(ValueError, match="empty json"):
        StepChatJsonDataset(str(tmp_path / "empty.json"))
    with pytest.raises(StepChatSampleFormatError):
        StepChatJsonDataset.convert_dialog(["not", "a", "dict"])
    with pytest.raises(ValueError, match="Invalid content message part"):
        StepChatJsonDataset.convert_content_part({"type": "video", "value": "x"})
    # sub-sampling: the share asked for, the same draw every time
    many = [{"conversations": [{"role": "user", "content": f"q{i}"}, {"role": "assistant", "content": f"a{i}"}]} for i in range(40)]
    (tmp_path / "many.json").write_text(json.dumps(many))
    src = DataSourceFile(str(tmp_path / "many.json"), subsample_rate=0.25)
    one, two = StepChatJsonDataset([src]), StepChatJsonDataset([src])
    pick = lambda ds: [d["conversations"][0]["content"][0]["value"] for d in ds.data]
    assert len(one) == 10 and pick(one) == pick(two) and len(set(pick(one))) == 10
    both, counts = StepChatJsonDataset.read_from_file([src, str(tmp_path / "a.json")])
    assert len(both) == 11 and counts[str(tmp_path / "many.json")] == 10
