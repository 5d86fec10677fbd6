"""Chat templating with loss masks (reference ``steptronoss/data/chat_templates/text_template.py:21-98``).

A conversation becomes ``{"tokens": int32[n], "loss_mask": float16[n]}``.  Only assistant turns that come after the
LAST user turn and carry ``loss_mask == 1`` are trained.  Token ranges are found by templating growing prefixes of the
conversation; a prefix that ends with anything but an assistant turn is rendered WITH the generation prompt, so the
header that opens the next assistant turn belongs to the prefix: the model is trained on the answer, not on the header
it is prompted with.  Tool schemas (``tool_schemas`` of the first message) are handed to the tokenizer's template, and
``tool_calls`` / ``reasoning_content`` / ``name`` of a message travel with it.
"""
from __future__ import annotations

import numpy as np

_PASS_THROUGH = ("tool_calls", "reasoning_content", "name")


class HuggingFaceTemplate:
    """Wraps a HF tokenizer's ``apply_chat_template``; falls back to a ChatML rendering when the tokenizer has no
    template.  ``system_prompt`` is put in front of conversations that do not start with a system turn."""

    def __init__(self, tokenizer, system_prompt: str | None = None):
        self.tok = self.tokenizer = tokenizer
        self.system_prompt = system_prompt

    def apply_chat_template(self, messages: list, tokenize: bool = True, tools=None):
        """Tokens (or text) of ``messages``; the generation prompt is added when the last message is not the
        assistant's."""
        prompt = messages[-1]["role"] != "assistant"
        if getattr(self.tok, "chat_template", None):
            kw = {"tools": tools} if tools else {}
            out = self.tok.apply_chat_template(messages, tokenize=tokenize, add_generation_prompt=prompt, **kw)
            return out if isinstance(out, (list, str)) else out["input_ids"]
        text = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in messages)
        text += "<|im_start|>assistant\n" if prompt else ""
        return self.tok.encode(text, add_special_tokens=False) if tokenize else text

    def __call__(self, data) -> dict:
        conversations = data["conversations"] if isinstance(data, dict) else list(data)
        if self.system_prompt and (not conversations or conversations[0]["role"] != "system"):
            conversations = [{"role": "system", "content": self.system_prompt, "loss_mask": 0}] + list(conversations)
        if not conversations or conversations[-1]["role"] != "assistant":
            raise ValueError("a training conversation ends with an assistant turn")
        tools = conversations[0].get("tool_schemas") or None
        msgs = []
        for c in conversations:
            m = {"role": c["role"], "content": _content_text(c)}
            m.update({k: c[k] for k in _PASS_THROUGH if c.get(k)})
            msgs.append(m)
        last_user = max((i for i, m in enumerate(msgs) if m["role"] == "user"), default=-1)
        if last_user < 0:
            raise ValueError("no user turn in the conversation: nothing tells where the trained part starts")
        tokens = self.apply_chat_template(msgs, True, tools)
        mask = np.zeros(len(tokens), dtype=np.float16)
        pos = len(self.apply_chat_template(msgs[: last_user + 1], True, tools))
        for i in range(last_user + 1, len(msgs)):
            end = len(self.apply_chat_template(msgs[: i + 1], True, tools))
            if msgs[i]["role"] == "assistant" and float(conversations[i].get("loss_mask", 1)) == 1.0:
                mask[pos:end] = 1.0
            pos = end
        return {"tokens": np.asarray(tokens, dtype=np.int32), "loss_mask": mask}


def _content_text(turn: dict) -> str:
    c = turn.get("content", turn.get("value", ""))
    if isinstance(c, list):
        return "".join(p if isinstance(p, str) else str(p.get("value", p.get("text", ""))) for p in c if p is not None)
    return "" if c is None else str(c)
