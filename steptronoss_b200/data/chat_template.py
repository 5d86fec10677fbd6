"""Chat templating with loss masks (reference ``steptronoss/data/chat_templates/text_template.py:25-72``):
a conversation becomes ``{"tokens": int32[n], "loss_mask": float16[n]}``; only assistant turns that come after
the LAST user turn and are flagged ``loss_mask == 1`` contribute to the loss."""
from __future__ import annotations

import numpy as np


class HuggingFaceTemplate:
    """Wraps a HF tokenizer's ``apply_chat_template``; falls back to a ChatML rendering when the tokenizer has
    no template."""

    def __init__(self, tokenizer, system_prompt: str | None = None):
        self.tok = tokenizer
        self.system_prompt = system_prompt

    def _render(self, messages: list, add_generation_prompt: bool = False) -> str:
        if getattr(self.tok, "chat_template", None):
            return self.tok.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt)
        text = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in messages)
        return text + ("<|im_start|>assistant\n" if add_generation_prompt else "")

    def _encode(self, text: str) -> list:
        return self.tok.encode(text, add_special_tokens=False)

    def __call__(self, conversations: list) -> dict:
        msgs = [{"role": c["role"], "content": _content_text(c)} for c in conversations]
        if self.system_prompt and (not msgs or msgs[0]["role"] != "system"):
            msgs = [{"role": "system", "content": self.system_prompt}] + msgs
            conversations = [{"role": "system", "content": self.system_prompt, "loss_mask": 0}] + list(conversations)
        last_user = max((i for i, m in enumerate(msgs) if m["role"] == "user"), default=-1)
        tokens, mask = [], []
        prev = 0
        for i in range(len(msgs)):
            upto = self._encode(self._render(msgs[: i + 1]))
            piece = upto[prev:]
            prev = len(upto)
            train = msgs[i]["role"] == "assistant" and i > last_user and float(conversations[i].get("loss_mask", 1)) == 1
            tokens += piece
            mask += [1.0 if train else 0.0] * len(piece)
        return {"tokens": np.asarray(tokens, dtype=np.int32), "loss_mask": np.asarray(mask, dtype=np.float16)}


def _content_text(turn: dict) -> str:
    c = turn.get("content", "")
    if isinstance(c, list):
        return "".join(str(p.get("value", p.get("text", ""))) for p in c)
    return str(c)
