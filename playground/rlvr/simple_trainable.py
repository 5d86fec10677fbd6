"""A rollout item that asks the experiment's inference router for one completion and rewards a correct
``\\boxed{...}`` answer (reference ``playground/rlvr/simple_trainable.py``).

The router endpoint and the served model name are resolved at call time (getters), so an item pickled before a
restart still reaches the restarted services.  Reward: 1 for a final boxed answer equal to the ground truth, 0
otherwise and for completions cut off by the length limit.
"""
from __future__ import annotations

import hashlib
import json
import re

from steptronoss_b200.exp.rl import EnvTrajectory, StopType
from steptronoss_b200.generation.base_generatable import TrainableItem

_BOXED = re.compile(r"\\boxed\{([^{}]*)\}")


class SimpleTrainable(TrainableItem):
    def __init__(self, prompt_text: str, gt: str, endpoint_getter, model_name_getter, sampling_params: dict | None = None,
                 max_tokens: int = 1024, timeout_s: float = 7200.0):
        super().__init__()
        self.prompt_text, self.gt = prompt_text, gt
        self.endpoint_getter, self.model_name_getter = endpoint_getter, model_name_getter
        self.timeout_s = timeout_s
        self.sampling_params = {"temperature": 1.0, "top_p": 1.0, "top_k": -1, "max_tokens": max_tokens}
        self.sampling_params.update(sampling_params or {})

    @staticmethod
    def extract_boxed(text: str) -> str:
        found = _BOXED.findall(text or "")
        return found[-1].strip() if found else ""

    def request(self) -> dict:
        return dict(self.sampling_params, model=self.model_name_getter(), prompt=self.prompt_text, return_token_ids=True)

    async def generate(self) -> dict:
        import aiohttp

        async with aiohttp.request("POST", f"{self.endpoint_getter()}/v1/completions", json=self.request(),
                                   timeout=aiohttp.ClientTimeout(total=self.timeout_s)) as r:
            out = await r.json()
        if "choices" not in out:
            raise ValueError(f"unexpected completion response: {str(out)[:500]}")
        return {"choice": out["choices"][0], "prompt": self.prompt_text}

    def fingerprint(self) -> str:
        blob = json.dumps({"type": type(self).__name__, "prompt": self.prompt_text, "sampling_params": self.sampling_params},
                          ensure_ascii=False, sort_keys=True, separators=(",", ":"))
        return f"{type(self).__name__}:v1:{hashlib.sha256(blob.encode()).hexdigest()}"

    def score(self, choice: dict) -> EnvTrajectory:
        prompt_ids, new_ids = list(choice["prompt_token_ids"]), list(choice["token_ids"])
        cut = choice.get("finish_reason", "") == "length"
        right = self.extract_boxed(choice.get("text") or "") == self.gt.strip()
        logprobs = None
        lp = choice.get("logprobs") or {}
        if isinstance(lp, dict) and lp.get("token_logprobs") and len(lp["token_logprobs"]) == len(new_ids):
            logprobs = [float(x) for x in lp["token_logprobs"]]
        return EnvTrajectory(trajectory=prompt_ids + new_ids, is_gen_mask=[0] * len(prompt_ids) + [1] * len(new_ids),
                             raw_reward=0.0 if cut else float(right), logprobs=logprobs,
                             stop_type=StopType.MAX_LEN if cut else StopType.STOP_STRING)

    async def generate_for_train(self) -> list:
        return [self.score((await self.generate())["choice"])]
