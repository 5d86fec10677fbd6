"""Generation-based evaluation (reference ``steptronoss/exp/gen_eval.py:12-32`` and
``playground/eval/eval_sets/simple_eval.py``): expand benchmark cases into generatable items, run them
through the worker pool against the experiment's inference router, score and dump."""
from __future__ import annotations

import json
import os

from ..config import Config
from ..generation.base_benchmark import Generated, SamplingParams
from ..generation.base_generatable import GenableItem


class ChatCaseGenable(GenableItem):
    """One benchmark case as a request to an OpenAI-compatible endpoint."""

    def __init__(self, case, endpoint_getter, model_name_getter, timeout_s: float = 7200.0):
        super().__init__()
        self.case, self.endpoint_getter, self.model_name_getter, self.timeout_s = case, endpoint_getter, model_name_getter, timeout_s

    def payload(self) -> tuple[str, dict]:
        p = self.case.prompt
        body = {"model": self.model_name_getter()}
        body.update(p.sampling_params.to_dict() if p.sampling_params else {})
        if p.messages is not None:
            return "/v1/chat/completions", dict(body, messages=p.messages)
        return "/v1/completions", dict(body, prompt=p.tokens)

    async def generate(self) -> Generated:
        import aiohttp

        route, body = self.payload()
        try:
            async with aiohttp.request("POST", self.endpoint_getter() + route, json=body,
                                       timeout=aiohttp.ClientTimeout(total=self.timeout_s)) as r:
                out = await r.json()
            ch = out["choices"][0]
            msg = ch.get("message") or {}
            return Generated(self.case, {"finish_reason": ch.get("finish_reason"), "raw": ch},
                             msg.get("content") or ch.get("text") or "", msg.get("reasoning_content"))
        except Exception as e:
            return Generated(self.case, error=f"{type(e).__name__}: {e}")

    def fingerprint(self) -> str:
        import hashlib

        return "ChatCaseGenable:v1:" + hashlib.sha256(
            json.dumps(self.case.prompt.to_dict(), sort_keys=True, ensure_ascii=False).encode()).hexdigest()


class GenableEvalConfig(Config):
    """Evaluation that needs no trainer: build prompts, generate, compute metrics."""

    record_eval_rollout: bool = False
    num_workers: int | None = None
    max_concurrent_genables: int | None = None

    def get_prompts(self) -> list:
        raise NotImplementedError

    def build_controller(self):
        from ..generation.async_generation import GenerationController

        return GenerationController(self.num_workers, self.max_concurrent_genables)

    def eval(self) -> list:
        controller = self.build_controller()
        try:
            return [result for _item, result in controller.generate(self.get_prompts())]
        finally:
            controller.shutdown()


class BenchmarkEvalConfig(GenableEvalConfig):
    """Run a list of :class:`~steptronoss_b200.generation.base_benchmark.BaseBenchmark` objects."""

    router_addr_key: str = "default"
    model_name_template: str = "deployed-model-{EXP_ID}"
    temperature: float | None = 0.6
    top_p: float | None = 0.95
    max_tokens: int | None = 32768
    seed: int | None = 0
    dump_dir: str | None = None

    def build_benchmarks(self) -> list:
        raise NotImplementedError

    def sampling_params(self, run_index: int) -> SamplingParams:
        seed = None if self.seed is None else self.seed + run_index
        return SamplingParams(self.temperature, self.top_p, None, self.max_tokens, seed)

    def items_for(self, bench) -> list:
        from ..generation.base_generatable import EndpointGetter, ModelNameGetter

        ep, mn = EndpointGetter(self.router_addr_key), ModelNameGetter(self.model_name_template)
        return [ChatCaseGenable(c.with_sampling_params(self.sampling_params(c.evaluation.run_index)), ep, mn)
                for c in bench.get_cases()]

    def get_prompts(self) -> list:
        return [it for b in self.build_benchmarks() for it in self.items_for(b)]

    def eval(self) -> dict:
        benches = {b.name: b for b in self.build_benchmarks()}
        controller = self.build_controller()
        try:
            items = [it for b in benches.values() for it in self.items_for(b)]
            per: dict = {n: [] for n in benches}
            for _item, res in controller.generate(items):
                per[res.case.benchmark.benchmark_name].append(res)
        finally:
            controller.shutdown()
        out = {}
        for name, results in per.items():
            results.sort(key=lambda r: (r.case.evaluation.prompt_index, r.case.evaluation.run_index))
            out[name] = benches[name].evaluate(results)
            if self.dump_dir and self.record_eval_rollout:
                os.makedirs(self.dump_dir, exist_ok=True)
                with open(os.path.join(self.dump_dir, f"{name}.jsonl"), "w", encoding="utf-8") as f:
                    for r in results:
                        f.write(json.dumps(r.to_dict(), ensure_ascii=False) + "\n")
        return out
