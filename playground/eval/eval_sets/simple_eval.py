"""The standard evaluation set: AIME 2025, HMMT 2025, GPQA-Diamond, MMLU-Pro and IFBench against the experiment's
inference router, with a persistent cache of generations (reference ``playground/eval/eval_sets/simple_eval.py``).

``datasets_dir`` holds one sub-directory per benchmark (``AIME2025/test.jsonl``, ``HMMT2025/test.jsonl``,
``GPQA_DIAMOND/test.jsonl``, ``MMLU_PRO/test.jsonl``, ``IFBENCH/IFBench_test.jsonl``).  Every request is keyed by
its fingerprint (prompt + sampling parameters): answers found in ``save_dir/predictions.jsonl`` are not generated
again, which makes an interrupted evaluation resumable; ``rerun_level="error"`` retries only the failed requests,
``"all"`` ignores the cache.  The summary (per benchmark metric and finish-reason counts) goes to
``save_dir/summary.json``.
"""
from __future__ import annotations

import json
import os

from playground.eval.benchmarks.ifbench import IFBenchBenchmark
from playground.eval.benchmarks.math_boxed import AIME25Benchmark, HMMT25Benchmark
from playground.eval.benchmarks.multiple_choice import GPQADiamondBenchmark, MMLUProBenchmark
from steptronoss_b200.config import Ref
from steptronoss_b200.exp.base_exp import TokenizerConfig
from steptronoss_b200.exp.gen_eval import BenchmarkEvalConfig, ChatCaseGenable
from steptronoss_b200.generation.base_benchmark import Generated, SamplingParams
from steptronoss_b200.utils.logger import logger


class PredictionCache:
    """Append-only jsonl of ``{"fingerprint", "generated"}`` with an in-memory index (last entry wins)."""

    def __init__(self, path: str):
        self.path = path
        self.index: dict = {}
        if os.path.exists(path):
            with open(path, encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        rec = json.loads(line)
                        self.index[rec["fingerprint"]] = rec["generated"]
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        self._out = open(path, "a", encoding="utf-8")

    def get(self, fingerprint: str):
        d = self.index.get(fingerprint)
        return None if d is None else Generated.from_dict(json.loads(json.dumps(d)))

    def put(self, fingerprint: str, generated: Generated) -> None:
        d = generated.to_dict()
        self.index[fingerprint] = d
        self._out.write(json.dumps({"fingerprint": fingerprint, "generated": d}, ensure_ascii=False) + "\n")
        self._out.flush()

    def close(self) -> None:
        self._out.close()


class SimpleBenchmarksEvalConfig(BenchmarkEvalConfig):
    selected_datasets: str | None = None
    """comma list of benchmark names to run; None = all that are present in ``datasets_dir``"""
    sample_per_prompt: dict = {"AIME2025": 32, "HMMT2025": 32, "GPQA_DIAMOND": 8, "MMLU_PRO": 1, "IFBENCH": 1}
    chat_template_args: dict = {"enable_thinking": True}
    shuffle_prompts: bool = True
    down_sample_to: int | None = None
    datasets_dir: str = "./datasets"
    save_dir: str = Ref("..log_path", "./eval_out")
    max_decode_steps: int = 128 * 1024
    num_concurrent_requests: int = 4096
    tokenizer_cfg: TokenizerConfig = TokenizerConfig
    router_addr_key: str = Ref("..vllm_cfg.router_addr_key", "default")
    model_name_template: str = Ref("..vllm_cfg.model_name_template", "deployed-model-{EXP_ID}")
    max_model_len: int = Ref("..vllm_cfg.max_seq_len", 65536)
    rerun_level: str | None = None
    """None: use every cached answer; "error": generate failed requests again; "all": ignore the cache"""
    benchmark_options: dict = {}
    """extra constructor arguments per benchmark name, e.g. ``{"IFBENCH": {"sampling_params": {"temperature": 1.0}}}``
    (``sampling_params`` may be given as a dict of :class:`SamplingParams` fields)"""

    BENCHMARKS = {"AIME2025": (AIME25Benchmark, "test.jsonl"), "HMMT2025": (HMMT25Benchmark, "test.jsonl"),
                  "GPQA_DIAMOND": (GPQADiamondBenchmark, "test.jsonl"), "MMLU_PRO": (MMLUProBenchmark, "test.jsonl"),
                  "IFBENCH": (IFBenchBenchmark, None)}

    @property
    def predictions_path(self) -> str:
        return os.path.join(self.save_dir, "predictions.jsonl")

    @property
    def summary_path(self) -> str:
        return os.path.join(self.save_dir, "summary.json")

    def sanity_check(self):
        super().sanity_check()
        if self.rerun_level not in (None, "error", "all"):
            raise AssertionError(f"rerun_level must be None, 'error' or 'all', got {self.rerun_level!r}")

    def build_controller(self):
        from steptronoss_b200.generation.async_generation import GenerationController

        return GenerationController(self.num_workers, self.max_concurrent_genables or self.num_concurrent_requests)

    def build_benchmarks(self) -> list:
        wanted = None if not self.selected_datasets else {s.strip() for s in self.selected_datasets.split(",") if s.strip()}
        unknown = (wanted or set()) - set(self.BENCHMARKS)
        if unknown:
            raise ValueError(f"unknown benchmarks {sorted(unknown)}; known: {sorted(self.BENCHMARKS)}")
        tok = self.tokenizer_cfg.build_tokenizer()
        out = []
        for name, (cls, file) in self.BENCHMARKS.items():
            if wanted is not None and name not in wanted:
                continue
            root = os.path.join(self.datasets_dir, name)
            path = root if file is None else os.path.join(root, file)
            if not os.path.exists(path):
                if wanted is not None:
                    raise FileNotFoundError(f"benchmark {name} selected but {path} does not exist")
                logger.warning(f"benchmark {name} skipped: {path} does not exist")
                continue
            extra = dict(self.benchmark_options.get(name, {}))
            if isinstance(extra.get("sampling_params"), dict):
                extra["sampling_params"] = SamplingParams(**extra["sampling_params"])
            out.append(cls(path, tok, self.sample_per_prompt.get(name, 1), self.down_sample_to, self.shuffle_prompts,
                           dict(self.chat_template_args), **extra))
        if not out:
            raise FileNotFoundError(f"no benchmark data under {self.datasets_dir}")
        return out

    def sampling_params(self, run_index: int, own: SamplingParams | None = None, prompt_tokens: int = 0) -> SamplingParams:
        """A benchmark's own sampling parameters (IFBench is greedy) win over the configured ones; the decode limit
        always fits the engine's context."""
        base = super().sampling_params(run_index)
        room = max(self.max_model_len - prompt_tokens - 1, 1)
        limit = min(self.max_decode_steps, room)
        if own is None:
            return SamplingParams(base.temperature, base.top_p, base.top_k, limit, base.seed)
        return SamplingParams(own.temperature if own.temperature is not None else base.temperature,
                              own.top_p if own.top_p is not None else base.top_p, own.top_k,
                              min(own.max_tokens or limit, limit), own.seed if own.seed is not None else base.seed,
                              extra_body=getattr(own, "extra_body", None) or {})

    def items_for(self, bench) -> list:
        from steptronoss_b200.generation.base_generatable import EndpointGetter, ModelNameGetter

        ep, mn = EndpointGetter(self.router_addr_key), ModelNameGetter(self.model_name_template)
        items = []
        for c in bench.get_cases():
            sp = self.sampling_params(c.evaluation.run_index, c.prompt.sampling_params, c.prompt.prompt_token_count or 0)
            items.append(ChatCaseGenable(c.with_sampling_params(sp), ep, mn))
        return items

    def eval(self) -> dict:
        benches = {b.name: b for b in self.build_benchmarks()}
        items = [it for b in benches.values() for it in self.items_for(b)]
        cache = PredictionCache(self.predictions_path)
        per: dict = {n: [] for n in benches}
        todo = []
        for it in items:
            hit = None if self.rerun_level == "all" else cache.get(it.fingerprint())
            if hit is not None and not (hit.error and self.rerun_level == "error"):
                per[it.case.benchmark.benchmark_name].append(Generated(it.case, hit.choice, hit.response,
                                                                       hit.reasoning_content, hit.error))
            else:
                todo.append(it)
        logger.info(f"{len(items) - len(todo)} of {len(items)} requests answered from {self.predictions_path}")
        if todo:
            controller = self.build_controller()
            try:
                for item, res in controller.generate(todo):
                    if isinstance(res, Exception):
                        res = Generated(item.case, error=f"{type(res).__name__}: {res}")
                    cache.put(item.fingerprint(), res)
                    per[res.case.benchmark.benchmark_name].append(res)
            finally:
                controller.shutdown()
        cache.close()
        summary = {}
        for name, results in per.items():
            results.sort(key=lambda r: (r.case.evaluation.prompt_index, r.case.evaluation.run_index))
            reasons: dict = {}
            for r in results:
                reasons[r.finish_reason] = reasons.get(r.finish_reason, 0) + 1
            summary[name] = {"metric": benches[name].evaluate(results).to_dict(), "num_results": len(results),
                             "finish_reasons": reasons}
        os.makedirs(self.save_dir, exist_ok=True)
        with open(self.summary_path, "w", encoding="utf-8") as f:
            json.dump(summary, f, ensure_ascii=False, indent=1)
        return summary
