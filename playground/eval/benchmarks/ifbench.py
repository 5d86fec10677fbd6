"""IFBench: verifiable instruction following (reference ``playground/eval/benchmarks/IFBench/benchmark.py:14-243``).

``data_path`` is the IFBENCH resource directory holding ``IFBench_test.jsonl`` (one record per line: ``key``,
``prompt``, ``instruction_id_list``, ``kwargs``).  Every prompt is one user turn, sampled greedily by default.  A
response is scored in two modes: *strict* checks the response as it is, *loose* also accepts the response without
its first and / or last line and without ``*``.  A sample counts as a success when it follows all of its
instructions in the configured mode; the metric also carries prompt-level and instruction-level accuracy for both
modes.  Leading ``<think>...</think>``-style reasoning is removed before scoring.
"""
from __future__ import annotations

import copy
import json
import os
import re
from dataclasses import dataclass, field

from steptronoss_b200.generation.base_benchmark import BaseMetric, Generated, SamplingParams

from . import ifbench_checks
from .common import JsonlChatBenchmark

_REASONING = tuple(re.compile(p, re.DOTALL) for p in (
    r"^\s*<think>.*?</think>\s*", r"^\s*<thinking>.*?</thinking>\s*", r"^\s*<reasoning>.*?</reasoning>\s*",
    r"^\s*<analysis>.*?</analysis>\s*", r"^\s*<\|begin_of_thought\|>.*?<\|end_of_thought\|>\s*"))


@dataclass
class IFBenchMetric(BaseMetric):
    evaluation_mode: str = "loose"
    official_metrics: dict = field(default_factory=dict)

    def to_dict(self) -> dict:
        d = super().to_dict()
        d["evaluation_mode"] = self.evaluation_mode
        d["official_metrics"] = copy.deepcopy(self.official_metrics)
        return d


@dataclass
class FollowReport:
    instruction_ids: list
    followed: list

    @property
    def follow_all(self) -> bool:
        return all(self.followed)


def accuracy_report(reports: list) -> dict:
    """Prompt-level / instruction-level accuracy, and instruction-level accuracy per id and per id family."""
    per_id: dict = {}
    for rep in reports:
        for i, ok in zip(rep.instruction_ids, rep.followed):
            a = per_id.setdefault(i, [0, 0])
            a[0] += int(ok)
            a[1] += 1
    fam: dict = {}
    for i, (ok, n) in per_id.items():
        a = fam.setdefault(i.split(":")[0], [0, 0])
        a[0] += ok
        a[1] += n
    n_inst = sum(n for _, n in per_id.values())
    return {
        "prompt_level_accuracy": sum(r.follow_all for r in reports) / len(reports) if reports else float("nan"),
        "instruction_level_accuracy": sum(ok for ok, _ in per_id.values()) / n_inst if n_inst else float("nan"),
        "by_category": {k: ok / n for k, (ok, n) in sorted(fam.items())},
        "by_instruction": {k: ok / n for k, (ok, n) in sorted(per_id.items())},
    }


class IFBenchBenchmark(JsonlChatBenchmark):
    dataset_name = "IFBENCH"
    prompt_file = "IFBench_test.jsonl"

    def __init__(self, data_path: str, tokenizer, sample_per_prompt: int, down_sample_to: int | None = None,
                 shuffle_prompts: bool = False, chat_template_options: dict | None = None,
                 evaluation_mode: str = "loose", strip_reasoning: bool = True,
                 sampling_params: SamplingParams | None = None):
        if data_path.endswith(".jsonl"):
            raise ValueError(f"data_path must be the IFBENCH resource directory, not the prompt file: {data_path}")
        if evaluation_mode not in ("loose", "strict"):
            raise ValueError(f"evaluation_mode must be 'loose' or 'strict', got {evaluation_mode!r}")
        self.resource_root = data_path
        path = os.path.join(data_path, self.prompt_file)
        if not os.path.isfile(path):
            raise FileNotFoundError(f"IFBench prompt file is missing: expected {path}")
        self.evaluation_mode, self.strip_reasoning = evaluation_mode, strip_reasoning
        self.sampling_params = SamplingParams(temperature=0.0) if sampling_params is None else copy.deepcopy(sampling_params)
        super().__init__(path, tokenizer, sample_per_prompt, down_sample_to, shuffle_prompts, chat_template_options)

    def _load_records(self) -> list:
        if self._records is None:
            recs = []
            with open(self.data_path, encoding="utf-8") as f:
                for n, line in enumerate(f):
                    if not line.strip():
                        continue
                    raw = json.loads(line)
                    missing = {"key", "prompt", "instruction_id_list", "kwargs"} - set(raw)
                    if missing:
                        raise ValueError(f"{self.data_path}:{n + 1}: missing {sorted(missing)}")
                    ids, kws = raw["instruction_id_list"], raw["kwargs"]
                    if not isinstance(raw["prompt"], str) or not isinstance(ids, list) or not isinstance(kws, list):
                        raise TypeError(f"{self.data_path}:{n + 1}: prompt must be str, instruction_id_list and kwargs lists")
                    unknown = [i for i in ids if i not in ifbench_checks.REGISTRY]
                    if unknown:
                        raise KeyError(f"{self.data_path}:{n + 1}: unknown instruction ids {unknown}")
                    kws = [{k: v for k, v in (kw or {}).items() if v is not None} for kw in kws]
                    ctx = {"key": str(raw["key"]), "prompt": raw["prompt"], "instruction_id_list": list(ids), "kwargs": kws}
                    recs.append((self.dataset_name, [{"role": "user", "content": raw["prompt"]}], str(raw["key"]), ctx))
            self._records = recs
        return super()._load_records()

    def get_cases(self) -> list:
        return [c.with_sampling_params(copy.deepcopy(self.sampling_params)) for c in super().get_cases()]

    # ------------------------------------------------------------------ scoring
    def response_for_scoring(self, result: Generated) -> str:
        if result.error:
            return ""
        text = result.response or ""
        if self.strip_reasoning:
            for pat in _REASONING:
                text = pat.sub("", text, count=1)
        return text.strip()

    def follow(self, result: Generated, mode: str) -> FollowReport:
        ctx = result.case.benchmark.context
        ids, kws = ctx["instruction_id_list"], ctx["kwargs"]
        text = self.response_for_scoring(result)
        variants = [text] if mode == "strict" else [v for v in ifbench_checks.loose_variants(text)]
        followed = []
        for i, inst in enumerate(ids):
            kw = dict(kws[i]) if i < len(kws) else {}
            if inst in ("repeat:repeat_change", "repeat:repeat_span") and "prompt_to_repeat" not in kw:
                kw["prompt_to_repeat"] = ctx["prompt"]
            followed.append(any(ifbench_checks.check(inst, v, **kw) for v in variants))
        return FollowReport(list(ids), followed)

    def evaluate(self, results: list) -> BaseMetric:
        strict = [self.follow(r, "strict") for r in results]
        loose = [self.follow(r, "loose") for r in results]
        primary = strict if self.evaluation_mode == "strict" else loose
        ok = {id(r): rep.follow_all for r, rep in zip(results, primary)}
        base = BaseMetric.from_samples(results, [1.0 if rep.follow_all else 0.0 for rep in primary],
                                       self.sample_per_prompt, lambda r: ok[id(r)])
        return IFBenchMetric(base.score_avg, base.score_std, dict(base.pass_at_k), self.evaluation_mode,
                             {"strict": accuracy_report(strict), "loose": accuracy_report(loose)})
