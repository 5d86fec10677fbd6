"""Benchmarks stored as jsonl chat records (reference ``playground/eval/benchmarks/common.py``).

One line per item: ``{"dataset": str, "messages": [{"role", "content"}...], "source_item": {"item_id": str,
...scoring context...}}``.  A trailing empty assistant turn is dropped; every item is expanded into
``sample_per_prompt`` cases.
"""
from __future__ import annotations

import copy
import json
import random

from steptronoss_b200.generation.base_benchmark import (BaseBenchmark, BaseMetric, BenchmarkMeta, EvaluationCase,
                                                       EvaluationMeta, Generated, Prompt)


def parse_record(rec: dict) -> tuple[str, list, str, dict]:
    if not isinstance(rec, dict) or not isinstance(rec.get("dataset"), str):
        raise TypeError("benchmark record needs a string 'dataset'")
    msgs = rec.get("messages")
    if not isinstance(msgs, list) or not all(
            isinstance(m, dict) and isinstance(m.get("role"), str) and isinstance(m.get("content"), str) for m in msgs):
        raise TypeError("messages must be a list of {role, content} objects")
    src = rec.get("source_item")
    if not isinstance(src, dict) or not isinstance(src.get("item_id"), str):
        raise TypeError("source_item.item_id must be a string")
    ctx = {k: v for k, v in src.items() if k != "item_id"}
    clean = [{k: m[k] for k in ("role", "content", "ground_truth") if k in m} for m in msgs]
    return rec["dataset"], clean, src["item_id"], ctx


class JsonlChatBenchmark(BaseBenchmark):
    dataset_name: str | None = None

    def __init__(self, data_path: str, tokenizer, sample_per_prompt: int, down_sample_to: int | None = None,
                 shuffle_prompts: bool = False, chat_template_options: dict | None = None):
        if not self.dataset_name:
            raise ValueError(f"{type(self).__name__} must define dataset_name")
        self.name = self.dataset_name
        self.data_path, self.tokenizer, self.sample_per_prompt = data_path, tokenizer, sample_per_prompt
        self.down_sample_to, self.shuffle_prompts = down_sample_to, shuffle_prompts
        self.chat_template_options = dict(chat_template_options or {})
        self._records: list | None = None

    def _load_records(self) -> list:
        if self._records is None:
            with open(self.data_path, encoding="utf-8") as f:
                self._records = [parse_record(json.loads(line)) for line in f if line.strip()]
        recs = list(self._records)
        if self.shuffle_prompts:
            random.Random(1234).shuffle(recs)
        return recs[: self.down_sample_to] if self.down_sample_to is not None else recs

    @staticmethod
    def _normalize_messages(messages: list) -> list:
        msgs = copy.deepcopy(messages)
        if msgs and msgs[-1].get("role") == "assistant" and not msgs[-1].get("content"):
            msgs = msgs[:-1]
        return msgs

    def get_cases(self) -> list:
        cases = []
        for pi, (_ds, messages, item_id, ctx) in enumerate(self._load_records()):
            msgs = self._normalize_messages(messages)
            n_tok = len(self.tokenizer.apply_chat_template(msgs, tokenize=True, add_generation_prompt=True,
                                                           **self.chat_template_options))
            for ri in range(self.sample_per_prompt):
                cases.append(EvaluationCase(Prompt(messages=copy.deepcopy(msgs), prompt_token_count=n_tok),
                                            BenchmarkMeta(self.name, item_id, copy.deepcopy(ctx)),
                                            EvaluationMeta(pi, ri)))
        return cases

    def count_response_tokens(self, response: str) -> int:
        return len(self.tokenizer.encode(response, add_special_tokens=False))

    @staticmethod
    def _gold_answer(result: Generated) -> str:
        a = result.case.benchmark.context.get("answer")
        return a.strip() if isinstance(a, str) else str(a).strip()

    def is_correct(self, result: Generated) -> bool:
        """Default: the generation finished by itself."""
        return result.error is None and result.finish_reason == "stop"

    def evaluate(self, results: list) -> BaseMetric:
        values = [1.0 if self.is_correct(r) else 0.0 for r in results]
        return BaseMetric.from_samples(results, values, self.sample_per_prompt, self.is_correct)
