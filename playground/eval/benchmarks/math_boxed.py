"""Competition-math benchmarks scored on the last ``\\boxed{...}`` of the response (AIME 2025, HMMT 2025;
reference ``playground/eval/benchmarks/AIME25/benchmark.py``, ``HMMT25``)."""
from __future__ import annotations

from steptronoss_b200.text_processing.math_utils import is_equal, last_boxed_only_string, remove_boxed

from .common import JsonlChatBenchmark


class BoxedMathBenchmark(JsonlChatBenchmark):
    symbolic_fallback: bool = True

    @staticmethod
    def extract_answer(response: str) -> str:
        if not response:
            return ""
        inner = remove_boxed(last_boxed_only_string(response))
        return (inner if inner is not None else response).strip()

    @staticmethod
    def normalize(text: str) -> str:
        for a, b in ((r"\dfrac", r"\frac"), (r"\tfrac", r"\frac"), (r"\left", ""), (r"\right", ""), (" ", ""), ("\n", "")):
            text = text.replace(a, b)
        return text.strip()

    def is_correct(self, result) -> bool:
        if result.error:
            return False
        gold, pred = self._gold_answer(result), self.extract_answer(result.response)
        if self.normalize(pred) == self.normalize(gold):
            return True
        if not self.symbolic_fallback or not pred or len(pred) > 256:
            return False
        try:
            return bool(is_equal(pred, gold))
        except Exception:
            return False


class AIME25Benchmark(BoxedMathBenchmark):
    dataset_name = "AIME2025"


class HMMT25Benchmark(BoxedMathBenchmark):
    dataset_name = "HMMT2025"
