"""Multiple-choice benchmarks scored on the last option letter of the response, boxed letters first
(GPQA-Diamond: A-D, MMLU-Pro: A-J; reference ``playground/eval/benchmarks/GPQADiamond``, ``MMLUPro``)."""
from __future__ import annotations

import re

from .common import JsonlChatBenchmark

_BOXED = re.compile(r"\\boxed\{([^}]*)\}")


class MultipleChoiceBenchmark(JsonlChatBenchmark):
    options: str = "ABCD"

    def _pattern(self):
        return re.compile(r"(?<![a-zA-Z0-9_])[%s](?![a-zA-Z0-9_])" % self.options)

    def extract_choice(self, response: str) -> str:
        if not response:
            return ""
        pat = self._pattern()
        for cand in reversed(_BOXED.findall(response)):
            m = pat.findall(cand.upper())
            if m:
                return m[-1]
        m = pat.findall(response.upper())
        return m[-1] if m else ""

    def is_correct(self, result) -> bool:
        return not result.error and self.extract_choice(result.response) == self._gold_answer(result).upper()


class GPQADiamondBenchmark(MultipleChoiceBenchmark):
    dataset_name = "GPQA_DIAMOND"
    options = "ABCD"


class MMLUProBenchmark(MultipleChoiceBenchmark):
    dataset_name = "MMLU_PRO"
    options = "ABCDEFGHIJ"
