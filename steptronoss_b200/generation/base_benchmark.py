"""Data model of offline benchmarks (reference ``steptronoss/generation/base_benchmark.py:1-369``).

Ownership: the benchmark owns :class:`Prompt` (what is sent to the model) and :class:`BenchmarkMeta` (what is
needed to score, never sent); the runner owns :class:`EvaluationMeta` (indices of the expanded prompt and of
the repeated sample); :class:`Generated` ties a model answer to all three.  Everything serialises to plain
JSON so that prediction dumps can be re-scored later.
"""
from __future__ import annotations

import math
from abc import ABC, abstractmethod
from dataclasses import dataclass, field, replace
from typing import TypeAlias, TypedDict

# ---- shapes of the JSON payloads that travel through prompts and prediction dumps ------------------------------
JsonScalar: TypeAlias = None | bool | int | float | str
JsonValue: TypeAlias = JsonScalar | list["JsonValue"] | dict[str, "JsonValue"]
JsonObject: TypeAlias = dict[str, JsonValue]


class GroundTruthValue(TypedDict):
    """Which benchmark item a turn of an exported conversation refers to."""

    item_id: str
    dataset: str


class GroundTruth(TypedDict):
    value: GroundTruthValue


class ChatMessage(TypedDict, total=False):
    """One chat turn as the tokenizer template and the chat API take it; ``ground_truth`` rides along on exported
    assistant turns and is never rendered."""

    role: str
    content: str
    ground_truth: GroundTruth


Messages: TypeAlias = list[ChatMessage]


class CompletionMessage(TypedDict, total=False):
    """``message`` of a chat/completions choice."""

    content: str
    reasoning_content: str


class CompletionChoice(TypedDict, total=False):
    """A sampled completion as kept in prediction dumps: ``text`` from completion-style back-ends, ``message`` from
    chat-style ones, ``raw`` the back-end's own object."""

    finish_reason: str
    text: str
    message: CompletionMessage
    raw: JsonObject


@dataclass(frozen=True)
class SamplingParams:
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    max_tokens: int | None = None
    seed: int | None = None
    extra_body: dict = field(default_factory=dict)

    def to_dict(self) -> dict:
        out = dict(self.extra_body)
        for k in ("temperature", "top_p", "top_k", "max_tokens", "seed"):
            v = getattr(self, k)
            if v is not None:
                out[k] = v
        return out


@dataclass(frozen=True)
class Prompt:
    """Exactly one of ``tokens`` (token API) or ``messages`` (chat API)."""

    tokens: list | None = None
    messages: list | None = None
    prompt_token_count: int | None = None
    sampling_params: SamplingParams | None = None

    def __post_init__(self):
        if (self.tokens is None) == (self.messages is None):
            raise ValueError("Prompt must define exactly one of tokens or messages")
        if self.prompt_token_count is not None and self.prompt_token_count < 0:
            raise ValueError("Prompt.prompt_token_count must be non-negative")
        if self.tokens is not None and self.prompt_token_count is None:
            object.__setattr__(self, "prompt_token_count", len(self.tokens))

    def with_sampling_params(self, sp: SamplingParams) -> "Prompt":
        return replace(self, sampling_params=sp)

    def to_dict(self) -> dict:
        out: dict = {}
        if self.tokens is not None:
            out["tokens"] = list(self.tokens)
        if self.messages is not None:
            out["messages"] = [dict(m) for m in self.messages]
        if self.prompt_token_count is not None:
            out["prompt_token_count"] = self.prompt_token_count
        out["sampling_params"] = None if self.sampling_params is None else self.sampling_params.to_dict()
        return out


@dataclass(frozen=True)
class BenchmarkMeta:
    benchmark_name: str
    item_id: str
    context: dict = field(default_factory=dict)

    def to_dict(self) -> dict:
        return {"benchmark_name": self.benchmark_name, "item_id": self.item_id, "context": dict(self.context)}


@dataclass(frozen=True)
class EvaluationMeta:
    prompt_index: int
    run_index: int

    def to_dict(self) -> dict:
        return {"prompt_index": self.prompt_index, "run_index": self.run_index}


@dataclass(frozen=True)
class EvaluationCase:
    prompt: Prompt
    benchmark: BenchmarkMeta
    evaluation: EvaluationMeta

    def with_sampling_params(self, sp: SamplingParams) -> "EvaluationCase":
        return EvaluationCase(self.prompt.with_sampling_params(sp), self.benchmark, self.evaluation)


@dataclass
class Generated:
    case: EvaluationCase
    choice: dict | None = None
    response: str = ""
    reasoning_content: str | None = None
    error: str | None = None

    @property
    def finish_reason(self) -> str:
        if self.error:
            return "error"
        fr = (self.choice or {}).get("finish_reason")
        return fr if isinstance(fr, str) and fr else "unknown"

    def to_dict(self) -> dict:
        return {"prompt": self.case.prompt.to_dict(), "benchmark": self.case.benchmark.to_dict(),
                "evaluation": self.case.evaluation.to_dict(), "choice": None if self.choice is None else dict(self.choice),
                "response": self.response, "reasoning_content": self.reasoning_content, "error": self.error}

    @classmethod
    def from_dict(cls, d: dict) -> "Generated":
        sp = d["prompt"].get("sampling_params")
        prompt = Prompt(tokens=d["prompt"].get("tokens"), messages=d["prompt"].get("messages"),
                        prompt_token_count=d["prompt"].get("prompt_token_count"),
                        sampling_params=None if sp is None else SamplingParams(
                            **{k: sp.pop(k) for k in ("temperature", "top_p", "top_k", "max_tokens", "seed") if k in sp},
                            extra_body=sp))
        case = EvaluationCase(prompt, BenchmarkMeta(**d["benchmark"]), EvaluationMeta(**d["evaluation"]))
        return cls(case, d.get("choice"), d.get("response", ""), d.get("reasoning_content"), d.get("error"))


def build_demo_generated(response: str = "3") -> Generated:
    """The smallest complete prompt -> answer record, for documentation and for tests of new benchmarks."""
    case = EvaluationCase(
        prompt=Prompt(messages=[ChatMessage(role="user", content="How many r are in strawberry?")], prompt_token_count=3,
                      sampling_params=SamplingParams(seed=0, max_tokens=8)),
        benchmark=BenchmarkMeta(benchmark_name="demo_count_r", item_id="strawberry_r_count_0", context={"answer": "3"}),
        evaluation=EvaluationMeta(prompt_index=0, run_index=0))
    return Generated(case=case, response=response)


def estimate_pass_at_k(num_samples: int, num_successes: int, k: int) -> float:
    """Unbiased estimator ``1 - C(n-c, k) / C(n, k)`` (``k`` clipped to ``n``)."""
    if num_samples <= 0 or not 0 <= num_successes <= num_samples or k <= 0:
        raise ValueError("need n > 0, 0 <= c <= n, k > 0")
    k = min(k, num_samples)
    if num_successes == 0:
        return 0.0
    if num_samples - num_successes < k:
        return 1.0
    return 1.0 - math.prod(1.0 - k / d for d in range(num_samples - num_successes + 1, num_samples + 1))


@dataclass
class BaseMetric:
    score_avg: float
    score_std: float
    pass_at_k: dict = field(default_factory=dict)

    def __repr__(self) -> str:
        f = lambda v: "nan" if math.isnan(v) else f"{v:.4f}"  # noqa: E731
        p = ", ".join(f"{k}: {f(v)}" for k, v in sorted(self.pass_at_k.items()))
        return f"BaseMetric(score_avg={f(self.score_avg)}, score_std={f(self.score_std)}, pass_at_k={{ {p} }})"

    def to_dict(self) -> dict:
        return {"score_avg": self.score_avg, "score_std": self.score_std,
                "pass_at_k": {str(k): v for k, v in self.pass_at_k.items()}, "repr": repr(self)}

    @classmethod
    def from_samples(cls, results: list, values: list, sample_per_prompt: int, is_success) -> "BaseMetric":
        """Mean / population std of the per-sample scores and pass@k for k = 1, 2, 4, ..., samples per prompt."""
        if not results:
            return cls(math.nan, math.nan, {})
        avg = sum(values) / len(values)
        std = math.sqrt(sum((v - avg) ** 2 for v in values) / len(values))
        groups: dict = {}
        for r in results:
            groups.setdefault(r.case.benchmark.item_id, []).append(r)
        ks, k = {1, sample_per_prompt}, 2
        while k < sample_per_prompt:
            ks.add(k)
            k *= 2
        pak = {}
        for k in sorted(ks):
            tot = sum(estimate_pass_at_k(len(g), sum(1 for r in g if is_success(r)), k) for g in groups.values())
            pak[k] = tot / max(len(groups), 1)
        return cls(avg, std, pak)


class BaseBenchmark(ABC):
    name: str

    @abstractmethod
    def get_cases(self) -> list:
        """Evaluation cases in the order the scorer expects."""

    @abstractmethod
    def evaluate(self, results: list) -> BaseMetric:
        """Aggregate per-sample outputs into the benchmark metric."""
