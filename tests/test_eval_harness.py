"""Benchmark data model, pass@k, jsonl benchmarks and the benchmark eval config with in-process generation."""
import json
import math

import pytest

from steptronoss_b200.generation.base_benchmark import (BenchmarkMeta, EvaluationCase, EvaluationMeta, Generated, Prompt,
                                                       SamplingParams, estimate_pass_at_k)


def test_pass_at_k_matches_combinatorics():
    for n, c, k in [(8, 3, 1), (8, 3, 4), (8, 0, 2), (8, 8, 8), (5, 2, 8)]:
        kk = min(k, n)
        want = 1 - math.comb(n - c, kk) / math.comb(n, kk) if n - c >= kk else 1.0
        assert abs(estimate_pass_at_k(n, c, k) - (0.0 if c == 0 else want)) < 1e-12


def test_prompt_validation_and_round_trip():
    with pytest.raises(ValueError):
        Prompt()
    with pytest.raises(ValueError):
        Prompt(tokens=[1], messages=[])
    case = EvaluationCase(Prompt(tokens=[1, 2, 3], sampling_params=SamplingParams(temperature=0.5, seed=3)),
                          BenchmarkMeta("b", "i0", {"answer": "7"}), EvaluationMeta(0, 1))
    g = Generated(case, {"finish_reason": "stop"}, "x")
    assert case.prompt.prompt_token_count == 3 and g.finish_reason == "stop"
    back = Generated.from_dict(json.loads(json.dumps(g.to_dict())))
    assert back.to_dict() == g.to_dict()


class _Tok:
    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True, **kw):
        return [1] * sum(len(m["content"].split()) for m in messages)

    def encode(self, text, add_special_tokens=False):
        return text.split()


def _write(path, rows):
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")


def test_boxed_math_and_multiple_choice_scoring(tmp_path):
    from playground.eval.benchmarks.math_boxed import AIME25Benchmark
    from playground.eval.benchmarks.multiple_choice import GPQADiamondBenchmark

    p = tmp_path / "aime.jsonl"
    _write(p, [{"dataset": "AIME2025", "messages": [{"role": "user", "content": "what is 1+1"}, {"role": "assistant", "content": ""}],
                "source_item": {"item_id": "q0", "answer": "\\frac{1}{2}"}},
               {"dataset": "AIME2025", "messages": [{"role": "user", "content": "q"}], "source_item": {"item_id": "q1", "answer": "42"}}])
    b = AIME25Benchmark(str(p), _Tok(), sample_per_prompt=2)
    b.symbolic_fallback = False
    cases = b.get_cases()
    assert len(cases) == 4 and len(cases[0].prompt.messages) == 1
    answers = ["so \\boxed{\\dfrac{1}{2}}", "\\boxed{3}", "I think \\boxed{42}", "no box 42"]
    res = [Generated(c, {"finish_reason": "stop"}, a) for c, a in zip(cases, answers)]
    m = b.evaluate(res)
    assert abs(m.score_avg - 0.5) < 1e-9 and abs(m.pass_at_k[1] - 0.5) < 1e-9 and m.pass_at_k[2] == 1.0
    p2 = tmp_path / "gpqa.jsonl"
    _write(p2, [{"dataset": "GPQA_DIAMOND", "messages": [{"role": "user", "content": "pick"}], "source_item": {"item_id": "g0", "answer": "C"}}])
    g = GPQADiamondBenchmark(str(p2), _Tok(), sample_per_prompt=3)
    out = [Generated(c, {"finish_reason": "stop"}, a) for c, a in
           zip(g.get_cases(), ["The answer is C.", "\\boxed{B} although C", "A or D... final: (c)"])]
    assert [g.is_correct(r) for r in out] == [True, False, True]


def test_benchmark_eval_config_runs_items(tmp_path):
    from playground.eval.benchmarks.multiple_choice import GPQADiamondBenchmark
    from steptronoss_b200.exp.gen_eval import BenchmarkEvalConfig
    from steptronoss_b200.generation.async_generation import SingleGenerationController
    from steptronoss_b200.generation.base_generatable import GenableItem

    p = tmp_path / "g.jsonl"
    _write(p, [{"dataset": "GPQA_DIAMOND", "messages": [{"role": "user", "content": "pick"}], "source_item": {"item_id": f"g{i}", "answer": "ABCD"[i % 4]}}
               for i in range(6)])

    class Canned(GenableItem):
        def __init__(self, case):
            super().__init__()
            self.case = case

        async def generate(self):
            return Generated(self.case, {"finish_reason": "stop"}, "answer: A")

    class Cfg(BenchmarkEvalConfig):
        def build_benchmarks(self):
            return [GPQADiamondBenchmark(str(p), _Tok(), sample_per_prompt=2)]

        def items_for(self, bench):
            return [Canned(c) for c in bench.get_cases()]

        def build_controller(self):
            c = SingleGenerationController()
            c.shutdown_orig, c.shutdown = c.shutdown, (lambda: None)
            return c

    cfg = Cfg()
    cfg.dump_dir, cfg.record_eval_rollout = str(tmp_path / "dump"), True
    out = cfg.eval()
    assert abs(out["GPQA_DIAMOND"].score_avg - 2 / 6) < 1e-9
    assert sum(1 for _ in open(tmp_path / "dump" / "GPQA_DIAMOND.jsonl")) == 12


def test_demo_record_round_trips_and_payload_shapes_are_plain_dicts():
    from steptronoss_b200.generation.base_benchmark import (ChatMessage, CompletionChoice, CompletionMessage, Generated,
                                                            GroundTruth, GroundTruthValue, build_demo_generated)

    g = build_demo_generated()
    assert g.response == "3" and g.case.benchmark.context == {"answer": "3"} and g.finish_reason == "unknown"
    again = Generated.from_dict(g.to_dict())
    assert again.case == g.case and again.response == "3"
    gt: GroundTruth = {"value": GroundTruthValue(item_id="q1", dataset="demo")}
    msg = ChatMessage(role="assistant", content="3", ground_truth=gt)
    choice = CompletionChoice(finish_reason="stop", message=CompletionMessage(content="3"), raw={"index": 0})
    assert msg == {"role": "assistant", "content": "3", "ground_truth": {"value": {"item_id": "q1", "dataset": "demo"}}}
    g.choice = choice
    assert g.finish_reason == "stop" and Generated.from_dict(g.to_dict()).choice == dict(choice)
