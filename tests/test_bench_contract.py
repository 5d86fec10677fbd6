"""bench.py: command-line defaults, layout parsing, the FLOP model, the clock-sample summary, the reference arm's
refusal line (what the driver reads must keep its shape)."""
import json
import os
import subprocess
import sys

import pytest

import bench


def test_defaults_follow_the_model(monkeypatch):
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    a = bench.parse()
    assert (a.gpus, a.steps, a.warmup, a.impl, a.model, a.seqs_per_gpu, a.seq_len) == (1, 3, 3, "ours", "qwen3_8b", 8, 8192)
    monkeypatch.setattr(sys, "argv", ["bench.py", "--model", "qwen3_30b_a3b", "--gpus", "8"])
    a = bench.parse()
    assert (a.seqs_per_gpu, a.seq_len, a.dispatcher, a.moe_capacity_factor) == (32, 4096, "peer", 0.0)   # 256 x 4096 at 8 GPUs
    assert a.seqs_per_micro_batch == 1
    monkeypatch.setattr(sys, "argv", ["bench.py", "--model", "qwen3_30b_a3b", "--seqs-per-micro-batch", "4"])
    assert bench.parse().seqs_per_micro_batch == 4
    monkeypatch.setattr(sys, "argv", ["bench.py", "--seqs-per-micro-batch", "3"])       # 8 sequences per GPU
    with pytest.raises(SystemExit):
        bench.parse()


def test_layouts():
    assert [bench.default_parallelism(n) for n in (1, 2, 4, 8)] == ["dp1", "tp2dp1", "tp4dp1", "tp4dp2"]
    assert bench.parse_parallelism("tp2cp2pp2") == {"tp": 2, "dp": 1, "pp": 2, "cp": 2, "ep": 1}
    assert bench.parse_parallelism("ep8dp8")["ep"] == 8


def test_flop_model_matches_a_hand_count():
    # Qwen3-8B: per token 6 x (dense parameters that multiply a token) + 6 x attention MACs at the average context
    dense = 36 * (4096 * (32 + 16) * 128 + 32 * 128 * 4096 + 3 * 4096 * 12288) + 151936 * 4096
    want = 6 * dense + 6 * 36 * 2 * 32 * 128 * 1000
    assert bench.model_flops_per_token(36, 4096, 32, 8, 128, 12288, 151936, 1000) == want
    moe = bench.model_flops_per_token(48, 2048, 32, 4, 128, 8 * 768, 151936, 2048, router_experts=128)
    assert moe > 6 * 48 * 3 * 2048 * 8 * 768                                    # the routed experts are in


def test_clock_summary_reads_reasons_and_median(tmp_path):
    p = tmp_path / "clocks.csv"
    p.write_text("0, 1965, 1965, 700.1, 0x0, Not Active, Not Active, Not Active, Not Active\n"
                 "0, 1500, 1965, 990.0, 0x4, Not Active, Not Active, Not Active, Active\n"
                 "0, 1400, 1965, 995.0, 0x4, Not Active, Not Active, Not Active, Active\n"
                 "garbage line\n")
    s = bench.ClockSampler(str(p), 1)
    s.proc = type("P", (), {"terminate": lambda self: None, "wait": lambda self, timeout=None: 0})()
    s.f = open(p)
    out = s.stop()
    assert out == {"sm_mhz": 1500.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    assert bench.ClockSampler(str(p), 1).stop()["reasons"] == ["unsampled"]     # never started


def test_reference_arm_says_why_it_cannot_run_the_moe_model():
    out = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--model", "qwen3_30b_a3b"],
                         capture_output=True, text=True, timeout=120, cwd=bench.ROOT)
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and "\n" not in line["unavailable"]


def test_run_all_lists_single_and_multi_rank_benchmarks(tmp_path):
    from benchmarks import run_all

    one = run_all.commands(str(tmp_path), 1, set())
    # the multi-rank benchmarks other than the MoE layer need two GPUs
    assert [n for n, _ in one] == ["gemm", "fp8_gemm", "attention", "moe", "muon", "moe_layer"]
    eight = dict(run_all.commands(str(tmp_path), 8, {"attention"}))
    assert set(eight) == {"gemm", "fp8_gemm", "moe", "muon", "moe_layer", "zero", "fused_tp", "cp_attention",
                          "peer_bandwidth"} and "--nproc-per-node=8" in eight["zero"]
    for cmd in list(dict(one).values()) + list(eight.values()):
        script = next(c for c in cmd if c.endswith(".py"))
        assert os.path.exists(script)
