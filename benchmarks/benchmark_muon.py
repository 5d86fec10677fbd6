"""Newton-Schulz orthogonalisation of the Qwen3-8B hidden matrices: this repository's ``zeropower`` (bf16 on the
tcgen05 GEMM) against the reference's own ``zeropower`` (``steptronoss/optimizer/_helpers.py:66-98``, fp16 on
``torch.matmul``), 5 iterations with the coefficients (3.4445, -4.7750, 2.0315), 1 x B200.

Matrices at full size (what Muon works on after the gather of the TP shards) and as the per-rank shapes of TP=2.
CUDA events, best of ``--iters`` after 2 warm-up calls.  The reference function is imported from the unmodified tree
under ``baseline/_ref``; without that tree only this repository's column is printed.

    python benchmarks/benchmark_muon.py --json out.json
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _reference_zeropower():
    path = os.path.join(ROOT, "baseline", "_ref", "steptronoss", "optimizer", "_helpers.py")
    if not os.path.exists(path):
        return None
    try:
        spec = importlib.util.spec_from_file_location("ref_muon_helpers", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod.zeropower
    except Exception as e:     # the helpers import only torch, but stay honest if that changes
        print(f"reference helpers not importable: {e}", flush=True)
        return None


def _time(fn, iters):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b))
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    from benchmarks.common import measured_peaks
    from steptronoss_b200.optim import zeropower as zp

    ref = _reference_zeropower()
    coeffs = (3.4445, -4.7750, 2.0315)
    peak = measured_peaks()["bf16_tflops"]
    dev = torch.device("cuda")
    shapes = [("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 24576, 4096), ("down", 4096, 12288),
              ("qkv, TP=2 shard", 3072, 4096), ("down, TP=2 shard", 4096, 6144)]
    rows = []
    for name, r, c in shapes:
        g = torch.randn(r, c, device=dev, dtype=torch.bfloat16)
        m, n = min(r, c), max(r, c)
        flops = 5 * (4.0 * m * m * n + 2.0 * m * m * m)
        ours = _time(lambda: zp.zeropower(g, 5, True, coeffs), args.iters)
        row = {"matrix": name, "rows": r, "cols": c, "ours_ms": ours, "ours_tflops": flops / ours / 1e9,
               "ours_frac_of_measured_peak": flops / ours / 1e9 / peak}
        if ref is not None:
            t = _time(lambda: ref(g, 5, True, coeffs), args.iters)
            row["reference_ms"] = t
            row["speedup"] = t / ours
            a = zp.zeropower(g, 5, True, coeffs).float()
            b = ref(g, 5, True, coeffs).float()
            row["rel_diff"] = float((a - b).norm() / b.norm())
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.json:
        json.dump({"peak_bf16_tflops": peak, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
