"""tcgen05 GEMM throughput on the projection shapes of Qwen3-8B (8192 tokens), forward / dgrad /
wgrad layouts, against the measured cuBLAS bf16 peak.  ``--library`` also times torch.matmul on the
same shapes for orientation.

    python benchmarks/benchmark_gemm.py [--library] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from benchmarks.common import measured_peaks, time_cuda  # noqa: E402
from steptronoss_b200.ops import gemm  # noqa: E402
from steptronoss_b200.ops import native  # noqa: E402

SHAPES = {  # name: (tokens M, out N, in K)
    "qkv": (8192, 6144, 4096),
    "o": (8192, 4096, 4096),
    "w1": (8192, 24576, 4096),
    "w2": (8192, 4096, 12288),
    "head_chunk": (2048, 151936, 4096),
    "qkv_tp4": (8192, 1536, 4096),
    "w2_tp4": (8192, 4096, 3072),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--library", action="store_true")
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    peaks = measured_peaks()
    peak = peaks["bf16_tflops"]
    rows = []
    for name, (M, N, K) in SHAPES.items():
        if args.only and name not in args.only.split(","):
            continue
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        g = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
        dw = torch.zeros(N, K, device="cuda", dtype=torch.float32)
        flops = 2.0 * M * N * K
        cases = {
            "fwd": lambda: gemm(x, w, out=y),
            "dgrad": lambda: gemm(g, w, b_mn_major=True, out=dx),
            "wgrad_acc_fp32": lambda: gemm(g, x, a_mn_major=True, b_mn_major=True, out=dw, accumulate=True),
        }
        for cname, fn in cases.items():
            t = time_cuda(fn)
            tf = flops / (t["best_ms"] * 1e-3) / 1e12
            row = {"shape": name, "case": cname, "M": M, "N": N, "K": K, "best_ms": t["best_ms"],
                   "median_ms": t["median_ms"], "tflops": tf, "frac_of_measured_peak": tf / peak}
            if args.library:
                lib_fn = {"fwd": lambda: torch.matmul(x, w.t()), "dgrad": lambda: torch.matmul(g, w),
                          "wgrad_acc_fp32": lambda: torch.matmul(g.t(), x)}[cname]
                tl = time_cuda(lib_fn)
                row["library_ms"] = tl["best_ms"]
                row["library_tflops"] = flops / (tl["best_ms"] * 1e-3) / 1e12
            rows.append(row)
            print(json.dumps(row), flush=True)
        del x, w, g, y, dx, dw
        torch.cuda.empty_cache()
    native.raise_if_kernel_error()
    if args.json:
        json.dump({"peaks": peaks, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
