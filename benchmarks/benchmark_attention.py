"""tcgen05 flash attention forward / backward throughput on Qwen3-8B shapes (32 query heads, 8 KV
heads, head_dim 128, packed documents), reported as a fraction of the measured bf16 peak with the
causal-halved FLOP count.  ``--library`` also times flash-attn 2 (the reference's kernel) when it is
importable.

    python benchmarks/benchmark_attention.py [--library]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from benchmarks.common import measured_peaks, time_cuda  # noqa: E402
from steptronoss_b200.ops import native  # noqa: E402
from steptronoss_b200.ops.attention import attention  # noqa: E402


def causal_flops(lens, hq, d):
    # QK^T and PV, 2 flops per MAC, causal half
    return sum(4.0 * hq * d * (l * (l + 1) / 2.0) for l in lens)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--library", action="store_true")
    ap.add_argument("--only", default=None, help="comma list of case names")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    peak = measured_peaks()["bf16_tflops"]
    hq, hkv, d = 32, 8, 128
    cases = {"1x8192": [8192], "2x4096": [4096, 4096], "mixed": [3000, 700, 2500, 1992], "8x1024": [1024] * 8}
    for name, lens in cases.items():
        if args.only and name not in args.only.split(","):
            continue
        T = sum(lens)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
        q = torch.randn(T, hq, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        k = torch.randn(T, hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        v = torch.randn(T, hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        g = torch.randn(T, hq, d, device="cuda", dtype=torch.bfloat16)
        fl = causal_flops(lens, hq, d)
        tf = time_cuda(lambda: attention(q, k, v, cu, cu, max(lens)), iters=args.iters)
        o = attention(q, k, v, cu, cu, max(lens))

        def bwd():
            o.backward(g, retain_graph=True)

        tb = time_cuda(bwd, iters=args.iters)
        row = {"case": name, "tokens": T, "fwd_ms": tf["best_ms"], "fwd_tflops": fl / tf["best_ms"] / 1e9,
               "fwd_frac_of_measured_peak": fl / tf["best_ms"] / 1e9 / peak, "bwd_ms": tb["best_ms"],
               "bwd_tflops_useful": 2.5 * fl / tb["best_ms"] / 1e9,
               "bwd_frac_of_measured_peak": 2.5 * fl / tb["best_ms"] / 1e9 / peak}
        if args.library:
            try:
                from flash_attn import flash_attn_varlen_func

                ql, kl, vl = (t.detach().clone().requires_grad_() for t in (q, k, v))
                tl = time_cuda(lambda: flash_attn_varlen_func(ql, kl, vl, cu, cu, max(lens), max(lens), causal=True))
                ol = flash_attn_varlen_func(ql, kl, vl, cu, cu, max(lens), max(lens), causal=True)
                tlb = time_cuda(lambda: ol.backward(g, retain_graph=True))
                row["library_fwd_ms"], row["library_bwd_ms"] = tl["best_ms"], tlb["best_ms"]
            except Exception as e:  # flash-attn missing or not built for this GPU
                row["library_error"] = f"{type(e).__name__}: {e}"[:200]
        print(json.dumps(row), flush=True)
    native.raise_if_kernel_error()


if __name__ == "__main__":
    main()
