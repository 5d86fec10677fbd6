"""Block-scaled fp8 (e4m3, 1 x 128 activation and 128 x 128 weight scales) grouped GEMM of the routed experts against
the bf16 grouped GEMM on the same rows (1 x B200).

Shapes of the MoE layer micro-benchmark: 4096 tokens x top-8 = 32768 expert rows of hidden 4096 spread over 16 local
experts, gate/up (N = 3072) and down (K = 1536) projections; and of Qwen3-30B-A3B (hidden 2048, expert width 768).
Times are CUDA events, best of ``--iters`` after 3 warm-up launches, 256 MB written between launches to flush L2.
The fp8 row times the product alone (operands already quantised); the quantisation kernels are timed separately.

    python benchmarks/benchmark_fp8_gemm.py --json out.json
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    from benchmarks.common import measured_peaks, time_cuda
    from steptronoss_b200.ops import fp8, native
    from steptronoss_b200.ops.grouped import grouped_gemm_rows, tile_groups_from_offsets

    dev = torch.device("cuda")
    peak = measured_peaks()["bf16_tflops"]
    rows_out = []
    cases = [("moe_layer gate_up", 32768, 3072, 4096, 16), ("moe_layer down", 32768, 4096, 1536, 16),
             ("qwen3_30b gate_up", 32768, 1536, 2048, 16), ("qwen3_30b down", 32768, 2048, 768, 16),
             ("dense 8192x4096x4096", 8192, 4096, 4096, 1)]
    for name, M, N, K, G in cases:
        torch.manual_seed(0)
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(G, N, K, device=dev) * 0.02).to(torch.bfloat16)
        offsets = torch.arange(G + 1, device=dev, dtype=torch.int32) * (M // G)
        tg = tile_groups_from_offsets(offsets, M)
        xq, sx = fp8.quantize_rows_1x128(x)
        wq, sw = fp8.quantize_blocks_128x128(w.view(G * N, K))
        flops = 2.0 * M * N * K
        t_bf16 = time_cuda(lambda: grouped_gemm_rows(x, w, offsets, tile_group=tg), iters=args.iters)["best_ms"]
        t_fp8 = time_cuda(lambda: fp8.grouped_gemm_fp8(xq, sx, wq, sw, offsets, G, tile_group=tg), iters=args.iters)["best_ms"]
        t_qx = time_cuda(lambda: fp8.quantize_rows_1x128(x), iters=args.iters)["best_ms"]
        t_qw = time_cuda(lambda: fp8.quantize_blocks_128x128(w.view(G * N, K)), iters=args.iters)["best_ms"]
        y8 = fp8.grouped_gemm_fp8(xq, sx, wq, sw, offsets, G, tile_group=tg).float()
        y16 = grouped_gemm_rows(x, w, offsets, tile_group=tg).float()
        row = {"case": name, "M": M, "N": N, "K": K, "groups": G, "bf16_ms": t_bf16, "fp8_ms": t_fp8,
               "bf16_tflops": flops / t_bf16 / 1e9, "fp8_tflops": flops / t_fp8 / 1e9,
               "fp8_over_measured_bf16_peak": flops / t_fp8 / 1e9 / peak, "quant_x_ms": t_qx, "quant_w_ms": t_qw,
               "rel_diff_fp8_vs_bf16": float((y8 - y16).norm() / y16.norm())}
        rows_out.append(row)
        print(json.dumps(row), flush=True)
    torch.cuda.synchronize()
    native.raise_if_kernel_error()
    if args.json:
        json.dump({"peak_bf16_tflops": peak, "rows": rows_out}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
