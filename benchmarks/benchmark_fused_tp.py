"""Fused GEMM + collective kernels on the Qwen3-8B sequence-parallel projections, one rank per GPU (TP = world size).

For 8192 tokens per TP group: all-gather -> qkv, all-gather -> gate/up, o_proj -> reduce-scatter, down ->
reduce-scatter and the gather-only launch, each against the NCCL collective + the same tcgen05 GEMM and against the
GEMM alone.  CUDA events on the launching stream, 3 warm-up + ``--iters`` timed launches, max over ranks.  With
``--trace`` the kernels' own per-CTA phase stamps (``%globaltimer``) are reported as well.

Roofline target of a fused kernel = the slower of FLOPs / measured cuBLAS bf16 peak and the bytes that must cross
NVLink / 770 GB/s (measured peer copy per direction per GPU); ``frac`` = target / achieved.

    NCCL_NVLS_ENABLE=0 python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29711 benchmarks/benchmark_fused_tp.py --json out.json
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBS = 770.0


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    beg.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    t = torch.tensor([beg.elapsed_time(end) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=12288)
    ap.add_argument("--qkv", type=int, default=6144)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--trace", action="store_true")
    ap.add_argument("--json", default=None)
    args = ap.parse_args()

    from benchmarks.common import measured_peaks
    from steptronoss_b200.ops import native
    from steptronoss_b200.ops.gemm import gemm
    from steptronoss_b200.parallel import symm
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    PM.new_parallel("TP", [list(range(PM.world_size))])
    group = PM.group_of("TP")
    rank, tp = PM.rank_in("TP"), PM.size_of("TP")
    dev = torch.device("cuda", torch.cuda.current_device())
    assert symm.enabled("TP"), "peer-memory arena could not be created"
    peak = measured_peaks()["bf16_tflops"] * 1e12
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    tokens, hidden = args.tokens, args.hidden
    rows = tokens // tp
    link_bytes = (tp - 1) * rows * hidden * 2            # every collective here moves rows of `hidden` bf16
    rows_out = []

    def record(name, m, n, k, fused, unfused, gemm_only, trace=None):
        target_ms = max(2.0 * m * n * k / peak, link_bytes / (NVLINK_GBS * 1e9)) * 1e3
        row = {"op": name, "tp": tp, "M": m, "N": n, "K": k, "nvlink_mb": link_bytes / 1e6, "target_us": target_ms * 1e3,
               "fused_us": fused * 1e3, "frac_of_roofline": target_ms / fused, "nccl_plus_gemm_us": unfused * 1e3,
               "gemm_only_us": gemm_only * 1e3 if gemm_only else None}
        if trace:
            row["trace"] = trace
        rows_out.append(row)
        if rank == 0:
            shown = {k: v for k, v in row.items() if k != "trace"}
            print(json.dumps(shown), flush=True)

    def traced(fn):
        if not args.trace:
            return None
        symm.trace(True)
        fn()
        torch.cuda.synchronize()
        out = symm.trace_summary()
        out["rows"] = symm.trace_rows()
        symm.trace(False)
        return out

    for name, n in (("ag_qkv", args.qkv // tp), ("ag_gate_up", 2 * args.ffn // tp)):
        x = torch.randn(rows, hidden, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(n, hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        full = torch.empty((tokens, hidden), dtype=x.dtype, device=dev)

        def nccl():
            dist.all_gather_into_tensor(full, x, group=group)
            return gemm(full, w)

        fused = _time(lambda: symm.all_gather_gemm(x, w, "TP"), args.iters)
        record(name, tokens, n, hidden, fused, _time(nccl, args.iters), _time(lambda: gemm(full, w), args.iters),
               traced(lambda: symm.all_gather_gemm(x, w, "TP")))
    # backward of the row projections: all-gather of the output gradient feeding dgrad (weight stored [K][N])
    for name, n in (("ag_dgrad_o_proj", hidden // tp), ("ag_dgrad_down", args.ffn // tp)):
        x = torch.randn(rows, hidden, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(hidden, n, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        full = torch.empty((tokens, hidden), dtype=x.dtype, device=dev)

        def nccl():
            dist.all_gather_into_tensor(full, x, group=group)
            return gemm(full, w, b_mn_major=True)

        fused = _time(lambda: symm.all_gather_gemm(x, w, "TP", b_mn_major=True), args.iters)
        record(name, tokens, n, hidden, fused, _time(nccl, args.iters),
               _time(lambda: gemm(full, w, b_mn_major=True), args.iters))
    xg = torch.randn(rows, hidden, device=dev, generator=g).to(torch.bfloat16)
    fullg = torch.empty((tokens, hidden), dtype=xg.dtype, device=dev)
    fused = _time(lambda: symm.all_gather_gemm(xg, None, "TP"), args.iters)
    record("gather_only", tokens, 0, hidden, fused,
           _time(lambda: dist.all_gather_into_tensor(fullg, xg, group=group), args.iters), None,
           traced(lambda: symm.all_gather_gemm(xg, None, "TP")))
    for name, k in (("rs_o_proj", hidden // tp), ("rs_down", args.ffn // tp)):
        a = torch.randn(tokens, k, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(hidden, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        out = torch.empty((rows, hidden), dtype=a.dtype, device=dev)

        def nccl():
            y = gemm(a, w)
            dist.reduce_scatter_tensor(out, y, group=group)
            return out

        fused = _time(lambda: symm.gemm_reduce_scatter(a, w, "TP"), args.iters)
        record(name, tokens, hidden, k, fused, _time(nccl, args.iters), _time(lambda: gemm(a, w), args.iters),
               traced(lambda: symm.gemm_reduce_scatter(a, w, "TP")))
    # backward of the column projections: dgrad (weight stored [K][N]) -> reduce-scatter
    for name, k in (("rs_dgrad_qkv", args.qkv // tp), ("rs_dgrad_gate_up", 2 * args.ffn // tp)):
        a = torch.randn(tokens, k, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(k, hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        out = torch.empty((rows, hidden), dtype=a.dtype, device=dev)

        def nccl():
            y = gemm(a, w, b_mn_major=True)
            dist.reduce_scatter_tensor(out, y, group=group)
            return out

        fused = _time(lambda: symm.gemm_reduce_scatter(a, w, "TP", b_mn_major=True), args.iters)
        record(name, tokens, hidden, k, fused, _time(nccl, args.iters),
               _time(lambda: gemm(a, w, b_mn_major=True), args.iters))
    torch.cuda.synchronize()
    native.raise_if_kernel_error()
    dist.barrier()
    if rank == 0 and args.json:
        json.dump({"tp": tp, "peak_bf16_tflops": peak / 1e12, "nvlink_gbs": NVLINK_GBS, "rows": rows_out},
                  open(args.json, "w"), indent=1)
    symm.shutdown()
    dist.barrier()


if __name__ == "__main__":
    main()
