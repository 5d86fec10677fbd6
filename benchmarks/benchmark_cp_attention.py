"""Context-parallel attention: keys gathered over peer memory and addressed by global position inside the kernels,
against the packed-keys statement over NCCL (all-gather, row gather per half, variable-length attention, index-add and
reduce-scatter in the backward).  One rank per GPU, CP = world size, Qwen3-8B heads (32 q / 8 kv, head_dim 128).

CUDA events on the launching stream, 3 warm-up + ``--iters`` timed calls, max over ranks.  Roofline target of one
call = the slower of (causal FLOPs of this rank / measured cuBLAS bf16 peak) and (K/V bytes that must arrive over
NVLink / 770 GB/s).

    NCCL_NVLS_ENABLE=0 python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29721 benchmarks/benchmark_cp_attention.py --seq-len 32768 --json out.json
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq-len", type=int, default=32768, help="tokens of the whole sequence (all CP ranks)")
    ap.add_argument("--docs", type=int, default=1, help="equal packed documents in the sequence")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()

    from benchmarks.common import measured_peaks
    from steptronoss_b200.exp.base_exp import ParallelConfig
    from steptronoss_b200.ops import native
    from steptronoss_b200.parallel import context_parallel as cpm
    from steptronoss_b200.parallel import symm
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    mesh = ParallelConfig()
    mesh.context_parallel_size = PM.world_size
    PM.set_mesh(mesh)
    cp, rank = PM.size_of("CP"), PM.rank_in("CP")
    dev = torch.device("cuda", torch.cuda.current_device())
    peak = measured_peaks()["bf16_tflops"] * 1e12
    T, hq, hkv, D = args.seq_len, args.heads, args.kv_heads, 128
    rows = T // cp
    cu = None
    if args.docs > 1:
        cu = torch.tensor([i * (T // args.docs) for i in range(args.docs)] + [T], dtype=torch.int32, device=dev)
    meta = cpm.build_cp_meta(cu, T, device=dev)
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    q = torch.randn(rows, hq, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
    k = torch.randn(rows, hkv, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
    v = torch.randn(rows, hkv, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
    do = torch.randn(rows, hq, D, device=dev, generator=g).to(torch.bfloat16)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        beg.record()
        for _ in range(args.iters):
            fn()
        end.record()
        torch.cuda.synchronize()
        t = torch.tensor([beg.elapsed_time(end) / args.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def fwd():
        with torch.no_grad():
            return cpm.cp_attention(q, k, v, meta, causal=True)

    def fwd_bwd():
        for t in (q, k, v):
            t.grad = None
        cpm.cp_attention(q, k, v, meta, causal=True).backward(do)

    # causal FLOPs of the whole sequence (documents of equal length), split evenly by the load-balanced layout
    doc = T // args.docs
    flops_fwd = args.docs * 4.0 * hq * D * doc * doc / 2 / cp
    kv_bytes = (cp - 1) * rows * 2 * hkv * D * 2
    res = {"cp": cp, "seq_len": T, "docs": args.docs, "rows_per_rank": rows, "kv_bytes_in": kv_bytes}
    for name, peer in (("peer", True), ("packed_nccl", False)):
        cpm.PEER_PATH = peer
        if peer:
            assert cpm._peer_path_ok(q, k, v, meta), "peer path unavailable"
        f = timed(fwd)
        fb = timed(fwd_bwd)
        res[name] = {"fwd_ms": f, "fwd_bwd_ms": fb, "bwd_ms": fb - f}
    tgt_f = max(flops_fwd / peak, kv_bytes / (NVLINK_GBS * 1e9)) * 1e3
    tgt_b = max(2.5 * flops_fwd / peak, 2 * kv_bytes / (NVLINK_GBS * 1e9)) * 1e3   # re-gather + dK/dV back
    res["target_fwd_ms"], res["target_bwd_ms"] = tgt_f, tgt_b
    res["peer"]["fwd_frac_of_roofline"] = tgt_f / res["peer"]["fwd_ms"]
    res["peer"]["bwd_frac_of_roofline"] = tgt_b / res["peer"]["bwd_ms"]
    torch.cuda.synchronize()
    native.raise_if_kernel_error()
    dist.barrier()
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
        if args.json:
            json.dump(res, open(args.json, "w"), indent=1)
    symm.shutdown()
    dist.barrier()


if __name__ == "__main__":
    main()
