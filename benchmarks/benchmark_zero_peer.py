"""ZeRO-1 step over peer memory against its NCCL statement, on a synthetic bucket (one rank per GPU of one node).

Times, per optimizer step of a flat bucket of ``--numel`` fp32 gradients / bf16 parameters:

* peer: publish + ``stb_zero_reduce`` (owner sums its shard over all ranks' buffers, squared norm as a by-product)
  + ``stb_adam_push`` (Adam on the shard, bf16 result stored into every rank's parameter buffer) + publish + wait;
* nccl: ``reduce_scatter_tensor`` + squared norm of the shard + ``stb_adam`` + ``all_gather_into_tensor``.

Roofline of the peer path per rank: NVLink carries (W-1)/W x numel x 4 bytes in (gradient shards read from peers)
and (W-1)/W x numel x 2 bytes out (parameter shard stored to peers); HBM carries the Adam state of the shard
(numel / W x 30 bytes).  Both results must agree (parameters after the step compared).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/benchmark_zero_peer.py
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--numel", type=int, default=1 << 28)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()

    from benchmarks.common import measured_peaks
    from steptronoss_b200.exp.base_exp import ParallelConfig
    from steptronoss_b200.ops import native
    from steptronoss_b200.optim import peer_zero
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    PM.set_mesh(ParallelConfig())                      # pure data parallel
    W, rank = PM.world_size, PM.world_rank
    dev = torch.device("cuda", torch.cuda.current_device())
    lib = native.load()
    n = args.numel // (W * 256) * (W * 256)
    shard = n // W
    lo, hi = rank * shard, (rank + 1) * shard
    assert peer_zero.group_supported("DP"), "needs 2-8 GPUs of one node over NCCL"
    pz = peer_zero.PeerZeroGroup("DP")

    class Bucket:  # what PeerZeroGroup reads from a bucket
        def own_range(self):
            return lo, hi

    b = Bucket()
    b.grad_buf = pz.allocate("k", n, torch.float32, "grad")
    b.param_buf = pz.allocate("k", n, torch.bfloat16, "param")
    pz.finish_allocation()
    g = torch.Generator(device=dev).manual_seed(rank)
    grads = torch.randn(n, device=dev, generator=g) * 1e-2
    params0 = (torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(99)) * 0.02).bfloat16()
    chunk = 1 << 16
    table = torch.frombuffer(bytearray(b"".join(struct.pack("<qiffi", o, min(chunk, shard - o), 1.0, 0.1, 0)
                                                 for o in range(0, shard, chunk))), dtype=torch.uint8).to(dev)
    n_chunks = (shard + chunk - 1) // chunk
    scalars = torch.tensor([0.0, 0.0, 1.0, 1.0], device=dev)
    sq = torch.zeros(1, device=dev)
    hp = dict(lr=1e-3, b1=0.9, b2=0.95, eps=1e-8, bc1=0.1, bc2=0.05, gs=1.0 / W)

    def fresh_state():
        return params0[lo:hi].float(), torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)

    ptrs = pz.param_ptrs("k", b)

    def peer_step(state):
        master, m, v = state
        pz.begin_step()
        pz.reduce("k", b, 1.0, sq, accumulate=False)
        rc = lib.stb_adam_push(master.data_ptr(), b.grad_buf[lo:hi].data_ptr(), m.data_ptr(), v.data_ptr(), ptrs, W,
                               table.data_ptr(), n_chunks, scalars.data_ptr(), hp["lr"], hp["b1"], hp["b2"], hp["eps"],
                               hp["bc1"], hp["bc2"], hp["gs"], 0, native.stream())
        native.check(rc, "adam_push")
        pz.end_step()
        pz.wait_params()

    gbuf = torch.empty(n, device=dev)
    pbuf = torch.empty(n, device=dev, dtype=torch.bfloat16)
    partial = torch.empty(lib.stb_sqnorm_grid(), device=dev)
    grp = PM.group_of("DP")

    def nccl_step(state):
        master, m, v = state
        dist.reduce_scatter_tensor(gbuf[lo:hi], gbuf, group=grp)
        native.check(lib.stb_sqnorm(gbuf[lo:hi].data_ptr(), shard, partial.data_ptr(), sq.data_ptr(), 0, native.stream()), "sqnorm")
        rc = lib.stb_adam(master.data_ptr(), gbuf[lo:hi].data_ptr(), m.data_ptr(), v.data_ptr(), pbuf[lo:hi].data_ptr(),
                          table.data_ptr(), n_chunks, scalars.data_ptr(), hp["lr"], hp["b1"], hp["b2"], hp["eps"],
                          hp["bc1"], hp["bc2"], hp["gs"], 0, native.stream())
        native.check(rc, "adam")
        dist.all_gather_into_tensor(pbuf, pbuf[lo:hi], group=grp)

    def timed(step, refill):
        times = []
        for it in range(args.iters + 2):
            state = fresh_state()
            refill()
            torch.cuda.synchronize()
            dist.barrier()
            a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step(state)
            e.record()
            torch.cuda.synchronize()
            if it >= 2:
                times.append(a.elapsed_time(e))
        t = torch.tensor([min(times)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def refill_peer():
        b.grad_buf.copy_(grads)
        b.param_buf.copy_(params0)

    def refill_nccl():
        gbuf.copy_(grads)
        pbuf.copy_(params0)

    ms_peer = timed(peer_step, refill_peer)
    sq_peer = float(sq)
    ms_nccl = timed(nccl_step, refill_nccl)
    err = float((b.param_buf.float() - pbuf.float()).abs().max())
    rel_sq = abs(sq_peer - float(sq)) / max(float(sq), 1e-30)
    torch.cuda.synchronize()
    native.raise_if_kernel_error()
    peaks = measured_peaks()
    link = 770.0                                             # measured peer copy, GB/s per direction
    t_link = (W - 1) / W * n * 4 / (link * 1e9) * 1e3        # inbound gradient shards dominate (outbound is half)
    t_hbm = (shard * 30 + n * 4 / W * (W - 1)) / (peaks["hbm_gbs"] * 1e9) * 1e3
    row = {"bench": "zero1_step", "ranks": W, "numel": n, "peer_ms": ms_peer, "nccl_ms": ms_nccl,
           "speedup": ms_nccl / ms_peer, "roofline_ms": max(t_link, t_hbm), "peer_frac_of_roofline": max(t_link, t_hbm) / ms_peer,
           "max_param_diff": err, "sqnorm_rel_diff": rel_sq}
    assert err <= 1e-2 and rel_sq < 1e-4, row
    dist.barrier()
    if rank == 0:
        print(json.dumps(row), flush=True)
        if args.json:
            json.dump(row, open(args.json, "w"))


if __name__ == "__main__":
    main()
