"""What one GPU moves to / from its peers over NVLink with the access patterns of the fused kernels.

Every rank copies ``--mb`` MiB between its own memory and the peer-mapped buffers of the other ranks (split evenly
over the peers), all ranks at once, and reports GB/s per direction per GPU (max time over ranks):

* ``push_st``    16-byte loads from local memory, 16-byte stores into the peer (the all-gather push of
  ``csrc/gemm_tp_sm100.cu``, the MoE dispatch, the ZeRO-1 parameter push);
* ``push_bulk``  ``cp.async.bulk`` local -> shared memory -> ``cp.async.bulk`` into the peer, per chunk size;
* ``pull_ld``    16-byte loads from the peer, stores to local memory (the ZeRO-1 gradient reduce);
* ``pull_bulk``  ``cp.async.bulk`` from the peer into shared memory, ``cp.async.bulk`` to local memory;
* ``memcpy``     ``cudaMemcpyAsync`` (copy engine) between the same buffers, for reference;

each over a range of grid sizes, which shows how many SMs a transfer needs to saturate the links.  The reference
prints an NCCL all-reduce bandwidth probe at start-up (``steptronoss/utils/utils.py:377-433``); this is the
corresponding probe for peer memory.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/benchmark_peer_bandwidth.py
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=192, help="MiB moved per rank and direction")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--ring-mb", type=int, default=32, help="MiB per rank moved by the ring variants")
    ap.add_argument("--ring-only", action="store_true", help="skip the plain / bulk sweeps")
    ap.add_argument("--no-ring", action="store_true", help="skip the ring variants")
    ap.add_argument("--json", default=None)
    args = ap.parse_args()

    from steptronoss_b200.ops import native
    from steptronoss_b200.parallel import symm
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    PM.new_parallel("TP", [list(range(PM.world_size))])
    W, rank = PM.world_size, PM.world_rank
    dev = torch.device("cuda", torch.cuda.current_device())
    lib = native.load()
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    native.register_signature("stb_peer_copy", [P, P, L, I, I, I, P, P])
    peers = [(rank + d) % W for d in range(1, W)]
    per_peer = (args.mb << 20) // len(peers) // 4096 * 4096
    total = per_peer * len(peers)
    buf = symm.SymmetricBuffer(total, PM.group_of("TP"), lib)     # every rank's landing / source zone
    local = torch.empty(total, dtype=torch.uint8, device=dev).random_(0, 255)
    buf.own_tensor().copy_(local)
    torch.cuda.synchronize()
    dist.barrier()
    status = native.status_word(dev)
    side = [torch.cuda.Stream() for _ in peers]

    def run(push: bool, bulk: int, grid: int, chunk: int):
        # one launch per peer on its own stream, each with grid / (W-1) CTAs
        g = max(1, grid // len(peers))
        cur = torch.cuda.current_stream()
        for i, p in enumerate(peers):
            side[i].wait_stream(cur)
            off = i * per_peer
            # push: my local slice i lands in the peer's zone at the offset reserved for me; pull: the reverse
            their_off = ((rank - p) % W - 1) * per_peer if push else off
            src = local.data_ptr() + off if push else buf.ptrs[p] + their_off
            dst = buf.ptrs[p] + their_off if push else local.data_ptr() + off
            rc = lib.stb_peer_copy(src, dst, per_peer, g, bulk, chunk, status.data_ptr(), side[i].cuda_stream)
            native.check(rc, "stb_peer_copy")
        for s in side:
            cur.wait_stream(s)

    cudart = ctypes.CDLL("libcudart.so.12")
    cudart.cudaMemcpyAsync.argtypes = [P, P, ctypes.c_size_t, I, P]

    def run_memcpy(push: bool):
        cur = torch.cuda.current_stream()
        for i, p in enumerate(peers):
            side[i].wait_stream(cur)
            off = i * per_peer
            their_off = ((rank - p) % W - 1) * per_peer if push else off
            src = local.data_ptr() + off if push else buf.ptrs[p] + their_off
            dst = buf.ptrs[p] + their_off if push else local.data_ptr() + off
            rc = cudart.cudaMemcpyAsync(dst, src, per_peer, 4, side[i].cuda_stream)   # 4 = cudaMemcpyDefault
            assert rc == 0, rc
        for s in side:
            cur.wait_stream(s)

    def timed(fn):
        for _ in range(2):
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
        return total / (float(t.item()) * 1e-3) / 1e9

    res = {"ranks": W, "mib_per_rank": total >> 20, "gbs": {}}
    for grid in (() if args.ring_only else (16, 32, 64, 148, 296)):
        res["gbs"][f"push_st_g{grid}"] = timed(lambda: run(True, 0, grid, 0))
        res["gbs"][f"pull_ld_g{grid}"] = timed(lambda: run(False, 0, grid, 0))
    for chunk in (() if args.ring_only else (2048, 8192, 32768)):
        for grid in (16, 32, 64, 148):
            res["gbs"][f"push_bulk_c{chunk}_g{grid}"] = timed(lambda: run(True, 1, grid, chunk))
            res["gbs"][f"pull_bulk_c{chunk}_g{grid}"] = timed(lambda: run(False, 1, grid, chunk))
    # the ring of the fused kernels at their transfer size, extras switched on one by one (`--ring-mb` per rank)
    native.register_signature("stb_peer_copy_ring", [P, P, P, P, L, I, I, I, I, P, P])
    ring_bytes = min(per_peer, (args.ring_mb << 20) // len(peers) // 4096 * 4096)
    scratch = torch.empty(ring_bytes, dtype=torch.uint8, device=dev)
    flags = symm.SymmetricBuffer(4096, PM.group_of("TP"), lib)

    def run_ring(grid, stages, feat):
        g = max(1, grid // len(peers))
        cur = torch.cuda.current_stream()
        for i, p in enumerate(peers):
            side[i].wait_stream(cur)
            their_off = ((rank - p) % W - 1) * per_peer
            rc = lib.stb_peer_copy_ring(local.data_ptr() + i * per_peer, buf.ptrs[p] + their_off, scratch.data_ptr(),
                                        flags.ptrs[p], ring_bytes, g, 32768, stages, feat, status.data_ptr(),
                                        side[i].cuda_stream)
            native.check(rc, "stb_peer_copy_ring")
        for s in side:
            cur.wait_stream(s)

    def timed_ring(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        beg.record()
        for _ in range(10):
            fn()
        end.record()
        torch.cuda.synchronize()
        t = torch.tensor([beg.elapsed_time(end) / 10], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return {"us": float(t.item()) * 1e3, "gbs": ring_bytes * len(peers) / (float(t.item()) * 1e-3) / 1e9}

    res["ring"] = {"mib_per_rank": ring_bytes * len(peers) >> 20}
    for grid in (() if args.no_ring else (16, 20, 32)):
        for stages in (4, 6):
            for feat in (0, 1, 2, 3, 4, 8, 15):
                res["ring"][f"g{grid}_s{stages}_f{feat}"] = timed_ring(lambda: run_ring(grid, stages, feat))
    res["gbs"]["memcpy_push"] = timed(lambda: run_memcpy(True))
    res["gbs"]["memcpy_pull"] = timed(lambda: run_memcpy(False))
    # correctness of the last push: what landed in my zone from each peer equals that peer's source slice
    run(True, 1, 64, 8192)
    torch.cuda.synchronize()
    dist.barrier()
    mine = buf.own_tensor()
    gathered = [torch.empty_like(local) for _ in range(W)]
    dist.all_gather(gathered, local)
    ok = True
    for p in peers:
        # peer p pushed its slice i_p (the index of me in p's peer list) to my offset ((p - me) % W - 1) * per_peer
        i_p = (rank - p) % W - 1
        mine_off = ((p - rank) % W - 1) * per_peer
        ok = ok and torch.equal(mine[mine_off: mine_off + per_peer], gathered[p][i_p * per_peer: (i_p + 1) * per_peer])
    res["push_landed_correctly"] = bool(ok)
    native.raise_if_kernel_error()
    dist.barrier()
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
        if args.json:
            with open(args.json, "w") as f:
                json.dump(res, f, indent=1)
    torch.cuda.synchronize()
    dist.barrier()
    buf.release()
    flags.release()
    dist.barrier()


if __name__ == "__main__":
    main()
