"""Worker for the peer-memory MoE dispatcher test (torch.distributed.run, one rank per GPU): the peer
dispatcher and the all-to-all dispatcher must give the same block output and gradients."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def _run(disp, x, ids, w, per_rank):
    x = x.clone().requires_grad_()
    w = w.clone().requires_grad_()
    xr, ids_r, w_r = disp.dispatch(x, ids, w)
    # a stand-in for the experts: expert e scales its input by (e + 1), weighted by the routing weight
    scale = torch.where(ids_r >= 0, (ids_r + 1 + disp.rank * per_rank).float() * w_r.float(), torch.zeros_like(w_r.float())).sum(1)
    y = (xr.float() * scale.unsqueeze(1)).to(xr.dtype)
    out = disp.combine(y)
    (out.float() * torch.linspace(0.5, 1.5, out.shape[1], device=out.device)).sum().backward()
    return out.detach().float(), x.grad.float(), w.grad.float()


def main():
    from steptronoss_b200.ops import native
    from steptronoss_b200.parallel.ep_dispatcher import AllToAllDispatcher
    from steptronoss_b200.parallel.peer_dispatcher import PeerMemoryDispatcher
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    PM.new_parallel("EP", [list(range(PM.world_size))])
    world, rank = PM.world_size, PM.world_rank
    dev = torch.device("cuda", torch.cuda.current_device())
    E, K, T, H = 8 * world, 4, 384, 256
    per_rank = E // world
    res = {}
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    peer, a2a = PeerMemoryDispatcher("EP", E), AllToAllDispatcher("EP", E)
    for it in range(4):  # several calls: slot reuse
        x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        ids = torch.stack([torch.randperm(E, device=dev, generator=g)[:K] for _ in range(T)])
        w = torch.rand(T, K, device=dev, generator=g)
        a = _run(peer, x, ids, w, per_rank)
        b = _run(a2a, x, ids, w, per_rank)
        for name, u, v in zip(("out", "gx", "gw"), a, b):
            err = float((u - v).abs().max() / v.abs().max().clamp_min(1e-6))
            res[f"{name}_{it}"] = err
            assert err < 2e-2, (name, it, err)
    torch.cuda.synchronize()
    native.raise_if_kernel_error()
    # timing of dispatch + combine (forward only)
    x = torch.randn(4096, 2048, device=dev, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=dev, generator=g)[:K] for _ in range(4096)])
    w = torch.rand(4096, K, device=dev, generator=g)

    def timed(d):
        for _ in range(3):
            xr, _i, _w = d.dispatch(x, ids, w)
            d.combine(xr)
        torch.cuda.synchronize()
        dist.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(10):
            xr, _i, _w = d.dispatch(x, ids, w)
            d.combine(xr)
        t1.record()
        torch.cuda.synchronize()
        t = torch.tensor([t0.elapsed_time(t1) / 10], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    with torch.no_grad():
        res["ms_peer"], res["ms_alltoall"] = timed(peer), timed(a2a)
    dist.barrier()
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
