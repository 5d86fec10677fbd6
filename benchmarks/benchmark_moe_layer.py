"""Expert-parallel MoE layer micro-benchmark: router -> dispatch -> grouped SwiGLU FFN -> combine, forward and
backward, one rank per GPU (EP = world size).

Workload: 4096 tokens per rank, hidden 4096, 128 experts with SwiGLU width 1536, top-8; router logits N(0,1)
("uniform") and the same logits plus the log of a Zipf(s=1.0) expert popularity ("zipf"); activations N(0,1) in
bf16, weights N(0,0.02).  Both token dispatchers are timed: ``alltoall`` (NCCL all-to-alls with a host exchange of
the split sizes, the structure of the reference's ``TokenDispatcher``, ``ep_dispatcher/token_dispatcher.py:14-118``)
and ``peer`` (rows written straight into the destination GPU's buffer over NVLink).  Times are CUDA events on
every rank, maximum over ranks.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/benchmark_moe_layer.py

``--impl reference`` times the same layer built from the unmodified reference framework under ``baseline/_ref``:
its ``TokenDispatcher`` (NCCL all-to-alls), its ``routed_grouped_ffn`` with the fastest expert GEMM it ships that
runs here (its Triton grouped GEMM; ``--ref-grouped-gemm default`` selects the per-expert loop) and its Triton
routing / scatter / gather kernels, in the manner of its own ``benchmarks/benchmark_dispatcher.py:20-157``.  The
router (top-k of the same logits) is this repository's on both arms and sits outside the timed region there.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run_reference(args):
    """The reference's dispatcher + grouped expert FFN + combine on the same workload, forward and backward."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "steptronoss")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/steptronoss is absent"}), flush=True)
        return
    sys.path.insert(0, os.path.join(root, "baseline", "shims"))
    sys.path.insert(0, ref)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")):
        os.environ.setdefault(k, v)
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    from steptronoss.core.parallel_state import PM as RPM
    from steptronoss.exp.base_exp import ParallelConfig as RParallelConfig
    from steptronoss.model.ep_dispatcher.token_dispatcher import TokenDispatcher
    from steptronoss.model.utils import moe_utils as rmoe
    from steptronoss.utils.optimizable import set_optimization

    from benchmarks.common import flush_l2, measured_peaks
    from steptronoss_b200.ops import moe as moe_ops          # the router only: outside the timed region

    if not dist.is_initialized():
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    world, rank = dist.get_world_size(), dist.get_rank()
    RPM.initialize(backend="nccl")
    mesh = RParallelConfig()
    mesh.tensor_model_parallel_size = mesh.pipeline_model_parallel_size = mesh.context_parallel_size = 1
    mesh.virtual_pipeline_model_parallel_size = 1
    mesh.expert_model_parallel_size, mesh.expert_tensor_parallel_size = world, 1
    RPM.set_mesh(mesh)
    choices = {"histogram": "triton", "index_compute": "triton", "moe_scatter": "triton", "moe_weighted_gather": "triton"}
    if args.ref_grouped_gemm != "default":
        choices["grouped_gemm"] = args.ref_grouped_gemm
    set_optimization(**choices)

    dev = torch.device("cuda", torch.cuda.current_device())
    T, H, E, F, K = args.tokens, args.hidden, args.experts, args.ffn, args.top_k
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    e_local = E // world
    w1 = (torch.randn(e_local, 2 * F, H, device=dev, generator=g) * 0.02).to(torch.bfloat16).requires_grad_()
    w2 = (torch.randn(e_local, H, F, device=dev, generator=g) * 0.02).to(torch.bfloat16).requires_grad_()
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16).requires_grad_()
    gout = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    base_logits = torch.randn(T, E, device=dev, generator=g)
    zipf = torch.log(1.0 / torch.arange(1, E + 1, device=dev, dtype=torch.float32))

    def act(v):
        a, b = torch.chunk(v, 2, dim=-1)
        return torch.nn.functional.silu(a) * b

    peaks = measured_peaks()
    rows = []
    for routing, logits in (("uniform", base_logits), ("zipf", base_logits + zipf)):
        ids, w, _ps, _hist, _stats = moe_ops.fused_router(logits, None, K, False, True, 0.0)
        ids, w = ids.long(), w.detach().float().requires_grad_()
        dispatcher = TokenDispatcher("EP", num_experts=E) if world > 1 else None

        def step():
            if dispatcher is not None:
                h, lid, lw = dispatcher.dispatch(x, ids, w)
            else:
                h, lid, lw = x, ids, w
            y = rmoe.routed_grouped_ffn(w1, w2, act, h, lid.to(torch.int32), lw)
            out = dispatcher.combine(y) if dispatcher is not None else y
            return out, torch.autograd.grad(out, [x, w, w1, w2], gout)

        for _ in range(args.warmup):
            step()
        times = []
        for _ in range(args.iters):
            dist.barrier()
            flush_l2()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            step()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        t = torch.tensor([min(times), sorted(times)[len(times) // 2]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        flops = 3 * 2.0 * float(T * K * world) * H * 3 * F
        row = {"bench": "moe_layer_fwd_bwd", "impl": "reference", "routing": routing,
               "dispatcher": "TokenDispatcher (NCCL all-to-all)", "optimizable": choices, "ep": world,
               "tokens_per_rank": T, "hidden": H, "experts": E, "ffn": F, "top_k": K, "best_ms": float(t[0]),
               "median_ms": float(t[1]), "tokens_per_s_all_ranks": T * world / (float(t[0]) * 1e-3),
               "expert_gemm_tflops_per_gpu": flops / world / (float(t[0]) * 1e-3) / 1e12,
               "frac_of_measured_bf16_peak": flops / world / (float(t[0]) * 1e-3) / 1e12 / peaks["bf16_tflops"]}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    dist.barrier()
    if rank == 0 and args.json:
        json.dump({"peaks": peaks, "rows": rows}, open(args.json, "w"), indent=1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--ffn", type=int, default=1536)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default=None)
    ap.add_argument("--fp8", action="store_true",
                    help="forward expert GEMMs in block-scaled e4m3 (1x128 activation, 128x128 weight scales)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-grouped-gemm", default="triton_grouped_gemm",
                    help="reference arm: alternative of its grouped_gemm switch, or 'default' for the per-expert loop")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    from benchmarks.common import flush_l2, measured_peaks
    from steptronoss_b200.config import Config
    from steptronoss_b200.exp.base_exp import MegatronTPConfig, ParallelConfig
    from steptronoss_b200.models.common.moe_block import MoEBlock, MoEConfig
    from steptronoss_b200.ops import moe as moe_ops
    from steptronoss_b200.ops import native
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    world, rank = PM.world_size, PM.world_rank
    mesh = ParallelConfig()
    mesh.expert_model_parallel_size, mesh.expert_tensor_parallel_size = world, 1
    PM.set_mesh(mesh)
    cuda = torch.cuda.is_available()  # CPU ranks (gloo) only smoke-test the script
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    T, H, E, F, K = args.tokens, args.hidden, args.experts, args.ffn, args.top_k

    class Holder(Config):
        tp_cfg = MegatronTPConfig
        params_dtype = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        moe_cfg = MoEConfig

    holders = []

    def build(kind):
        h = Holder()
        c = h.moe_cfg
        c.hidden_size, c.moe_num_experts, c.moe_top_k, c.moe_hidden_size = H, E, K, F
        c.moe_layer_list, c.dispatcher, c.norm_expert_weight = [0], kind, True
        c.fp8 = bool(args.fp8)
        holders.append(h)
        with torch.device(dev):
            return MoEBlock(c, 0)

    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    blocks = {k: build(k) for k in ("alltoall", "peer")} if world > 1 else {"local": build("alltoall")}
    first = next(iter(blocks.values()))
    with torch.no_grad():
        for w in (first.experts.w1, first.experts.w2):
            w.copy_(torch.randn(w.shape, device=dev, generator=g) * 0.02)
    for b in blocks.values():
        b.load_state_dict(first.state_dict())

    act = torch.bfloat16 if cuda else torch.float32
    x = torch.randn(T, H, device=dev, generator=g).to(act).requires_grad_()
    gout = torch.randn(T, H, device=dev, generator=g).to(act)
    route = moe_ops.fused_router if cuda else moe_ops.router_reference
    base_logits = torch.randn(T, E, device=dev, generator=g)
    zipf = torch.log(1.0 / torch.arange(1, E + 1, device=dev, dtype=torch.float32))
    peaks = measured_peaks()
    rows = []
    for routing, logits in (("uniform", base_logits), ("zipf", base_logits + zipf)):
        logits = logits.clone().requires_grad_()
        outs = {}
        for kind, blk in blocks.items():
            fn = blk.forward_experts_ep if world > 1 else blk.forward_experts_tp

            def step():
                ids, w, _ps, _hist, _stats = route(logits, None, K, False, True, 0.0)
                out = fn(x, ids, w)
                return out, torch.autograd.grad(out, [x, logits, blk.experts.w1, blk.experts.w2], gout)

            out, grads = step()
            outs[kind] = (out.detach().float(), grads[0].float(), grads[2].float())
            for _ in range(args.warmup):
                step()
            times = []
            for _ in range(args.iters):
                if world > 1:
                    dist.barrier()
                if not cuda:
                    import time
                    t0 = time.perf_counter()
                    step()
                    times.append((time.perf_counter() - t0) * 1e3)
                    continue
                flush_l2()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                step()
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b))
            t = torch.tensor([min(times), sorted(times)[len(times) // 2]], device=dev, dtype=torch.float64)
            slots = torch.tensor([float(T * K)], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                dist.all_reduce(slots)
            flops = 3 * 2.0 * float(slots) * H * 3 * F  # forward + 2x backward of the two expert GEMMs, all ranks
            row = {"bench": "moe_layer_fwd_bwd", "routing": routing, "dispatcher": kind, "ep": world,
                   "expert_forward": "fp8 e4m3, 1x128 / 128x128 block scales" if args.fp8 else "bf16",
                   "tokens_per_rank": T, "hidden": H, "experts": E, "ffn": F, "top_k": K, "best_ms": float(t[0]),
                   "median_ms": float(t[1]), "tokens_per_s_all_ranks": T * world / (float(t[0]) * 1e-3),
                   "expert_gemm_tflops_per_gpu": flops / world / (float(t[0]) * 1e-3) / 1e12,
                   "frac_of_measured_bf16_peak": flops / world / (float(t[0]) * 1e-3) / 1e12 / peaks["bf16_tflops"]}
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
        if len(outs) == 2:  # both dispatchers must agree
            for name, a, b in zip(("out", "dx", "dw1"), outs["peer"], outs["alltoall"]):
                err = float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))
                assert err < 2e-2, (routing, name, err)
    if cuda:
        torch.cuda.synchronize()
        native.raise_if_kernel_error()
    if world > 1:
        dist.barrier()
    if rank == 0 and args.json:
        json.dump({"peaks": peaks, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
