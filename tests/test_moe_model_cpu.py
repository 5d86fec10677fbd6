"""MoE decoder on CPU: trains in one process, and expert parallelism over 2 gloo ranks reproduces the
single-process block output and gradients."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from steptronoss_b200.config import Config
from steptronoss_b200.exp.base_exp import MegatronTPConfig, ParallelConfig


def _moe_cfg(E=4, K=2, H=32, F=16):
    from steptronoss_b200.models.common.moe_block import MoEConfig

    class Holder(Config):
        tp_cfg = MegatronTPConfig
        params_dtype = torch.float32
        moe_cfg = MoEConfig

    h = Holder()
    c = h.moe_cfg
    c.hidden_size, c.moe_num_experts, c.moe_top_k, c.moe_hidden_size = H, E, K, F
    c.moe_aux_loss_coef = 0.01
    c.moe_layer_list = [0]
    return h, c


def _build_block(seed=0):
    from steptronoss_b200.models.common.moe_block import MoEBlock
    from steptronoss_b200.parallel.layers import init_parallel_weight_, set_defaults_if_not_set_tensor_model_parallel_attributes

    holder, cfg = _moe_cfg()
    blk = MoEBlock(cfg, 0)
    for n, p in blk.named_parameters():
        set_defaults_if_not_set_tensor_model_parallel_attributes(p)
        init_parallel_weight_(p, n, seed, 0.3)
    blk._holder = holder
    return blk


def _inputs(rank=None, world=1):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(24, 32, generator=g)
    if rank is None:
        return x
    return x.chunk(world)[rank].clone()


def test_moe_block_single_process_router_properties():
    blk = _build_block()
    x = _inputs().requires_grad_()
    out = blk(x)
    assert out.shape == x.shape
    out.sum().backward()
    assert blk.experts.w1.grad is not None and blk.gate.weight.grad is not None
    ids, w, aux = blk.forward_router(blk.gate(x.detach()))
    assert ids.shape == (24, 2) and torch.allclose(w.sum(-1), torch.ones(24), atol=1e-5)
    assert float(aux) > 0


def _ep_worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    from steptronoss_b200.parallel.state import PM

    PM.initialize(backend="gloo")
    pc = ParallelConfig()
    pc.expert_model_parallel_size = 2
    pc.expert_tensor_parallel_size = 1
    PM.set_mesh(pc)
    blk = _build_block()
    x = _inputs(rank, world).requires_grad_()
    out = blk(x)
    out.sum().backward()
    q.put((rank, out.detach().numpy(), x.grad.numpy(), blk.experts.w1.grad.numpy(), blk.gate.weight.grad.numpy()))
    torch.distributed.barrier()


def test_expert_parallel_2_ranks_matches_single_process():
    torch.set_num_threads(1)
    os.environ.pop("WORLD_SIZE", None)
    blk = _build_block()
    x = _inputs().requires_grad_()
    # single process sees the two halves as two independent "micro-batches" (router statistics are per rank)
    outs, gxs = [], []
    for part in x.detach().chunk(2):
        part = part.clone().requires_grad_()
        o = blk(part)
        o.sum().backward()
        outs.append(o.detach())
        gxs.append(part.grad)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=300) for _ in range(2)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    w1_full = blk.experts.w1.grad
    for rank, out, gx, gw1, ggate in res:
        assert torch.allclose(torch.from_numpy(out), outs[rank], atol=1e-5), f"rank {rank} output"
        # expert weight gradients: rank r owns experts [2r, 2r+2) and received tokens of both ranks
        assert torch.allclose(torch.from_numpy(gw1), w1_full[2 * rank: 2 * rank + 2], atol=1e-4)


def test_router_options_scale_balance_and_raw_weights():
    """``routed_scaling_factor`` multiplies the block output, ``force_balance`` deals tokens out round-robin,
    ``norm_expert_weight=False`` keeps the raw softmax probabilities of the chosen experts."""
    x = _inputs()
    base = _build_block()
    ref = base(x)
    scaled = _build_block()
    scaled.cfg.routed_scaling_factor = 2.5
    assert torch.allclose(scaled(x), ref * 2.5, atol=1e-6)

    forced = _build_block()
    forced.cfg.force_balance = True
    ids, w, _ = forced.forward_router(forced.gate(x))
    assert ids.reshape(-1).tolist() == [i % 4 for i in range(48)]                 # 24 tokens x top-2 over 4 experts
    assert torch.bincount(ids.reshape(-1), minlength=4).tolist() == [12, 12, 12, 12]
    assert torch.allclose(w.sum(-1), torch.ones(24), atol=1e-5)

    raw = _build_block()
    raw.cfg.norm_expert_weight = False
    logits = raw.gate(x)
    ids, w, _ = raw.forward_router(logits)
    prob = torch.softmax(logits.float(), dim=1)
    assert torch.allclose(w, prob.gather(1, ids), atol=1e-6) and bool((w.sum(-1) < 1).all())


def test_zero_centred_norm_weight_and_clamped_swiglu():
    from steptronoss_b200.models.common.rms_norm import RMSNorm
    from steptronoss_b200.ops import rmsnorm
    from steptronoss_b200.ops.fused import swiglu_reference

    torch.manual_seed(0)
    x = torch.randn(5, 16)
    plain, zero = RMSNorm(16, 1e-6, params_dtype=torch.float32), RMSNorm(16, 1e-6, use_zero_init=True, params_dtype=torch.float32)
    assert plain.weight.init_kind == "ones" and zero.weight.init_kind == "zeros"
    with torch.no_grad():
        plain.weight.fill_(1.0)
        zero.weight.zero_()                                                      # gamma = weight + 1
    assert torch.allclose(plain(x), zero(x), atol=1e-6)
    with torch.no_grad():
        zero.weight.fill_(0.5)
    want = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * 1.5
    assert torch.allclose(zero(x), want, atol=1e-5)
    xg = x.clone().requires_grad_(True)
    rmsnorm(xg, zero.weight, 1e-6, True).sum().backward()
    assert zero.weight.grad is not None and xg.grad is not None

    h = torch.tensor([[10.0, -10.0, 1.0, 20.0, -20.0, 2.0]])                     # gate | up
    out = swiglu_reference(h, limit=7.0)
    # the activated gate is capped above (silu(10) = 9.9995 -> 7), the up branch on both sides
    act = torch.nn.functional.silu(torch.tensor([10.0, -10.0, 1.0])).clamp(max=7.0)
    assert float(act[0]) == 7.0
    assert torch.allclose(out, act * torch.tensor([7.0, -7.0, 2.0]))
    assert not torch.allclose(out, swiglu_reference(h))
    # a gate of exactly the limit is not cut: silu(7) < 7
    assert float(swiglu_reference(torch.tensor([[7.0, 1.0]]), limit=7.0)) == pytest.approx(7.0 / (1 + 2.718281828 ** -7), rel=1e-6)
    from steptronoss_b200.models.common.feed_forward import FeedForwardConfig

    assert torch.equal(FeedForwardConfig().activation(h, swiglu_limit=7.0), out)


def test_detailed_router_metrics_are_filled_when_asked_for():
    from steptronoss_b200.utils.metrics import GlobalMetrics, Metric

    names = ("router_logits_max", "router_logits_std", "moe_minp", "moe_sumk", "moe_std", "moe_avg", "moe_max",
             "expert_coef")
    for n in names:
        GlobalMetrics.register(n, Metric(is_group=True).mean("time"))
    try:
        blk = _build_block()
        blk.cfg.detailed_router_metrics = True
        x = _inputs()
        logits = blk.gate(x)
        blk.forward_router(logits)
        got = GlobalMetrics.reduce_all()
        prob = torch.softmax(logits.float(), dim=1)
        key = lambda n: next(k for k in got if k.startswith(n))
        assert abs(float(got[key("moe_avg")]) - 1.0 / prob.shape[1]) < 1e-6            # softmax rows sum to one
        assert abs(float(got[key("moe_minp")]) - float(prob.min(1).values.mean())) < 1e-6
        assert abs(float(got[key("moe_sumk")]) - float(prob.topk(2, dim=1).values.sum(1).mean())) < 1e-6
        assert abs(float(got[key("router_logits_std")]) - float(logits.float().std(1).mean())) < 1e-5
        assert float(got[key("moe_max")]) >= float(got[key("moe_minp")])
    finally:
        GlobalMetrics.clear()
