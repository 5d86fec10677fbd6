"""MoE decoder on CPU: trains in one process, and expert parallelism over 2 gloo ranks reproduces the
single-process block output and gradients."""
import os
import socket

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
