"""Worker (torch.distributed.run, one rank per GPU): an expert-parallel MoE block gives the same output and
gradients with the peer-memory dispatcher as with the all-to-all dispatcher."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    from steptronoss_b200.config import Config
    from steptronoss_b200.exp.base_exp import MegatronTPConfig, ParallelConfig
    from steptronoss_b200.models.common.moe_block import MoEBlock, MoEConfig
    from steptronoss_b200.ops import native
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    mesh = ParallelConfig()
    mesh.expert_model_parallel_size, mesh.expert_tensor_parallel_size = PM.world_size, 1
    PM.set_mesh(mesh)
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")

    class Holder(Config):
        tp_cfg = MegatronTPConfig
        params_dtype = torch.bfloat16
        moe_cfg = MoEConfig

    def build(kind):
        h = Holder()
        c = h.moe_cfg
        c.hidden_size, c.moe_num_experts, c.moe_top_k, c.moe_hidden_size = 256, 8, 2, 128
        c.moe_aux_loss_coef, c.moe_layer_list, c.dispatcher = 0.01, [0], kind
        with torch.device(dev):
            blk = MoEBlock(c, 0)
        blk._holder = h
        return blk

    blocks = {k: build(k) for k in ("alltoall", "peer")}
    blocks["peer_capacity"] = build("peer")
    blocks["peer_capacity"].cfg.capacity_factor = 1.5
    gw = torch.Generator(device=dev).manual_seed(3)                     # the router is replicated
    ge = torch.Generator(device=dev).manual_seed(100 + PM.world_rank)   # the experts are not
    first = blocks["alltoall"]
    with torch.no_grad():
        first.gate.weight.copy_(torch.randn(first.gate.weight.shape, device=dev, generator=gw) * 0.1)
        for w in (first.experts.w1, first.experts.w2):
            w.copy_(torch.randn(w.shape, device=dev, generator=ge) * 0.05)
    for k in ("peer", "peer_capacity"):
        blocks[k].load_state_dict(first.state_dict())

    g = torch.Generator(device=dev).manual_seed(11 + PM.world_rank)
    res = {}
    for it in range(3):
        x = torch.randn(384, 256, device=dev, generator=g).to(torch.bfloat16)
        outs = {}
        for kind, blk in blocks.items():
            xi = x.clone().requires_grad_()
            for p in blk.parameters():
                p.grad = None
            o = blk(xi)
            o.float().pow(2).sum().backward()
            outs[kind] = (o.detach().float(), xi.grad.float(), blk.experts.w1.grad.float(), blk.gate.weight.grad.float())
        for kind in ("peer", "peer_capacity"):
            for name, a, b in zip(("out", "dx", "dw1", "dgate"), outs[kind], outs["alltoall"]):
                err = float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))
                res[f"{kind}_{name}_{it}"] = err
                assert err < 2e-2, (kind, name, it, err)
    if dev.type == "cuda":
        torch.cuda.synchronize()
        native.raise_if_kernel_error()
    dist.barrier()
    if PM.world_rank == 0:
        print("RESULT " + json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
