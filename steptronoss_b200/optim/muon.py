"""Muon: momentum orthogonalised by Newton-Schulz for matrix parameters, AdamW for the rest.

Reference: ``steptronoss/optimizer/muon.py:19-195`` (nesterov momentum 0.95, update scaled by
``lr * 0.2 * sqrt(max(rows, cols))`` of the *full* matrix, decoupled weight decay) with TP shards
gathered into the full matrix before the iteration and sliced back afterwards
(``exp/optimizer.py:125-147``).

Two front-ends share the update rule:

* ``Muon``: a ``torch.optim.Optimizer`` over parameter groups (``is_muon_param`` selects the rule),
  usable stand-alone;
* ``FlatMuon``: driven by the gradient manager on the whole matrices this data-parallel rank owns
  (ZeRO-1 never splits a parameter, which is what makes the per-matrix iteration possible).  Matrices
  of equal shape are stacked and orthogonalised as one batch.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..parallel.layers import shard_of_full
from ..parallel.state import PM
from .zeropower import adjust_ratio_for_muon, get_zeropower_fn


def gather_full_matrix(shard: torch.Tensor, param) -> torch.Tensor:
    """Full (unsharded) matrix from this rank's TP shard of ``param``-shaped data."""
    if not getattr(param, "tensor_model_parallel", False):
        return shard
    group_name = getattr(param, "partition_group", "TP")
    world = PM.size_of(group_name)
    if world == 1:
        return shard
    dim = param.partition_dim
    blocks = getattr(param, "partition_blocks", None)
    peer = _gather_over_peer_memory(shard, dim, group_name, world)
    if peer is not None:
        parts = list(peer)
    else:
        parts = [torch.empty_like(shard) for _ in range(world)]
        dist.all_gather(parts, shard.contiguous(), group=PM.group_of(group_name))
    if not blocks:
        return torch.cat(parts, dim=dim) if peer is None or dim != 0 else peer.reshape(-1, shard.shape[1])
    per = [b // world for b in blocks]
    pieces = [p.split(per, dim=dim) for p in parts]
    return torch.cat([torch.cat([pieces[r][i] for r in range(world)], dim=dim) for i in range(len(blocks))], dim=dim)


def _gather_over_peer_memory(shard: torch.Tensor, dim: int, group_name: str, world: int):
    """``[world, *shard.shape]`` view of every rank's shard, gathered by the push kernel of the fused
    all-gather (each rank stores its rows into every peer's buffer over NVLink; no NCCL call), or ``None``
    when the shard does not fit that kernel (not bf16 on the GPU, not 2-D, row count not a multiple of 128)
    or the group has no peer-memory arena.  The view lives in the group's symmetric memory and is consumed
    (copied by ``cat`` / normalised by the first Newton-Schulz step) before the second-next gather."""
    if not (shard.is_cuda and shard.dim() == 2 and shard.dtype == torch.bfloat16):
        return None
    from ..parallel import symm

    x = shard.contiguous()
    if not (symm.enabled(group_name) and symm.usable(x.shape[0], x.shape[1], 8, x)):
        return None
    _, gathered = symm.all_gather_gemm(x, None, group_name, need_gathered=True)
    return gathered.view(world, x.shape[0], x.shape[1])


def slice_own_shard(full: torch.Tensor, param) -> torch.Tensor:
    if not getattr(param, "tensor_model_parallel", False):
        return full
    group_name = getattr(param, "partition_group", "TP")
    world = PM.size_of(group_name)
    if world == 1:
        return full
    return shard_of_full(full, param.partition_dim, getattr(param, "partition_blocks", None), PM.rank_in(group_name),
                         world).contiguous()


def muon_update(grad: torch.Tensor, buf: torch.Tensor, param, *, momentum: float, nesterov: bool, ns_steps: int,
                ns_fn, run_ns_in_fp16: bool, matched_adamw_rms: float) -> torch.Tensor:
    """Momentum + orthogonalisation for one (shard of a) matrix; returns the unit-lr update for the shard."""
    buf.mul_(momentum).add_(grad)
    g = grad.add(buf, alpha=momentum) if nesterov else buf
    g = g.bfloat16() if run_ns_in_fp16 else g.float()
    full = gather_full_matrix(g, param)
    if full.dim() == 3:  # stacked expert matrices: one iteration per expert
        ortho = torch.stack([ns_fn(m, steps=ns_steps) for m in full])
    else:
        ortho = ns_fn(full, steps=ns_steps)
    ortho = ortho.float() * adjust_ratio_for_muon(matched_adamw_rms, full.shape)
    return slice_own_shard(ortho, param)


class Muon(torch.optim.Optimizer):
    def __init__(self, param_groups, lr=2e-2, weight_decay=0.1, matched_adamw_rms=0.2, momentum=0.95, nesterov=True,
                 ns_steps=5, adamw_betas=(0.95, 0.95), adamw_eps=1e-8, run_ns_in_fp16=True, newtonschulz_fn="default"):
        defaults = dict(lr=lr, weight_decay=weight_decay, matched_adamw_rms=matched_adamw_rms, momentum=momentum,
                        nesterov=nesterov, ns_steps=ns_steps, adamw_betas=adamw_betas, adamw_eps=adamw_eps)
        super().__init__(param_groups, defaults)
        self.run_ns_in_fp16 = run_ns_in_fp16
        self.ns_fn = get_zeropower_fn(newtonschulz_fn, run_ns_in_fp16)

    @torch.no_grad()
    def step(self):
        for group in self.param_groups:
            lr, wd = group["lr"], group["weight_decay"]
            if group.get("is_muon_param", False):
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    st = self.state[p]
                    if "muon_buffer" not in st:
                        st["muon_buffer"] = torch.zeros_like(p.grad)
                    upd = muon_update(p.grad, st["muon_buffer"], p, momentum=group["momentum"],
                                      nesterov=group["nesterov"], ns_steps=group["ns_steps"], ns_fn=self.ns_fn,
                                      run_ns_in_fp16=self.run_ns_in_fp16, matched_adamw_rms=group["matched_adamw_rms"])
                    p.mul_(1 - lr * wd)
                    p.add_(upd.to(p.dtype), alpha=-lr)
            else:
                b1, b2 = group["adamw_betas"]
                eps = group["adamw_eps"]
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    st = self.state[p]
                    if "step" not in st:
                        st["step"], st["moment1"], st["moment2"] = 0, torch.zeros_like(p.grad), torch.zeros_like(p.grad)
                    st["step"] += 1
                    st["moment1"].lerp_(p.grad, 1 - b1)
                    st["moment2"].lerp_(p.grad.square(), 1 - b2)
                    bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                    upd = st["moment1"] / (eps + st["moment2"].sqrt()) * (bc2 ** 0.5 / bc1)
                    p.mul_(1 - lr * wd)
                    p.add_(upd, alpha=-lr)


class FlatMuon:
    """Muon over the whole matrices a data-parallel rank owns inside the gradient manager's buckets."""

    def __init__(self, opt_cfg, bucket_items: list):
        self.cfg = opt_cfg
        self.ns_fn = get_zeropower_fn(opt_cfg.muon_newtonschulz_fn, opt_cfg.muon_run_ns_in_fp16)
        self.entries = []
        for bucket, slots in bucket_items:
            for s in slots:
                grad = bucket.grad_buf[s.offset : s.offset + s.numel].view(s.param.shape)
                low = bucket.param_buf[s.offset : s.offset + s.numel].view(s.param.shape)
                self.entries.append({"slot": s, "grad": grad, "low": low, "master": low.float(),
                                     "buf": torch.zeros(s.param.shape, dtype=torch.float32, device=low.device)})

    @torch.no_grad()
    def step(self, lr: float, weight_decay: float, grad_scale: float, scalars) -> None:
        c = self.cfg
        if scalars is not None:
            scale = scalars[2] * grad_scale  # device scalar: clip coefficient x averaging factor
        else:
            scale = grad_scale
        for e in self.entries:
            p = e["slot"].param
            g = e["grad"] * scale
            upd = muon_update(g, e["buf"], p, momentum=c.muon_momentum, nesterov=c.muon_nesterov,
                              ns_steps=c.muon_ns_steps, ns_fn=self.ns_fn, run_ns_in_fp16=c.muon_run_ns_in_fp16,
                              matched_adamw_rms=c.muon_matched_adamw_rms)
            wd = weight_decay * float(c.scale_wd_cond(e["slot"].name, p))
            lr_eff = lr * float(c.scale_lr_func(e["slot"].name, p))
            e["master"].mul_(1 - lr_eff * wd).add_(upd, alpha=-lr_eff)
            e["low"].copy_(e["master"])

    def state_dict(self) -> dict:
        return {e["slot"].name: {"muon_buffer": e["buf"].cpu(), "master": e["master"].cpu()} for e in self.entries}

    def load_state_dict(self, sd: dict) -> None:
        for e in self.entries:
            st = sd.get(e["slot"].name)
            if st:
                e["buf"].copy_(st["muon_buffer"])
                e["master"].copy_(st["master"])
                e["low"].copy_(e["master"])

    def to(self, device) -> None:
        for e in self.entries:
            e["buf"] = e["buf"].to(device)
            e["master"] = e["master"].to(device)
