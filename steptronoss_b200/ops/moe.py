"""Mixture-of-experts token routing ops.

Semantics of the reference ops (``steptronoss/model/utils/moe_utils.py:85-453``): ``histogram``
(ids equal to -1 are ignored), ``index_compute`` (stable expert-major position of every
(token, k) slot), ``moe_scatter`` (copy rows into expert-major order), ``moe_weighted_gather``
(``out[t] = sum_k w[t,k] * y[pos[t,k]]``) and their composition ``routed_grouped_ffn``.

Differences that follow from the grouped tcgen05 GEMM: every expert's segment starts at a multiple
of 128 rows and padding rows are zero (one row tile = one expert, whole 64-row reduction blocks),
and all sizes stay on the device: the expert-major buffer has a static worst-case row count, so no
``.item()`` / ``batch_sizes.tolist()`` synchronisation remains.
"""
from __future__ import annotations

import torch

from . import native
from .fused import swiglu
from .gemm import count_launch
from .grouped import SEGMENT_ALIGNMENT, grouped_gemm_reduce, grouped_gemm_rows, tile_groups_from_offsets


def histogram(ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Count of every expert id in ``ids``; entries equal to -1 (foreign experts) are ignored."""
    flat = ids.reshape(-1)
    valid = flat >= 0
    return torch.bincount(torch.where(valid, flat, torch.zeros_like(flat)), weights=valid.to(torch.float32),
                          minlength=num_experts)[:num_experts].to(torch.int32)


def padded_rows(num_slots: int, num_experts: int) -> int:
    """Static upper bound of the expert-major buffer height (multiple of 128)."""
    worst = num_slots + num_experts * (SEGMENT_ALIGNMENT - 1)
    return (worst + SEGMENT_ALIGNMENT - 1) // SEGMENT_ALIGNMENT * SEGMENT_ALIGNMENT


def index_compute(ids: torch.Tensor, num_experts: int):
    """Destination row of every (token, k) slot in the expert-major buffer.

    Returns ``(dest [T,k] int64 with -1 for ignored slots, offsets [E+1] int32 aligned segment
    starts, counts [E] int32)``.  Inside an expert the slots keep their token order (stable)."""
    T, K = ids.shape
    flat = ids.reshape(-1).to(torch.int64)
    valid = flat >= 0
    key = torch.where(valid, flat, torch.full_like(flat, num_experts))
    order = torch.sort(key, stable=True).indices
    counts = torch.bincount(key, minlength=num_experts + 1)[:num_experts]
    aligned = (counts + SEGMENT_ALIGNMENT - 1) // SEGMENT_ALIGNMENT * SEGMENT_ALIGNMENT
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=ids.device)
    offsets[1:] = torch.cumsum(aligned, 0)
    starts_sorted = torch.zeros(num_experts + 1, dtype=torch.int64, device=ids.device)
    starts_sorted[1:] = torch.cumsum(counts, 0)
    sorted_key = key[order]
    rank = torch.arange(flat.numel(), device=ids.device) - starts_sorted[sorted_key.clamp(max=num_experts)]
    dest_sorted = torch.where(sorted_key < num_experts, offsets[sorted_key.clamp(max=num_experts - 1)] + rank,
                              torch.full_like(rank, -1))
    dest = torch.empty_like(dest_sorted)
    dest[order] = dest_sorted
    return dest.view(T, K), offsets.to(torch.int32), counts.to(torch.int32)


class _ScatterFn(torch.autograd.Function):
    """rows of x copied to ``dest`` (one copy per slot); backward sums the k copies of each token."""

    @staticmethod
    def forward(ctx, x, dest, rows):
        T, K = dest.shape
        out = torch.zeros((rows, x.shape[1]), dtype=x.dtype, device=x.device)
        d = dest.reshape(-1)
        valid = d >= 0
        src = torch.arange(T, device=x.device).repeat_interleave(K)
        out.index_copy_(0, d[valid], x.index_select(0, src[valid]))
        ctx.save_for_backward(dest)
        ctx.t = T
        return out

    @staticmethod
    def backward(ctx, g):
        (dest,) = ctx.saved_tensors
        T, K = dest.shape
        d = dest.reshape(-1)
        valid = (d >= 0).unsqueeze(-1)
        picked = g.index_select(0, d.clamp(min=0)).float() * valid
        return picked.view(T, K, -1).sum(1).to(g.dtype), None, None


def moe_scatter(x, dest, rows):
    return _ScatterFn.apply(x, dest, rows)


class _WeightedGatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, dest, weights):
        T, K = dest.shape
        d = dest.reshape(-1)
        valid = (d >= 0).view(T, K, 1)
        picked = y.index_select(0, d.clamp(min=0)).view(T, K, -1).float() * valid
        out = (picked * weights.float().unsqueeze(-1)).sum(1).to(y.dtype)
        ctx.save_for_backward(y, dest, weights)
        return out

    @staticmethod
    def backward(ctx, g):
        y, dest, weights = ctx.saved_tensors
        T, K = dest.shape
        d = dest.reshape(-1)
        validf = (d >= 0)
        gy = torch.zeros_like(y)
        contrib = (g.float().unsqueeze(1) * weights.float().unsqueeze(-1)).view(T * K, -1)
        gy.index_copy_(0, d[validf], contrib[validf].to(y.dtype))
        picked = y.index_select(0, d.clamp(min=0)).view(T, K, -1).float() * validf.view(T, K, 1)
        gw = (picked * g.float().unsqueeze(1)).sum(-1).to(weights.dtype)
        return gy, None, gw


def moe_weighted_gather(y, dest, weights):
    """``out[t] = sum_k weights[t,k] * y[dest[t,k]]`` (ignored slots contribute nothing)."""
    return _WeightedGatherFn.apply(y, dest, weights)


class _GroupedLinearFn(torch.autograd.Function):
    """Per-expert ``x_g @ w[g].T`` over expert-major rows; wgrad accumulates into ``w.main_grad``."""

    @staticmethod
    def forward(ctx, x, w, offsets):
        tile_group = tile_groups_from_offsets(offsets, x.shape[0]) if x.is_cuda else None
        y = grouped_gemm_rows(x, w, offsets, trans_b=True, tile_group=tile_group)
        ctx.save_for_backward(x, w, offsets, tile_group if tile_group is not None else offsets)
        ctx.w_ref = w
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w, offsets, tile_group = ctx.saved_tensors
        gy = gy.contiguous()
        G = w.shape[0]
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = grouped_gemm_rows(gy, w, offsets, trans_b=False, tile_group=tile_group if x.is_cuda else None)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(ctx.w_ref, "main_grad", None)
            if main_grad is not None and x.is_cuda:
                grouped_gemm_reduce(gy, x, offsets, G, out=main_grad, accumulate=True)
                ctx.w_ref.grad_added_to_main_grad = True
            else:
                dw = grouped_gemm_reduce(gy, x, offsets, G)
        return dx, dw, None


def grouped_linear(x, w, offsets):
    return _GroupedLinearFn.apply(x, w, offsets)


def routed_grouped_ffn(x, expert_ids, weights, w1, w2, limit: float = 0.0):
    """Top-k routed SwiGLU experts on one rank.

    ``x [T,H]``, ``expert_ids [T,k]`` (local expert index or -1), ``weights [T,k]``,
    ``w1 [E, 2F, H]`` (gate | up), ``w2 [E, H, F]``.  Returns ``[T,H]``."""
    E = w1.shape[0]
    T, K = expert_ids.shape
    dest, offsets, _ = index_compute(expert_ids, E)
    rows = padded_rows(T * K, E)
    xe = moe_scatter(x, dest, rows)
    h = grouped_linear(xe, w1, offsets)
    a = swiglu(h, limit)
    y = grouped_linear(a, w2, offsets)
    return moe_weighted_gather(y, dest, weights)


def routed_grouped_ffn_reference(x, expert_ids, weights, w1, w2, limit: float = 0.0):
    """Plain loop over experts (oracle)."""
    from .fused import swiglu_reference

    out = torch.zeros_like(x, dtype=torch.float32)
    E = w1.shape[0]
    for e in range(E):
        tok, slot = (expert_ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = x[tok].float() @ w1[e].float().t()
        a = swiglu_reference(h, limit)
        y = a @ w2[e].float().t()
        out.index_add_(0, tok, y * weights[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)
