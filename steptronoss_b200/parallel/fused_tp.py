"""Sequence-parallel projections: all-gather -> column GEMM and row GEMM -> reduce-scatter.

The reference performs these as an NCCL collective followed (or preceded) by a cuBLAS GEMM inside
one autograd function (``steptronoss/core/tensor_parallel/layers.py:151-346``).  Here each pair is
one autograd function with two bodies:

* the NCCL statement (any backend, also gloo on CPU): collective, then ``ops.gemm``;
* the peer-memory path (CUDA, all ranks of the group on one node): one kernel per projection
  (``csrc/gemm_tp_sm100.cu``) whose extra warps pull the peers' rows over NVLink while the tcgen05
  GEMM consumes the row tiles that have arrived, or whose epilogue stores partial tiles into the
  owner's memory where they are summed in fixed rank order.

Backward mirrors the reference: the column layer needs its gathered input for the weight gradient and
reduce-scatters the input gradient; the row layer all-gathers the output gradient.  The reference
re-gathers the column layer's input in backward to keep only 1/TP of it alive.  On the peer-memory path
the gathered rows are kept instead (``STB200_TP_KEEP_GATHERED``, default on): one copy out of the
gathered slot costs a fifth of a second all-gather over NVLink, and tokens x hidden bf16 per column layer
is small against 180 GB; ``0`` restores the re-gather.
"""
from __future__ import annotations

import os

import torch

from ..ops.gemm import gemm
from . import comm
from .state import PM


KEEP_GATHERED = os.environ.get("STB200_TP_KEEP_GATHERED", "1") != "0"


def _ag_rows(x, group_name):
    n = PM.size_of(group_name)
    x = x.contiguous()
    out = torch.empty((x.shape[0] * n, x.shape[1]), dtype=x.dtype, device=x.device)
    comm.all_gather_into_tensor(out, x, group=PM.group_of(group_name))
    return out


def _rs_rows(x, group_name):
    n = PM.size_of(group_name)
    x = x.contiguous()
    out = torch.empty((x.shape[0] // n, x.shape[1]), dtype=x.dtype, device=x.device)
    comm.reduce_scatter_tensor(out, x, group=PM.group_of(group_name))
    return out


def _peer(group_name, rows_local, k, n, *tensors) -> bool:
    """True when this projection runs as one fused kernel over peer memory."""
    if not tensors[0].is_cuda:
        return False
    from . import symm

    return symm.usable(rows_local, k, n, *tensors) and symm.enabled(group_name)


def _wgrad(weight, g2, x2):
    main_grad = getattr(weight, "main_grad", None)
    if main_grad is not None and g2.is_cuda:
        gemm(g2, x2, a_mn_major=True, b_mn_major=True, out=main_grad, accumulate=True)
        weight.grad_added_to_main_grad = True
        return None
    return gemm(g2, x2, a_mn_major=True, b_mn_major=True, out_dtype=weight.dtype)


class _AllGatherLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group_name, out_dtype):
        ctx.group_name = group_name
        ctx.weight_ref = w
        ctx.full = None
        if _peer(group_name, x.shape[0], x.shape[1], w.shape[0], x, w):
            from . import symm

            keep = KEEP_GATHERED and ctx.needs_input_grad[1]   # not under no_grad (first pass of a recomputed block)
            y, full = symm.all_gather_gemm(x, w, group_name, out_dtype=out_dtype, need_gathered=keep)
            if keep:
                # the gathered slot is reused by the second-next all-gather of the group: keep a private copy
                ctx.full = full.clone()
            ctx.save_for_backward(x, w)
            return y
        ctx.save_for_backward(x, w)  # only the local 1/TP slice is kept
        full = _ag_rows(x, group_name)
        return gemm(full, w, out_dtype=out_dtype or x.dtype)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        name = ctx.group_name
        g2 = gy if gy.dtype == w.dtype else gy.to(w.dtype)
        g2 = g2.contiguous()
        dx = dw = None
        peer = _peer(name, x.shape[0], x.shape[1], w.shape[0], x, w, g2)
        if peer:
            from . import symm
        if ctx.needs_input_grad[0]:
            if peer:
                dx = symm.gemm_reduce_scatter(g2, w, name, b_mn_major=True)
            else:
                dx = _rs_rows(gemm(g2, w, b_mn_major=True, out_dtype=x.dtype), name)
        if ctx.needs_input_grad[1]:
            if ctx.full is not None:
                full, ctx.full = ctx.full, None
            else:
                full = symm.all_gather_gemm(x, None, name)[1] if peer else _ag_rows(x, name)
            dw = _wgrad(ctx.weight_ref, g2, full)
        return dx, dw, None, None


class _LinearReduceScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group_name):
        ctx.group_name = group_name
        ctx.weight_ref = w
        ctx.save_for_backward(x, w)
        tp = PM.size_of(group_name)
        if x.shape[0] % tp == 0 and _peer(group_name, x.shape[0] // tp, x.shape[1], w.shape[0], x, w):
            from . import symm

            return symm.gemm_reduce_scatter(x, w, group_name)
        return _rs_rows(gemm(x, w, out_dtype=x.dtype), group_name)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        name = ctx.group_name
        g = gy if gy.dtype == w.dtype else gy.to(w.dtype)
        g = g.contiguous()
        dx = dw = None
        if _peer(name, g.shape[0], g.shape[1], w.shape[1], g, w, x):
            from . import symm

            # dx = all_gather(g) @ w in the same launch that gathers g for the weight gradient
            dx, gfull = symm.all_gather_gemm(g, w if ctx.needs_input_grad[0] else None, name, b_mn_major=True)
        else:
            gfull = _ag_rows(g, name)
            if ctx.needs_input_grad[0]:
                dx = gemm(gfull, w, b_mn_major=True, out_dtype=x.dtype)
        if ctx.needs_input_grad[1]:
            dw = _wgrad(ctx.weight_ref, gfull, x)
        return dx, dw, None


def all_gather_linear(x, w, group_name: str = "TP", out_dtype=None):
    """``all_gather_rows(x) @ w.T`` for a sequence-parallel column projection."""
    if PM.size_of(group_name) == 1:
        from ..ops import linear

        return linear(x, w, out_dtype)
    return _AllGatherLinearFn.apply(x, w, group_name, out_dtype)


def linear_reduce_scatter(x, w, group_name: str = "TP"):
    """``reduce_scatter_rows(x @ w.T)`` for a sequence-parallel row projection."""
    if PM.size_of(group_name) == 1:
        from ..ops import linear

        return linear(x, w)
    return _LinearReduceScatterFn.apply(x, w, group_name)
