"""Sequence-parallel projections: all-gather -> column GEMM and row GEMM -> reduce-scatter.

The reference performs these as an NCCL collective followed (or preceded) by a cuBLAS GEMM inside
one autograd function (``steptronoss/core/tensor_parallel/layers.py:151-346``).  Here each pair is
one autograd function with two bodies:

* the NCCL statement (any backend, also gloo on CPU): collective, then ``ops.gemm``;
* the peer-memory path (CUDA + symmetric arena available): the activations live in a symmetric
  buffer, peers' row blocks are pulled over NVLink chunk by chunk on a copy stream while the
  tcgen05 GEMM of the chunks that already arrived runs, and the reduce-scatter is performed by a
  kernel that reads the partial tiles from every peer's buffer in fixed rank order.

Backward mirrors the reference: the column layer re-gathers its input for the weight gradient and
reduce-scatters the input gradient; the row layer all-gathers the output gradient.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops.gemm import gemm
from . import comm
from .state import PM


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


def _peer_path(x) -> bool:
    if not x.is_cuda:
        return False
    from . import symm

    return symm.enabled()


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
        if _peer_path(x):
            from . import symm

            full = symm.all_gather_rows(x, group_name)
        else:
            full = _ag_rows(x, group_name)
        y = gemm(full, w, out_dtype=out_dtype or x.dtype)
        ctx.save_for_backward(x, w)  # only the local 1/TP slice is kept
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        name = ctx.group_name
        g2 = gy if gy.dtype == w.dtype else gy.to(w.dtype)
        g2 = g2.contiguous()
        dx = dw = None
        peer = _peer_path(x)
        if ctx.needs_input_grad[0]:
            dfull = gemm(g2, w, b_mn_major=True, out_dtype=x.dtype)
            if peer:
                from . import symm

                dx = symm.reduce_scatter_rows(dfull, name)
            else:
                dx = _rs_rows(dfull, name)
        if ctx.needs_input_grad[1]:
            if peer:
                from . import symm

                full = symm.all_gather_rows(x, name)
            else:
                full = _ag_rows(x, name)
            dw = _wgrad(ctx.weight_ref, g2, full)
        return dx, dw, None, None


class _LinearReduceScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group_name):
        ctx.group_name = group_name
        ctx.weight_ref = w
        ctx.save_for_backward(x, w)
        y = gemm(x, w, out_dtype=x.dtype)
        if _peer_path(x):
            from . import symm

            return symm.reduce_scatter_rows(y, group_name)
        return _rs_rows(y, group_name)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        name = ctx.group_name
        g = gy if gy.dtype == w.dtype else gy.to(w.dtype)
        if _peer_path(x):
            from . import symm

            gfull = symm.all_gather_rows(g, name)
        else:
            gfull = _ag_rows(g, name)
        dx = dw = None
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
