"""bf16 GEMM front-end and the linear-layer autograd function.

On CUDA every product is the hand-written tcgen05 kernel (``csrc/gemm_sm100.cu``); on CPU tensors
the same functions run plain PyTorch so that the whole framework is testable without a GPU.
Replaces the cuBLAS calls of the reference linear layers
(``steptronoss/core/tensor_parallel/layers.py:178-218,251-255,299``) and apex's fp32
weight-gradient accumulation (``layers.py:244-249``).
"""
from __future__ import annotations

import os

import torch

from . import native

_FORCE_LIBRARY_GEMM = os.environ.get("STB200_DEBUG_LIBRARY_GEMM", "0") == "1"
_LAUNCHES = 0


def launch_count() -> int:
    """Number of native kernel launches issued through this module family since import."""
    return _LAUNCHES


def count_launch(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def _tma_compatible(*tensors: torch.Tensor) -> bool:
    """TMA wants 16-byte aligned bases and row pitches; odd shapes (a router with 4 experts, a gate column
    count that is not a multiple of 8, whatever the output type) go to the library GEMM instead."""
    for t in tensors:
        if t.data_ptr() % 16 or (t.stride(0) * t.element_size()) % 16 or t.stride(-1) != 1:
            return False
    return True


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn_major: bool = False,
    b_mn_major: bool = False,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    accumulate: bool = False,
    alpha: float = 1.0,
    addend: torch.Tensor | None = None,
    beta: float = 1.0,
    upper_only: bool = False,
) -> torch.Tensor:
    """``C[M,N] (+)= alpha * A * B^T`` in the operand conventions of the kernel.

    ``addend`` (bf16 ``[M, N]``): ``C = alpha * A B^T + beta * addend`` in the epilogue of the product (bf16 output,
    no ``accumulate``).  ``upper_only``: the result is known to be symmetric (``X X^T``, the square of a symmetric
    matrix, possibly plus a symmetric addend); only the tiles that reach the diagonal are computed and the lower
    triangle is filled from the upper one by a second small kernel.

    ``a`` is stored ``[M, K]`` (K-major) or ``[K, M]`` (``a_mn_major``); ``b`` is stored ``[N, K]``
    (K-major) or ``[K, N]`` (``b_mn_major``).  Row strides may exceed the row length (views of a
    wider buffer are fine) but the last dimension must be contiguous.
    """
    if a_mn_major:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn_major:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"reduction extents differ: {K} vs {Kb}")
    if out is None:
        out_dtype = out_dtype or a.dtype
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        accumulate = False
    if not a.is_cuda or _FORCE_LIBRARY_GEMM or N % 8 or not _tma_compatible(a, b, out):
        am = a.t() if a_mn_major else a
        bm = b if b_mn_major else b.t()
        if a.is_cuda:
            res = torch.matmul(am, bm).float()
        else:
            res = torch.matmul(am.float(), bm.float())
        res = res * alpha if alpha != 1.0 else res
        if addend is not None:
            res = res + beta * addend.float()
        if accumulate:
            out.add_(res.to(out.dtype))
        else:
            out.copy_(res.to(out.dtype))
        return out
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("native GEMM takes bf16 operands")
    if a.stride(-1) != 1 or b.stride(-1) != 1 or out.stride(-1) != 1:
        raise ValueError("last dimension of every GEMM operand must be contiguous")
    lib = native.load()
    if addend is not None or upper_only:
        if accumulate or out.dtype != torch.bfloat16:
            raise ValueError("addend / upper_only take a bf16 output without accumulate")
        if addend is not None and (addend.dtype != torch.bfloat16 or addend.shape != out.shape or addend.stride(-1) != 1):
            raise ValueError("addend must be a bf16 [M, N] matrix with a contiguous last dimension")
        rc = lib.stb_gemm_bf16_ex(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
            int(a_mn_major), int(b_mn_major), float(alpha), native.ptr(addend),
            addend.stride(0) if addend is not None else 0, float(beta), int(upper_only),
            native.status_word(a.device).data_ptr(), native.stream(),
        )
        native.check(rc, f"gemm M={M} N={N} K={K} (addend / upper_only)")
        count_launch()
        if upper_only:
            native.check(lib.stb_mirror_upper_bf16(out.data_ptr(), M, out.stride(0), native.stream()), "mirror_upper")
            count_launch()
        return out
    rc = lib.stb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn_major), int(b_mn_major), int(out.dtype == torch.float32), int(accumulate), float(alpha),
        native.status_word(a.device).data_ptr(), native.stream(),
    )
    native.check(rc, f"gemm M={M} N={N} K={K}")
    count_launch()
    return out


class _LinearFn(torch.autograd.Function):
    """y = x @ w.T with the weight gradient optionally accumulated straight into ``w.main_grad``."""

    @staticmethod
    def forward(ctx, x, w, out_dtype):
        ctx.save_for_backward(x, w)
        ctx.weight_ref = w
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, w, out_dtype=out_dtype or x.dtype)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        weight = ctx.weight_ref
        g2 = gy.reshape(-1, gy.shape[-1])
        if g2.dtype != w.dtype:
            g2 = g2.to(w.dtype)
        if g2.stride(-1) != 1:
            g2 = g2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(g2, w, b_mn_major=True, out_dtype=x.dtype).view_as(x)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                gemm(g2, x2, a_mn_major=True, b_mn_major=True, out=main_grad, accumulate=True)
                weight.grad_added_to_main_grad = True
                dw = None
            else:
                dw = gemm(g2, x2, a_mn_major=True, b_mn_major=True, out_dtype=w.dtype)
        return dx, dw, None


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x @ w.T`` (no bias). On CUDA: three tcgen05 GEMMs (fwd, dgrad, wgrad) through autograd."""
    if not x.is_cuda:
        y = torch.nn.functional.linear(x, w)
        return y.to(out_dtype) if out_dtype is not None and out_dtype != y.dtype else y
    return _LinearFn.apply(x, w, out_dtype)
