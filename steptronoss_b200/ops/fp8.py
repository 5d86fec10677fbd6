"""Block-scaled fp8 (e4m3) products: 1 x 128 scales on activations, 128 x 128 scales on weights.

``Y = sum_kb sx[:, kb] * sw[n_block, kb] * (Xq[:, kb] @ Wq[:, kb].T)`` with fp32 accumulation
(``csrc/gemm_fp8_sm100.cu``).  The reference keeps this recipe as an unused Triton kernel next to its bf16
grouped GEMM back-ends (``steptronoss/model/utils/moe_utils.py:423-453``); here it is the forward of the routed
expert FFN when ``MoEConfig.fp8`` is set, with the backward products in bf16.

The PyTorch restatements (``*_reference``) define the numbers: quantise with ``scale = amax / 448`` per block,
round to e4m3, multiply back.  Without a GPU they are what runs.
"""
from __future__ import annotations

import torch

from . import native
from .gemm import count_launch
from .grouped import tile_groups_from_offsets

E4M3_MAX = 448.0
P, I, L = native.P, native.I, native.L
native.register_signature("stb_gemm_fp8_block_scaled", [P, P, P, P, P, P, I, I, I, I, L, L, L, P, P])
native.register_signature("stb_quant_rows_1x128", [P, L, P, L, P, L, I, P])
native.register_signature("stb_quant_blocks_128x128", [P, L, P, L, P, L, I, P])


# ----------------------------------------------------------------------------------------------- quantisation
def quantize_rows_1x128_reference(x: torch.Tensor):
    """``x [M, K]`` -> ``(q [M, K] float8_e4m3fn, scales [M, K/128] fp32)``."""
    M, K = x.shape
    b = x.float().view(M, K // 128, 128)
    amax = b.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (b / scale.unsqueeze(-1)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(M, K), scale


def quantize_blocks_128x128_reference(w: torch.Tensor):
    """``w [R, K]`` (R, K multiples of 128) -> ``(q [R, K] float8_e4m3fn, scales [R/128, K/128] fp32)``."""
    R, K = w.shape
    b = w.float().view(R // 128, 128, K // 128, 128)
    amax = b.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (b / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(R, K), scale


def quantize_rows_1x128(x: torch.Tensor):
    if not x.is_cuda:
        return quantize_rows_1x128_reference(x)
    M, K = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and K % 128 == 0
    q = torch.empty((M, K), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((M, K // 128), dtype=torch.float32, device=x.device)
    rc = native.load().stb_quant_rows_1x128(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), s.data_ptr(), M, K,
                                            native.stream())
    native.check(rc, "quantize_rows_1x128")
    count_launch()
    return q, s


def quantize_blocks_128x128(w: torch.Tensor):
    if not w.is_cuda:
        return quantize_blocks_128x128_reference(w)
    R, K = w.shape
    assert w.dtype == torch.bfloat16 and w.stride(1) == 1 and K % 128 == 0 and R % 128 == 0
    q = torch.empty((R, K), dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty((R // 128, K // 128), dtype=torch.float32, device=w.device)
    rc = native.load().stb_quant_blocks_128x128(w.data_ptr(), w.stride(0), q.data_ptr(), q.stride(0), s.data_ptr(), R, K,
                                                native.stream())
    native.check(rc, "quantize_blocks_128x128")
    count_launch()
    return q, s


def dequantize_rows(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    M, K = q.shape
    return (q.float().view(M, K // 128, 128) * s.unsqueeze(-1)).view(M, K)


def dequantize_blocks(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    R, K = q.shape
    return (q.float().view(R // 128, 128, K // 128, 128) * s[:, None, :, None]).view(R, K)


# ----------------------------------------------------------------------------------------------- products
def grouped_gemm_fp8_reference(xq, sx, wq, sw, offsets, num_groups: int) -> torch.Tensor:
    """Dequantise, then fp32 matmul per group.  ``wq [G*N, K]``, ``sw [G*N/128, K/128]``."""
    M = xq.shape[0]
    N = wq.shape[0] // num_groups
    x = dequantize_rows(xq, sx)
    w = dequantize_blocks(wq, sw).view(num_groups, N, -1)
    out = torch.zeros((M, N), dtype=torch.float32, device=xq.device)
    o = offsets.tolist()
    for g in range(num_groups):
        if o[g + 1] > o[g]:
            out[o[g]:o[g + 1]] = x[o[g]:o[g + 1]] @ w[g].t()
    return out.to(torch.bfloat16)


def grouped_gemm_fp8(xq, sx, wq, sw, offsets, num_groups: int, tile_group: torch.Tensor | None = None,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """``y[rows of g] = dequant(xq)[rows of g] @ dequant(wq[g]).T`` in bf16; segment starts are multiples of 128.

    ``offsets=None`` with ``num_groups == 1`` is the dense product."""
    M, K = xq.shape
    N = wq.shape[0] // num_groups
    if not xq.is_cuda:
        if offsets is None:
            offsets = torch.tensor([0, M], dtype=torch.int32)
        return grouped_gemm_fp8_reference(xq, sx, wq, sw, offsets, num_groups)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=xq.device)
    if tile_group is None and offsets is not None:
        tile_group = tile_groups_from_offsets(offsets, M)
    rc = native.load().stb_gemm_fp8_block_scaled(
        xq.data_ptr(), sx.data_ptr(), wq.data_ptr(), sw.data_ptr(), out.data_ptr(), native.ptr(tile_group), M, N, K,
        num_groups, xq.stride(0), wq.stride(0), out.stride(0), native.status_word(xq.device).data_ptr(), native.stream())
    native.check(rc, f"grouped_gemm_fp8 M={M} N={N} K={K} G={num_groups}")
    count_launch()
    return out


def gemm_fp8(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` with both operands quantised on the fly (bf16 in, bf16 out)."""
    xq, sx = quantize_rows_1x128(x)
    wq, sw = quantize_blocks_128x128(w)
    return grouped_gemm_fp8(xq, sx, wq, sw, None, 1)
