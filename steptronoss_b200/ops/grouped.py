"""Grouped (per-expert) GEMMs over expert-major row segments.

Rows of the activation matrix are grouped by expert; every segment starts at a multiple of 128 rows
(``segment_alignment``) and padding rows are zero, so that each 128-row tile belongs to exactly one
expert and the reduction of the weight-gradient product can run over whole 64-row blocks.  The
group sizes stay on the device (``offsets`` int32 ``[G+1]``): unlike the reference's grouped GEMM
back-ends there is no host ``batch_sizes`` and no synchronisation
(``steptronoss/model/utils/moe_utils.py:423-453``).
"""
from __future__ import annotations

import torch

from . import native
from .gemm import count_launch

SEGMENT_ALIGNMENT = 128


def tile_groups_from_offsets(offsets: torch.Tensor, total_rows: int) -> torch.Tensor:
    """``tile_group[t]`` = expert owning rows ``[128 t, 128 t + 128)`` or -1 past the last segment."""
    n_tiles = (total_rows + SEGMENT_ALIGNMENT - 1) // SEGMENT_ALIGNMENT
    starts = torch.arange(n_tiles, device=offsets.device, dtype=torch.int32) * SEGMENT_ALIGNMENT
    g = torch.searchsorted(offsets[1:].contiguous(), starts, right=True).to(torch.int32)
    G = offsets.numel() - 1
    return torch.where(g < G, g, torch.full_like(g, -1))


def grouped_gemm_rows(x: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, trans_b: bool = True,
                      out: torch.Tensor | None = None, tile_group: torch.Tensor | None = None) -> torch.Tensor:
    """``y[rows of g] = x[rows of g] @ (w[g].T if trans_b else w[g])``.

    ``w`` is ``[G, N, K]`` (``trans_b``) or ``[G, K, N]``.  Segment starts must be multiples of 128."""
    G = w.shape[0]
    M, K = x.shape
    N = w.shape[1] if trans_b else w.shape[2]
    if not x.is_cuda:
        outs = torch.zeros((M, N), dtype=x.dtype, device=x.device) if out is None else out
        o = offsets.tolist()
        for g in range(G):
            if o[g + 1] > o[g]:
                wg = w[g].t() if trans_b else w[g]
                outs[o[g]:o[g + 1]] = (x[o[g]:o[g + 1]].float() @ wg.float()).to(x.dtype)
        return outs
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    if tile_group is None:
        tile_group = tile_groups_from_offsets(offsets, M)
    lib = native.load()
    w2 = w.reshape(G * w.shape[1], w.shape[2])
    rc = lib.stb_gemm_bf16_grouped_rows(x.data_ptr(), w2.data_ptr(), out.data_ptr(), tile_group.data_ptr(), M, N, K, G,
                                        x.stride(0), w2.stride(0), out.stride(0), int(not trans_b),
                                        int(out.dtype == torch.float32), 0,
                                        native.status_word(x.device).data_ptr(), native.stream())
    native.check(rc, "grouped_gemm_rows")
    count_launch()
    return out


def grouped_gemm_reduce(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor, num_groups: int,
                        out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """``out[g] (+)= a[rows of g].T @ b[rows of g]`` -> ``[G, a.shape[1], b.shape[1]]`` (expert wgrad)."""
    Ma, Na = a.shape[1], b.shape[1]
    if not a.is_cuda:
        res = torch.zeros((num_groups, Ma, Na), dtype=torch.float32, device=a.device)
        o = offsets.tolist()
        for g in range(num_groups):
            res[g] = a[o[g]:o[g + 1]].float().t() @ b[o[g]:o[g + 1]].float()
        if out is None:
            return res.to(a.dtype)
        if accumulate:
            out.add_(res.to(out.dtype))
        else:
            out.copy_(res.to(out.dtype))
        return out
    if out is None:
        out = torch.empty((num_groups, Ma, Na), dtype=a.dtype, device=a.device)
        accumulate = False
    lib = native.load()
    rc = lib.stb_gemm_bf16_grouped_reduce(a.data_ptr(), b.data_ptr(), out.data_ptr(), offsets.data_ptr(), a.shape[0], Ma,
                                          Na, num_groups, a.stride(0), b.stride(0), out.stride(1),
                                          int(out.dtype == torch.float32), int(accumulate),
                                          native.status_word(a.device).data_ptr(), native.stream())
    native.check(rc, "grouped_gemm_reduce")
    count_launch()
    return out
