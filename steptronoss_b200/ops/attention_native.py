"""Autograd wrapper of the tcgen05 flash-attention kernels (``csrc/attention_sm100.cu``).

The block schedule (which 128-row block belongs to which packed segment) is computed on the device
from ``cu_seqlens`` with a handful of tiny tensor ops and cached per ``cu_seqlens`` tensor, so all
layers of a micro-batch share it and nothing synchronises with the host.
"""
from __future__ import annotations

import math
import weakref

import torch

from . import native
from .gemm import count_launch

_BLOCK = 128
_SCHED_CACHE: dict = {}


def _schedule(cu: torch.Tensor, total_rows: int):
    """(blk_seg, blk_row0, num_blocks) for 128-row blocks that never straddle two segments."""
    key = (cu.data_ptr(), cu._version, total_rows, cu.numel())
    hit = _SCHED_CACHE.get(key)
    if hit is not None and hit[0]() is cu:
        return hit[1]
    nseg = cu.numel() - 1
    max_blocks = (total_rows + _BLOCK - 1) // _BLOCK + nseg
    cu64 = cu.to(torch.int64)
    lens = cu64[1:] - cu64[:-1]
    nblk = (lens + _BLOCK - 1) // _BLOCK
    ends = torch.cumsum(nblk, 0)
    starts = ends - nblk
    b = torch.arange(max_blocks, device=cu.device, dtype=torch.int64)
    seg = torch.searchsorted(ends, b, right=True)
    valid = seg < nseg
    seg_c = seg.clamp(max=nseg - 1)
    row0 = cu64[:-1][seg_c] + (b - starts[seg_c]) * _BLOCK
    blk_seg = torch.where(valid, seg, torch.full_like(seg, -1)).to(torch.int32)
    blk_row0 = torch.where(valid, row0, torch.zeros_like(row0)).to(torch.int32)
    out = (blk_seg, blk_row0, max_blocks)
    if len(_SCHED_CACHE) > 64:
        _SCHED_CACHE.clear()
    _SCHED_CACHE[key] = (weakref.ref(cu), out)
    return out


def _default_cu(total: int, device) -> torch.Tensor:
    key = ("default", total, str(device))
    hit = _SCHED_CACHE.get(key)
    if hit is None:
        t = torch.tensor([0, total], dtype=torch.int32, device=device)
        _SCHED_CACHE[key] = (lambda: None, t)
        return t
    return hit[1]


_FORCE_SPLITS = 0   # tests set this to exercise the split dK/dV path on shapes that would not choose it


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, causal, window, scale):
        lib = native.load()
        Tq, hq, D = q.shape
        Tk, hkv, _ = k.shape
        if q.stride(2) != 1 or q.stride(1) != D:
            q = q.contiguous()
        if k.stride(2) != 1 or k.stride(1) != D:
            k = k.contiguous()
        if v.stride(2) != 1 or v.stride(1) != D:
            v = v.contiguous()
        o = torch.empty((Tq, hq, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((hq, Tq), dtype=torch.float32, device=q.device)
        qs, qr, nq = _schedule(cu_q, Tq)
        rc = lib.stb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), cu_q.data_ptr(),
                              cu_k.data_ptr(), qs.data_ptr(), qr.data_ptr(), nq, Tq, Tk, hq, hkv, D, q.stride(0),
                              k.stride(0), v.stride(0), int(causal), int(window), float(scale), None, None, None, 0, 0,
                              native.status_word(q.device).data_ptr(), native.stream())
        native.check(rc, "attention forward")
        count_launch()
        ctx.save_for_backward(q, k, v, o, lse, cu_q, cu_k)
        ctx.cfg = (causal, window, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        lib = native.load()
        q, k, v, o, lse, cu_q, cu_k = ctx.saved_tensors
        causal, window, scale = ctx.cfg
        Tq, hq, D = q.shape
        Tk, hkv, _ = k.shape
        do = do.contiguous()
        dq = torch.empty((Tq, hq, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((Tk, hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((Tk, hkv, D), dtype=q.dtype, device=q.device)
        delta = torch.empty((hq, Tq), dtype=torch.float32, device=q.device)
        qs, qr, nq = _schedule(cu_q, Tq)
        ks, kr, nk = _schedule(cu_k, Tk)
        # few kv heads x key blocks: the q heads of a group are split over several CTAs (fp32 partials, ordered sum)
        splits = _FORCE_SPLITS or lib.stb_attn_bwd_splits(hq, hkv, nk)
        part = torch.empty((splits, 2, Tk, hkv, D), dtype=torch.float32, device=q.device) if splits > 1 else None
        rc = lib.stb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                              delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu_q.data_ptr(),
                              cu_k.data_ptr(), qs.data_ptr(), qr.data_ptr(), nq, ks.data_ptr(), kr.data_ptr(), nk, Tq, Tk,
                              hq, hkv, D, q.stride(0), k.stride(0), v.stride(0), dv.stride(0), int(causal), int(window),
                              float(scale), native.ptr(part), splits, None, None, None, 0, 0,
                              native.status_word(q.device).data_ptr(), native.stream())
        native.check(rc, "attention backward")
        count_launch(3 + (splits > 1))
        return dq, dk, dv, None, None, None, None, None


# --------------------------------------------------------------------------- keys addressed by global position
class GatheredKeyPlan:
    """Segments of one call whose keys live in a rank-major ``[cp][2*chunk_len]`` buffer (context parallelism).

    ``pieces``: list of ``(q_begin, q_end, k_begin)`` in *global* positions, one per document piece of the local q
    rows of this call (``k_end == q_end``); ``q_local0``: global position of the call's first q row.  Device
    tables are built once per micro-batch and shared by all layers."""

    def __init__(self, pieces, cp: int, chunk_len: int, device):
        self.cp, self.chunk_len = cp, chunk_len
        q_lens = [qe - qs for qs, qe, _ in pieces]
        k_begin = [ks // _BLOCK * _BLOCK for _, _, ks in pieces]
        k_skip = [ks - kb for (_, _, ks), kb in zip(pieces, k_begin)]
        k_len = [qe - kb for (_, qe, _), kb in zip(pieces, k_begin)]
        i32 = dict(dtype=torch.int32, device=device)
        self.cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0).tolist()), **i32)
        self.seg_k_begin = torch.tensor(k_begin, **i32)
        self.seg_k_len = torch.tensor(k_len, **i32)
        self.seg_k_skip = torch.tensor(k_skip, **i32)
        # q-block schedule from cu_q; key-block schedule: 128-row blocks of every segment's key range (global rows)
        self.q_sched = _schedule(self.cu_q, sum(q_lens))
        seg, row0 = [], []
        for i, (kb, kl) in enumerate(zip(k_begin, k_len)):
            for b in range((kl + _BLOCK - 1) // _BLOCK):
                seg.append(i)
                row0.append(kb + b * _BLOCK)
        self.k_blk_seg = torch.tensor(seg, **i32)
        self.k_blk_row0 = torch.tensor(row0, **i32)
        self.num_k_blocks = len(seg)


def gathered_attention_fwd(q, k_buf, v_buf, plan: GatheredKeyPlan, causal: bool, window: int, scale: float):
    """Forward over keys addressed by global position; returns ``(o, lse)``.  ``k_buf`` / ``v_buf``: ``[cp*2L,hkv,D]``."""
    lib = native.load()
    Tq, hq, D = q.shape
    Tk, hkv, _ = k_buf.shape
    o = torch.empty((Tq, hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((hq, Tq), dtype=torch.float32, device=q.device)
    qs, qr, nq = plan.q_sched
    rc = lib.stb_attn_fwd(q.data_ptr(), k_buf.data_ptr(), v_buf.data_ptr(), o.data_ptr(), lse.data_ptr(),
                          plan.cu_q.data_ptr(), None, qs.data_ptr(), qr.data_ptr(), nq, Tq, Tk, hq, hkv, D, q.stride(0),
                          k_buf.stride(0), v_buf.stride(0), int(causal), int(window), float(scale),
                          plan.seg_k_begin.data_ptr(), plan.seg_k_len.data_ptr(), plan.seg_k_skip.data_ptr(), plan.cp,
                          plan.chunk_len, native.status_word(q.device).data_ptr(), native.stream())
    native.check(rc, "attention forward (gathered keys)")
    count_launch()
    return o, lse


def gathered_attention_bwd(q, k_buf, v_buf, o, do, lse, plan: GatheredKeyPlan, causal: bool, window: int, scale: float,
                           dk_buf, dv_buf):
    """Backward: returns ``dq``; writes this call's dK / dV into the rows of ``dk_buf`` / ``dv_buf`` (rank-major, like
    the key buffers) that its segments cover, leaving every other row untouched."""
    lib = native.load()
    Tq, hq, D = q.shape
    Tk, hkv, _ = k_buf.shape
    dq = torch.empty((Tq, hq, D), dtype=q.dtype, device=q.device)
    delta = torch.empty((hq, Tq), dtype=torch.float32, device=q.device)
    qs, qr, nq = plan.q_sched
    splits = _FORCE_SPLITS or lib.stb_attn_bwd_splits(hq, hkv, plan.num_k_blocks)
    part = torch.zeros((splits, 2, Tk, hkv, D), dtype=torch.float32, device=q.device) if splits > 1 else None
    rc = lib.stb_attn_bwd(q.data_ptr(), k_buf.data_ptr(), v_buf.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                          delta.data_ptr(), dq.data_ptr(), dk_buf.data_ptr(), dv_buf.data_ptr(), plan.cu_q.data_ptr(),
                          None, qs.data_ptr(), qr.data_ptr(), nq, plan.k_blk_seg.data_ptr(), plan.k_blk_row0.data_ptr(),
                          plan.num_k_blocks, Tq, Tk, hq, hkv, D, q.stride(0), k_buf.stride(0), v_buf.stride(0),
                          dv_buf.stride(0), int(causal), int(window), float(scale), native.ptr(part), splits,
                          plan.seg_k_begin.data_ptr(), plan.seg_k_len.data_ptr(), plan.seg_k_skip.data_ptr(), plan.cp,
                          plan.chunk_len, native.status_word(q.device).data_ptr(), native.stream())
    native.check(rc, "attention backward (gathered keys)")
    count_launch(3 + (splits > 1))
    return dq


def flash_attention(q, k, v, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen=None, causal=True, window=0, scale=None):
    """q ``[Tq,hq,128]``, k/v ``[Tk,hkv,128]`` (v may be a strided view) -> ``[Tq,hq,128]``."""
    Tq, hq, D = q.shape
    if D != 128 or q.dtype != torch.bfloat16:
        raise NotImplementedError("native attention: head_dim 128, bf16")
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if cu_seqlens_q is None:
        cu_seqlens_q = _default_cu(Tq, q.device)
    if cu_seqlens_k is None:
        cu_seqlens_k = cu_seqlens_q if k.shape[0] == Tq else _default_cu(k.shape[0], q.device)
    if cu_seqlens_q.dtype != torch.int32:
        cu_seqlens_q = cu_seqlens_q.to(torch.int32)
    if cu_seqlens_k.dtype != torch.int32:
        cu_seqlens_k = cu_seqlens_k.to(torch.int32)
    return _FlashAttnFn.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, bool(causal), int(window or 0), float(scale))
