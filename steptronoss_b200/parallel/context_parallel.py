"""Context parallelism: load-balanced ("zigzag") sequence sharding with gathered keys and values.

Semantics of the reference (``steptronoss/core/context_parallel/context_parallel.py:10-178`` and
``model/common/grouped_query_attention.py:276-329``): the sequence is cut into ``2·CP`` chunks, rank
``r`` keeps chunks ``r`` and ``2·CP-1-r`` (so that every rank gets the same amount of causal work);
queries stay local, K and V are all-gathered over the CP group (backward: reduce-scatter); each half
of the local queries attends, per packed document, to the keys from the document start up to its own
end.

Two implementations.  On GPUs of one node the keys never get packed: K and V of all ranks are gathered over peer
memory (one launch of the gather kernel of ``csrc/gemm_tp_sm100.cu``) into a rank-major buffer, and the attention
kernels address a key by its *global position* (``key_row`` in ``csrc/attention_common.cuh``), with one segment
per document piece; the forward is a single launch over both halves, the backward one launch group per half
whose dK / dV land in rank-major buffers that are summed and reduce-scattered.  K / V are gathered again in the
backward instead of being kept.  Elsewhere (CPU, other nodes) the two halves become two calls of the
variable-length attention whose q segments are the tail of their key segments; the keys each half needs are
packed from the gathered tensor with one row gather, whose backward sums the contributions of overlapping ranges.
"""
from __future__ import annotations

import math
import os
import weakref
from dataclasses import dataclass, field

import torch

from ..ops import attention
from . import comm
from .state import PM

PEER_PATH = os.environ.get("STB200_CP_PEER", "1") != "0"


def _cp():
    return PM.size_of("CP"), PM.rank_in("CP")


def balanced_chunk_ids(rank: int, cp: int) -> tuple[int, int]:
    return rank, 2 * cp - 1 - rank


def scatter_to_balanced_cp_region(x: torch.Tensor, dim: int = 0) -> torch.Tensor:
    """Keep chunks ``r`` and ``2·CP-1-r`` of ``2·CP`` equal chunks along ``dim`` (no communication: every
    CP rank holds the full tensor)."""
    cp, r = _cp()
    if cp == 1:
        return x
    if x.shape[dim] % (2 * cp):
        raise ValueError(f"length {x.shape[dim]} is not divisible by 2*CP = {2 * cp}")
    chunks = x.chunk(2 * cp, dim=dim)
    a, b = balanced_chunk_ids(r, cp)
    return torch.cat([chunks[a], chunks[b]], dim=dim)


class _GatherBalanced(torch.autograd.Function):
    """All-gather over CP and restore the global order; backward reduce-scatters in the zigzag layout."""

    @staticmethod
    def forward(ctx, x):
        cp, _ = _cp()
        full = torch.empty((cp * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
        comm.all_gather_into_tensor(full, x.contiguous(), group=PM.group_of("CP"))
        half = x.shape[0] // 2
        parts = full.view(cp, 2, half, *x.shape[1:])
        order = [None] * (2 * cp)
        for rank in range(cp):
            a, b = balanced_chunk_ids(rank, cp)
            order[a], order[b] = parts[rank, 0], parts[rank, 1]
        return torch.cat(order, dim=0)

    @staticmethod
    def backward(ctx, g):
        cp, _ = _cp()
        chunks = g.chunk(2 * cp, dim=0)
        zig = []
        for rank in range(cp):
            a, b = balanced_chunk_ids(rank, cp)
            zig += [chunks[a], chunks[b]]
        full = torch.cat(zig, dim=0).contiguous()
        out = torch.empty((full.shape[0] // cp, *full.shape[1:]), dtype=g.dtype, device=g.device)
        comm.reduce_scatter_tensor(out, full, group=PM.group_of("CP"))
        return out


def gather_from_balanced_cp_region(x: torch.Tensor) -> torch.Tensor:
    """Local ``[2L, ...]`` (two zigzag chunks) -> global ``[2·CP·L, ...]`` in sequence order."""
    if PM.size_of("CP") == 1:
        return x
    return _GatherBalanced.apply(x)


@dataclass
class HalfPlan:
    cu_q: torch.Tensor            # int32 [n+1] over the half's local q rows
    cu_k: torch.Tensor            # int32 [n+1] over the packed keys of the half
    key_index: torch.Tensor       # int64 [sum k] rows of the *global-order* K/V to pack
    max_q: int = 0
    max_k: int = 0


@dataclass
class CPMeta:
    chunk_len: int
    token_index: torch.Tensor     # int64 [2L] global positions of this rank's tokens
    halves: list = field(default_factory=list)
    pieces: list = field(default_factory=list)    # per half: [(q_begin, q_end, k_begin)] in global positions
    cp: int = 1
    _gathered: tuple | None = None                # (plan over both halves, [plan of half 0, plan of half 1])

    def gathered_plans(self, device):
        """Segment tables of the global-position kernels, built on first use."""
        if self._gathered is None:
            from ..ops.attention_native import GatheredKeyPlan

            both = GatheredKeyPlan(self.pieces[0] + self.pieces[1], self.cp, self.chunk_len, device)
            self._gathered = (both, [GatheredKeyPlan(p, self.cp, self.chunk_len, device) for p in self.pieces])
        return self._gathered

    def local_position_id(self, position_id: torch.Tensor) -> torch.Tensor:
        return position_id.index_select(0, self.token_index.to(position_id.device))


def cu_seqlens_to_balanced_cp(cu_seqlens: list, total: int, cp: int, rank: int) -> list:
    """Per half of rank ``rank``: list of ``(q_begin, q_end, k_begin)`` in global positions, one entry per
    document piece that falls into the half (``k_end == q_end``)."""
    L = total // (2 * cp)
    out = []
    for c in balanced_chunk_ids(rank, cp):
        lo, hi = c * L, (c + 1) * L
        pieces = []
        for ds, de in zip(cu_seqlens[:-1], cu_seqlens[1:]):
            qs, qe = max(ds, lo), min(de, hi)
            if qe > qs:
                pieces.append((qs, qe, ds))
        if not pieces or pieces[-1][1] < hi:  # tokens after the last document (padding) attend to themselves
            start = pieces[-1][1] if pieces else lo
            pieces.append((start, hi, start))
        out.append(pieces)
    return out


_META_CACHE: dict = {}


def build_cp_meta(cu_seqlens, total: int, device=None) -> CPMeta:
    cp, rank = _cp()
    if cu_seqlens is None:
        cu_list = [0, total]
    else:
        key = (id(cu_seqlens), cu_seqlens._version, total, cp, rank)
        hit = _META_CACHE.get(key)
        if hit is not None and hit[0]() is cu_seqlens:  # same tensor object, not a recycled address
            return hit[1]
        cu_list = [int(v) for v in cu_seqlens.tolist()]  # host read, once per micro-batch
    if total % (2 * cp):
        raise ValueError(f"sequence length {total} is not divisible by 2*CP = {2 * cp}")
    device = device or (cu_seqlens.device if cu_seqlens is not None else "cpu")
    L = total // (2 * cp)
    a, b = balanced_chunk_ids(rank, cp)
    token_index = torch.cat([torch.arange(a * L, (a + 1) * L), torch.arange(b * L, (b + 1) * L)]).to(device)
    meta = CPMeta(L, token_index, cp=cp)
    for pieces in cu_seqlens_to_balanced_cp(cu_list, total, cp, rank):
        meta.pieces.append(pieces)
        q_lens = [qe - qs for qs, qe, _ in pieces]
        k_lens = [qe - ks for _, qe, ks in pieces]
        cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=device)
        cu_k = torch.tensor([0] + list(torch.tensor(k_lens).cumsum(0)), dtype=torch.int32, device=device)
        idx = torch.cat([torch.arange(ks, qe) for _, qe, ks in pieces]).to(device)
        meta.halves.append(HalfPlan(cu_q, cu_k, idx, max(q_lens), max(k_lens)))
    if cu_seqlens is not None:
        if len(_META_CACHE) > 32:
            _META_CACHE.clear()
        _META_CACHE[key] = (weakref.ref(cu_seqlens), meta)
    return meta


class _PeerCPAttention(torch.autograd.Function):
    """Attention of the local queries against the keys of all CP ranks, addressed by global position."""

    @staticmethod
    def _gather(kv_local):
        from . import symm

        _, buf = symm.all_gather_gemm(kv_local, None, "CP")
        return buf

    @staticmethod
    def forward(ctx, q, k, v, meta, causal, window):
        from ..ops import attention_native as an

        rows, hkv, D = k.shape
        scale = 1.0 / math.sqrt(D)
        q = q.contiguous()
        kv_local = torch.cat([k.reshape(rows, hkv * D), v.reshape(rows, hkv * D)], dim=1)
        buf = _PeerCPAttention._gather(kv_local).view(-1, 2, hkv, D)     # valid until the next gather on the group
        both, _ = meta.gathered_plans(q.device)
        o, lse = an.gathered_attention_fwd(q, buf[:, 0], buf[:, 1], both, causal, window, scale)
        ctx.save_for_backward(q, kv_local, o, lse)
        ctx.cfg = (meta, causal, window, scale, hkv, D)
        return o

    @staticmethod
    def backward(ctx, do):
        from ..ops import attention_native as an

        q, kv_local, o, lse = ctx.saved_tensors
        meta, causal, window, scale, hkv, D = ctx.cfg
        L, cp = meta.chunk_len, meta.cp
        do = do.contiguous()
        buf = _PeerCPAttention._gather(kv_local).view(-1, 2, hkv, D)
        _, halves = meta.gathered_plans(q.device)
        # [half][dK | dV][rank-major key rows]: a half writes only the rows its segments cover
        part = torch.zeros((2, 2, buf.shape[0], hkv, D), dtype=q.dtype, device=q.device)
        dq = []
        for h, plan in enumerate(halves):
            rows = slice(h * L, (h + 1) * L)
            dq.append(an.gathered_attention_bwd(q[rows], buf[:, 0], buf[:, 1], o[rows], do[rows],
                                                lse[:, rows].contiguous(), plan, causal, window, scale,
                                                part[h, 0], part[h, 1]))
        total = part[0].add_(part[1])
        dkv = torch.empty((2, 2 * L, hkv, D), dtype=q.dtype, device=q.device)
        for i in range(2):                       # rank-major rows: exactly the layout reduce-scatter cuts
            comm.reduce_scatter_tensor(dkv[i], total[i], group=PM.group_of("CP"))
        return torch.cat(dq, dim=0), dkv[0], dkv[1], None, None, None


def _peer_path_ok(q, k, v, meta: CPMeta) -> bool:
    if not (PEER_PATH and q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and meta.chunk_len % 128 == 0):
        return False
    from . import symm

    return symm.enabled("CP") and symm.usable(2 * meta.chunk_len, 2 * k.shape[1] * k.shape[2], 0)


def cp_attention(q, k, v, meta: CPMeta, causal: bool = True, window: int = 0):
    """q ``[2L,hq,D]`` (local zigzag chunks), k/v ``[2L,hkv,D]`` local -> ``[2L,hq,D]``."""
    L = meta.chunk_len
    if _peer_path_ok(q, k, v, meta):
        return _PeerCPAttention.apply(q, k, v, meta, causal, window)
    k_all = gather_from_balanced_cp_region(k.contiguous())
    v_all = gather_from_balanced_cp_region(v.contiguous())
    outs = []
    for h, plan in enumerate(meta.halves):
        qh = q[h * L : (h + 1) * L]
        kh = k_all.index_select(0, plan.key_index)
        vh = v_all.index_select(0, plan.key_index)
        outs.append(attention(qh, kh, vh, plan.cu_q, plan.cu_k, plan.max_k, causal=causal, window=window))
    return torch.cat(outs, dim=0)
