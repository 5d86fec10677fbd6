"""Variable-length causal attention with grouped-query heads.

``attention`` is the single entry point of the framework: on CUDA it runs the hand-written
tcgen05 flash-attention kernels (``csrc/attention_sm100.cu``), on CPU tensors the PyTorch
restatement below, which follows the fallback path of the reference ``AttentionCore``
(``steptronoss/model/common/attention_core.py:270-400``): a loop over the ``cu_seqlens`` segments
with per-segment causal / sliding-window masks and separate q and k segment tables (needed by
context parallelism, where a rank's queries are a slice of the keys it sees).
"""
from __future__ import annotations

import math
import os

import torch



def _segment_mask(lq: int, lk: int, causal: bool, window: int, device):
    """Boolean [lq, lk] mask, True = attend. Causality is aligned to the end of the key segment."""
    if not causal and window <= 0:
        return None
    qi = torch.arange(lq, device=device).unsqueeze(1) + (lk - lq)
    kj = torch.arange(lk, device=device).unsqueeze(0)
    mask = torch.ones(lq, lk, dtype=torch.bool, device=device)
    if causal:
        mask &= kj <= qi
    if window > 0:
        mask &= kj > qi - window
    return mask


def attention_reference(q, k, v, cu_seqlens_q=None, cu_seqlens_k=None, causal=True, window=0, scale=None):
    """q ``[Tq,hq,D]``, k/v ``[Tk,hkv,D]`` -> ``[Tq,hq,D]``. fp32 softmax, output in q's dtype."""
    Tq, hq, D = q.shape
    Tk, hkv, _ = k.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if cu_seqlens_q is None:
        cu_seqlens_q = torch.tensor([0, Tq], dtype=torch.int32)
    if cu_seqlens_k is None:
        cu_seqlens_k = cu_seqlens_q if Tq == Tk else torch.tensor([0, Tk], dtype=torch.int32)
    cq = cu_seqlens_q.tolist()
    ck = cu_seqlens_k.tolist()
    rep = hq // hkv
    outs = []
    for i in range(len(cq) - 1):
        qs = q[cq[i] : cq[i + 1]].transpose(0, 1).float()  # [hq, lq, D]
        ks = k[ck[i] : ck[i + 1]].transpose(0, 1).float()
        vs = v[ck[i] : ck[i + 1]].transpose(0, 1).float()
        if rep > 1:
            ks = ks.repeat_interleave(rep, dim=0)
            vs = vs.repeat_interleave(rep, dim=0)
        lq, lk = qs.shape[1], ks.shape[1]
        if lq == 0:
            continue
        if lk == 0:
            outs.append(torch.zeros(lq, hq, D, dtype=q.dtype, device=q.device))
            continue
        s = torch.matmul(qs, ks.transpose(1, 2)) * scale
        mask = _segment_mask(lq, lk, causal, window, q.device)
        if mask is not None:
            s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)  # rows with no visible key
        outs.append(torch.matmul(p, vs).transpose(0, 1).to(q.dtype))
    if not outs:
        return torch.zeros_like(q)
    out = torch.cat(outs, dim=0)
    if out.shape[0] < Tq:  # rows after the last segment (padding) produce zeros
        out = torch.cat([out, torch.zeros(Tq - out.shape[0], hq, D, dtype=q.dtype, device=q.device)])
    return out


def _native_attention_enabled() -> bool:
    return os.environ.get("STB200_DEBUG_REFERENCE_ATTENTION", "0") != "1"


def attention(q, k, v, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen: int | None = None, causal: bool = True,
              window: int = 0, scale: float | None = None):
    """Packed variable-length attention. Segments are given by ``cu_seqlens_*`` (int32, device);
    ``None`` means one segment spanning all rows."""
    if q.is_cuda and _native_attention_enabled():
        from .attention_native import flash_attention

        return flash_attention(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen, causal, window, scale)
    return attention_reference(q, k, v, cu_seqlens_q, cu_seqlens_k, causal, window, scale)
