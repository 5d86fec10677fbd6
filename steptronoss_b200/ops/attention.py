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

from ..utils.optimizable import optimizable


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


def _attention_reference_alt(q, k, v, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen=None, causal=True, window=0,
                             scale=None):
    cu_q = cu_seqlens_q.cpu() if cu_seqlens_q is not None else None
    cu_k = cu_seqlens_k.cpu() if cu_seqlens_k is not None else None
    return attention_reference(q, k, v, cu_q, cu_k, causal, window, scale)


# ``set_optimization(AttentionCore="flash-attn-3")`` of an experiment file written for the reference selects the kernel
# path (there is one); ``"sdpa"`` / ``"reference"`` select the PyTorch statement above.
@optimizable({"reference": _attention_reference_alt, "sdpa": _attention_reference_alt}, aliases=("AttentionCore",),
             native_names=("flash-attn", "flash-attn-3"))
def attention(q, k, v, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen: int | None = None, causal: bool = True,
              window: int = 0, scale: float | None = None):
    """Packed variable-length attention. Segments are given by ``cu_seqlens_*`` (int32, device);
    ``None`` means one segment spanning all rows."""
    if q.is_cuda and _native_attention_enabled():
        from .attention_native import flash_attention

        return flash_attention(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen, causal, window, scale)
    return attention_reference(q, k, v, cu_seqlens_q, cu_seqlens_k, causal, window, scale)


def parse_cu_seqlens(cu_seqlens, max_seq_len=None):
    """``cu_seqlens`` is one int tensor (queries and keys share the segments) or ``{"q": ..., "k": ...}``;
    ``max_seq_len`` an int, a ``{"q", "k"}`` dict or None (then taken from the tables).
    Returns ``(cu_q, cu_k, max_q, max_k)`` with int32 tables (reference: model/common/attention_core.py:11-32)."""
    if isinstance(cu_seqlens, dict):
        cu_q, cu_k = cu_seqlens["q"].to(torch.int32), cu_seqlens["k"].to(torch.int32)
    else:
        cu_q = cu_k = cu_seqlens.to(torch.int32)
    if isinstance(max_seq_len, dict):
        max_q, max_k = max_seq_len.get("q"), max_seq_len.get("k")
    else:
        max_q = max_k = max_seq_len
    if max_q is None:
        max_q = int((cu_q[1:] - cu_q[:-1]).max())
    if max_k is None:
        max_k = int((cu_k[1:] - cu_k[:-1]).max())
    return cu_q, cu_k, max_q, max_k


class AttentionCore(torch.nn.Module):
    """Module form of ``attention`` with the call surface of the reference's ``AttentionCore`` / ``FlashAttention``
    (model/common/attention_core.py:270-400): ``q [b, s, hq, D]``, ``k / v [b, s_k, hkv, D]`` -> ``[b, s, hq, D]``.

    Without ``cu_seqlens`` every batch row is one sequence; with it the rows of all batch entries are read as one
    packed stream cut at ``cu_seqlens`` (one table, or ``{"q", "k"}`` when queries are the tail of longer key
    segments).  ``sliding_window = w >= 0`` shows a query the ``w`` keys before it and itself (flash-attn's
    ``window_size=(w, w)`` under a causal mask); -1 means no window.  Causality is aligned to the end of the key
    segment, as flash-attn does it.  Dropout on the probabilities is applied only by the PyTorch path, which this
    module takes whenever ``attention_dropout > 0`` in training."""

    def __init__(self, causal: bool = True, attention_dropout: float = 0.0, sliding_window: int = -1, **kwargs):
        super().__init__()
        self.causal = bool(causal)
        self.attention_dropout = float(attention_dropout)
        self.sliding_window = (sliding_window, sliding_window)
        if not self.causal and sliding_window is not None and sliding_window >= 0:
            raise ValueError("a sliding window needs causal attention here")

    def _with_dropout(self, q, k, v, cu_q, cu_k, window):
        outs, rep = [], q.shape[1] // k.shape[1]
        for i in range(cu_q.numel() - 1):
            qs = q[int(cu_q[i]):int(cu_q[i + 1])].transpose(0, 1)
            ks = k[int(cu_k[i]):int(cu_k[i + 1])].transpose(0, 1).repeat_interleave(rep, 0)
            vs = v[int(cu_k[i]):int(cu_k[i + 1])].transpose(0, 1).repeat_interleave(rep, 0)
            mask = _segment_mask(qs.shape[1], ks.shape[1], self.causal, window, q.device)
            o = torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, attn_mask=mask, dropout_p=self.attention_dropout)
            outs.append(o.transpose(0, 1))
        return torch.cat(outs, 0)

    def forward(self, q, k, v, cu_seqlens=None, max_seq_len=None):
        b, s, hq, d = q.shape
        sk = k.shape[1]
        if cu_seqlens is None:
            cu_q = torch.arange(b + 1, dtype=torch.int32, device=q.device) * s
            cu_k = cu_q if sk == s else torch.arange(b + 1, dtype=torch.int32, device=q.device) * sk
            max_q = s
        else:
            cu_q, cu_k, max_q, _ = parse_cu_seqlens(cu_seqlens, max_seq_len)
        w = self.sliding_window[0]
        window = w + 1 if w is not None and w >= 0 else 0
        qf, kf, vf = q.reshape(b * s, hq, d), k.reshape(b * sk, -1, d), v.reshape(b * sk, -1, d)
        if self.training and self.attention_dropout > 0:
            out = self._with_dropout(qf, kf, vf, cu_q.cpu(), cu_k.cpu(), window)
        else:
            out = attention(qf, kf, vf, cu_q, cu_k, int(max_q), causal=self.causal, window=window)
        return out.reshape(b, s, hq, d)


FlashAttention = FlashAttention3 = AttentionCore     # one implementation; the reference's class names keep working
