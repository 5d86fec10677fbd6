"""Adam on flat fp32 shards.

Hyper-parameters and update rule of ``torch.optim.Adam`` as the reference configures it
(``steptronoss/exp/optimizer.py:33-62``: coupled L2 decay, no decay on biases / 1-D parameters,
per-parameter lr multipliers), or decoupled AdamW (``mode="adamw"``, used for the non-Muon groups
of the Muon optimizer, ``steptronoss/optimizer/muon.py:136-195``).  On CUDA one kernel launch
updates a whole shard: it applies the gradient averaging factor and the device-resident clip
coefficient, updates master/m/v and writes the bf16 parameter copy in the same pass.
"""
from __future__ import annotations

import math
import struct

import torch

from ..ops import native
from ..ops.gemm import count_launch

_CHUNK = 1 << 16


class FlatAdamShard:
    """State + update for one contiguous shard ``[lo, hi)`` of a bucket."""

    def __init__(self, bucket, lo: int, hi: int, segments: list, mode: str = "adam"):
        """``segments``: ``(offset_in_shard, numel, lr_mult, wd_mult)`` for every owned parameter."""
        self.bucket, self.lo, self.hi = bucket, lo, hi
        self.mode = mode
        dev = bucket.param_buf.device
        n = hi - lo
        self.master = bucket.param_buf[lo:hi].float()
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        self.segments = segments
        self.peer = None
        """``(PeerZeroGroup, pointer array)`` when the bucket's parameter buffers are peer-mapped: the update then
        stores the new bf16 values into every rank's buffer (``stb_adam_push``)."""
        self._chunks = None
        self._chunk_wd = None

    def _chunk_table(self, weight_decay: float):
        if self._chunks is not None and self._chunk_wd == weight_decay:
            return self._chunks
        rows = []
        for off, numel, lr_mult, wd_mult in self.segments:
            pos = 0
            while pos < numel:
                ln = min(_CHUNK, numel - pos)
                rows.append(struct.pack("<qiffi", off + pos, ln, float(lr_mult), float(weight_decay * wd_mult), 0))
                pos += ln
        raw = b"".join(rows)
        t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(self.master.device) if raw else None
        self._chunks, self._chunk_wd = (t, len(rows)), weight_decay
        return self._chunks

    def step(self, step: int, lr: float, weight_decay: float, beta1: float, beta2: float, eps: float,
             grad_scale: float, scalars: torch.Tensor | None):
        g = self.bucket.grad_buf[self.lo:self.hi]
        p_lp = self.bucket.param_buf[self.lo:self.hi]
        bc1 = 1.0 - beta1 ** step
        bc2 = 1.0 - beta2 ** step
        if self.master.is_cuda:
            table, n = self._chunk_table(weight_decay)
            if n == 0:
                return
            lib = native.load()
            if self.peer is not None and p_lp.dtype == torch.bfloat16:
                pz, ptrs = self.peer
                native.check(lib.stb_adam_push(self.master.data_ptr(), g.data_ptr(), self.exp_avg.data_ptr(),
                                               self.exp_avg_sq.data_ptr(), ptrs, pz.world, table.data_ptr(), n,
                                               native.ptr(scalars), lr, beta1, beta2, eps, bc1, bc2, grad_scale,
                                               0 if self.mode == "adam" else 1, native.stream()), "adam_push")
                count_launch()
                return
            lp_ptr = p_lp.data_ptr() if p_lp.dtype == torch.bfloat16 else None
            native.check(lib.stb_adam(self.master.data_ptr(), g.data_ptr(), self.exp_avg.data_ptr(),
                                      self.exp_avg_sq.data_ptr(), lp_ptr, table.data_ptr(), n,
                                      native.ptr(scalars), lr, beta1, beta2, eps, bc1, bc2, grad_scale,
                                      0 if self.mode == "adam" else 1, native.stream()), "adam")
            count_launch()
            if lp_ptr is None:
                p_lp.copy_(self.master)
            return
        clip = float(scalars[2]) if scalars is not None else 1.0
        if scalars is not None and float(scalars[3]) == 0.0:
            return
        for off, numel, lr_mult, wd_mult in self.segments:
            sl = slice(off, off + numel)
            gv = g[sl] * (grad_scale * clip)
            p = self.master[sl]
            wd = weight_decay * wd_mult
            lr_eff = lr * lr_mult
            if self.mode == "adam":
                gv = gv + wd * p
            else:
                p.mul_(1.0 - lr_eff * wd)
            self.exp_avg[sl].mul_(beta1).add_(gv, alpha=1 - beta1)
            self.exp_avg_sq[sl].mul_(beta2).addcmul_(gv, gv, value=1 - beta2)
            denom = (self.exp_avg_sq[sl].sqrt() / math.sqrt(bc2)).add_(eps)
            p.addcdiv_(self.exp_avg[sl], denom, value=-(lr_eff / bc1))
        p_lp.copy_(self.master)

    def state_dict(self) -> dict:
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq}

    def load_state_dict(self, sd: dict) -> None:
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
