"""Rotary position embedding tables with YaRN / NTK frequency blending.

Reference: ``steptronoss/model/common/rope.py:38-250`` (half-split rotation, fp32 caches that stay
fp32 when the module is cast, per-token position ids for packed samples).  The rotation itself is
fused with the per-head QK RMSNorm in ``ops.qknorm_rope``; this module owns the tables.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ...ops import rope_tables


def yarn_inv_freq(inv_freq: torch.Tensor, rot_dim: int, theta: float, scaling_factor: float,
                  original_max_position: int, beta_fast: float = 32.0, beta_slow: float = 1.0,
                  ntk_interp_ratio: float = 1.0) -> torch.Tensor:
    """Blend interpolated (``/scaling_factor``) and extrapolated frequencies with the YaRN ramp."""
    if scaling_factor <= 1.0:
        return inv_freq

    def correction_dim(num_rot):
        return (rot_dim * math.log(original_max_position / (num_rot * 2 * math.pi))) / (2 * math.log(theta))

    low = max(math.floor(correction_dim(beta_fast)), 0)
    high = min(math.ceil(correction_dim(beta_slow)), rot_dim // 2 - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(rot_dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
    extrap_weight = (1 - ramp) * ntk_interp_ratio + (1 - ntk_interp_ratio) * 0.0 if ntk_interp_ratio != 1.0 else (1 - ramp)
    return inv_freq / scaling_factor * (1 - extrap_weight) + inv_freq * extrap_weight


class RotaryEmbedding(nn.Module):
    """Holds fp32 ``cos``/``sin`` tables ``[max_pos, rot_dim/2]``, grown on demand."""

    def __init__(self, rot_dim: int, theta: float = 10000.0, max_position: int = 8192, scaling_factor: float = 1.0,
                 original_max_position: int | None = None, beta_fast: float = 32.0, beta_slow: float = 1.0,
                 ntk_interp_ratio: float = 1.0):
        super().__init__()
        self.rot_dim, self.theta = rot_dim, theta
        self.scaling = None
        if scaling_factor > 1.0:
            omp = original_max_position or max_position
            self.scaling = lambda f: yarn_inv_freq(f, rot_dim, theta, scaling_factor, omp, beta_fast, beta_slow,
                                                   ntk_interp_ratio)
        self._max = 0
        self._cos = self._sin = None
        self._want = max_position

    def _apply(self, fn, recurse=True):  # keep the caches fp32 through .to(bf16)/.half()
        return super()._apply(fn, recurse)

    def tables(self, device, need: int | None = None):
        need = max(need or 0, min(self._want, 1 << 16))
        if self._cos is None or self._cos.device != device or need > self._max:
            size = max(need, self._max)
            self._cos, self._sin = rope_tables(size, self.rot_dim, self.theta, device, self.scaling)
            self._max = size
        return self._cos, self._sin
