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


def ropen_linspace(start, end, steps, **kwargs):
    """``steps`` points from ``start`` in equal strides that stop one stride short of ``end``:
    ``ropen_linspace(0, 1, 4) = [0, .25, .5, .75]`` (the exponents ``2i / C`` of the rotary frequencies)."""
    return torch.linspace(start, end, steps + 1, **kwargs)[:-1]


def ntk_by_rotations_inv_freq(inv_freq: torch.Tensor, max_position: int, ratio: float, beta_fast: float = 32.0,
                              beta_slow: float = 1.0) -> torch.Tensor:
    """The reference's YaRN rule (model/common/rope.py ``_get_frequencies``), switched on by ``ntk_interp_ratio != 1``.

    A frequency that turns at least ``beta_fast`` times over ``max_position`` tokens keeps its value, one that turns
    at most ``beta_slow`` times is divided by ``ratio``, and in between the two are blended linearly in the number
    of turns (HF's YaRN ramps linearly in the channel index instead; that one is ``yarn_inv_freq`` above)."""
    if ratio == 1.0:
        return inv_freq
    turns = max_position * inv_freq / (2 * math.pi)
    keep = ((turns - beta_slow) / (beta_fast - beta_slow)).clamp(0, 1)
    return inv_freq * keep + inv_freq / ratio * (1 - keep)


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
        elif ntk_interp_ratio != 1.0:
            if not max_position:
                raise ValueError("ntk_interp_ratio != 1 needs max_position_embeddings (the context the turns are counted over)")
            self.scaling = lambda f: ntk_by_rotations_inv_freq(f, max_position, ntk_interp_ratio, beta_fast, beta_slow)
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


class YARNRoPE(nn.Module):
    """Stand-alone rotary embedding with the constructor and call of the reference's class (model/common/rope.py:38-250):
    ``feature [B, S, H, C]`` rotated in fp32 over the half-split channel pairs (or adjacent pairs), positions
    ``0..S-1`` or ``position_id [S]`` for packed samples.  The decoder does not call this module - its rotation is
    fused with the QK norm kernel - but ViT-style code and tests written against the reference do."""

    def __init__(self, dim: int, theta: float = 10000.0, ntk_interp_ratio: float = 1.0, yarn_beta_slow: float = 1,
                 yarn_beta_fast: float = 32, max_position_embeddings: int | None = None, use_adjacent_pair: bool = False):
        super().__init__()
        self.dim, self.theta, self.ntk_interp_ratio = dim, theta, ntk_interp_ratio
        self.max_position_embeddings, self.use_adjacent_pair = max_position_embeddings, use_adjacent_pair
        self.tables_owner = RotaryEmbedding(dim, theta, max_position_embeddings or 8192, 1.0, None, yarn_beta_fast,
                                            yarn_beta_slow, ntk_interp_ratio)

    @staticmethod
    def rotate_half(x: torch.Tensor) -> torch.Tensor:
        a, b = x.chunk(2, dim=-1)
        return torch.cat((-b, a), dim=-1)

    def forward(self, feature: torch.Tensor, position_id: torch.Tensor | None = None) -> torch.Tensor:
        b, s, h, c = feature.shape
        if position_id is not None:
            need = self.max_position_embeddings or int(position_id.max()) + 1
            cos, sin = self.tables_owner.tables(feature.device, need)
            cos, sin = cos[position_id.long()], sin[position_id.long()]
        else:
            cos, sin = (t[:s] for t in self.tables_owner.tables(feature.device, s))
        cos, sin = (torch.cat([t, t], -1)[None, :, None, :] for t in (cos, sin))
        x = feature
        if self.use_adjacent_pair:                       # (x0, x1), (x2, x3) ... -> the half-split order
            x = x.view(b, s, h, c // 2, 2).transpose(4, 3).reshape(b, s, h, c)
        x = x.float()
        return (x * cos + self.rotate_half(x) * sin).to(feature.dtype)


def _rope_config_cls():
    from ...exp.abstract import ModelConfig

    class RoPEConfig(ModelConfig):
        """Config node that builds a ``YARNRoPE`` (reference: model/common/rope.py:19-35)."""

        dim: int = 128
        theta: float = 10000.0
        ntk_interp_ratio: float = 1.0
        yarn_beta_slow: float = 1.0
        yarn_beta_fast: float = 32.0
        max_position_embeddings: int | None = None

        def build_model(self):
            return YARNRoPE(dim=self.dim, theta=self.theta, ntk_interp_ratio=self.ntk_interp_ratio,
                            yarn_beta_slow=self.yarn_beta_slow, yarn_beta_fast=self.yarn_beta_fast,
                            max_position_embeddings=self.max_position_embeddings)

    return RoPEConfig


RoPEConfig = _rope_config_cls()
