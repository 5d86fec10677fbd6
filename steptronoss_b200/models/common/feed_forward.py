"""Dense SwiGLU feed-forward block (reference ``steptronoss/model/common/feed_forward.py:9-74``):
``w1`` column-parallel ``[H -> 2F]`` laid out ``[gate | up]`` per shard, SwiGLU with optional
clamps, ``w2`` row-parallel."""
from __future__ import annotations

import torch
import torch.nn as nn

from ...config import Config, Ref
from ...ops import swiglu
from ...ops.fused import swiglu_linear
from ...parallel.state import PM
from ...parallel.layers import ColumnParallelLinear, RowParallelLinear


class FeedForwardConfig(Config):
    tp_cfg = Ref("..tp_cfg")
    params_dtype = Ref("..params_dtype", torch.bfloat16)
    hidden_size: int
    ffn_hidden_size: int
    layernorm_epsilon: float = 1e-6
    rms_norm_zero_gamma: bool = False
    swiglu_recompute_silu_out_proj: bool = False
    swiglu_limit: float | list | None = None

    def activation(self, x, swiglu_limit=None):
        """SwiGLU on ``[gate | up]`` halves of the last dimension, optionally clamped (gate above, up on both sides).
        The PyTorch statement of what the fused kernel computes (reference: model/common/feed_forward.py:20-26)."""
        from ...ops.fused import swiglu_reference

        return swiglu_reference(x, float(swiglu_limit) if swiglu_limit else 0.0)

    def build_model(self, layer_id: int = 0):
        return FeedForward(self, layer_id)


class FeedForward(nn.Module):
    def __init__(self, cfg: FeedForwardConfig, layer_id: int = 0, ffn_hidden_size: int | None = None):
        super().__init__()
        F = ffn_hidden_size or cfg.ffn_hidden_size
        sp = bool(cfg.tp_cfg.sequence_parallel)
        self.w1 = ColumnParallelLinear(cfg.hidden_size, 2 * F, params_dtype=cfg.params_dtype, sequence_parallel=sp,
                                       blocks=[F, F])
        self.w2 = RowParallelLinear(F, cfg.hidden_size, params_dtype=cfg.params_dtype, sequence_parallel=sp)
        lim = cfg.swiglu_limit
        if isinstance(lim, (list, tuple)):
            lim = lim[layer_id]
        self.limit = float(lim) if lim else 0.0
        self.fuse_act = bool(cfg.swiglu_recompute_silu_out_proj) and PM.size_of("TP") == 1

    def forward(self, x):
        h = self.w1(x)
        if self.fuse_act:
            # the activation is recomputed inside the down projection's backward instead of being stored
            return swiglu_linear(h, self.w2.weight, self.limit)
        return self.w2(swiglu(h, self.limit))
