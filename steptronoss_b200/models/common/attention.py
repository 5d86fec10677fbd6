"""Grouped-query attention block.

Reference: ``steptronoss/model/common/grouped_query_attention.py:18-349``.  One fused column-
parallel projection produces q, k, v (and optional head-wise gate logits); q and k are RMS-normalised
per head and rotated (one fused kernel); packed variable-length causal attention; row-parallel
output projection.  Layout of the fused projection per TP shard: ``[q heads | k heads | v heads |
gate]`` (the reference interleaves k and v per group; the HF reshaper accounts for the difference).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ...config import Config, Ref
from ...ops import attention, qknorm_rope
from ...parallel.layers import ColumnParallelLinear, RowParallelLinear
from ...parallel.state import PM
from .rope import RotaryEmbedding


def _per_layer(v, layer_id):
    return v[layer_id] if isinstance(v, (list, tuple)) else v


class AttentionConfig(Config):
    tp_cfg = Ref("..tp_cfg")
    params_dtype = Ref("..params_dtype", torch.bfloat16)
    causal: bool = True
    attention_dropout: float = 0.0
    use_sliding_window: bool | list = False
    num_attention_heads: int
    num_attention_groups: int
    head_dim: int | None = None
    hidden_size: int
    use_headwise_attn_gate: bool = False
    use_qkv_bias: bool = False
    sliding_window_size: int | None = -1
    use_qk_norm: bool = False
    """Reference semantics (inverted): ``False`` ENABLES the per-head q/k RMSNorm
    (``grouped_query_attention.py:127``). ``qk_norm`` below, when not None, overrides it directly."""
    qk_norm: bool | None = None
    layernorm_epsilon: float = 1e-6
    rms_norm_zero_gamma: bool = False
    recompute_qknorm_rope: bool = False
    qk_rope_head_dim: int | list | None = None
    rope_theta: float | list = 10000.0
    yarn_beta_slow: float = 1.0
    yarn_beta_fast: float = 32.0
    ntk_interp_ratio: float = 1.0
    rope_scaling_factor: float = 1.0
    rope_use_adjacent_pair: bool = False
    """rotate the pairs (2i, 2i+1) instead of (i, i + rot/2): q and k are brought into the half-split order first (as
    the reference's ``RotaryEmbedding(use_adjacent_pair=True)`` does, ``model/common/rope.py:242-246``) and stay in it,
    which leaves every q.k product unchanged"""
    original_max_position_embeddings: int | None = None
    max_position_embeddings: int = 32768
    num_attention_heads_per_layer: list | None = None

    @property
    def qk_norm_enabled(self) -> bool:
        return (not self.use_qk_norm) if self.qk_norm is None else bool(self.qk_norm)

    def build_model(self, layer_id: int):
        return GroupedQueryAttention(cfg=self, layer_id=layer_id)


class GroupedQueryAttention(nn.Module):
    def __init__(self, cfg: AttentionConfig, layer_id: int = 0):
        super().__init__()
        self.cfg = cfg
        self.layer_id = layer_id
        tp = PM.size_of("TP")
        nh = _per_layer(cfg.num_attention_heads_per_layer, layer_id) if cfg.num_attention_heads_per_layer else cfg.num_attention_heads
        self.head_dim = cfg.head_dim or cfg.hidden_size // nh
        self.hq, self.hkv = nh // tp, max(cfg.num_attention_groups // tp, 1)
        if nh % tp or cfg.num_attention_groups % tp:
            raise ValueError(f"heads {nh}/{cfg.num_attention_groups} not divisible by TP={tp}")
        D = self.head_dim
        self.use_gate = bool(cfg.use_headwise_attn_gate)
        self.num_heads, self.num_kv_heads = nh, cfg.num_attention_groups   # global (un-sharded) counts
        self.wqkv_extra_dims = nh if self.use_gate else 0                    # head-wise gate rows of wqkv
        sp = bool(cfg.tp_cfg.sequence_parallel)
        dtype = cfg.params_dtype
        blocks = [nh * D, cfg.num_attention_groups * D, cfg.num_attention_groups * D]
        if self.use_gate:
            blocks.append(nh)
        self.wqkv = ColumnParallelLinear(cfg.hidden_size, sum(blocks), params_dtype=dtype, sequence_parallel=sp,
                                         blocks=blocks, bias=bool(cfg.use_qkv_bias))
        self.wo = RowParallelLinear(nh * D, cfg.hidden_size, params_dtype=dtype, sequence_parallel=sp)
        self.use_qk_norm = cfg.qk_norm_enabled
        if self.use_qk_norm:
            self.q_norm = nn.Module()
            self.k_norm = nn.Module()
            for m in (self.q_norm, self.k_norm):
                m.weight = nn.Parameter(torch.empty(D, dtype=dtype))
                m.weight.init_kind = "zeros" if cfg.rms_norm_zero_gamma else "ones"
                # replicated over TP but every rank only sees its own heads: the gradient is a partial sum
                m.weight.tp_partial_grad = True
        self.rot_dim = _per_layer(cfg.qk_rope_head_dim, layer_id) or D
        theta = float(_per_layer(cfg.rope_theta, layer_id))
        self.rope = RotaryEmbedding(self.rot_dim, theta, cfg.max_position_embeddings, cfg.rope_scaling_factor,
                                    cfg.original_max_position_embeddings, cfg.yarn_beta_fast, cfg.yarn_beta_slow,
                                    cfg.ntk_interp_ratio)
        self.pair_perm = None
        if cfg.rope_use_adjacent_pair:
            r = self.rot_dim
            self.pair_perm = torch.tensor(list(range(0, r, 2)) + list(range(1, r, 2)) + list(range(r, D)))
        sw = _per_layer(cfg.use_sliding_window, layer_id)
        # ``sliding_window_size = w`` is handed to flash-attn as ``window_size=(w, w)`` by the reference
        # (model/common/grouped_query_attention.py:125, attention_core.py:102): a query sees the w keys before it and
        # itself.  The kernels here count the visible keys, so that is w + 1.
        self.window = int(cfg.sliding_window_size) + 1 if sw and cfg.sliding_window_size and cfg.sliding_window_size > 0 else 0

    def forward(self, x, position_id, cu_seqlens=None, max_seqlen=None, cp_meta=None):
        """x ``[tokens(/TP), H]`` -> same shape. ``position_id`` int32 ``[tokens]`` (full sequence on this CP rank)."""
        D, hq, hkv = self.head_dim, self.hq, self.hkv
        qkv = self.wqkv(x)
        T = qkv.shape[0]
        gate = None
        if self.use_gate:
            gate = qkv[:, (hq + 2 * hkv) * D :]
        need = int(max_seqlen) if max_seqlen is not None else None
        cos, sin = self.rope.tables(qkv.device, need if need is not None else self.cfg.max_position_embeddings)
        qw = self.q_norm.weight if self.use_qk_norm else None
        kw = self.k_norm.weight if self.use_qk_norm else None
        if self.pair_perm is not None:
            perm = self.pair_perm.to(qkv.device)
            n_qk = (hq + hkv) * D
            qk = qkv[:, :n_qk].reshape(T, hq + hkv, D).index_select(-1, perm).reshape(T, n_qk)
            qkv = torch.cat([qk, qkv[:, n_qk:]], dim=1)
            if self.use_qk_norm:                       # the per-dimension norm weights move with their dimensions
                qw, kw = qw.index_select(0, perm), kw.index_select(0, perm)
        q, k, v = qknorm_rope(qkv if not self.use_gate else qkv[:, : (hq + 2 * hkv) * D], qw, kw, cos, sin, position_id,
                              hq, hkv, D, self.rot_dim, self.cfg.layernorm_epsilon, self.use_qk_norm,
                              self.cfg.rms_norm_zero_gamma)
        if cp_meta is not None:
            from ...parallel.context_parallel import cp_attention

            o = cp_attention(q, k, v, cp_meta, causal=self.cfg.causal, window=self.window)
        else:
            o = attention(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, causal=self.cfg.causal, window=self.window)
        o = o.reshape(T, hq * D)
        if gate is not None:
            o = (o.view(T, hq, D) * torch.sigmoid(gate.float()).to(o.dtype).unsqueeze(-1)).reshape(T, hq * D)
        return self.wo(o)
