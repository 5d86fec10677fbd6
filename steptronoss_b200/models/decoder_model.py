"""Decoder-only transformer with a pipeline layer map.

Reference: ``steptronoss/model/decoder_model.py:39-301``.  ``DecoderLLMConfig.build_layer_map``
assigns global layer ids (with per-layer options such as ``recompute``) to every
``(pipeline rank, virtual chunk)``; ``LlamaLikeModel`` builds the layers of its own chunk.
Activations are ``[tokens(/TP), hidden]``; the packed micro-batch travels as ``input_ids [1, S]``
plus ``cu_seqlens``, ``position_id`` and ``max_seq_len``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..exp.base_exp import Megatron3DParallelModelConfig, MegatronTPConfig
from ..ops import residual_add
from ..parallel.random import checkpoint, get_rng_tracker
from ..parallel.state import PM
from ..utils.general import get_position_id_from_cu_seqlens, list_split
from .common.attention import AttentionConfig
from .common.feed_forward import FeedForwardConfig
from .common.parallel_embedding import InputEmbeddingConfig, OutputEmbeddingConfig
from .common.rms_norm import RMSNorm
from .module import MegatronModule

_ALL_PARTS = ["attention", "attn_norm", "feed_forward", "ffn_norm"]


class DecoderLLMConfig(Megatron3DParallelModelConfig):
    num_layers: int
    hidden_size: int
    layernorm_epsilon: float = 1e-6
    rms_norm_zero_gamma: bool = False
    recompute: list | bool = []
    """Per-block recompute: any of 'attention', 'attn_norm', 'feed_forward', 'ffn_norm'; True = all
    (one checkpoint around the whole block). A custom ``pp_vp_allocation`` overrides it per layer."""
    recompute_num_layers: int | None = None
    """When set, ``recompute`` applies to the first ``recompute_num_layers`` layers of every pipeline chunk
    only; the remaining layers keep their activations (a memory / speed dial for 180 GB parts)."""
    tie_embedding: bool = False
    init_std: float = 0.02

    tp_cfg: MegatronTPConfig = MegatronTPConfig
    ffn_cfg: FeedForwardConfig = FeedForwardConfig
    attn_cfg: AttentionConfig = AttentionConfig
    tok_embed_cfg: InputEmbeddingConfig = InputEmbeddingConfig
    out_embed_cfg: OutputEmbeddingConfig = OutputEmbeddingConfig

    def pp_vp_allocation(self, abs_pp_rank: int) -> list:
        chunks = PM.get_vpp_size() * PM.size_of("PP")
        n = len(list_split(list(range(self.num_layers)), chunks)[abs_pp_rank])
        return [{} for _ in range(n)]

    def build_layer_map(self) -> dict:
        layer_map, layer_id = {}, 0
        for vp in range(PM.get_vpp_size()):
            for pp in range(PM.size_of("PP")):
                chunk = layer_map.setdefault(pp, {}).setdefault(vp, {})
                for pos, opts in enumerate(self.pp_vp_allocation(vp * PM.size_of("PP") + pp)):
                    opts = dict(opts)
                    partial = self.recompute_num_layers is not None and pos >= self.recompute_num_layers
                    opts.setdefault("recompute", False if partial else self.recompute)
                    chunk[layer_id] = opts
                    layer_id += 1
        return layer_map

    def build_block(self, layer_id: int, opts: dict):
        if opts.get("noop", False):
            return NoopTransformerBlock()
        return TransformerBlock(self, layer_id, opts.get("recompute", False))

    def build_model(self, vpp_rank: int | None = None):
        return LlamaLikeModel(cfg=self, layer_map=self.build_layer_map(), vpp_rank=vpp_rank)

    def sanity_check(self):
        super().sanity_check()
        if self.tie_embedding and self.parallel_cfg.pipeline_model_parallel_size != 1:
            raise NotImplementedError("Tie embedding for PP > 1")


class NoopTransformerBlock(nn.Module):
    """Placeholder layer used by uneven layer maps (keeps layer numbering, does nothing)."""

    def forward(self, x, **kw):
        return x


class TransformerBlock(nn.Module):
    """Pre-norm residual block: ``x + attn(norm(x))`` then ``x + ffn(norm(x))``."""

    def __init__(self, cfg: DecoderLLMConfig, layer_id: int, recompute=False):
        super().__init__()
        self.cfg, self.layer_id = cfg, layer_id
        if recompute is True:
            self.recompute_all, self.recompute = True, list(_ALL_PARTS)
        else:
            self.recompute_all, self.recompute = False, list(recompute or [])
        sp = bool(cfg.tp_cfg.sequence_parallel)
        # with sequence parallelism the block input is already 1/TP per rank: nothing left to distribute
        self.distribute_saved_activations = bool(cfg.tp_cfg.distribute_saved_activations) and not sp
        self.attention_norm = RMSNorm(cfg.hidden_size, cfg.layernorm_epsilon, sequence_parallel=sp,
                                      use_zero_init=cfg.rms_norm_zero_gamma, params_dtype=cfg.params_dtype)
        self.ffn_norm = RMSNorm(cfg.hidden_size, cfg.layernorm_epsilon, sequence_parallel=sp,
                                use_zero_init=cfg.rms_norm_zero_gamma, params_dtype=cfg.params_dtype)
        self.attention = cfg.attn_cfg.build_model(layer_id=layer_id)
        self.feed_forward = cfg.ffn_cfg.build_model(layer_id=layer_id)

    def _maybe(self, part: str, fn, *args):
        if part in self.recompute and not self.recompute_all and torch.is_grad_enabled():
            return checkpoint(fn, *args, distribute_saved_activations=self.distribute_saved_activations)
        return fn(*args)

    def _body(self, x, position_id, cu_seqlens, max_seqlen, cp_meta):
        h = self._maybe("attn_norm", self.attention_norm, x)
        a = self._maybe("attention", lambda t: self.attention(t, position_id, cu_seqlens, max_seqlen, cp_meta), h)
        if "ffn_norm" in self.recompute and not self.recompute_all:
            x = residual_add(x, a)
            h = self._maybe("ffn_norm", self.ffn_norm, x)
        else:
            x, h = self.ffn_norm.forward_with_residual(x, a)   # x + a and its norm in one pass
        f = self._maybe("feed_forward", self.feed_forward, h)
        return residual_add(x, f)

    def forward(self, x, position_id=None, cu_seqlens=None, max_seqlen=None, cp_meta=None):
        if self.recompute_all and torch.is_grad_enabled() and x.requires_grad:
            return checkpoint(lambda t: self._body(t, position_id, cu_seqlens, max_seqlen, cp_meta), x,
                              distribute_saved_activations=self.distribute_saved_activations)
        return self._body(x, position_id, cu_seqlens, max_seqlen, cp_meta)


class LlamaLikeModel(MegatronModule):
    def __init__(self, cfg: DecoderLLMConfig, layer_map: dict, vpp_rank: int | None = None):
        super().__init__(vpp_rank)
        self.cfg = cfg
        my = layer_map[PM.rank_in("PP")][self.vpp_rank]
        self.layer_ids = list(my.keys())
        self.layers = nn.ModuleDict({str(i): cfg.build_block(i, my[i]) for i in self.layer_ids})
        if self.is_first_stage:
            self.tok_embeddings = cfg.tok_embed_cfg.build_model()
        if self.is_last_stage:
            tied = self.tok_embeddings.word_embeddings.weight if (cfg.tie_embedding and self.is_first_stage) else None
            self.out_embeddings = cfg.out_embed_cfg.build_model(tied_embedding_weight=tied)
        self.sequence_parallel = bool(cfg.tp_cfg.sequence_parallel) and PM.size_of("TP") > 1
        self.name_parameters()

    def name_parameters(self) -> None:
        """Names under which gradient norms are logged: one per layer, the embeddings, the output head (with the
        final norm), anything else (a vision encoder, ...) as ``other`` (reference ``model/decoder_model.py:288-301``)."""
        for p in self.parameters():
            p._log_name = "other"
        for i in self.layer_ids:
            for p in self.layers[str(i)].parameters():
                p._log_name = f"layer{i}"
        if hasattr(self, "tok_embeddings"):
            for p in self.tok_embeddings.parameters():
                p._log_name = "tok_embeddings"
        if hasattr(self, "out_embeddings"):
            for p in self.out_embeddings.parameters():
                p._log_name = "output"

    # ------------------------------------------------------------------ stages
    def _cp_meta(self, data):
        if PM.size_of("CP") == 1:
            return None
        from ..parallel.context_parallel import build_cp_meta

        return build_cp_meta(data.get("cu_seqlens"), data["input_ids"].numel() if "input_ids" in data else None)

    def forward_head(self, input_ids=None, **data):
        ids = input_ids.reshape(-1)
        if PM.size_of("CP") > 1:
            from ..parallel.context_parallel import scatter_to_balanced_cp_region

            ids = scatter_to_balanced_cp_region(ids, dim=0)
        return self.tok_embeddings(ids)

    def forward_chunk(self, hidden, input_ids=None, cu_seqlens=None, position_id=None, max_seq_len=None, **data):
        total = None
        if position_id is None:
            if cu_seqlens is not None:
                position_id = get_position_id_from_cu_seqlens(cu_seqlens)
            else:
                total = hidden.shape[0] * (PM.size_of("TP") if self.sequence_parallel else 1) * PM.size_of("CP")
                position_id = torch.arange(total, dtype=torch.int32, device=hidden.device)
        position_id = position_id.reshape(-1).to(torch.int32)
        cp_meta = None
        if PM.size_of("CP") > 1:
            from ..parallel.context_parallel import build_cp_meta

            cp_meta = build_cp_meta(cu_seqlens, position_id.numel(), device=hidden.device)
            position_id = cp_meta.local_position_id(position_id)
        max_seqlen = int(max_seq_len) if max_seq_len is not None else None
        if cu_seqlens is not None:
            cu_seqlens = cu_seqlens.to(device=hidden.device, dtype=torch.int32)
        ctx = get_rng_tracker().fork() if self.sequence_parallel else _null()
        with ctx:
            for i in self.layer_ids:
                hidden = self.layers[str(i)](hidden, position_id=position_id, cu_seqlens=cu_seqlens,
                                             max_seqlen=max_seqlen, cp_meta=cp_meta)
        return hidden

    def forward_tail(self, hidden, labels=None, loss_masks=None, loss_scale=None, return_logits=False, **data):
        """With ``labels`` (training): dict(loss, per-token loss, predictions, ...) through the fused
        projection + cross-entropy; the loss is ``loss_scale * CP * sum(mask * CE) / sum(mask)`` with
        the mask sum taken over the whole (global) sequence. Otherwise vocab-sharded logits
        ``[tokens, V/TP]``."""
        if labels is not None and not return_logits:
            lab = labels.reshape(-1)
            if loss_masks is None:
                loss_masks = torch.ones(lab.shape, dtype=torch.float32, device=lab.device)
            mask = loss_masks.reshape(-1).float()
            cp = PM.size_of("CP")
            scale = (1.0 if loss_scale is None else float(loss_scale)) * cp
            w = mask * (scale / mask.sum().clamp_min(1e-8))
            if cp > 1:
                from ..parallel.context_parallel import scatter_to_balanced_cp_region

                lab = scatter_to_balanced_cp_region(lab, dim=0)
                w = scatter_to_balanced_cp_region(w, dim=0)
            loss, loss_tok, pred = self.out_embeddings.loss(hidden, lab, w)
            return {"loss": loss, "token_loss": loss_tok, "pred": pred, "labels": lab, "weights": w}
        return self.out_embeddings(hidden)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def _moe_types():
    from .common.moe_block import MoEConfig, MoEFeedForwardConfig

    return MoEConfig, MoEFeedForwardConfig


class MoEDecoderLLMConfig(DecoderLLMConfig):
    """Decoder whose feed-forward blocks are routed experts on the layers of ``moe_cfg.moe_layer_list``
    (dense SwiGLU elsewhere).  After every optimizer step the aux-loss-free router bias is updated."""

    moe_cfg = _moe_types()[0]
    ffn_cfg = _moe_types()[1]
