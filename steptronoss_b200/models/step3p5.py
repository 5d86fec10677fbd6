"""Step-3.5 decoder: per-layer choice between sliding-window and full attention, routed experts with a
shared expert and an aux-loss-free router bias, head-wise gated attention.

Reference: ``steptronoss/model/step3p5.py:15-316``.  ``swa_layer_list[i]`` selects ``swa_cfg`` (a second
:class:`AttentionConfig`, typically with ``use_sliding_window=True`` and its own head count / RoPE base)
for layer ``i``; every other layer uses ``attn_cfg``.  Both attention flavours run the same
varlen flash-attention kernel, the window being one of its arguments.  The HF <-> native weight
mapping follows the reference's script list (``step3p5.py:86-316``).
"""
from __future__ import annotations

from .common.attention import AttentionConfig
from .common.moe_block import MoEConfig, MoEFeedForwardConfig
from .decoder_model import DecoderLLMConfig, LlamaLikeModel, NoopTransformerBlock, TransformerBlock


class Step3p5Block(TransformerBlock):
    """A transformer block whose attention module comes from ``swa_cfg`` on sliding-window layers."""

    def __init__(self, cfg: "Step3p5ModelConfig", layer_id: int, recompute=False):
        super().__init__(cfg, layer_id, recompute)
        if cfg.swa_layer_list[layer_id]:
            self.attention = cfg.swa_cfg.build_model(layer_id=layer_id)
        self.is_swa = bool(cfg.swa_layer_list[layer_id])


class Step3p5ModelConfig(DecoderLLMConfig):
    swa_cfg: AttentionConfig = AttentionConfig
    moe_cfg: MoEConfig = MoEConfig
    ffn_cfg: MoEFeedForwardConfig = MoEFeedForwardConfig
    swa_layer_list: list = []

    def build_block(self, layer_id: int, opts: dict):
        if opts.get("noop", False):
            return NoopTransformerBlock()
        return Step3p5Block(self, layer_id, opts.get("recompute", False))

    def build_model(self, vpp_rank: int | None = None):
        return Step3p5Model(cfg=self, layer_map=self.build_layer_map(), vpp_rank=vpp_rank)

    def sanity_check(self):
        super().sanity_check()
        if len(self.swa_layer_list) != self.num_layers:
            raise AssertionError(
                f"swa_layer_list has {len(self.swa_layer_list)} entries for {self.num_layers} layers")


class Step3p5Model(LlamaLikeModel):
    @property
    def reshaper(self):
        return self.build_reshaper()

    @reshaper.setter
    def reshaper(self, value):  # the base class may assign a default mapping
        pass

    def build_reshaper(self):
        from ..checkpointing.reshape_ops import (ColumnParallel, Duplicate, FFNMergeGateUp, GQAMergeQKVG, KeepThisEP,
                                                 KeepThisTP, OnlineReshaper, Rename, RowParallel, Script, VocabPad)

        cfg, scripts = self.cfg, []

        def dup(src, dst):
            return Script(src=src, dst=dst, op=Duplicate() + KeepThisTP() + Rename(f"{dst}: {src}"))

        if self.is_first_stage:
            scripts.append(Script(
                src="model.embed_tokens.weight", dst="tok_embeddings.word_embeddings.weight",
                op=VocabPad(cfg.tok_embed_cfg.vocab_size, 0) + ColumnParallel() + KeepThisTP()
                + Rename("tok_embeddings.word_embeddings.weight: model.embed_tokens.weight")))
        if self.is_last_stage:
            scripts.append(Script(
                src="lm_head.weight", dst="out_embeddings.output.weight",
                op=VocabPad(cfg.out_embed_cfg.vocab_size, 0) + ColumnParallel() + KeepThisTP()
                + Rename("out_embeddings.output.weight: lm_head.weight")))
            scripts.append(dup("model.norm.weight", "out_embeddings.norm.weight"))
        for i in self.layer_ids:
            block = self.layers[str(i)]
            if isinstance(block, NoopTransformerBlock):
                continue
            s, d = f"model.layers.{i}", f"layers.{i}"
            att = block.attention
            scripts.append(Script(
                src=f"{s}.self_attn.[qkvg]_proj.weight", dst=f"{d}.attention.wqkv.weight",
                op=GQAMergeQKVG(att.num_kv_heads, att.head_dim, gate_dims=att.wqkv_extra_dims) + KeepThisTP()
                + Rename(f"{d}.attention.wqkv.weight: {s}.self_attn.qkv_proj.weight")))
            scripts.append(Script(
                src=f"{s}.self_attn.o_proj.weight", dst=f"{d}.attention.wo.weight",
                op=RowParallel() + KeepThisTP() + Rename(f"{d}.attention.wo.weight: {s}.self_attn.o_proj.weight")))
            scripts.append(dup(f"{s}.input_layernorm.weight", f"{d}.attention_norm.weight"))
            scripts.append(dup(f"{s}.post_attention_layernorm.weight", f"{d}.ffn_norm.weight"))
            if getattr(att, "q_norm", None) is not None:
                scripts.append(dup(f"{s}.self_attn.q_norm.weight", f"{d}.attention.q_norm.weight"))
                scripts.append(dup(f"{s}.self_attn.k_norm.weight", f"{d}.attention.k_norm.weight"))
            ff = block.feed_forward
            if hasattr(ff, "moe"):
                scripts.append(dup(f"{s}.moe.gate.weight", f"{d}.feed_forward.moe.gate.weight"))
                if ff.moe.router_balance_bias is not None:
                    scripts.append(dup(f"{s}.moe.router_bias", f"{d}.feed_forward.moe.router_balance_bias"))
                scripts.append(Script(
                    src=f"{s}.moe.[gu]*_proj.weight", dst=f"{d}.feed_forward.moe.experts.w1",
                    op=FFNMergeGateUp(group="ETP") + KeepThisTP(group="ETP") + KeepThisEP()
                    + Rename(f"{d}.feed_forward.moe.experts.w1: {s}.moe.gate_up_proj.weight")))
                scripts.append(Script(
                    src=f"{s}.moe.down_proj.weight", dst=f"{d}.feed_forward.moe.experts.w2",
                    op=RowParallel(group="ETP") + KeepThisTP(group="ETP") + KeepThisEP()
                    + Rename(f"{d}.feed_forward.moe.experts.w2: {s}.moe.down_proj.weight")))
                if getattr(ff, "enable_share_expert", False):
                    scripts.append(Script(
                        src=f"{s}.share_expert.[gu]*_proj.weight", dst=f"{d}.feed_forward.share_expert.w1.weight",
                        op=FFNMergeGateUp() + KeepThisTP()
                        + Rename(f"{d}.feed_forward.share_expert.w1.weight: {s}.share_expert.gate_up_proj.weight")))
                    scripts.append(Script(
                        src=f"{s}.share_expert.down_proj.weight", dst=f"{d}.feed_forward.share_expert.w2.weight",
                        op=RowParallel() + KeepThisTP()
                        + Rename(f"{d}.feed_forward.share_expert.w2.weight: {s}.share_expert.down_proj.weight")))
            else:
                scripts.append(Script(
                    src=f"{s}.mlp.[gu]*_proj.weight", dst=f"{d}.feed_forward.w1.weight",
                    op=FFNMergeGateUp() + KeepThisTP()
                    + Rename(f"{d}.feed_forward.w1.weight: {s}.mlp.gate_up_proj.weight")))
                scripts.append(Script(
                    src=f"{s}.mlp.down_proj.weight", dst=f"{d}.feed_forward.w2.weight",
                    op=RowParallel() + KeepThisTP() + Rename(f"{d}.feed_forward.w2.weight: {s}.mlp.down_proj.weight")))
        return OnlineReshaper(scripts)
