"""Qwen3 dense and MoE decoders (reference ``steptronoss/model/qwen_dense.py:6-231``): the generic
decoder plus the HF <-> native weight mapping."""
from __future__ import annotations

from .decoder_model import DecoderLLMConfig, LlamaLikeModel


class QwenModel(LlamaLikeModel):
    def __init__(self, cfg: DecoderLLMConfig, layer_map: dict, vpp_rank: int | None = None):
        super().__init__(cfg, layer_map, vpp_rank)
        try:
            from ..checkpointing.reshape_ops import build_qwen_reshaper

            self.reshaper = build_qwen_reshaper(cfg, self.layer_ids, self.is_first_stage, self.is_last_stage)
        except ImportError:
            self.reshaper = None
