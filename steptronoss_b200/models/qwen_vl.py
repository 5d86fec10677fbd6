"""Qwen decoder with a decoupled vision encoder and image-token insertion (reference
``steptronoss/model/qwen_vl.py:1-12``): the text weights keep the Qwen HF mapping, the vision encoder and the
projector add theirs, so a checkpoint in HF layout loads and exports whole."""
from __future__ import annotations

from .common.image_insert import ImageInsertDecoderMixin, ImageInsertInputEmbeddingConfig
from .decoder_model import DecoderLLMConfig
from .qwen_dense import QwenModel


class QwenImageInsertModel(ImageInsertDecoderMixin, QwenModel):
    def __init__(self, cfg, layer_map, vpp_rank=None):
        super().__init__(cfg, layer_map, vpp_rank)
        self.build_multimodal_modules()
        self.name_parameters()


class QwenImageInsertModelConfig(DecoderLLMConfig):
    tok_embed_cfg: ImageInsertInputEmbeddingConfig = ImageInsertInputEmbeddingConfig

    def build_model(self, vpp_rank=None):
        return QwenImageInsertModel(cfg=self, layer_map=self.build_layer_map(), vpp_rank=vpp_rank)
