"""Vision-language decoders: a text decoder (Qwen-style dense or Step-3.5 MoE) whose first stage splices
vision-encoder features into the token embeddings (reference ``playground/pretrain/step3v/step3v_10b.py`` and
``steptronoss/model/common/image_insert_decoder.py``)."""
from __future__ import annotations

from .common.image_insert import ImageInsertDecoderMixin, ImageInsertInputEmbeddingConfig
from .decoder_model import DecoderLLMConfig, LlamaLikeModel
from .step3p5 import Step3p5Model, Step3p5ModelConfig


class _VLInit:
    def __init__(self, cfg, layer_map, vpp_rank=None):
        super().__init__(cfg, layer_map, vpp_rank)
        self.build_multimodal_modules()
        self.name_parameters()


class QwenVLModel(_VLInit, ImageInsertDecoderMixin, LlamaLikeModel):
    pass


class Step3VModel(_VLInit, ImageInsertDecoderMixin, Step3p5Model):
    pass


class QwenVLModelConfig(DecoderLLMConfig):
    tok_embed_cfg: ImageInsertInputEmbeddingConfig = ImageInsertInputEmbeddingConfig

    def build_model(self, vpp_rank=None):
        return QwenVLModel(cfg=self, layer_map=self.build_layer_map(), vpp_rank=vpp_rank)


class Step3VModelConfig(Step3p5ModelConfig):
    tok_embed_cfg: ImageInsertInputEmbeddingConfig = ImageInsertInputEmbeddingConfig

    def build_model(self, vpp_rank=None):
        return Step3VModel(cfg=self, layer_map=self.build_layer_map(), vpp_rank=vpp_rank)
