"""Step3-VL-10B model configuration: the Qwen3-8B text stack plus a 47-layer vision transformer (patch 14 on 728 px
images, hidden 1536, 2-D RoPE, layer scale, two stride-2 convolutional down-samplers), whose features are spliced
into the token embeddings after every image start token (reference ``playground/pretrain/step3v/step3v_10b.py``)."""
import torch

from playground.pretrain.qwen3.qwen3_8b import (Qwen3AttentionConfig, Qwen3FeedForwardConfig,
                                                Qwen3OutputEmbeddingConfig, Qwen3ParallelConfig)
from steptronoss_b200.config import Ref
from steptronoss_b200.models.common.image_insert import ImageInsertInputEmbeddingConfig
from steptronoss_b200.models.common.vit import VisionTransformerConfig
from steptronoss_b200.models.step3v import QwenVLModelConfig


class Step3VVisionConfig(VisionTransformerConfig):
    def __init__(self):
        super().__init__()
        self.in_channels, self.image_size, self.patch_size = 3, 728, 14
        self.hidden_size, self.ffn_hidden_size, self.num_layers, self.num_attention_heads = 1536, 8960, 47, 16
        self.vit_downsampler_hidden_dim = 3072
        self.output_dim = self.hidden_size * 4
        self.layernorm_epsilon = 1e-5
        self.use_rope2d = True
        self.rope_theta, self.rope_max_freq, self.rope_num_freqs, self.rope_theta_rescale_factor = 10000, 10, 1, 1.0
        self.layer_scale_init_value = 0.1
        self.use_cls_token, self.use_ln_pre, self.patch_embed_bias = False, True, False
        self.vit_downsampler1_kernel_size, self.vit_downsampler1_padding = 3, 1
        self.vit_downsampler2_kernel_size, self.vit_downsampler2_padding = 3, 1


class Step3VInputEmbeddingConfig(ImageInsertInputEmbeddingConfig):
    encoder_cfg = Step3VVisionConfig
    image_token_id: int = 151679
    """placeholder id of an image feature slot"""
    img_end_token: int = 151681
    patch_start_token: int = 151689
    patch_end_token: int = 151690
    patch_new_line_token: int = 151691

    def __init__(self):
        super().__init__()
        self.vocab_size = 151936
        self.hidden_size = Ref("..hidden_size")
        self.img_start_token = 151680
        self.encoder_no_grad = True
        self.projector_bias = False


class Step3V10BConfig(QwenVLModelConfig):
    ffn_cfg = Qwen3FeedForwardConfig
    attn_cfg = Qwen3AttentionConfig
    tok_embed_cfg = Step3VInputEmbeddingConfig
    out_embed_cfg = Qwen3OutputEmbeddingConfig
    parallel_cfg = Qwen3ParallelConfig

    def __init__(self):
        super().__init__()
        self.num_layers, self.hidden_size = 36, 4096
        self.layernorm_epsilon = 1e-6
        self.tie_embedding = False
        self.params_dtype = torch.bfloat16
        self.variable_seq_lengths = True
        self.attn_cfg.max_position_embeddings = 40960


Step3VL10BConfig = Step3V10BConfig
