"""Qwen3-1.7B dense decoder (model configuration only; the SFT / RLVR / eval experiments import it): 28 layers,
hidden 2048, 16 query / 8 KV heads of 128, SwiGLU 6144, per-head QK-norm, RoPE theta 1e6, vocabulary 151936,
tied input / output embeddings."""
from playground.pretrain.qwen3.qwen3_8b import (Qwen3_8BConfig, Qwen3AttentionConfig, Qwen3FeedForwardConfig,
                                                Qwen3InputEmbeddingConfig, Qwen3OutputEmbeddingConfig)


class Qwen3_1p7BAttentionConfig(Qwen3AttentionConfig):
    def __init__(self):
        super().__init__()
        self.num_attention_heads = 16
        self.num_attention_groups = 8
        self.hidden_size = 2048
        self.max_position_embeddings = 327680


class Qwen3_1p7BFeedForwardConfig(Qwen3FeedForwardConfig):
    def __init__(self):
        super().__init__()
        self.hidden_size = 2048
        self.ffn_hidden_size = 6144


class Qwen3_1p7BInputEmbeddingConfig(Qwen3InputEmbeddingConfig):
    def __init__(self):
        super().__init__()
        self.hidden_size = 2048


class Qwen3_1p7BOutputEmbeddingConfig(Qwen3OutputEmbeddingConfig):
    def __init__(self):
        super().__init__()
        self.hidden_size = 2048


class Qwen3_1p7BConfig(Qwen3_8BConfig):
    ffn_cfg = Qwen3_1p7BFeedForwardConfig
    attn_cfg = Qwen3_1p7BAttentionConfig
    tok_embed_cfg = Qwen3_1p7BInputEmbeddingConfig
    out_embed_cfg = Qwen3_1p7BOutputEmbeddingConfig

    def __init__(self):
        super().__init__()
        self.num_layers = 28
        self.hidden_size = 2048
        self.tie_embedding = True
