"""Qwen3-30B-A3B-shape mixture of experts: 48 layers, hidden 2048, 32 query / 4 KV heads of 128,
128 experts of SwiGLU width 768 on every layer, softmax router top-8 with renormalised weights,
no shared expert, vocabulary 151936.  Default layout: experts sharded over EP=8 (16 per rank),
attention data-parallel.

Run: ``torchrun --nproc-per-node 8 -m playground.pretrain.qwen3.qwen3_30a3b [key=value ...]``.
"""
import torch

from playground.pretrain.qwen3.qwen3_8b import Exp as DenseExp
from steptronoss_b200.exp.base_exp import ParallelConfig
from steptronoss_b200.exp.ntp import MoEPretrainMetricConfig
from steptronoss_b200.models.common.attention import AttentionConfig
from steptronoss_b200.models.common.moe_block import MoEConfig, MoEFeedForwardConfig
from steptronoss_b200.models.common.parallel_embedding import InputEmbeddingConfig, OutputEmbeddingConfig
from steptronoss_b200.models.decoder_model import MoEDecoderLLMConfig


class Qwen3MoEAttentionConfig(AttentionConfig):
    def __init__(self):
        super().__init__()
        self.num_attention_heads = 32
        self.num_attention_groups = 4
        self.head_dim = 128
        self.hidden_size = 2048
        self.use_qk_norm = False  # reference convention: False enables QK-norm
        self.layernorm_epsilon = 1e-6
        self.rope_theta = 1_000_000.0
        self.max_position_embeddings = 40960


class Qwen3MoEFFNConfig(MoEFeedForwardConfig):
    def __init__(self):
        super().__init__()
        self.hidden_size = 2048
        self.ffn_hidden_size = 6144  # dense fallback width (unused: every layer is MoE)
        self.layernorm_epsilon = 1e-6


class Qwen3MoEConfig(MoEConfig):
    def __init__(self):
        super().__init__()
        self.hidden_size = 2048
        self.moe_num_experts = 128
        self.moe_top_k = 8
        self.moe_hidden_size = 768
        self.moe_aux_loss_coef = 0.0         # as the reference's experiment; HF's config for this model says 1e-3
        self.norm_expert_weight = True
        self.share_expert_dim = 0
        self.moe_layer_list = list(range(48))


class Qwen3MoEInputEmbeddingConfig(InputEmbeddingConfig):
    def __init__(self):
        super().__init__()
        self.vocab_size = 151936
        self.hidden_size = 2048


class Qwen3MoEOutputEmbeddingConfig(OutputEmbeddingConfig):
    def __init__(self):
        super().__init__()
        self.vocab_size = 151936
        self.hidden_size = 2048


class Qwen3MoEParallelConfig(ParallelConfig):
    def __init__(self):
        super().__init__()
        self.tensor_model_parallel_size = 1
        self.expert_model_parallel_size = 8
        self.expert_tensor_parallel_size = 1


class Qwen3_30A3BConfig(MoEDecoderLLMConfig):
    ffn_cfg = Qwen3MoEFFNConfig
    attn_cfg = Qwen3MoEAttentionConfig
    moe_cfg = Qwen3MoEConfig
    tok_embed_cfg = Qwen3MoEInputEmbeddingConfig
    out_embed_cfg = Qwen3MoEOutputEmbeddingConfig
    parallel_cfg = Qwen3MoEParallelConfig

    def __init__(self):
        super().__init__()
        self.num_layers = 48
        self.hidden_size = 2048
        self.layernorm_epsilon = 1e-6
        self.params_dtype = torch.bfloat16
        self.variable_seq_lengths = True
        self.recompute = False

    def build_model(self, vpp_rank=None):
        from steptronoss_b200.models.qwen_dense import QwenModel

        return QwenModel(cfg=self, layer_map=self.build_layer_map(), vpp_rank=vpp_rank)


class Exp(DenseExp):
    model_cfg = Qwen3_30A3BConfig
    metric_cfg = MoEPretrainMetricConfig

    def __init__(self):
        super().__init__()
        t = self.trainer_cfg
        t.global_batch_size = 256
        t.global_seq_length = 4096
        t.micro_batch_size = 1
        self.data_cfg.max_doc_len = 4096


if __name__ == "__main__":
    Exp().train()
