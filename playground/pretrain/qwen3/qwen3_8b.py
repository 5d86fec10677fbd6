"""Qwen3-8B dense decoder: 36 layers, hidden 4096, 32 query / 8 KV heads of 128, SwiGLU 12288,
RMSNorm + per-head QK-norm (eps 1e-6), RoPE theta 1e6, vocabulary 151936, untied embeddings.

Default layout TP=4 with sequence parallelism (data parallel over the remaining ranks, ZeRO-1).
Run: ``torchrun --nproc-per-node 8 -m playground.pretrain.qwen3.qwen3_8b [key=value ...]``.
"""
import torch

from steptronoss_b200.data.synthetic import SyntheticDataConfig
from steptronoss_b200.exp.base_exp import GradientManagerConfig, ParallelConfig, ProfilerConfig
from steptronoss_b200.exp.checkpointing import CheckpointConfig
from steptronoss_b200.exp.lr_schedulers import ConstantSchedulerConfig
from steptronoss_b200.exp.ntp import NTPTrainerConfig, PretrainExp, PretrainMetricConfig
from steptronoss_b200.exp.resources import TorchrunResourceConfig
from steptronoss_b200.models.common.attention import AttentionConfig
from steptronoss_b200.models.common.feed_forward import FeedForwardConfig
from steptronoss_b200.models.common.parallel_embedding import InputEmbeddingConfig, OutputEmbeddingConfig
from steptronoss_b200.models.decoder_model import DecoderLLMConfig


class Qwen3AttentionConfig(AttentionConfig):
    def __init__(self):
        super().__init__()
        self.causal = True
        self.num_attention_heads = 32
        self.num_attention_groups = 8
        self.head_dim = 128
        self.hidden_size = 4096
        self.use_qk_norm = False  # reference convention: False enables the per-head q/k RMSNorm
        self.layernorm_epsilon = 1e-6
        self.rope_theta = 1_000_000.0
        self.max_position_embeddings = 40960


class Qwen3FeedForwardConfig(FeedForwardConfig):
    def __init__(self):
        super().__init__()
        self.hidden_size = 4096
        self.ffn_hidden_size = 12288
        self.layernorm_epsilon = 1e-6
        self.swiglu_recompute_silu_out_proj = True


class Qwen3InputEmbeddingConfig(InputEmbeddingConfig):
    def __init__(self):
        super().__init__()
        self.vocab_size = 151936
        self.hidden_size = 4096


class Qwen3OutputEmbeddingConfig(OutputEmbeddingConfig):
    def __init__(self):
        super().__init__()
        self.vocab_size = 151936
        self.hidden_size = 4096
        self.layernorm_epsilon = 1e-6


class Qwen3ParallelConfig(ParallelConfig):
    def __init__(self):
        super().__init__()
        self.tensor_model_parallel_size = 4
        self.expert_tensor_parallel_size = 1


class Qwen3_8BConfig(DecoderLLMConfig):
    ffn_cfg = Qwen3FeedForwardConfig
    attn_cfg = Qwen3AttentionConfig
    tok_embed_cfg = Qwen3InputEmbeddingConfig
    out_embed_cfg = Qwen3OutputEmbeddingConfig
    parallel_cfg = Qwen3ParallelConfig

    def __init__(self):
        super().__init__()
        self.num_layers = 36
        self.hidden_size = 4096
        self.layernorm_epsilon = 1e-6
        self.recompute = False
        self.tie_embedding = False
        self.params_dtype = torch.bfloat16
        self.variable_seq_lengths = True
        self.tp_cfg.sequence_parallel = True

    def build_model(self, vpp_rank=None):
        from steptronoss_b200.models.qwen_dense import QwenModel

        return QwenModel(cfg=self, layer_map=self.build_layer_map(), vpp_rank=vpp_rank)


class OneNodeResourceConfig(TorchrunResourceConfig):
    def __init__(self):
        super().__init__()
        self.replica = 1
        self.gpu = 8


class Exp(PretrainExp):
    log_dir = "./tensorboard_logs/"
    resource_cfg = OneNodeResourceConfig
    trainer_cfg = NTPTrainerConfig
    model_cfg = Qwen3_8BConfig
    optimizer_cfg = GradientManagerConfig
    scheduler_cfg = ConstantSchedulerConfig
    data_cfg = SyntheticDataConfig
    checkpoint_cfg = CheckpointConfig
    metric_cfg = PretrainMetricConfig
    profiler_cfg = ProfilerConfig

    def __init__(self):
        super().__init__()
        t = self.trainer_cfg
        t.global_batch_size = 64
        t.global_seq_length = 8192
        t.micro_batch_size = 1
        t.train_iters = 100
        s = self.scheduler_cfg
        s.lr = 1e-5
        s.weight_decay = 0.1
        s.warmup_schedule = 0
        self.checkpoint_cfg.save_interval = None


if __name__ == "__main__":
    Exp().train()
