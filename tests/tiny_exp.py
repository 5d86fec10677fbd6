"""Tiny Qwen3-style experiment used across the tests and by the smoke entry point."""
from __future__ import annotations

import torch

from steptronoss_b200.data.synthetic import SyntheticDataConfig
from steptronoss_b200.exp.base_exp import GradientManagerConfig, ProfilerConfig
from steptronoss_b200.exp.lr_schedulers import ConstantSchedulerConfig
from steptronoss_b200.exp.ntp import NTPTrainerConfig, PretrainExp, PretrainMetricConfig
from steptronoss_b200.models.decoder_model import DecoderLLMConfig


class TinyModel(DecoderLLMConfig):
    chunk_lengths: list | None = None
    """layers per (virtual) pipeline chunk, in chunk order; None: the even split of the base class"""
    noop_chunks: list = []
    """chunks whose layers are placeholders that pass their input through"""

    def pp_vp_allocation(self, abs_pp_rank: int) -> list:
        if self.chunk_lengths is None:
            return super().pp_vp_allocation(abs_pp_rank)
        opts = {"noop": True} if abs_pp_rank in self.noop_chunks else {}
        return [dict(opts) for _ in range(self.chunk_lengths[abs_pp_rank])]


class TinyExp(PretrainExp):
    trainer_cfg = NTPTrainerConfig
    model_cfg = TinyModel
    optimizer_cfg = GradientManagerConfig
    scheduler_cfg = ConstantSchedulerConfig
    data_cfg = SyntheticDataConfig
    metric_cfg = PretrainMetricConfig
    profiler_cfg = ProfilerConfig


def make_tiny_exp(dtype=torch.float32, hidden=256, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1024, layers=2,
                  seq=128, gbs=4, iters=10, lr=1e-3, wd=0.1, tp=1, pp=1, cp=1, vpp=1, sp=False, zero1=True, recompute=False,
                  min_doc=16, max_doc=64, clip=1.0) -> TinyExp:
    e = TinyExp()
    m = e.model_cfg
    m.num_layers, m.hidden_size, m.params_dtype = layers, hidden, dtype
    m.variable_seq_lengths = True
    m.recompute = recompute
    m.tp_cfg.sequence_parallel = sp
    a = m.attn_cfg
    a.num_attention_heads, a.num_attention_groups, a.head_dim, a.hidden_size = heads, kv_heads, head_dim, hidden
    a.rope_theta, a.layernorm_epsilon, a.use_qk_norm = 1e6, 1e-6, False
    f = m.ffn_cfg
    f.hidden_size, f.ffn_hidden_size = hidden, ffn
    m.tok_embed_cfg.vocab_size = m.out_embed_cfg.vocab_size = vocab
    m.tok_embed_cfg.hidden_size = m.out_embed_cfg.hidden_size = hidden
    p = m.parallel_cfg
    p.tensor_model_parallel_size, p.pipeline_model_parallel_size, p.context_parallel_size = tp, pp, cp
    p.expert_tensor_parallel_size = 1
    p.virtual_pipeline_model_parallel_size = vpp
    t = e.trainer_cfg
    t.global_batch_size, t.global_seq_length, t.train_iters, t.writer_backend = gbs, seq, iters, []
    s = e.scheduler_cfg
    s.lr, s.weight_decay, s.warmup_schedule = lr, wd, 0
    e.optimizer_cfg.use_distributed_optimizer = zero1
    e.optimizer_cfg.clip_grad = clip
    e.data_cfg.min_doc_len, e.data_cfg.max_doc_len = min_doc, max_doc
    e.data_cfg.pin_memory = False
    return e
