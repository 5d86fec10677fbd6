"""Input word embedding and output head (reference ``steptronoss/model/common/parallel_embedding.py``).

``WordEmbedding``: vocab-parallel table, output scattered to the sequence-parallel region.
``OutputEmbedding``: final RMSNorm + vocab-parallel LM head.  Besides ``forward`` (logits, as in the
reference) it offers ``loss``: the fused projection + cross-entropy that never builds fp32 logits.
``OneDimensionalOutputEmbedding`` is the scalar value head used by the PPO critic.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ...config import Config, Ref
from ...ops import fused_linear_cross_entropy, linear
from ...parallel import mappings
from ...parallel.layers import ColumnParallelLinear, VocabParallelEmbedding
from ...parallel.state import PM
from .rms_norm import RMSNorm


class InputEmbeddingConfig(Config):
    tp_cfg = Ref("..tp_cfg")
    params_dtype = Ref("..params_dtype", torch.bfloat16)
    vocab_size: int
    hidden_size: int
    embedding_weights_in_fp32: bool = False
    fp32_residual_connection: bool = False

    def build_model(self):
        return WordEmbedding(self)


class OutputEmbeddingConfig(Config):
    tp_cfg = Ref("..tp_cfg")
    params_dtype = Ref("..params_dtype", torch.bfloat16)
    vocab_size: int
    hidden_size: int
    fp32_rms_norm: bool = True
    rms_norm_zero_gamma: bool = False
    layernorm_epsilon: float = 1e-6
    gather_output: bool = False
    fp32_lm_head_out: bool = False
    ce_chunk_tokens: int = 2048

    def build_model(self, tied_embedding_weight=None):
        return OutputEmbedding(self, tied_embedding_weight)


class WordEmbedding(nn.Module):
    def __init__(self, cfg: InputEmbeddingConfig):
        super().__init__()
        self.cfg = cfg
        dtype = torch.float32 if cfg.embedding_weights_in_fp32 else cfg.params_dtype
        self.word_embeddings = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, params_dtype=dtype,
                                                      sequence_parallel=bool(cfg.tp_cfg.sequence_parallel))

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        """``input_ids [tokens]`` -> ``[tokens(/TP), H]``."""
        h = self.word_embeddings(input_ids.reshape(-1))
        if h.dtype != self.cfg.params_dtype and not self.cfg.fp32_residual_connection:
            h = h.to(self.cfg.params_dtype)
        return h


class OutputEmbedding(nn.Module):
    def __init__(self, cfg: OutputEmbeddingConfig, tied_embedding_weight=None):
        super().__init__()
        self.cfg = cfg
        sp = bool(cfg.tp_cfg.sequence_parallel)
        self.sequence_parallel = sp and PM.size_of("TP") > 1
        self.norm = RMSNorm(cfg.hidden_size, cfg.layernorm_epsilon, sequence_parallel=sp,
                            use_zero_init=cfg.rms_norm_zero_gamma, params_dtype=cfg.params_dtype)
        self.output = ColumnParallelLinear(cfg.hidden_size, cfg.vocab_size, params_dtype=cfg.params_dtype,
                                           gather_output=cfg.gather_output, sequence_parallel=sp,
                                           out_dtype=torch.float32 if cfg.fp32_lm_head_out else None)
        if tied_embedding_weight is not None:
            self.output.weight = tied_embedding_weight
        per = cfg.vocab_size // PM.size_of("TP")
        self.vocab_start = PM.rank_in("TP") * per

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.output(self.norm(x))

    def loss(self, x, labels, weights):
        """Weighted CE sum over this rank's (CP-local) tokens, per-token loss and predictions."""
        h = self.norm(x)
        if self.sequence_parallel:
            h = mappings.gather_from_sequence_parallel_region(h, "TP")
        else:
            h = mappings.copy_to_tensor_model_parallel_region(h, "TP")
        group = PM.group_of("TP") if PM.size_of("TP") > 1 else None
        return fused_linear_cross_entropy(h, self.output.weight, labels.reshape(-1), weights.reshape(-1),
                                          self.vocab_start, group, self.cfg.ce_chunk_tokens)


class OneDimensionalOutputEmbedding(nn.Module):
    """RMSNorm + replicated ``[1, H]`` projection producing one scalar per token (critic value head)."""

    def __init__(self, cfg: OutputEmbeddingConfig):
        super().__init__()
        self.cfg = cfg
        sp = bool(cfg.tp_cfg.sequence_parallel)
        self.sequence_parallel = sp and PM.size_of("TP") > 1
        self.norm = RMSNorm(cfg.hidden_size, cfg.layernorm_epsilon, sequence_parallel=sp,
                            use_zero_init=cfg.rms_norm_zero_gamma, params_dtype=cfg.params_dtype)
        self.output = nn.Module()
        self.output.weight = nn.Parameter(torch.empty(8, cfg.hidden_size, dtype=cfg.params_dtype))
        self.output.weight.sequence_parallel = sp

    def forward(self, x):
        h = self.norm(x)
        v = linear(h, self.output.weight)[..., :1].float()
        if self.sequence_parallel:
            v = mappings.gather_from_sequence_parallel_region_no_reduce(v, "TP")
        return v
