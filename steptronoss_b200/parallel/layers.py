"""Tensor-parallel linears (with sequence parallelism) and the vocab-parallel embedding.

Counterpart of ``steptronoss/core/tensor_parallel/layers.py:78-970``.  Activations are token-major
2-D tensors ``[tokens, hidden]`` (the packed micro-batch of the reference, ``[S, B=1, H]``, with
the unit batch dimension dropped); under sequence parallelism a rank holds ``tokens / TP`` rows
between blocks.

* ``ColumnParallelLinear``: weight ``[out/TP, in]``; forward = (all-gather rows when SP) -> GEMM.
* ``RowParallelLinear``: weight ``[out, in/TP]``; forward = GEMM -> reduce-scatter rows (SP) or
  all-reduce.
* Weight gradients are accumulated by the wgrad GEMM epilogue straight into ``weight.main_grad``
  (fp32) when the gradient manager has attached one.

The reference leaves parameters uninitialised (``torch.empty``); here every parameter carries the
description of its full (unsharded) shape so that ``init_parallel_weight_`` can draw the same
N(0, std) matrix on every layout and keep this rank's slice: the initial model is independent of
the TP/EP degree.
"""
from __future__ import annotations

import zlib

import torch
import torch.nn as nn

from ..ops import embedding, linear
from . import mappings
from .state import PM

_TP_ATTR_DEFAULTS = {
    "tensor_model_parallel": False,
    "partition_dim": -1,
    "partition_stride": 1,
    "expert_model_parallel": False,
    "is_muon_param": False,
    "sequence_parallel": False,
    "micro_dp": False,
    "shared": False,
}


def set_tensor_model_parallel_attributes(param, is_parallel: bool, dim: int, stride: int = 1, blocks=None,
                                         group: str = "TP") -> None:
    param.tensor_model_parallel = is_parallel
    param.partition_dim = dim
    param.partition_stride = stride
    param.partition_blocks = blocks  # full sizes of the stacked sub-matrices along `dim`
    param.partition_group = group


def set_defaults_if_not_set_tensor_model_parallel_attributes(param) -> None:
    for k, v in _TP_ATTR_DEFAULTS.items():
        if not hasattr(param, k):
            setattr(param, k, v)
    if not hasattr(param, "partition_blocks"):
        param.partition_blocks = None
    if not hasattr(param, "partition_group"):
        param.partition_group = "TP"


def copy_tensor_model_parallel_attributes(dst, src) -> None:
    for k in list(_TP_ATTR_DEFAULTS) + ["partition_blocks", "partition_group", "manual_grad_bucket_prefix", "merge_op",
                                        "_log_name", "_lr_scale", "init_std", "init_kind"]:
        if hasattr(src, k):
            setattr(dst, k, getattr(src, k))


def shard_of_full(full: torch.Tensor, dim: int, blocks, rank: int, world: int) -> torch.Tensor:
    """This rank's slice of a full matrix made of stacked ``blocks`` along ``dim``."""
    if world == 1:
        return full
    if not blocks:
        return full.chunk(world, dim=dim)[rank]
    parts = full.split(list(blocks), dim=dim)
    return torch.cat([p.chunk(world, dim=dim)[rank] for p in parts], dim=dim)


def _name_seed(seed: int, name: str) -> int:
    return (int(seed) * 1000003 + zlib.crc32(name.encode())) % (2**63 - 1)


@torch.no_grad()
def init_parallel_weight_(param: torch.Tensor, name: str, seed: int, std: float = 0.02) -> None:
    """Fill ``param`` with this rank's slice of a N(0, std) matrix determined by ``(seed, name)``."""
    kind = getattr(param, "init_kind", "normal")
    if kind == "ones":
        param.fill_(1.0)
        return
    if kind == "zeros":
        param.zero_()
        return
    std = getattr(param, "init_std", None) or std
    gen = torch.Generator(device=param.device)
    gen.manual_seed(_name_seed(seed, name))
    if getattr(param, "tensor_model_parallel", False):
        group = getattr(param, "partition_group", "TP")
        world, rank = PM.size_of(group), PM.rank_in(group)
        dim = param.partition_dim
        full_shape = list(param.shape)
        full_shape[dim] *= world
        if param.dim() == 3 and getattr(param, "expert_model_parallel", False):
            ep, er = PM.size_of("EP"), PM.rank_in("EP")
            full_shape[0] *= ep
        else:
            ep, er = 1, 0
        # rows are drawn in blocks so that the transient fp32 matrix stays bounded
        full = torch.empty(full_shape, dtype=torch.float32, device=param.device).normal_(0.0, std, generator=gen)
        if ep > 1:
            full = full.chunk(ep, dim=0)[er]
        param.copy_(shard_of_full(full, dim, getattr(param, "partition_blocks", None), rank, world))
    elif getattr(param, "expert_model_parallel", False) and param.dim() == 3:
        ep, er = PM.size_of("EP"), PM.rank_in("EP")
        full_shape = list(param.shape)
        full_shape[0] *= ep
        full = torch.empty(full_shape, dtype=torch.float32, device=param.device).normal_(0.0, std, generator=gen)
        param.copy_(full.chunk(ep, dim=0)[er])
    else:
        param.copy_(torch.empty(param.shape, dtype=torch.float32, device=param.device).normal_(0.0, std, generator=gen))


class ColumnParallelLinear(nn.Module):
    def __init__(self, input_size: int, output_size: int, *, params_dtype=torch.bfloat16, gather_output: bool = False,
                 sequence_parallel: bool = False, group: str = "TP", blocks=None, out_dtype=None, device=None,
                 bias: bool = False):
        super().__init__()
        self.group = group
        world = PM.size_of(group)
        if output_size % world:
            raise ValueError(f"output size {output_size} not divisible by {group}={world}")
        if blocks is not None and any(b % world for b in blocks):
            raise ValueError(f"stacked blocks {blocks} not divisible by {group}={world}")
        self.input_size, self.output_size = input_size, output_size
        self.output_size_per_partition = output_size // world
        self.gather_output = gather_output
        self.sequence_parallel = sequence_parallel and world > 1
        self.out_dtype = out_dtype
        self.weight = nn.Parameter(torch.empty(self.output_size_per_partition, input_size, dtype=params_dtype, device=device))
        set_tensor_model_parallel_attributes(self.weight, world > 1, 0, 1, blocks, group)
        self.bias = None
        if bias:                                   # split like the rows of the weight; starts at zero
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition, dtype=params_dtype, device=device))
            set_tensor_model_parallel_attributes(self.bias, world > 1, 0, 1, blocks, group)
            self.bias.init_kind = "zeros"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel:
            from .fused_tp import all_gather_linear

            y = all_gather_linear(x, self.weight, self.group, self.out_dtype)
        else:
            x = mappings.copy_to_tensor_model_parallel_region(x, self.group)
            y = linear(x, self.weight, self.out_dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        if self.gather_output:
            y = mappings.gather_from_tensor_model_parallel_region(y, self.group)
        return y


class RowParallelLinear(nn.Module):
    def __init__(self, input_size: int, output_size: int, *, params_dtype=torch.bfloat16, input_is_parallel: bool = True,
                 sequence_parallel: bool = False, group: str = "TP", device=None):
        super().__init__()
        self.group = group
        world = PM.size_of(group)
        if input_size % world:
            raise ValueError(f"input size {input_size} not divisible by {group}={world}")
        self.input_size, self.output_size = input_size, output_size
        self.input_size_per_partition = input_size // world
        self.input_is_parallel = input_is_parallel
        self.sequence_parallel = sequence_parallel and world > 1
        self.weight = nn.Parameter(torch.empty(output_size, self.input_size_per_partition, dtype=params_dtype, device=device))
        set_tensor_model_parallel_attributes(self.weight, world > 1, 1, 1, None, group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.input_is_parallel:
            x = mappings.scatter_to_tensor_model_parallel_region(x, self.group)
        if self.sequence_parallel:
            from .fused_tp import linear_reduce_scatter

            return linear_reduce_scatter(x, self.weight, self.group)
        y = linear(x, self.weight)
        return mappings.reduce_from_tensor_model_parallel_region(y, self.group)


class VocabParallelEmbedding(nn.Module):
    """Embedding table sharded over the vocabulary; foreign ids contribute zero rows that the TP
    reduction fills in (``layers.py:78-139``).  With sequence parallelism the reduction is a
    reduce-scatter over tokens."""

    def __init__(self, num_embeddings: int, embedding_dim: int, *, params_dtype=torch.bfloat16,
                 sequence_parallel: bool = False, group: str = "TP", device=None):
        super().__init__()
        self.group = group
        world, rank = PM.size_of(group), PM.rank_in(group)
        if num_embeddings % world:
            raise ValueError(f"vocab {num_embeddings} not divisible by {group}={world}")
        self.num_embeddings = num_embeddings
        per = num_embeddings // world
        self.vocab_start, self.vocab_end = rank * per, (rank + 1) * per
        self.sequence_parallel = sequence_parallel and world > 1
        self.weight = nn.Parameter(torch.empty(per, embedding_dim, dtype=params_dtype, device=device))
        set_tensor_model_parallel_attributes(self.weight, world > 1, 0, 1, None, group)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        out = embedding(ids, self.weight, self.vocab_start, self.vocab_end)
        if self.sequence_parallel:
            return mappings.reduce_scatter_to_sequence_parallel_region(out, self.group)
        return mappings.reduce_from_tensor_model_parallel_region(out, self.group)
