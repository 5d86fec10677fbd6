"""Small tensor and partition helpers of the tensor-parallel layer.

The reference keeps these in ``core/utils.py`` (``divide``, viewless tensors), ``core/tensor_parallel/utils.py``
(splitting along the last dimension, flat 1-D shards and their gather), ``core/tensor_parallel/cross_entropy.py``
(``VocabUtility``) and ``core/tensor_parallel/layers.py`` / ``model/module.py`` (which parameter copies count once in
a norm).  Model code ported from the reference imports them by these names.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .state import PM


def ensure_divisibility(numerator: int, denominator: int) -> None:
    if numerator % denominator:
        raise AssertionError(f"{numerator} is not divisible by {denominator}")


def divide(numerator: int, denominator: int) -> int:
    """``numerator / denominator`` for sizes that must split evenly."""
    ensure_divisibility(numerator, denominator)
    return numerator // denominator


class VocabUtility:
    """Half-open range ``[first, last)`` of the vocabulary rows a rank owns."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition_vocab_size: int, rank: int, world_size: int = 1):
        return rank * per_partition_vocab_size, (rank + 1) * per_partition_vocab_size

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab_size: int, rank: int, world_size: int):
        return VocabUtility.vocab_range_from_per_partition_vocab_size(divide(global_vocab_size, world_size), rank, world_size)


def split_tensor_along_last_dim(tensor: torch.Tensor, num_partitions: int, contiguous_split_chunks: bool = False):
    """``num_partitions`` equal views along the last dimension (copies when ``contiguous_split_chunks``)."""
    parts = tensor.split(divide(tensor.shape[-1], num_partitions), dim=-1)
    return tuple(p.contiguous() for p in parts) if contiguous_split_chunks else parts


def _tp_family(use_expert_tp: bool) -> str:
    return "ETP" if use_expert_tp else "TP"


def split_tensor_into_1d_equal_chunks(tensor: torch.Tensor, new_buffer: bool = False, use_expert_tp: bool = False):
    """This rank's ``1 / TP`` of the flattened tensor: a view, or a copy with ``new_buffer``."""
    fam = _tp_family(use_expert_tp)
    n = tensor.numel() // PM.size_of(fam)
    piece = tensor.reshape(-1)[n * PM.rank_in(fam): n * (PM.rank_in(fam) + 1)]
    return piece.clone() if new_buffer else piece


def gather_split_1d_tensor(tensor: torch.Tensor, use_expert_tp: bool = False) -> torch.Tensor:
    """Inverse of ``split_tensor_into_1d_equal_chunks``: the flat shards of all ranks of the family, in rank order."""
    fam = _tp_family(use_expert_tp)
    world = PM.size_of(fam)
    flat = tensor.reshape(-1).contiguous()
    if world == 1:
        return flat.clone()
    out = torch.empty(flat.numel() * world, dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out, flat, group=PM.group_of(fam))
    return out


# ---- viewless tensors ------------------------------------------------------------------------------------------
# A view keeps its base tensor alive.  Activations that are stored across micro-batches (pipeline buffers, the
# hidden state handed from layer to layer) are therefore re-wrapped in a tensor that shares the storage but has no
# ``_base``, so that dropping ``.data`` later really releases the memory.
def _rewrap(t: torch.Tensor, requires_grad: bool) -> torch.Tensor:
    out = torch.empty((1,), dtype=t.dtype, device=t.device, requires_grad=requires_grad)
    out.data = t.data
    return out


class MakeViewlessTensor(torch.autograd.Function):
    """The re-wrap as a graph node: gradients pass through unchanged."""

    @staticmethod
    def forward(ctx, t, requires_grad):
        return _rewrap(t, requires_grad)

    @staticmethod
    def backward(ctx, g):
        return g, None


def make_viewless_tensor(inp: torch.Tensor, requires_grad: bool, keep_graph: bool) -> torch.Tensor:
    if inp._base is None:
        return inp
    return MakeViewlessTensor.apply(inp, requires_grad) if keep_graph else _rewrap(inp, requires_grad)


def assert_viewless_tensor(tensor, extra_msg: str | None = None):
    if isinstance(tensor, list):
        for t in tensor:
            assert_viewless_tensor(t, extra_msg)
        return tensor
    if isinstance(tensor, torch.Tensor) and tensor._base is not None:
        raise AssertionError("a view was about to be stored or to get new .data: its base tensor would stay alive. "
                             f"{extra_msg or ''}")
    return tensor


def safely_set_viewless_tensor_data(tensor: torch.Tensor, new_data_tensor: torch.Tensor) -> None:
    assert_viewless_tensor(tensor, f"base shape {None if tensor._base is None else tuple(tensor._base.shape)}, "
                                   f"new data shape {tuple(new_data_tensor.shape)}")
    tensor.data = new_data_tensor


# ---- which copy of a parameter counts (norms, zero counts) -----------------------------------------------------
def param_is_not_tensor_parallel_duplicate(param) -> bool:
    """Sharded parameters count on every TP rank, replicated ones on TP rank 0 only."""
    return bool(getattr(param, "tensor_model_parallel", False)) or PM.i_am("TP", 0)


def param_is_not_expert_parallel_duplicate(param) -> bool:
    return bool(getattr(param, "expert_model_parallel", False)) or PM.i_am("TP", 0)


def param_is_not_shared(param) -> bool:
    return not getattr(param, "shared", False)
