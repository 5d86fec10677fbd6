"""Autograd-aware collectives between tensor-parallel regions.

Same set as the reference (``steptronoss/core/tensor_parallel/mappings.py:10-375``): identity
forward / all-reduce backward and its dual, scatter / gather on the last or the first (sequence)
dimension, reduce-scatter / all-gather for sequence parallelism.  Every function takes the *name*
of a process-group family (``"TP"``, ``"ETP"``, ``"CP"`` ...) and is an identity when that family
has one member.  These are the NCCL statements; the fused GEMM+collective kernels in
``parallel/fused_tp.py`` replace the pairs that sit next to a projection.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import comm
from .state import PM


def _size(name: str) -> int:
    return PM.size_of(name) if PM.has(name) else 1


def _all_reduce(x, name):
    if _size(name) == 1:
        return x
    x = x.contiguous()
    dist.all_reduce(x, group=PM.group_of(name))
    return x


def _split_last(x, name):
    n = _size(name)
    if n == 1:
        return x
    return x.chunk(n, dim=-1)[PM.rank_in(name)].contiguous()


def _split_first(x, name):
    n = _size(name)
    if n == 1:
        return x
    if x.shape[0] % n:
        raise ValueError(f"first dimension {x.shape[0]} not divisible by {name} size {n}")
    return x.chunk(n, dim=0)[PM.rank_in(name)].contiguous()


def _gather_last(x, name):
    n = _size(name)
    if n == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=PM.group_of(name))
    return torch.cat(parts, dim=-1)


def _gather_first(x, name):
    n = _size(name)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] * n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    comm.all_gather_into_tensor(out, x, group=PM.group_of(name))
    return out


def _reduce_scatter_first(x, name):
    n = _size(name)
    if n == 1:
        return x
    x = x.contiguous()
    if x.shape[0] % n:
        raise ValueError(f"first dimension {x.shape[0]} not divisible by {name} size {n}")
    out = torch.empty((x.shape[0] // n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    comm.reduce_scatter_tensor(out, x, group=PM.group_of(name))
    return out


def _make(fwd, bwd, doc):
    class _Fn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, name):
            ctx.name = name
            return fwd(x, name)

        @staticmethod
        def backward(ctx, g):
            return bwd(g, ctx.name), None

    _Fn.__doc__ = doc

    def apply(x, group: str = "TP"):
        if _size(group) == 1:
            return x
        return _Fn.apply(x, group)

    apply.__doc__ = doc
    return apply


_ident = lambda x, name: x  # noqa: E731

copy_to_tensor_model_parallel_region = _make(_ident, _all_reduce, "identity forward, all-reduce backward")
reduce_from_tensor_model_parallel_region = _make(_all_reduce, _ident, "all-reduce forward, identity backward")
scatter_to_tensor_model_parallel_region = _make(_split_last, _gather_last, "split last dim / gather")
gather_from_tensor_model_parallel_region = _make(_gather_last, _split_last, "gather last dim / split")
scatter_to_sequence_parallel_region = _make(_split_first, _gather_first, "split first dim / gather")
gather_from_sequence_parallel_region = _make(_gather_first, _reduce_scatter_first,
                                             "all-gather first dim forward, reduce-scatter backward")
gather_from_sequence_parallel_region_no_reduce = _make(_gather_first, _split_first,
                                                       "all-gather first dim forward, split backward")
reduce_scatter_to_sequence_parallel_region = _make(_reduce_scatter_first, _gather_first,
                                                   "reduce-scatter first dim forward, all-gather backward")
slice_sequence_parallel_region = _make(_split_first, _gather_first, "take this rank's slice of the first dim")
slice_to_sequence_parallel_region = slice_sequence_parallel_region      # the reference's spelling


def split_along_first_dim_with_padding(input_, contiguous: bool = True, group: str = "TP"):
    """This rank's share of dimension 0 when its length does not divide by the group: every rank takes
    ``ceil(len / world)`` rows and the last one fills up with uninitialised rows.  Returns ``(share, padding rows)``;
    a group of one returns the input as it is (no tuple), as the reference does
    (core/tensor_parallel/mappings.py:127-156)."""
    world, rank = _size(group), PM.rank_in(group) if _size(group) > 1 else 0
    if world == 1:
        return input_
    n = input_.shape[0]
    if n <= (world - 1) ** 2:
        raise AssertionError(f"{n} rows are too few to pad for {world} ranks: an earlier rank would run past the end")
    share = -(-n // world)
    pad = share * world - n
    out = input_[rank * share:(rank + 1) * share]
    if rank == world - 1 and pad:
        out = torch.cat([out, input_.new_empty((pad, *input_.shape[1:]))])
    return (out.contiguous() if contiguous else out), pad
