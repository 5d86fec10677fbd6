"""Thin collective helpers that behave the same on NCCL and gloo (gloo lacks reduce-scatter)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def _is_gloo(group) -> bool:
    try:
        return dist.get_backend(group) == "gloo"
    except Exception:
        return False


def reduce_scatter_tensor(out: torch.Tensor, inp: torch.Tensor, group=None) -> None:
    """``out = sum over ranks of this rank's slice of inp``; ``out`` may alias that slice."""
    if _is_gloo(group):
        n = dist.get_world_size(group)
        r = dist.get_rank(group)
        tmp = inp.clone()
        dist.all_reduce(tmp, group=group)
        per = tmp.shape[0] // n
        out.copy_(tmp[r * per : (r + 1) * per].view_as(out))
        return
    dist.reduce_scatter_tensor(out, inp, group=group)


def all_gather_into_tensor(out: torch.Tensor, inp: torch.Tensor, group=None) -> None:
    if _is_gloo(group) and inp.untyped_storage().data_ptr() == out.untyped_storage().data_ptr():
        inp = inp.clone()
    dist.all_gather_into_tensor(out, inp, group=group)
