"""Flat parameter / gradient storage.

The reference keeps one contiguous fp32 gradient buffer per bucket key and gives every parameter
an fp32 ``main_grad`` view into it; whole parameters are assigned to data-parallel shards by greedy
size balancing, never split (``steptronoss/model/utils/comm_buffer.py:14-171``) because Muon needs
whole matrices.  This module keeps those rules and goes one step further for 180 GB parts: the
bf16 parameters themselves are re-seated as views of a second flat buffer with the same layout, so
the ZeRO-1 parameter all-gather lands directly in the tensors the GEMMs read (no copy-in/copy-out),
and the sharded Adam kernel streams one contiguous range.

Layout of a bucket of ``dp`` shards: ``[shard 0 | shard 1 | ...]`` each ``shard_size`` elements
(padded to the largest shard); shard ``r`` holds the whole parameters owned by DP rank ``r``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parallel.state import PM

_ALIGN = 64  # elements; keeps every parameter 128-byte aligned in bf16 (TMA needs 16 B)


@dataclass(frozen=True)
class BucketKey:
    dtype: torch.dtype
    reduce_group: str  # "DP" or "EDP"
    is_muon: bool
    tp_replicated: bool  # parameter identical on all TP ranks (norms, router ...)

    def __str__(self) -> str:
        return f"{str(self.dtype).split('.')[-1]}:{self.reduce_group}:MUON:{self.is_muon}:REP:{self.tp_replicated}"


@dataclass
class ParamSlot:
    name: str
    param: torch.nn.Parameter
    owner: int
    offset: int  # element offset in the bucket buffer
    numel: int


@dataclass
class Bucket:
    key: BucketKey
    slots: list = field(default_factory=list)
    shard_size: int = 0
    world: int = 1
    rank: int = 0
    param_buf: torch.Tensor | None = None  # params_dtype [world*shard_size]
    grad_buf: torch.Tensor | None = None   # fp32 [world*shard_size]

    @property
    def numel(self) -> int:
        return self.world * self.shard_size

    def own_range(self) -> tuple[int, int]:
        return self.rank * self.shard_size, (self.rank + 1) * self.shard_size

    def own_slots(self):
        return [s for s in self.slots if s.owner == self.rank]


def _round_up(n: int, a: int = _ALIGN) -> int:
    return (n + a - 1) // a * a


def balanced_assignment(sizes: list[int], parts: int) -> list[int]:
    """Greedy: biggest first onto the currently lightest part. Deterministic for equal inputs."""
    load = [0] * parts
    owner = [0] * len(sizes)
    for i in sorted(range(len(sizes)), key=lambda j: (-sizes[j], j)):
        r = min(range(parts), key=lambda q: (load[q], q))
        owner[i] = r
        load[r] += _round_up(sizes[i])
    return owner


def bucket_key_of(param, shard_over_dp: bool = True) -> BucketKey:
    expert = bool(getattr(param, "expert_model_parallel", False))
    rep = not bool(getattr(param, "tensor_model_parallel", False)) and not expert
    return BucketKey(param.dtype, "EDP" if expert else "DP", bool(getattr(param, "is_muon_param", False)), rep)


def build_buffers(named_params: list, shard: bool = True, allocator=None) -> dict:
    """Create the buckets, re-seat every parameter into its bucket's ``param_buf`` and attach
    ``param.main_grad``.  ``shard=False`` gives one shard per bucket (no ZeRO).  ``allocator(key, numel, dtype,
    kind)`` may supply the zeroed flat buffers (``kind`` is ``"param"`` or ``"grad"``) or return ``None`` to leave a
    bucket to ``torch.zeros``; it is called for every bucket in the same order on every rank."""
    groups: dict[BucketKey, list] = {}
    for name, p in named_params:
        if not p.requires_grad:
            continue
        groups.setdefault(bucket_key_of(p), []).append((name, p))
    buckets: dict[BucketKey, Bucket] = {}
    for key, items in groups.items():
        world = PM.size_of(key.reduce_group) if shard else 1
        rank = PM.rank_in(key.reduce_group) if shard else 0
        sizes = [p.numel() for _, p in items]
        owners = balanced_assignment(sizes, world)
        per_rank = [0] * world
        slots = []
        for (name, p), o in zip(items, owners):
            slots.append(ParamSlot(name, p, o, per_rank[o], p.numel()))
            per_rank[o] += _round_up(p.numel())
        shard_size = max(_round_up(max(per_rank)), _ALIGN)
        for s in slots:
            s.offset += s.owner * shard_size
        dev = items[0][1].device
        b = Bucket(key, slots, shard_size, world, rank)
        n = world * shard_size
        b.param_buf = allocator(key, n, key.dtype, "param") if allocator is not None else None
        b.grad_buf = allocator(key, n, torch.float32, "grad") if allocator is not None else None
        if b.param_buf is None:
            b.param_buf = torch.zeros(n, dtype=key.dtype, device=dev)
        if b.grad_buf is None:
            b.grad_buf = torch.zeros(n, dtype=torch.float32, device=dev)
        for s in slots:
            view = b.param_buf[s.offset : s.offset + s.numel].view(s.param.shape)
            view.copy_(s.param.data)
            s.param.data = view
            s.param.main_grad = b.grad_buf[s.offset : s.offset + s.numel].view(s.param.shape)
            s.param.grad_added_to_main_grad = False
        buckets[key] = b
    return buckets


# the reference's names for the same things (model/utils/comm_buffer.py)
ParamBucketKey = BucketKey
get_bucket_key_from_param_attrs = bucket_key_of
