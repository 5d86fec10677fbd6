"""Object-level collectives (reference ``steptronoss/utils/dist_utils.py:49-850``): broadcast or
exchange nested containers of tensors, pack dicts into byte tensors, gather dicts, balanced maps.

Tensors travel as tensors (one collective each, on the group's device); the container skeleton
travels pickled.
"""
from __future__ import annotations

import io
from typing import Any, Callable

import torch
import torch.distributed as dist


class _TensorSlot:
    __slots__ = ("index", "shape", "dtype")

    def __init__(self, index, shape, dtype):
        self.index, self.shape, self.dtype = index, tuple(shape), dtype


def _strip(obj, tensors: list):
    from ..config import DataClass

    if torch.is_tensor(obj):
        tensors.append(obj)
        return _TensorSlot(len(tensors) - 1, obj.shape, obj.dtype)
    if isinstance(obj, dict):
        return {k: _strip(v, tensors) for k, v in obj.items()}
    if isinstance(obj, DataClass):
        new = obj.__class__.__new__(obj.__class__)
        for k, v in obj.items():
            object.__setattr__(new, k, _strip(v, tensors))
        return new
    if isinstance(obj, (list, tuple)):
        return type(obj)(_strip(v, tensors) for v in obj)
    return obj


def _fill(obj, tensors: list):
    from ..config import DataClass

    if isinstance(obj, _TensorSlot):
        return tensors[obj.index]
    if isinstance(obj, dict):
        return {k: _fill(v, tensors) for k, v in obj.items()}
    if isinstance(obj, DataClass):
        for k, v in list(obj.items()):
            object.__setattr__(obj, k, _fill(v, tensors))
        return obj
    if isinstance(obj, (list, tuple)):
        return type(obj)(_fill(v, tensors) for v in obj)
    return obj


def _comm_device(group, device):
    if device is not None:
        return torch.device(device)
    try:
        return torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
    except Exception:
        return torch.device("cpu")


def broadcast_tensors(obj: Any, src: int | None = None, group=None, device=None, src_rank: int | None = None):
    """Broadcast a nested container from global rank ``src`` (``src_rank`` is the reference's name for the same
    argument) to the group; tensors arrive on ``device``."""
    if src is None:
        src = src_rank
    if src is None:
        raise TypeError("broadcast_tensors needs the source rank (src= or src_rank=)")
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return obj
    dev = _comm_device(group, device)
    comm_dev = _comm_device(group, None)
    me = dist.get_rank()
    tensors: list = []
    skeleton = [_strip(obj, tensors)] if me == src else [None]
    dist.broadcast_object_list(skeleton, src=src, group=group)
    skeleton = skeleton[0]
    if me != src:
        slots: list = []
        _collect_slots(skeleton, slots)
        tensors = [None] * len(slots)
        for s in slots:
            tensors[s.index] = torch.empty(s.shape, dtype=s.dtype, device=comm_dev)
    out = []
    for t in tensors:
        buf = t.to(comm_dev).contiguous() if me == src else t
        dist.broadcast(buf, src=src, group=group)
        out.append(buf.to(dev))
    return _fill(skeleton, out)


def _collect_slots(obj, out: list):
    from ..config import DataClass

    if isinstance(obj, _TensorSlot):
        out.append(obj)
    elif isinstance(obj, dict):
        for v in obj.values():
            _collect_slots(v, out)
    elif isinstance(obj, DataClass):
        for v in obj.values():
            _collect_slots(v, out)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            _collect_slots(v, out)


def dict_to_tensor(d: Any, device=None) -> torch.Tensor:
    """Pickle any object (tensors included) into a uint8 tensor."""
    buf = io.BytesIO()
    torch.save(d, buf)
    return torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8).to(device or "cpu")


def tensor_to_dict(t: torch.Tensor) -> Any:
    return torch.load(io.BytesIO(t.cpu().numpy().tobytes()), weights_only=False)


def all_gather_object(obj: Any, group=None) -> list:
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [obj]
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, obj, group=group)
    return out


def all_gather_dict(d: Any, group=None) -> list:
    """Every rank receives every rank's object (tensors moved to CPU on the way)."""
    from .general import recur_to

    return all_gather_object(recur_to(d, "cpu"), group=group)


def gather_dict(d: Any, dst: int = 0, group=None):
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [d]
    from .general import recur_to

    out = [None] * dist.get_world_size(group) if dist.get_rank() == dst else None
    dist.gather_object(recur_to(d, "cpu"), out, dst=dst, group=group)
    return out


def all_to_all_objects(send: list, group=None) -> list:
    """``send[i]`` goes to group rank ``i``; returns what every rank sent to this one."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return list(send)
    n = dist.get_world_size(group)
    if len(send) != n:
        raise ValueError(f"need {n} objects, got {len(send)}")
    gathered = all_gather_object(send, group=group)
    me = dist.get_rank(group)
    return [gathered[src][me] for src in range(n)]


def all_to_all_dicts(send: list, group=None) -> list:
    return all_to_all_objects(send, group=group)


def send_tensors(obj: Any, dst: int, group=None) -> None:
    tensors: list = []
    skeleton = _strip(obj, tensors)
    dist.send_object_list([skeleton], dst=dst, group=group)
    dev = _comm_device(group, None)
    for t in tensors:
        dist.send(t.to(dev).contiguous(), dst=dst, group=group)


def recv_tensors(src: int, group=None, device=None):
    box = [None]
    dist.recv_object_list(box, src=src, group=group)
    slots: list = []
    _collect_slots(box[0], slots)
    dev = _comm_device(group, None)
    tensors = [None] * len(slots)
    for s in sorted(slots, key=lambda s: s.index):
        t = torch.empty(s.shape, dtype=s.dtype, device=dev)
        dist.recv(t, src=src, group=group)
        tensors[s.index] = t.to(device) if device is not None else t
    return _fill(box[0], tensors)


def redistributed_tp(chunks: list, dim: int, new_tp: int) -> list:
    """Re-split a tensor given as TP shards along ``dim`` into ``new_tp`` shards."""
    full = torch.cat(chunks, dim=dim)
    return list(full.chunk(new_tp, dim=dim))


def list_balance(items: list, sizes: list, parts: int) -> list:
    from .general import balanced_list_split

    return balanced_list_split(items, sizes, parts)


def balanced_map(fn: Callable, items: list, sizes: list | None = None, group=None) -> list:
    """Apply ``fn`` to ``items`` with the work split over the group's ranks (size-balanced); every
    rank receives all results in the original order."""
    n = dist.get_world_size(group) if dist.is_initialized() else 1
    if n == 1:
        return [fn(x) for x in items]
    me = dist.get_rank(group)
    sizes = sizes or [1] * len(items)
    parts = list_balance(list(range(len(items))), sizes, n)
    mine = {i: fn(items[i]) for i in parts[me]}
    merged: dict = {}
    for d in all_gather_object(mine, group=group):
        merged.update(d)
    return [merged[i] for i in range(len(items))]
