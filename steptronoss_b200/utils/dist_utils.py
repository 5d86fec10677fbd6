"""Object-level collectives (reference ``steptronoss/utils/dist_utils.py:49-850``): broadcast or
exchange nested containers of tensors, pack dicts into byte tensors, gather dicts, balanced maps.

Tensors travel as tensors (one collective each, on the group's device); the container skeleton
travels pickled.
"""
from __future__ import annotations

import io
import pickle
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


def object_to_tensor(obj, device):
    """Pickle ``obj`` into a uint8 tensor on ``device``; returns ``(bytes, length)`` (the length as a 1-element int64
    tensor, ready to be exchanged before the payload)."""
    raw = pickle.dumps(obj)
    data = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
    return data, torch.tensor([len(raw)], dtype=torch.int64, device=device)


def tensor_to_object(tensor: torch.Tensor, tensor_size):
    """Inverse of ``object_to_tensor``; ``tensor`` may be longer than the pickled bytes (padded for a collective)."""
    return pickle.loads(tensor.cpu().numpy().tobytes()[: int(tensor_size)])


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


# ------------------------------------------------------------------ tensors between all ranks of a group
def all_to_all_tensors(tensors: list, group=None, dtype=None, device=None, async_op: bool = False):
    """``tensors[i]`` goes to group rank ``i``; shapes may differ per pair (they are exchanged first).  Returns the
    received tensors (with ``async_op`` the pair ``(work handle, received tensors)``)."""
    n = dist.get_world_size(group) if dist.is_initialized() else 1
    if len(tensors) != n:
        raise ValueError(f"need {n} tensors, got {len(tensors)}")
    if n == 1:
        return (None, list(tensors)) if async_op else list(tensors)
    me = dist.get_rank(group)
    dev = _comm_device(group, device)
    dtype = dtype or tensors[0].dtype
    shapes = all_gather_object([tuple(t.shape) for t in tensors], group=group)
    recv = [torch.empty(shapes[src][me], dtype=dtype, device=dev) for src in range(n)]
    send = [t.to(device=dev, dtype=dtype).contiguous() for t in tensors]
    if dist.get_backend(group) == "gloo":            # gloo has no list all-to-all: pairwise exchange
        work = [dist.isend(send[d], dist.get_global_rank(group, d) if group is not None else d, group=group)
                for d in range(n) if d != me]
        work += [dist.irecv(recv[s_], dist.get_global_rank(group, s_) if group is not None else s_, group=group)
                 for s_ in range(n) if s_ != me]
        recv[me].copy_(send[me])
        handle = _WorkList(work)
        if async_op:
            return handle, recv
        handle.wait()
        return recv
    handle = dist.all_to_all(recv, send, group=group, async_op=async_op)
    return (handle, recv) if async_op else recv


class _WorkList:
    def __init__(self, work):
        self.work = work

    def wait(self):
        wait_all(self.work)


def wait_all(handles) -> None:
    for h in handles:
        if h is not None:
            h.wait()


def gather_object(objects, group=None, dst: int = 0):
    """Group rank ``dst`` receives every rank's ``objects`` (a list, in rank order); the others receive empty lists."""
    n = dist.get_world_size(group) if dist.is_initialized() else 1
    send = [[] for _ in range(n)]
    send[dst] = objects
    return all_to_all_objects(send, group=group)


def concat_list_in_group(local_list: list, group=None) -> list:
    """The concatenation of every rank's list, in rank order, on every rank.  When only one rank holds data it is
    broadcast as tensors instead of being pickled through an all-gather (lower peak memory)."""
    sizes = all_gather_object(len(local_list), group=group)
    holders = [r for r, n in enumerate(sizes) if n > 0]
    if len(sizes) > 1 and len(holders) == 1:
        src = holders[0]
        src_global = dist.get_global_rank(group, src) if group is not None else src
        return broadcast_tensors(local_list if dist.get_rank(group) == src else None, src=src_global, group=group)
    out: list = []
    for part in all_gather_object(local_list, group=group):
        out += part
    return out


# ------------------------------------------------------------------ objects between two ranks
def _pickle_to_tensor(obj, device) -> torch.Tensor:
    buf = io.BytesIO()
    torch.save(obj, buf)
    return torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8).to(device)


def isend_obj(obj, dst: int, group=None) -> list:
    """Start sending a picklable object to global rank ``dst``; returns the work handles (``wait_all``)."""
    dev = _comm_device(group, None)
    payload = _pickle_to_tensor(obj, dev)
    size = torch.tensor([payload.numel()], dtype=torch.int64, device=dev)
    handles = [dist.isend(size, dst=dst, group=group), dist.isend(payload, dst=dst, group=group)]
    handles.append(_KeepAlive(size, payload))
    return handles


class _KeepAlive:
    """Holds the buffers of an asynchronous send until the caller has waited."""

    def __init__(self, *tensors):
        self.tensors = tensors

    def wait(self):
        self.tensors = ()


def send_obj(obj, dst: int, group=None) -> None:
    wait_all(isend_obj(obj, dst, group))


def recv_obj(src: int, group=None, device=None):
    dev = _comm_device(group, None)
    size = torch.zeros(1, dtype=torch.int64, device=dev)
    dist.recv(size, src=src, group=group)
    payload = torch.empty(int(size.item()), dtype=torch.uint8, device=dev)
    dist.recv(payload, src=src, group=group)
    obj = torch.load(io.BytesIO(payload.cpu().numpy().tobytes()), weights_only=False)
    if device is not None:
        from .general import recur_to

        obj = recur_to(obj, device)
    return obj


# ------------------------------------------------------------------ named tensors as one byte buffer
_PACK_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.int16, torch.int8,
                torch.uint8, torch.bool, torch.float64]


def pack_tensors(tensors: dict, names: list) -> tuple:
    """``(table, payload)``: ``table`` is int64 ``[len(names), 3]`` with ``(rows, cols, dtype id)`` per name
    (``-1`` three times for a missing / ``None`` entry), ``payload`` the tensors' bytes back to back.  Tensors have
    at most two dimensions; plain ints travel as one-element int64 tensors."""
    rows, chunks = [], []
    dev = None
    for name in names:
        t = tensors.get(name)
        if t is None:
            rows.append([-1, -1, -1])
            continue
        if not torch.is_tensor(t):
            if not isinstance(t, int):
                raise TypeError(f"{name}: only tensors and ints can be packed, got {type(t).__name__}")
            t = torch.tensor([t], dtype=torch.int64)
        if t.dim() > 2:
            raise ValueError(f"{name}: at most two dimensions, got {tuple(t.shape)}")
        if t.dtype not in _PACK_DTYPES:
            raise TypeError(f"{name}: dtype {t.dtype} cannot be packed")
        shape = [1, 1] if t.dim() == 0 else ([t.shape[0], 1] if t.dim() == 1 else list(t.shape))
        rows.append(shape + [_PACK_DTYPES.index(t.dtype)])
        dev = dev or t.device
        chunks.append(t.contiguous().reshape(-1).view(torch.uint8) if t.numel() else torch.empty(0, dtype=torch.uint8,
                                                                                                    device=t.device))
    dev = dev or torch.device("cpu")
    table = torch.tensor(rows, dtype=torch.int64, device=dev).reshape(len(names), 3)
    payload = torch.cat([c.to(dev) for c in chunks]) if chunks else torch.empty(0, dtype=torch.uint8, device=dev)
    return table, payload


def unpack_tensors(table: torch.Tensor, payload: torch.Tensor, names: list, keep_2d: tuple = ("input",)) -> dict:
    """Inverse of :func:`pack_tensors`.  A second dimension of 1 is dropped again except for the names in
    ``keep_2d`` (a one-column matrix and a vector are not distinguishable in the table)."""
    out, off = {}, 0
    info = table.cpu().tolist()
    for name, (r, c, d) in zip(names, info):
        if r == -1:
            out[name] = None
            continue
        dtype = _PACK_DTYPES[d]
        shape = [r] if c == 1 and name not in keep_2d else [r, c]
        nbytes = r * c * torch.empty((), dtype=dtype).element_size()
        out[name] = payload[off: off + nbytes].clone().view(dtype).reshape(shape)
        off += nbytes
    return out


def isend_packed_tensors(tensors: dict, dst: int, group=None) -> list:
    """Send named tensors as two messages (table, payload); the receiver names them with the same list."""
    dev = _comm_device(group, None)
    table, payload = pack_tensors(tensors, list(tensors.keys()))
    table, payload = table.to(dev), payload.to(dev)
    return [dist.isend(table, dst=dst, group=group), dist.isend(payload, dst=dst, group=group), _KeepAlive(table, payload)]


def recv_packed_tensors(names: list, src: int, group=None) -> dict:
    dev = _comm_device(group, None)
    table = torch.empty((len(names), 3), dtype=torch.int64, device=dev)
    dist.recv(table, src=src, group=group)
    total = sum(r * c * torch.empty((), dtype=_PACK_DTYPES[d]).element_size() for r, c, d in table.cpu().tolist() if r != -1)
    payload = torch.empty(total, dtype=torch.uint8, device=dev)
    dist.recv(payload, src=src, group=group)
    return unpack_tensors(table, payload, names)


# ------------------------------------------------------------------ balancing work over a group
def split_by_size(items: list, sizes: list, parts: int) -> list:
    from .general import balanced_list_split

    return balanced_list_split(items, sizes, parts)


def _even_ranges(total: int, parts: int) -> list:
    base, extra = divmod(total, parts)
    out, lo = [], 0
    for i in range(parts):
        hi = lo + base + (1 if i < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def list_balance(data: list, group=None) -> tuple:
    """Even out per-rank lists: the concatenation of all ranks' ``data`` (rank order) is re-cut into equal
    consecutive parts, e.g. rank 0 ``[0,1,2,3,4]``, rank 1 ``[5]`` -> ``[0,1,2]`` and ``[3,4,5]``.
    Returns ``(balanced_data, restore_info)``; :func:`list_unbalance` sends results back."""
    n = dist.get_world_size(group) if dist.is_initialized() else 1
    if n == 1:
        return list(data), (None, None, group)
    me = dist.get_rank(group)
    lens = all_gather_object(len(data), group=group)
    starts = [sum(lens[:r]) for r in range(n)]
    owned = [(starts[r], starts[r] + lens[r]) for r in range(n)]
    target = _even_ranges(sum(lens), n)
    my_lo = owned[me][0]
    send = [[data[g - my_lo] for g in range(max(owned[me][0], lo), min(owned[me][1], hi))] for lo, hi in target]
    from .general import recur_to

    got = all_to_all_objects(recur_to(send, "cpu"), group=group)
    return [x for part in got for x in part], (owned, target, group)


def list_unbalance(balanced_data: list, restore_info: tuple) -> list:
    """Inverse of :func:`list_balance`: items (or their results, same order) return to their original ranks."""
    owned, target, group = restore_info
    if owned is None:
        return list(balanced_data)
    n, me = dist.get_world_size(group), dist.get_rank(group)
    my_lo = target[me][0]
    send = [[balanced_data[g - my_lo] for g in range(max(target[me][0], lo), min(target[me][1], hi))] for lo, hi in owned]
    from .general import recur_to

    got = all_to_all_objects(recur_to(send, "cpu"), group=group)
    return [x for part in got for x in part]


def balanced_map(fn: Callable, data: list, group=None) -> list:
    """``[fn(x) for x in data]`` for this rank's ``data``, with the calls spread evenly over the group's ranks."""
    balanced, info = list_balance(data, group=group)
    return list_unbalance([fn(x) for x in balanced], info)


def replicated_map(fn: Callable, items: list, sizes: list | None = None, group=None) -> list:
    """Every rank holds the same ``items``; the calls are split over the ranks (balanced by ``sizes``) and every
    rank receives all results in the original order."""
    n = dist.get_world_size(group) if dist.is_initialized() else 1
    if n == 1:
        return [fn(x) for x in items]
    me = dist.get_rank(group)
    sizes = sizes or [1] * len(items)
    parts = split_by_size(list(range(len(items))), sizes, n)
    mine = {i: fn(items[i]) for i in parts[me]}
    merged: dict = {}
    for d in all_gather_object(mine, group=group):
        merged.update(d)
    return [merged[i] for i in range(len(items))]
