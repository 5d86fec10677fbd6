"""Helpers around checkpoint files: sizes, host copies, per-rank file names, the split of a state dict into expert and
non-expert parts, and a broadcast of byte strings too large for one message.  Same names and behaviour as the
reference's ``checkpointing/utils.py`` (its S3 listing aside: paths are local here)."""
from __future__ import annotations

import copy
import os
from collections.abc import Mapping
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from ..parallel.state import PM
from ..utils.dist_utils import broadcast_tensors
from .local_checkpoint import analyze_dir


def recur_stat(obj: Any) -> int:
    """Bytes held by the tensors and arrays inside nested dicts / lists (other leaves count nothing)."""
    if torch.is_tensor(obj):
        return obj.numel() * obj.element_size()
    if isinstance(obj, np.ndarray):
        return int(obj.nbytes)
    if isinstance(obj, Mapping):
        return sum(recur_stat(v) for v in obj.values())
    if isinstance(obj, (list, tuple)):
        return sum(recur_stat(v) for v in obj)
    return 0


def size_report(file_objects: Mapping[str, Any]) -> str:
    """``name: 1.2 G | other: NOTENSOR`` for the files of one checkpoint."""
    parts = []
    for name, obj in file_objects.items():
        gb = recur_stat(obj) / 1024 ** 3
        parts.append(f"{name}: {gb:.1f} G" if gb else f"{name}: NOTENSOR")
    return " | ".join(parts)


def move_tensor_to_memory(tensor: torch.Tensor) -> torch.Tensor:
    """A host copy that shares nothing with ``tensor`` (a CPU tensor is cloned)."""
    return tensor.detach().to("cpu", copy=True)


def move_to_memory(state: Any) -> Any:
    """Host copy of a nested state: tensors are copied to the CPU, containers rebuilt, other leaves deep-copied, so
    that a background writer can run while training overwrites the originals."""
    if torch.is_tensor(state):
        return move_tensor_to_memory(state)
    if type(state) in (dict, list):
        items = state.items() if isinstance(state, dict) else enumerate(state)
        out = type(state)() if isinstance(state, dict) else [None] * len(state)
        for k, v in items:
            out[k] = move_to_memory(v)
        return out
    return copy.deepcopy(state)


def get_rank_specific_name() -> str:
    return f"TP{PM.rank_in('TP'):02d}_PP{PM.rank_in('PP'):03d}_DP{PM.rank_in('DP'):03d}"


def find_rank_specific_path(path: str, use_dp0: bool = False) -> str:
    """The file of this rank inside the checkpoint directory ``path`` (``use_dp0``: the first data-parallel replica's,
    for state that every replica shares).  The directory must have been written with this TP and PP layout."""
    found = analyze_dir(path)
    if found["files"] and (found["tp"] != PM.size_of("TP") or found["pp"] != PM.size_of("PP")):
        raise AssertionError(f"checkpoint split mismatch: files are TP{found['tp']} x PP{found['pp']}, "
                             f"this job runs TP{PM.size_of('TP')} x PP{PM.size_of('PP')}")
    dp = 0 if use_dp0 else PM.rank_in("DP")
    return os.path.join(path, f"TP{PM.rank_in('TP'):02d}_PP{PM.rank_in('PP'):03d}_DP{dp:03d}.pt")


def split_state_dict(model_state_dict: Mapping[str, Any]) -> tuple[dict, dict]:
    """``(expert part, non-expert part)`` of a checkpoint's state.  Entries whose key starts with ``model`` are model
    chunks (name -> tensor): their parameters go to one side or the other by ``.experts.`` in the name; every other
    entry (iteration, RNG, ...) is kept on both sides."""
    shared = {k: v for k, v in model_state_dict.items() if not k.startswith("model")}
    experts, rest = dict(shared), dict(shared)
    for key, chunk in model_state_dict.items():
        if key.startswith("model"):
            experts[key] = {n: t for n, t in chunk.items() if ".experts." in n}
            rest[key] = {n: t for n, t in chunk.items() if ".experts." not in n}
    return experts, rest


def chunked_broadcast_bytes(data: bytes | None, src: int, group=None, chunk_size: int = 5 * 10 ** 9) -> bytes:
    """Broadcast ``data`` (given on global rank ``src``) to the group in pieces of ``chunk_size`` bytes."""
    me = dist.get_rank() if dist.is_initialized() else 0
    count = -(-len(data) // chunk_size) if me == src else None
    count = int(broadcast_tensors(count, src_rank=src, group=group))
    pieces = []
    for i in range(count):
        piece = data[i * chunk_size:(i + 1) * chunk_size] if me == src else None
        pieces.append(broadcast_tensors(piece, src_rank=src, group=group))
    return b"".join(pieces)
