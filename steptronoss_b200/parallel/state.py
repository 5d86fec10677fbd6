"""Process-group mesh manager (global ``PM``).

Behavioural counterpart of the reference ``ParallelManager``
(``steptronoss/core/parallel_state.py:38-266``): named families of process groups are derived
from rank-layout patterns such as ``"(p d t) -> (p d) t"``, meshes are cached per parallel
configuration and can be switched with ``use_mesh``, and named RNG streams can be registered
that differ across chosen families.

Differences that follow from the B200 design:

* a family's process group is created lazily, the first time it is asked for, and only for
  the row this rank belongs to (the reference eagerly creates every row of all ten families);
* a single-process run never initialises ``torch.distributed``: every family then has size 1
  and ``group_of`` returns ``None``;
* each family can own a symmetric peer-memory arena (see ``parallel/symm.py``) that the fused
  compute+collective kernels use instead of NCCL.
"""
from __future__ import annotations

import atexit
import os
import random
import re
from contextlib import contextmanager
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Any

import numpy as np
import torch
import torch.distributed as dist


# --------------------------------------------------------------------------- patterns
def _parse_side(text: str) -> list[list[str]]:
    """``"(p d) t"`` -> ``[["p", "d"], ["t"]]``."""
    out: list[list[str]] = []
    for grp, single in re.findall(r"\(([^)]*)\)|(\S+)", text.strip()):
        out.append(grp.split() if grp or not single else [single])
    return out


def layout_from_pattern(pattern: str, world_size: int, **sizes: int) -> list[list[int]]:
    """Rows of world ranks for one family.

    ``pattern`` is ``"<1-d source> -> <outer> <inner>"``; axes named in ``sizes`` take those
    extents, exactly one source axis may be left free and absorbs the rest of the world.  Each
    returned row is one process group (the ``inner`` axes vary inside a row).  Ranks beyond the
    largest multiple of the fixed extents form one trailing leftover row, as in the reference
    (``parallel_state.py:89-120``).
    """
    src_txt, dst_txt = (s.strip() for s in pattern.split("->"))
    src = _parse_side(src_txt)
    dst = _parse_side(dst_txt)
    if len(src) != 1:
        raise ValueError(f"source of {pattern!r} must be one parenthesised group")
    if len(dst) != 2:
        raise ValueError(f"destination of {pattern!r} must have two groups")
    axes = src[0]
    fixed = 1
    free = [a for a in axes if a not in sizes]
    for a in axes:
        if a in sizes:
            fixed *= int(sizes[a])
    if len(free) > 1:
        raise ValueError(f"{pattern!r}: more than one free axis {free}")
    usable = (world_size // fixed) * fixed
    if usable == 0:
        raise ValueError(f"cannot define {pattern!r} with {sizes}: need {fixed} ranks, have {world_size}")
    extent = {a: int(sizes[a]) for a in axes if a in sizes}
    if free:
        extent[free[0]] = usable // fixed
    elif usable != fixed:
        raise ValueError(f"{pattern!r}: all axes fixed ({fixed}) but world is {world_size}")
    shape = [extent[a] for a in axes]
    grid = np.arange(usable).reshape(shape)
    order = [axes.index(a) for a in dst[0] + dst[1]]
    if sorted(order) != list(range(len(axes))):
        raise ValueError(f"{pattern!r}: destination must use every source axis once")
    inner = int(np.prod([extent[a] for a in dst[1]])) if dst[1] else 1
    rows = grid.transpose(order).reshape(-1, inner).tolist()
    if usable != world_size:
        rows.append(list(range(usable, world_size)))
    return rows


@dataclass
class ParallelGroups:
    """One family: all rows, the row of this rank, and the lazily-created process group."""

    name: str
    ranks: list[list[int]]
    my_row: int
    valid_replicas: int
    group: Any = None  # dist.ProcessGroup | None
    created: bool = False
    extra: dict = field(default_factory=dict)


def _get_rng_state():
    cuda = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
    return (random.getstate(), np.random.get_state(), torch.get_rng_state(), cuda)


def _set_rng_state(state) -> None:
    random.setstate(state[0])
    np.random.set_state(state[1])
    torch.set_rng_state(state[2])
    if state[3] is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(state[3])


def _set_rng_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)


class GlobalMemoryBuffer:
    """Named scratch tensors that live for the whole job: ``get_tensor(shape, dtype, name)`` returns a view of one
    flat allocation per ``(name, dtype)``, grown when a larger request arrives.  Two users of the same name must not
    overlap in time.  (Reference ``steptronoss/core/utils.py:23-41``, used there for the sequence-parallel gather;
    the fused all-gather GEMM here keeps its landing area in the symmetric arena of ``parallel/symm.py`` instead.)"""

    def __init__(self) -> None:
        self.buffer: dict[tuple, torch.Tensor] = {}

    def get_tensor(self, tensor_shape, dtype: torch.dtype, name: str, device=None) -> torch.Tensor:
        need = 1
        for d in tensor_shape:
            need *= int(d)
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        cur = self.buffer.get((name, dtype))
        if cur is None or cur.numel() < need or cur.device != torch.device(device):
            cur = torch.empty(need, dtype=dtype, device=device, requires_grad=False)
            self.buffer[(name, dtype)] = cur
        return cur[:need].view(*tensor_shape)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.buffer.values())


_GLOBAL_MEMORY_BUFFER: GlobalMemoryBuffer | None = None


def get_global_memory_buffer() -> GlobalMemoryBuffer:
    global _GLOBAL_MEMORY_BUFFER
    if _GLOBAL_MEMORY_BUFFER is None:
        _GLOBAL_MEMORY_BUFFER = GlobalMemoryBuffer()
    return _GLOBAL_MEMORY_BUFFER


def destroy_global_memory_buffer() -> None:
    global _GLOBAL_MEMORY_BUFFER
    _GLOBAL_MEMORY_BUFFER = None


class ParallelManager:
    def __init__(self) -> None:
        self.world_size = 1
        self.world_rank = 0
        self.timeout_min = 10
        self.backend: str | None = None
        self.parallels: dict[str, ParallelGroups] = {}
        self.all_parallels: dict[str, dict[str, ParallelGroups]] = {}
        self.rng_states: dict[str, tuple] = {}
        self._rng_seeds: dict[str, int] = {}
        self._group_cache: dict[tuple, Any] = {}
        self._stack: list = []
        self._cur_cfg = None
        self._vpp_size = 1
        self._vpp_rank = 0

    # ------------------------------------------------------------------ init
    def initialize(self, backend: str | None = None, timeout_min: int = 300) -> None:
        """Join the job. Reads ``RANK/WORLD_SIZE/LOCAL_RANK/MASTER_*`` (torchrun's variables).

        ``backend`` defaults to NCCL when CUDA is present, gloo otherwise.  A world of one
        process stays un-initialised (no rendezvous, no communicator) unless
        ``STB200_FORCE_DIST=1``.
        """
        self.timeout_min = timeout_min
        world = int(os.getenv("WORLD_SIZE", "1"))
        rank = int(os.getenv("RANK", "0"))
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        self.backend = backend
        if torch.cuda.is_available() and (n := torch.cuda.device_count()) > 0:
            torch.cuda.set_device(int(os.getenv("LOCAL_RANK", "0")) % n)
        if dist.is_initialized():
            self.world_size, self.world_rank = dist.get_world_size(), dist.get_rank()
            return
        if world == 1 and os.getenv("STB200_FORCE_DIST", "0") != "1":
            self.world_size, self.world_rank = 1, 0
            return
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "23456")
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(
            backend=backend, world_size=world, rank=rank, timeout=timedelta(minutes=timeout_min), **kwargs
        )
        atexit.register(_destroy)
        self.world_size, self.world_rank = dist.get_world_size(), dist.get_rank()

    @property
    def initialized(self) -> bool:
        return dist.is_initialized()

    # ---------------------------------------------------------------- meshes
    def define_parallel(self, pattern: str, **sizes: int) -> list[list[int]]:
        return layout_from_pattern(pattern, self.world_size, **sizes)

    def new_parallel(self, name: str, ranks: list[list[int]]) -> ParallelGroups:
        if name in self.parallels:
            if ranks != self.parallels[name].ranks:
                raise AssertionError(f"family {name} redefined with different ranks")
            return self.parallels[name]
        full = len(ranks[0])
        my_row = next((i for i, r in enumerate(ranks) if self.world_rank in r), None)
        if my_row is None:
            raise RuntimeError(f"rank {self.world_rank} is in no row of family {name}")
        pg = ParallelGroups(
            name=name, ranks=ranks, my_row=my_row, valid_replicas=sum(1 for r in ranks if len(r) == full)
        )
        self.parallels[name] = pg
        return pg

    def set_mesh(self, parallel_cfg) -> dict[str, ParallelGroups]:
        self._cur_cfg = parallel_cfg
        identity = repr(sorted((k, repr(v)) for k, v in parallel_cfg.to_dict().items()))
        if identity not in self.all_parallels:
            self.parallels = {}
            for name, ranks in parallel_cfg.build_parallel().items():
                self.new_parallel(name, ranks)
            self.all_parallels[identity] = self.parallels
        self.parallels = self.all_parallels[identity]
        self._vpp_size = int(getattr(parallel_cfg, "virtual_pipeline_model_parallel_size", 1) or 1)
        return self.parallels

    @contextmanager
    def use_mesh(self, parallel_cfg):
        self._stack.append(self._cur_cfg)
        self.set_mesh(parallel_cfg)
        try:
            yield
        finally:
            prev = self._stack.pop()
            if prev is not None:
                self.set_mesh(prev)

    def reset(self) -> None:
        """Forget every mesh and RNG stream (tests)."""
        self.parallels, self.all_parallels = {}, {}
        self.rng_states, self._rng_seeds = {}, {}
        self._cur_cfg = None
        self._stack = []
        self._vpp_size, self._vpp_rank = 1, 0

    # ----------------------------------------------------------------- query
    def _fam(self, name: str) -> ParallelGroups | None:
        return self.parallels.get(name)

    def has(self, name: str) -> bool:
        return name in self.parallels

    def size_of(self, name: str) -> int:
        fam = self._fam(name)
        if fam is None:
            if self.world_size == 1 or not self.parallels:
                return 1
            raise KeyError(f"parallel family {name!r} is not defined")
        return len(fam.ranks[fam.my_row])

    def rank_in(self, name: str) -> int:
        fam = self._fam(name)
        if fam is None:
            if self.world_size == 1 or not self.parallels:
                return 0
            raise KeyError(f"parallel family {name!r} is not defined")
        return fam.ranks[fam.my_row].index(self.world_rank)

    def i_am(self, name: str, rank: int) -> bool:
        return rank % self.size_of(name) == self.rank_in(name)

    def ranks_of(self, name: str) -> list[int]:
        fam = self._fam(name)
        return [self.world_rank] if fam is None else fam.ranks[fam.my_row]

    def rank_of(self, name: str) -> int:
        fam = self._fam(name)
        return 0 if fam is None else fam.my_row

    def replica_of(self, name: str) -> int:
        fam = self._fam(name)
        return 1 if fam is None else fam.valid_replicas

    def world_ranks_of(self, name: str) -> list[list[int]]:
        fam = self._fam(name)
        return [[self.world_rank]] if fam is None else fam.ranks

    def group_of(self, name: str):
        """Process group of this rank's row, created on first use. ``None`` when the row has one
        member or the job is a single process."""
        fam = self._fam(name)
        if fam is None or not dist.is_initialized():
            return None
        if not fam.created:
            row = fam.ranks[fam.my_row]
            if len(row) == 1:
                fam.group = None
            elif len(row) == self.world_size:
                fam.group = dist.group.WORLD
            else:
                key = tuple(row)
                if key not in self._group_cache:
                    self._group_cache[key] = dist.new_group(
                        row, timeout=timedelta(minutes=self.timeout_min), use_local_synchronization=True
                    )
                fam.group = self._group_cache[key]
            fam.created = True
        return fam.group

    def barrier(self, name: str | None = None) -> None:
        if not dist.is_initialized():
            return
        if name is None:
            dist.barrier()
        elif (g := self.group_of(name)) is not None:
            dist.barrier(group=g)

    # ------------------------------------------------------- pipeline helpers
    def set_vpp_rank(self, r: int) -> None:
        self._vpp_rank = r

    def get_vpp_rank(self) -> int:
        return self._vpp_rank

    def get_vpp_size(self) -> int:
        return self._vpp_size

    def is_pipeline_first_stage(self, ignore_virtual: bool = False) -> bool:
        if not ignore_virtual and self._vpp_size > 1 and self._vpp_rank != 0:
            return False
        return self.rank_in("PP") == 0

    def is_pipeline_last_stage(self, ignore_virtual: bool = False) -> bool:
        if not ignore_virtual and self._vpp_size > 1 and self._vpp_rank != self._vpp_size - 1:
            return False
        return self.rank_in("PP") == self.size_of("PP") - 1

    def pipeline_next_rank(self) -> int:
        row = self.ranks_of("PP")
        return row[(self.rank_in("PP") + 1) % len(row)]

    def pipeline_prev_rank(self) -> int:
        row = self.ranks_of("PP")
        return row[(self.rank_in("PP") - 1) % len(row)]

    # ------------------------------------------------------------ data ranks
    def get_data_rank(self) -> int:
        """Index of the data shard this rank consumes: CP peers share a shard
        (reference ``parallel_state.py:382-394``)."""
        return self.rank_in("DP") // self.size_of("CP")

    def get_data_world_size(self) -> int:
        return max(1, self.size_of("DP") // self.size_of("CP"))

    # ---------------------------------------------------------------- RNG
    def register_rng(self, name: str, seed: int, diff_across: list[str] | None = None) -> None:
        offset, stride = 0, 1
        for pname in diff_across or []:
            offset += self.rank_in(pname) * stride
            stride *= self.size_of(pname)
        rng_seed = int(seed) + offset
        if name in self._rng_seeds:
            if self._rng_seeds[name] != rng_seed:
                raise RuntimeError(f"RNG '{name}' already registered with a different seed")
            return
        self._rng_seeds[name] = rng_seed
        old = _get_rng_state()
        _set_rng_seed(rng_seed)
        self.rng_states[name] = _get_rng_state()
        _set_rng_state(old)

    @contextmanager
    def use_rng(self, name: str):
        if name not in self.rng_states:
            raise RuntimeError(f"RNG '{name}' is not registered")
        outer = _get_rng_state()
        _set_rng_state(self.rng_states[name])
        try:
            yield
        finally:
            self.rng_states[name] = _get_rng_state()
            _set_rng_state(outer)

    def get_all_rng(self):
        return _get_rng_state(), dict(self.rng_states)

    def set_all_rng(self, saved) -> None:
        current, stashed = saved
        _set_rng_state(current)
        self.rng_states.clear()
        self.rng_states.update(stashed)

    def __repr__(self) -> str:
        lines = ["ParallelManager("]
        for n in self.parallels:
            lines.append(
                f"    {n} = I({self.rank_in(n)}/{self.size_of(n)}) E({self.rank_of(n)}/{self.replica_of(n)})"
            )
        lines.append(")")
        return "\n".join(lines)


def _destroy() -> None:
    try:
        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass


PM = ParallelManager()


def set_mpu_random_seed(seed: int) -> None:
    """Seed python/numpy/torch for this rank and register the model-parallel RNG streams.

    Seeding rule of the reference (``core/tensor_parallel/initialize.py:50-87``): the default
    stream is ``seed + 100·pp_rank`` (identical inside a TP group), the ``model-parallel-rng``
    stream adds ``2718 + tp_rank`` and the ``expert-model-parallel-rng`` stream adds
    ``3718 + etp_rank + ep_rank·ETP``.
    """
    from .random import get_rng_tracker

    pp = PM.rank_in("PP") if PM.has("PP") else 0
    base = seed + 100 * pp
    _set_rng_seed(base)
    tp = PM.rank_in("TP") if PM.has("TP") else 0
    etp = PM.rank_in("ETP") if PM.has("ETP") else 0
    ep = PM.rank_in("EP") if PM.has("EP") else 0
    etp_size = PM.size_of("ETP") if PM.has("ETP") else 1
    tracker = get_rng_tracker()
    tracker.reset()
    tracker.add("model-parallel-rng", base + 2718 + tp)
    tracker.add("expert-model-parallel-rng", base + 3718 + etp + ep * etp_size)


# ---------------------------------------------------------------------------------------------------------------
# Module-level spellings of the manager's queries.  Model and schedule code written against the reference calls
# these as free functions (core/parallel_state.py:269-394); each one asks ``PM``, so there is one source of truth.
# ---------------------------------------------------------------------------------------------------------------
def is_unitialized() -> bool:
    """True before any mesh was set (the reference's spelling, core/parallel_state.py:269)."""
    return not PM.has("DP")


def model_parallel_is_initialized() -> bool:
    return all(PM.has(f) for f in ("TP", "PP", "DP"))


def get_vpp_rank() -> int:
    return PM.get_vpp_rank()


def set_vpp_rank(rank: int) -> None:
    PM.set_vpp_rank(int(rank or 0))


def get_vpp_size() -> int:
    return PM.get_vpp_size()


def set_vpp_size(world_size: int | None) -> None:
    PM._vpp_size = int(world_size or 1)


def get_pipeline_model_parallel_world_size(ignore_virtual: bool = True) -> int:
    """Pipeline stages; with ``ignore_virtual=False`` the model chunks of the whole pipeline (stages x VPP)."""
    return PM.size_of("PP") * (1 if ignore_virtual else PM.get_vpp_size())


def get_pipeline_model_parallel_rank(ignore_virtual: bool = True) -> int:
    """Stage of this rank; with ``ignore_virtual=False`` the index of the current model chunk in pipeline order."""
    return PM.rank_in("PP") + (0 if ignore_virtual else PM.get_vpp_rank() * PM.size_of("PP"))


def get_pipeline_model_parallel_next_rank() -> int:
    return PM.pipeline_next_rank()


def get_pipeline_model_parallel_prev_rank() -> int:
    return PM.pipeline_prev_rank()


def is_pipeline_first_stage(ignore_virtual: bool = False) -> bool:
    return PM.is_pipeline_first_stage(ignore_virtual)


def is_pipeline_last_stage(ignore_virtual: bool = False) -> bool:
    return PM.is_pipeline_last_stage(ignore_virtual)


def get_data_rank() -> int:
    return PM.get_data_rank()


def get_data_world_size() -> int:
    return PM.get_data_world_size()
