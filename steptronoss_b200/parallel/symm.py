"""Peer-mapped ("symmetric") device memory of a process group and the fused GEMM+collective launches.

Every rank of a group allocates the same set of buffers with ``cudaMalloc``, publishes their CUDA IPC
handles through the group and maps the peers' buffers, so that a kernel on one GPU can load from and
store to the other GPUs of the node over NVLink.  On top of that arena sit the two fused launches of
``csrc/gemm_tp_sm100.cu``:

* :func:`all_gather_gemm`   ``all_gather_rows(x) @ w.T`` (or ``@ w``), also returning the gathered rows;
* :func:`gemm_reduce_scatter` ``reduce_scatter_rows(a @ w.T)`` (or ``a @ w``).

They stand where the reference issues an NCCL collective next to a cuBLAS GEMM
(``steptronoss/core/tensor_parallel/layers.py:151-346``).  The NCCL statement remains as the path for
CPU/gloo runs, groups that span nodes and shapes the kernels do not take (row blocks that are not a
multiple of 128).

Environment: ``STB200_PEER_TP=0`` disables the peer path; ``STB200_PEER_WAIT_S`` (default 30) bounds every
wait on another rank inside the kernels.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_void_p

import torch
import torch.distributed as dist

from ..ops import native
from ..ops.gemm import count_launch
from .state import PM

_MAX_RANKS = 8
_ARENAS: dict[str, "Arena | None"] = {}
_DISABLED = os.environ.get("STB200_PEER_TP", "1") == "0"
_WAIT_NS = int(float(os.environ.get("STB200_PEER_WAIT_S", "30")) * 1e9)
_TRACE = None  # int64 [SMs, 8] tensor set by trace(): per-CTA phase stamps of the next fused launches


def trace(enable: bool = True):
    """Start (or stop) recording the per-CTA phase stamps of the fused kernels; returns the buffer."""
    global _TRACE
    _TRACE = torch.zeros((256, 8), dtype=torch.int64, device="cuda") if enable else None
    return _TRACE


def trace_rows() -> list:
    """The raw per-CTA stamps (rows of CTAs that ran), columns as in :func:`trace_summary`."""
    t = _TRACE.cpu()
    return t[t[:, 0] > 0].tolist()


def trace_summary() -> dict:
    """Phase ends relative to the earliest CTA entry, in microseconds (max over CTAs)."""
    t = _TRACE.cpu()
    t = t[t[:, 0] > 0]
    t0 = int(t[:, 0].min())
    names = ["entry", "first_load", "producer_done", "mma_done", "epilogue_done", "aux_first", "aux_done", "exit"]
    out = {}
    for i, n in enumerate(names):
        col = t[:, i][t[:, i] > 0]
        if col.numel():
            out[n] = {"min_us": (int(col.min()) - t0) / 1e3, "max_us": (int(col.max()) - t0) / 1e3}
    return out

P, I, L, U, ULL = c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint, ctypes.c_ulonglong
native.register_signature("stb_tp_flag_words", [])
native.register_signature("stb_tp_ctr_words", [I])
native.register_signature("stb_symm_alloc", [P, ULL, P])
native.register_signature("stb_symm_open", [P, P])
native.register_signature("stb_symm_close", [P])
native.register_signature("stb_symm_free", [P])
native.register_signature(
    "stb_gemm_ag_bf16", [P, L, P, P, P, P, I, I, I, I, I, I, I, I, I, U, P, ULL, P, P, P]
)
native.register_signature(
    "stb_gemm_rs_bf16", [P, I, P, I, I, P, L, P, P, P, I, I, I, I, I, U, P, ULL, P, P, P]
)


class _DevicePointer:
    """Lets torch wrap memory it did not allocate (``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SymmetricBuffer:
    """One allocation per rank, mapped on every rank.  ``ptrs[r]`` is rank r's buffer in this process."""

    def __init__(self, nbytes: int, group, lib):
        self.nbytes = int(nbytes)
        self.group = group
        self.lib = lib
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        own = c_void_p()
        handle = ctypes.create_string_buffer(64)
        rc = lib.stb_symm_alloc(ctypes.byref(own), self.nbytes, handle)
        ok = torch.tensor([1 if rc == 0 else 0], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            if rc == 0:
                lib.stb_symm_free(own)
            raise RuntimeError(f"peer memory allocation of {nbytes} bytes failed on some rank (rc={rc})")
        self.own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, (os.getpid(), handle.raw), group=group)
        self.ptrs = [0] * self.world
        opened_ok = 1
        for r, (_, raw) in enumerate(handles):
            if r == self.rank:
                self.ptrs[r] = self.own
                continue
            p = c_void_p()
            rc = lib.stb_symm_open(ctypes.byref(p), raw)
            if rc != 0:
                opened_ok = 0
                break
            self.ptrs[r] = p.value
        ok = torch.tensor([opened_ok], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            self.release()
            raise RuntimeError("mapping a peer's memory failed on some rank")

    def own_tensor(self) -> torch.Tensor:
        """The own buffer as a uint8 tensor (no copy; the buffer outlives the tensor's uses by contract)."""
        if getattr(self, "_own_tensor", None) is None:
            self._own_tensor = torch.as_tensor(_DevicePointer(self.own, self.nbytes), device="cuda")
        return self._own_tensor

    def ptr_array(self, offset: int = 0):
        arr = (c_void_p * _MAX_RANKS)()
        for r in range(self.world):
            arr[r] = self.ptrs[r] + offset
        return arr

    def release(self):
        """Unmap the peers and free the own buffer; callers synchronise the group first."""
        for r, p in enumerate(self.ptrs):
            if p and r != self.rank:
                self.lib.stb_symm_close(c_void_p(p))
        if self.own:
            self.lib.stb_symm_free(c_void_p(self.own))
        self.ptrs, self.own = [], 0
        self._own_tensor = None


class Arena:
    """Flag page, gathered-matrix slots (all-gather) and receive slots (reduce-scatter) of one group."""

    def __init__(self, group_name: str):
        self.group_name = group_name
        self.group = PM.group_of(group_name)
        self.rank = PM.rank_in(group_name)
        self.world = PM.size_of(group_name)
        self.lib = native.load()
        self.flags = SymmetricBuffer(self.lib.stb_tp_flag_words() * 4, self.group, self.lib)
        self.stage: SymmetricBuffer | None = None   # 2 slots
        self.recv: SymmetricBuffer | None = None    # 2 slots
        self.stage_slot = 0
        self.recv_slot = 0
        self.partials: torch.Tensor | None = None   # local staging matrix of the reduce-scatter kernel
        self.ag_epoch = 0
        self.rs_epoch = 0
        self.ctrs = torch.zeros(self.lib.stb_tp_ctr_words(_MAX_RANKS * 1024), dtype=torch.int32, device="cuda")
        self._flag_arr = self.flags.ptr_array()
        dist.barrier(group=self.group)

    def _grow(self, which: str, slot_bytes: int):
        """All ranks reach this with the same arguments in the same call, so the exchange lines up."""
        slot_bytes = (slot_bytes + (1 << 20) - 1) & ~((1 << 20) - 1)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        old = getattr(self, which)
        if old is not None:
            old.release()
        setattr(self, which, SymmetricBuffer(2 * slot_bytes, self.group, self.lib))
        setattr(self, which + "_slot", slot_bytes)
        dist.barrier(group=self.group)

    def gathered_slot(self, need: int, epoch: int):
        """``(pointer array over ranks, own slot as uint8 tensor)`` of this call's gathered matrix."""
        if need > self.stage_slot:
            self._grow("stage", need)
        off = (epoch & 1) * self.stage_slot
        return self.stage.ptr_array(off), self.stage.own_tensor()[off: off + need]

    def partial_staging(self, need: int) -> torch.Tensor:
        """Local scratch for the partial products of one reduce-scatter launch (reused by the next launch: the
        kernel that read it has finished by then, launches on a group are stream-ordered)."""
        if self.partials is None or self.partials.numel() < need:
            self.partials = torch.empty((need + (1 << 20) - 1) & ~((1 << 20) - 1), dtype=torch.uint8, device="cuda")
        return self.partials

    def recv_ptrs(self, need: int, epoch: int):
        if need > self.recv_slot:
            self._grow("recv", need)
        return self.recv.ptr_array((epoch & 1) * self.recv_slot)


def _same_node(group) -> bool:
    import socket

    names = [None] * dist.get_world_size(group)
    dist.all_gather_object(names, socket.gethostname(), group=group)
    return len(set(names)) == 1


def arena(group_name: str) -> "Arena | None":
    """The group's arena, created on first use (collective); ``None`` when the peer path is unavailable."""
    if group_name in _ARENAS:
        return _ARENAS[group_name]
    a = None
    n = PM.size_of(group_name)
    if (not _DISABLED and torch.cuda.is_available() and dist.is_initialized() and 2 <= n <= _MAX_RANKS
            and dist.get_backend(PM.group_of(group_name)) == "nccl" and _same_node(PM.group_of(group_name))):
        try:
            a = Arena(group_name)
        except RuntimeError as e:  # every rank raises together (the outcome is all-reduced)
            from ..utils.logger import logger

            logger.warning(f"peer-memory path disabled for group {group_name}: {e}")
            a = None
    _ARENAS[group_name] = a
    return a


def enabled(group_name: str = "TP") -> bool:
    return arena(group_name) is not None


def usable(rows_local: int, k: int, n: int, *tensors) -> bool:
    """Shapes and dtypes the fused kernels take."""
    if rows_local <= 0 or rows_local % 128 or rows_local // 128 > 1024 or k % 8 or n % 8:
        return False
    return all(t.is_cuda and t.dtype == torch.bfloat16 and t.stride(-1) == 1 and t.data_ptr() % 16 == 0
               and (t.dim() < 2 or t.stride(0) % 8 == 0) for t in tensors)


def all_gather_gemm(x, w, group_name: str = "TP", *, b_mn_major: bool = False, out_dtype=None,
                    need_gathered: bool = True):
    """``(all_gather_rows(x) @ w.T  [or @ w], all_gather_rows(x))`` in one launch.  ``w=None`` gathers only;
    ``need_gathered=False`` returns ``None`` for the gathered rows and saves the copy of the own block.

    The gathered matrix is a view of the group's symmetric memory and stays valid until the NEXT fused all-gather
    on the group is launched: a peer may start writing the call after that one into the same slot as soon as it
    has seen this rank's rows of the next call.  Consume it on the launching stream, or copy it, before that."""
    a = arena(group_name)
    rows, k = x.shape
    m = rows * a.world
    if w is None:
        n = 0
    else:
        n = w.shape[1] if b_mn_major else w.shape[0]
    y = torch.empty((m, n), dtype=x.dtype, device=x.device) if n else None
    a.ag_epoch += 1
    ptrs, own = a.gathered_slot(m * k * 2, a.ag_epoch)
    gathered = own.view(torch.bfloat16).view(m, k)
    rc = a.lib.stb_gemm_ag_bf16(
        x.data_ptr(), x.stride(0), ptrs, a._flag_arr,
        w.data_ptr() if n else None, y.data_ptr() if n else None, rows, n, k,
        w.stride(0) if n else 8, y.stride(0) if n else 8, int(b_mn_major), int(need_gathered), a.rank, a.world,
        a.ag_epoch & 0xFFFFFFFF, a.ctrs.data_ptr(), _WAIT_NS, native.status_word(x.device).data_ptr(),
        _TRACE.data_ptr() if _TRACE is not None else None, native.stream(),
    )
    native.check(rc, f"all_gather_gemm rows={rows} N={n} K={k}")
    count_launch(2)
    if y is not None and out_dtype not in (None, y.dtype):
        y = y.to(out_dtype)
    return y, (gathered if need_gathered else None)


def gemm_reduce_scatter(x, w, group_name: str = "TP", *, b_mn_major: bool = False):
    """``reduce_scatter_rows(x @ w.T)`` (or ``x @ w``) in one launch; ``x`` is ``[tp*rows_local, K]``."""
    a = arena(group_name)
    m, k = x.shape
    rows = m // a.world
    n = w.shape[1] if b_mn_major else w.shape[0]
    out = torch.empty((rows, n), dtype=x.dtype, device=x.device)
    a.rs_epoch += 1
    recv = a.recv_ptrs(m * n * 2, a.rs_epoch)
    staging = a.partial_staging(m * n * 2)
    rc = a.lib.stb_gemm_rs_bf16(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), int(b_mn_major), out.data_ptr(), out.stride(0),
        staging.data_ptr(), recv, a._flag_arr, rows, n, k, a.rank, a.world, a.rs_epoch & 0xFFFFFFFF, a.ctrs.data_ptr(),
        _WAIT_NS, native.status_word(x.device).data_ptr(),
        _TRACE.data_ptr() if _TRACE is not None else None, native.stream(),
    )
    native.check(rc, f"gemm_reduce_scatter M={m} N={n} K={k}")
    count_launch(2)
    return out


def shutdown() -> None:
    """Release every arena (collective; call before destroying the process groups)."""
    for name, a in list(_ARENAS.items()):
        if a is None:
            continue
        torch.cuda.synchronize()
        dist.barrier(group=a.group)
        for buf in (a.stage, a.recv, a.flags):
            if buf is not None:
                buf.release()
    _ARENAS.clear()
