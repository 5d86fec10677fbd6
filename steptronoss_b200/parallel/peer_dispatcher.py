"""Expert-parallel dispatch / combine over peer memory (NVLink).

Semantics are those of :class:`~steptronoss_b200.parallel.ep_dispatcher.AllToAllDispatcher` (and of the
reference ``TokenDispatcher``, ``steptronoss/model/ep_dispatcher/token_dispatcher.py:14-118``): a token goes
once to every EP rank that hosts one of its top-k experts, with its expert ids rewritten to local indices
(-1 = foreign) and its weights (0 = foreign); the way back carries one partial row per (token, rank), which
the source adds up in rank order.

Instead of variable-size all-to-alls whose split sizes go through the host, every (token, destination) pair
has a fixed landing row: token ``t`` of source rank ``s`` lands in row ``s*T + t`` of the destination's receive
buffer, and its answer in row ``d*T + t`` of the source's return buffer.  Nothing is counted, prefix-summed or
exchanged before the payload moves: ``stb_ep_dispatch`` (``csrc/peer_rows.cu``) derives a token's destinations
from its k expert ids and stores the row and a small metadata row ``[call number | local ids | weights]`` into
the peers' memory; the receiver tells fresh rows from stale ones by the call number.  The receive buffer is
handed to the expert FFN as it is (``[world*T, H]`` with ids of -1 in the rows that did not arrive): the
expert-major scatter reads the arrived rows straight out of it, so there is no compaction copy.  One number
goes to the host per dispatch, the count of arrived (token, expert) slots, which sizes the expert-major buffers
that autograd keeps; with a ``capacity_factor`` not even that (the buffers take factor x the balanced load, and a
rank that receives more fails the step with an error status).

All ranks of the group must call with the same number of tokens ``T``.  CPU tensors (gloo tests), dtypes other
than bf16 and more than 15 experts per token take the all-to-all statement.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p

import torch
import torch.distributed as dist

from ..ops import native
from ..ops.gemm import count_launch
from .ep_dispatcher import AllToAllDispatcher
from .state import PM
from . import symm
from .symm import _WAIT_NS, SymmetricBuffer

P, I, L, U, ULL = c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint, ctypes.c_ulonglong
native.register_signature("stb_peer_scatter_rows", [P, L, I, P, P, P, I, P, L, P, I, I, I, U, P, P])
native.register_signature("stb_peer_wait_flags", [P, I, I, U, ULL, P, P])
native.register_signature("stb_ep_dispatch", [P, L, I, P, P, P, L, I, P, I, U, P, I, I, I, I, I, P])
native.register_signature("stb_ep_return", [P, I, P, P, P, L, P, I, U, P, I, I, I, I, P])
native.register_signature("stb_ep_sum", [P, I, P, P, P, P, I, I, I, I, I, P])

# buffer kinds: each has its own two slots, flag rows and call counter
_FWD, _BACK = 0, 1
_KINDS = 2


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class _PeerArena:
    """Flag page and the double-slotted receive / return buffers of one EP group."""

    def __init__(self, group_name: str):
        self.group = PM.group_of(group_name)
        self.rank, self.world = PM.rank_in(group_name), PM.size_of(group_name)
        self.lib = native.load()
        self.flags = SymmetricBuffer(2 * _KINDS * 8 * 4, self.group, self.lib)
        self.flags.own_tensor().zero_()
        self.bufs: list = [None] * _KINDS
        self.slot_bytes = [0] * _KINDS
        self.epoch = [0] * _KINDS
        self.done = torch.zeros(4, dtype=torch.int32, device="cuda")
        self._flag_arr = self.flags.ptr_array()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def slot(self, kind: int, need: int):
        """Advance the kind's call counter; ``(epoch, flag row, pointer array, own slot as bytes)``."""
        if need > self.slot_bytes[kind]:
            size = (need + (1 << 20) - 1) & ~((1 << 20) - 1)
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            if self.bufs[kind] is not None:
                self.bufs[kind].release()
            self.bufs[kind] = SymmetricBuffer(2 * size, self.group, self.lib)
            self.bufs[kind].own_tensor().zero_()       # call numbers start at 1: a zeroed row is never fresh
            self.slot_bytes[kind] = size
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        self.epoch[kind] += 1
        e = self.epoch[kind]
        off = (e & 1) * self.slot_bytes[kind]
        return e, 2 * kind + (e & 1), self.bufs[kind].ptr_array(off), self.bufs[kind].own_tensor()[off: off + need]

    def wait(self, flag_row: int, epoch: int, device) -> None:
        rc = self.lib.stb_peer_wait_flags(self.flags.own, flag_row, self.world, epoch & 0xFFFFFFFF, _WAIT_NS,
                                          native.status_word(device).data_ptr(), native.stream())
        native.check(rc, "peer wait")
        count_launch()


_ARENAS: dict = {}


def _arena(group_name: str) -> _PeerArena:
    if group_name not in _ARENAS:
        _ARENAS[group_name] = _PeerArena(group_name)
    return _ARENAS[group_name]


class _Plan:
    """What the four moves of one dispatch share."""

    def __init__(self, expert_ids: torch.Tensor, world: int, rank: int, per_rank: int):
        self.T, self.K = expert_ids.shape
        self.world, self.rank, self.per_rank = world, rank, per_rank
        self.ids = expert_ids.to(torch.int64).contiguous()
        self.valid = None      # uint8 [world*T]: receive-buffer rows that arrived in this dispatch
        self.slots = None      # number of (token, local expert) slots that arrived (host integer)


def _send_rows(ar: _PeerArena, plan: _Plan, x: torch.Tensor, weights):
    """Rows of ``x [T, H]`` (and metadata when ``weights`` is given) to the hosts of every token's experts; returns
    this rank's receive buffer ``[world*T, H]`` and metadata ``[world*T, 1+2K]`` (views of peer-mapped memory:
    consume them before the second-next call) and the call number that marks fresh metadata rows."""
    T, K, W = plan.T, plan.K, plan.world
    x = x.contiguous()
    row_bytes = x.shape[1] * x.element_size()
    meta_off = _align(W * T * row_bytes)
    meta_bytes = W * T * (1 + 2 * K) * 4 if weights is not None else 0
    e, flag_row, ptrs, own = ar.slot(_FWD, meta_off + meta_bytes)
    tag = e & 0x7FFFFFFF
    w32 = None if weights is None else weights.to(torch.float32).contiguous()
    rc = ar.lib.stb_ep_dispatch(x.data_ptr(), x.stride(0) * x.element_size(), row_bytes, plan.ids.data_ptr(),
                                native.ptr(w32), ptrs, meta_off, tag, ar._flag_arr, flag_row, e & 0xFFFFFFFF,
                                ar.done.data_ptr() + 4 * _FWD, T, K, W, plan.rank, plan.per_rank, native.stream())
    native.check(rc, "ep dispatch")
    count_launch()
    ar.wait(flag_row, e, x.device)
    recv = own[: W * T * row_bytes].view(x.dtype).view(W * T, x.shape[1])
    meta = own[meta_off: meta_off + meta_bytes].view(torch.int32).view(W * T, 1 + 2 * K) if weights is not None else None
    return recv, meta, tag


def _return_rows(ar: _PeerArena, plan: _Plan, rows: torch.Tensor, wrows, want_sum_dtype):
    """The way back: arrived rows of ``rows [world*T, H]`` (and ``wrows [world*T, K]`` fp32) go to their sources;
    returns per token the sum over its destinations ``[T, H]`` and the routing-weight gradients ``[T, K]``."""
    T, K, W = plan.T, plan.K, plan.world
    rows = rows.contiguous()
    H = rows.shape[1]
    row_bytes = H * rows.element_size()
    w_off = _align(W * T * row_bytes)
    w_bytes = W * T * K * 4 if wrows is not None else 0
    e, flag_row, ptrs, own = ar.slot(_BACK, w_off + w_bytes)
    w32 = None if wrows is None else wrows.to(torch.float32).contiguous()
    rc = ar.lib.stb_ep_return(rows.data_ptr(), row_bytes, native.ptr(w32), plan.valid.data_ptr(), ptrs, w_off,
                              ar._flag_arr, flag_row, e & 0xFFFFFFFF, ar.done.data_ptr() + 4 * _BACK, T, K, W,
                              plan.rank, native.stream())
    native.check(rc, "ep return")
    count_launch()
    ar.wait(flag_row, e, rows.device)
    out = torch.empty((T, H), dtype=want_sum_dtype, device=rows.device)
    gw = torch.empty((T, K), dtype=torch.float32, device=rows.device) if wrows is not None else None
    back_w = own[w_off: w_off + w_bytes] if wrows is not None else None
    rc = ar.lib.stb_ep_sum(own.data_ptr(), H, native.ptr(back_w), plan.ids.data_ptr(), out.data_ptr(), native.ptr(gw),
                           T, K, W, plan.rank, plan.per_rank, native.stream())
    native.check(rc, "ep sum")
    count_launch()
    return out, gw


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weights, disp):
        ar, plan = disp.arena, disp.plan
        K = plan.K
        recv, meta, tag = _send_rows(ar, plan, x, weights)
        fresh = meta[:, 0] == tag
        plan.valid = fresh.to(torch.uint8)
        ids_r = torch.where(fresh.unsqueeze(1), meta[:, 1: 1 + K], torch.full((), -1, dtype=torch.int32, device=x.device)).long()
        w_r = torch.where(fresh.unsqueeze(1), meta[:, 1 + K:].contiguous().view(torch.float32), torch.zeros((), device=x.device))
        if disp.capacity_factor:
            # no host read: the expert-major buffers take capacity_factor x the balanced load; the index kernel
            # drops what does not fit and raises the capacity error in the status word
            plan.slots = min(int(disp.capacity_factor * plan.T * K), plan.world * plan.T * K)
        else:
            plan.slots = int((ids_r >= 0).sum())       # the one host read of a dispatch
        ctx.disp, ctx.plan, ctx.w_dtype, ctx.x_dtype = disp, plan, weights.dtype, x.dtype
        ctx.mark_non_differentiable(ids_r)
        return recv, ids_r, w_r.to(weights.dtype)

    @staticmethod
    def backward(ctx, g_x, _g_ids, g_w):
        plan = ctx.plan
        if g_w is None:
            g_w = torch.zeros((plan.world * plan.T, plan.K), dtype=torch.float32, device=g_x.device)
        gx, gw = _return_rows(ctx.disp.arena, plan, g_x, g_w, ctx.x_dtype)
        return gx, gw.to(ctx.w_dtype), None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, disp):
        ctx.disp, ctx.plan = disp, disp.plan
        out, _ = _return_rows(disp.arena, disp.plan, y, None, y.dtype)
        return out

    @staticmethod
    def backward(ctx, g):
        recv, _meta, _tag = _send_rows(ctx.disp.arena, ctx.plan, g, None)
        return recv, None   # rows that did not arrive hold stale data: their ids are -1, nothing reads them


class PeerMemoryDispatcher:
    def __init__(self, group_name: str, num_experts: int, capacity_factor: float | None = None):
        self.group_name, self.num_experts = group_name, num_experts
        self.capacity_factor = capacity_factor
        """None: size the expert buffers by the exact number of arrived slots (one host read per dispatch).
        A factor f >= 1: size them for f x tokens x top-k slots without reading anything back; a rank that
        receives more fails the step with the capacity error instead of dropping tokens silently."""
        self.world, self.rank = PM.size_of(group_name), PM.rank_in(group_name)
        self.per_rank = num_experts // self.world
        self._fallback = AllToAllDispatcher(group_name, num_experts)
        self.arena: _PeerArena | None = None
        self.plan: _Plan | None = None
        self._used_fallback = False
        self.received_slots: int | None = None
        """(token, local expert) slots that arrived in the last dispatch; None on the all-to-all path."""
        self._group_decision: bool | None = None
        self._checked_tokens: set = set()

    def _group_ok(self) -> bool:
        """Decided once per dispatcher, collectively: the group is NCCL, 2 to 8 ranks, all on one node (peer memory
        is mapped through CUDA IPC, which does not cross nodes)."""
        if self._group_decision is None:
            ok = dist.is_initialized() and 2 <= self.world <= 8
            if ok:
                group = PM.group_of(self.group_name)
                ok = dist.get_backend(group) == "nccl" and symm._same_node(group)
            self._group_decision = bool(ok)
        return self._group_decision

    def _check_equal_tokens(self, tokens: int, device) -> None:
        """Landing rows are `source rank * T + token`: every rank of the group must dispatch the same number of
        tokens.  Checked once per token count with one small all-reduce; unequal counts raise on every rank."""
        if tokens in self._checked_tokens:
            return
        t = torch.tensor([tokens, -tokens], dtype=torch.int64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=PM.group_of(self.group_name))
        hi, lo = int(t[0].item()), -int(t[1].item())
        if hi != lo:
            raise ValueError(f"the peer-memory dispatcher needs the same token count on every rank of "
                             f"{self.group_name} (between {lo} and {hi} here); use the all-to-all dispatcher")
        self._checked_tokens.add(tokens)

    def _peer_ok(self, x: torch.Tensor, expert_ids: torch.Tensor) -> bool:
        return (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and expert_ids.shape[1] <= 15
                and self._group_ok())

    def dispatch(self, x, expert_ids, weights):
        self._used_fallback = not self._peer_ok(x, expert_ids)
        if self._used_fallback:
            self.received_slots = None
            return self._fallback.dispatch(x, expert_ids, weights)
        self._check_equal_tokens(x.shape[0], x.device)
        if self.arena is None:
            self.arena = _arena(self.group_name)
        self.plan = _Plan(expert_ids, self.world, self.rank, self.per_rank)
        out = _DispatchFn.apply(x, weights, self)
        self.received_slots = self.plan.slots
        return out

    def combine(self, y):
        if self._used_fallback:
            return self._fallback.combine(y)
        return _CombineFn.apply(y, self)
