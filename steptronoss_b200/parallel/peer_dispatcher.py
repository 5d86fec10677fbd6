"""Expert-parallel dispatch / combine over peer memory (NVLink), without host synchronisation.

Semantics are those of :class:`~steptronoss_b200.parallel.ep_dispatcher.AllToAllDispatcher` (and of the
reference ``TokenDispatcher``, ``steptronoss/model/ep_dispatcher/token_dispatcher.py:14-118``): a token goes
once to every EP rank that hosts one of its top-k experts, with its expert ids rewritten to local indices
(-1 = foreign) and its weights (0 = foreign); the way back carries one partial row per (token, rank).

Instead of variable-size all-to-alls whose split sizes go through the host, every (token, destination)
pair has a fixed landing row in the destination's receive buffer: source rank ``s`` owns rows
``[s*T, (s+1)*T)`` and fills them from the front in token order.  Rows travel with
``csrc/peer_rows.cu::stb_peer_scatter_rows`` (plain peer stores); each row of the small metadata buffer
starts with the call number, which is how the receiver tells fresh rows from stale ones, so no counts are
exchanged either.  The receive buffers have the worst-case capacity ``world * T`` rows; the fresh rows are then
compacted (one device-to-host read of their number per dispatch, where the all-to-all statement needs the
whole split-size matrix on the host before it can start), so that the expert GEMMs and what autograd keeps
are sized by the rows that actually arrived.

All ranks of the group must call with the same number of tokens ``T``.  CPU tensors (gloo tests) take the
all-to-all statement.
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
from .symm import _WAIT_NS, SymmetricBuffer

P, I, L, U, ULL = c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint, ctypes.c_ulonglong
native.register_signature("stb_peer_scatter_rows", [P, L, I, P, P, P, I, P, L, P, I, I, I, U, P, P])
native.register_signature("stb_peer_wait_flags", [P, I, I, U, ULL, P, P])

# buffer kinds: each has its own two slots, flag rows and call counter
_X, _META, _BACK, _BACK_W = 0, 1, 2, 3
_KINDS = 4


class _PeerArena:
    """Flag page and the double-slotted receive buffers of one EP group."""

    def __init__(self, group_name: str):
        self.group = PM.group_of(group_name)
        self.rank, self.world = PM.rank_in(group_name), PM.size_of(group_name)
        self.lib = native.load()
        self.flags = SymmetricBuffer(2 * _KINDS * 8 * 4, self.group, self.lib)
        self.bufs: list = [None] * _KINDS
        self.slot_bytes = [0] * _KINDS
        self.epoch = [0] * _KINDS
        self.done = torch.zeros(4, dtype=torch.int32, device="cuda")
        self._flag_arr = self.flags.ptr_array()
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
            self.slot_bytes[kind] = size
            dist.barrier(group=self.group)
        self.epoch[kind] += 1
        e = self.epoch[kind]
        off = (e & 1) * self.slot_bytes[kind]
        return e, 2 * kind + (e & 1), self.bufs[kind].ptr_array(off), self.bufs[kind].own_tensor()[off: off + need]


_ARENAS: dict = {}


def _arena(group_name: str) -> _PeerArena:
    if group_name not in _ARENAS:
        _ARENAS[group_name] = _PeerArena(group_name)
    return _ARENAS[group_name]


def _scatter(ar: _PeerArena, kind: int, src: torch.Tensor, src_row, dst_rank, dst_row, rows_cap: int) -> torch.Tensor:
    """Send rows of the 2-D tensor ``src`` to their landing rows on the peers, wait for everybody's rows and
    return this rank's receive buffer ``[rows_cap, src.shape[1]]`` (a view of peer-mapped memory: copy what
    must outlive the second-next call of the same kind)."""
    row_bytes = src.shape[1] * src.element_size()
    e, flag_row, ptrs, own = ar.slot(kind, rows_cap * row_bytes)
    st = native.stream()
    rc = ar.lib.stb_peer_scatter_rows(src.data_ptr(), src.stride(0) * src.element_size(), row_bytes,
                                      src_row.data_ptr(), dst_rank.data_ptr(), dst_row.data_ptr(), src_row.numel(),
                                      ptrs, row_bytes, ar._flag_arr, flag_row, ar.world, ar.rank, e & 0xFFFFFFFF,
                                      ar.done.data_ptr() + 4 * kind, st)
    native.check(rc, "peer scatter")
    rc = ar.lib.stb_peer_wait_flags(ar.flags.own, flag_row, ar.world, e & 0xFFFFFFFF, _WAIT_NS,
                                    native.status_word(src.device).data_ptr(), st)
    native.check(rc, "peer wait")
    count_launch(2)
    return own.view(src.dtype).view(rows_cap, src.shape[1])


class _Plan:
    """Where the rows of one dispatch go: computed once per call from the routing, reused by all four moves."""

    def __init__(self, expert_ids: torch.Tensor, world: int, rank: int, per_rank: int):
        T, K = expert_ids.shape
        dev = expert_ids.device
        dest = (expert_ids // per_rank).clamp(0, world - 1)
        hits = torch.zeros((T, world), dtype=torch.bool, device=dev)
        hits.scatter_(1, dest, expert_ids >= 0)
        pos = hits.to(torch.int32).cumsum(0, dtype=torch.int32) - 1             # row inside this rank's block
        self.T, self.K, self.world, self.rank = T, K, world, rank
        self.hits = hits
        # forward moves: pair (t, d) -> row rank*T + pos[t, d] on rank d
        self.pair_src = torch.arange(T, device=dev, dtype=torch.int32).repeat_interleave(world)
        self.pair_rank = torch.arange(world, device=dev, dtype=torch.int32).repeat(T)
        self.pair_row = torch.where(hits, pos + rank * T, torch.full_like(pos, -1)).reshape(-1).contiguous()
        # where the answers of rank d for token t come back to: row d*T + pos[t, d] of the back buffer
        self.back_index = (pos.clamp_min(0).long() + torch.arange(world, device=dev).long() * T)   # [T, world]
        # set by dispatch once the rows have arrived: which rows of the receive buffer are fresh (``sel``), and
        # where the answer to compact row i goes: source sel // T, row rank*T + sel % T of its back buffer
        self.sel = self.ret_src = self.ret_rank = self.ret_row = None

    def set_received(self, valid: torch.Tensor) -> None:
        sel = valid.nonzero(as_tuple=False).reshape(-1)          # host sync: number of received rows
        self.sel = sel
        self.ret_src = torch.arange(sel.numel(), device=sel.device, dtype=torch.int32)
        self.ret_rank = (sel // self.T).to(torch.int32)
        self.ret_row = (self.rank * self.T + sel % self.T).to(torch.int32)


def _sum_over_ranks(back: torch.Tensor, plan: "_Plan") -> torch.Tensor:
    """``[world*T, C]`` answers -> ``[T, C]``: per token the fp32 sum over the ranks it was sent to (rows of
    pairs that were never sent may hold anything, so they are selected out, not multiplied by zero)."""
    picked = back.index_select(0, plan.back_index.reshape(-1)).view(plan.T, plan.world, -1).float()
    return torch.where(plan.hits.unsqueeze(2), picked, torch.zeros((), device=back.device)).sum(1)


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weights, expert_ids, disp):
        ar, plan = disp.arena, disp.plan
        T, K, W = plan.T, plan.K, plan.world
        cap = W * T
        recv_x = _scatter(ar, _X, x.contiguous(), plan.pair_src, plan.pair_rank, plan.pair_row, cap)
        # metadata row per pair: [call number | local ids (k) | weights as bits (k)]
        local = expert_ids.unsqueeze(1) - (torch.arange(W, device=x.device) * disp.per_rank).view(1, W, 1)   # [T,W,K]
        foreign = (local < 0) | (local >= disp.per_rank) | (expert_ids.unsqueeze(1) < 0)
        local = torch.where(foreign, torch.full_like(local, -1), local).to(torch.int32)
        wbits = torch.where(foreign, torch.zeros((), device=x.device), weights.float().unsqueeze(1)).view(torch.int32)
        tag = torch.full((T, W, 1), (ar.epoch[_META] + 1) & 0x7FFFFFFF, dtype=torch.int32, device=x.device)
        meta_src = torch.cat([tag, local, wbits], dim=2).reshape(T * W, 1 + 2 * K).contiguous()
        pair_idx = torch.arange(T * W, device=x.device, dtype=torch.int32)
        meta = _scatter(ar, _META, meta_src, pair_idx, plan.pair_rank, plan.pair_row, cap)
        plan.set_received(meta[:, 0] == (ar.epoch[_META] & 0x7FFFFFFF))
        meta = meta.index_select(0, plan.sel)
        ids_r = meta[:, 1: 1 + K].long()
        w_r = meta[:, 1 + K:].contiguous().view(torch.float32)
        xr = recv_x.index_select(0, plan.sel)
        ctx.disp, ctx.plan, ctx.w_dtype = disp, plan, weights.dtype
        ctx.mark_non_differentiable(ids_r)
        return xr, ids_r, w_r.to(weights.dtype)

    @staticmethod
    def backward(ctx, g_x, _g_ids, g_w):
        ar, plan = ctx.disp.arena, ctx.plan
        T, K, W = plan.T, plan.K, plan.world
        back = _scatter(ar, _BACK, g_x.contiguous(), plan.ret_src, plan.ret_rank, plan.ret_row, W * T)
        gx = _sum_over_ranks(back, plan).to(g_x.dtype)
        gw = None
        if g_w is not None:
            back_w = _scatter(ar, _BACK_W, g_w.float().contiguous(), plan.ret_src, plan.ret_rank, plan.ret_row, W * T)
            gw = _sum_over_ranks(back_w, plan).to(ctx.w_dtype)
        return gx, gw, None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, disp):
        ar, plan = disp.arena, disp.plan
        T, W = plan.T, plan.world
        back = _scatter(ar, _BACK, y.contiguous(), plan.ret_src, plan.ret_rank, plan.ret_row, W * T)
        out = _sum_over_ranks(back, plan).to(y.dtype)
        ctx.disp, ctx.plan = disp, plan
        return out

    @staticmethod
    def backward(ctx, g):
        ar, plan = ctx.disp.arena, ctx.plan
        recv = _scatter(ar, _X, g.contiguous(), plan.pair_src, plan.pair_rank, plan.pair_row, plan.world * plan.T)
        return recv.index_select(0, plan.sel), None


class PeerMemoryDispatcher:
    def __init__(self, group_name: str, num_experts: int):
        self.group_name, self.num_experts = group_name, num_experts
        self.world, self.rank = PM.size_of(group_name), PM.rank_in(group_name)
        self.per_rank = num_experts // self.world
        self._fallback = AllToAllDispatcher(group_name, num_experts)
        self.arena: _PeerArena | None = None
        self.plan: _Plan | None = None
        self._used_fallback = False

    def _peer_ok(self, x: torch.Tensor) -> bool:
        return (x.is_cuda and dist.is_initialized() and 2 <= self.world <= 8
                and dist.get_backend(PM.group_of(self.group_name)) == "nccl")

    def dispatch(self, x, expert_ids, weights):
        self._used_fallback = not self._peer_ok(x)
        if self._used_fallback:
            return self._fallback.dispatch(x, expert_ids, weights)
        if self.arena is None:
            self.arena = _arena(self.group_name)
        self.plan = _Plan(expert_ids, self.world, self.rank, self.per_rank)
        return _DispatchFn.apply(x, weights, expert_ids, self)

    def combine(self, y):
        if self._used_fallback:
            return self._fallback.combine(y)
        return _CombineFn.apply(y, self)
