"""Expert-parallel token dispatch and combine.

Reference semantics (``steptronoss/model/ep_dispatcher/token_dispatcher.py:14-118``): a token is
sent once to every EP rank that hosts at least one of its top-k experts; it travels with its k
expert ids rewritten to local indices (-1 for experts of other ranks) and its k weights (0 for
foreign experts); the weighted sum over a token's local experts happens on the expert rank, so the
way back carries one partial row per (token, destination rank) that the source adds up.

``AllToAllDispatcher`` states this with two NCCL all-to-alls each way (one for the split sizes, one
for the payload packed as a single byte matrix: hidden row | ids | weights).  It works on gloo as
well, which is how the CPU tests run it.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..utils.optimizable import optimizable
from .state import PM


class _AllToAllRows(torch.autograd.Function):
    """Variable-split all-to-all over the first dimension; backward runs the inverse exchange."""

    @staticmethod
    def forward(ctx, x, send_counts, recv_counts, group):
        ctx.group, ctx.send_counts, ctx.recv_counts = group, send_counts, recv_counts
        out = torch.empty((sum(recv_counts), *x.shape[1:]), dtype=x.dtype, device=x.device)
        _a2a(out, x.contiguous(), recv_counts, send_counts, group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty((sum(ctx.send_counts), *g.shape[1:]), dtype=g.dtype, device=g.device)
        _a2a(out, g.contiguous(), ctx.send_counts, ctx.recv_counts, ctx.group)
        return out, None, None, None


def _a2a(out, inp, out_splits, in_splits, group):
    if dist.get_backend(group) == "gloo":
        # gloo has no all-to-all: pairwise send/recv (CPU tests only)
        n = dist.get_world_size(group)
        me = dist.get_rank(group)
        in_off = [0]
        out_off = [0]
        for a, b in zip(in_splits, out_splits):
            in_off.append(in_off[-1] + a)
            out_off.append(out_off[-1] + b)
        reqs, recv_bufs = [], {}
        for j in range(n):
            if j == me:
                out[out_off[j]:out_off[j + 1]].copy_(inp[in_off[j]:in_off[j + 1]])
                continue
            peer = dist.get_global_rank(group, j)
            if in_splits[j]:
                reqs.append(dist.isend(inp[in_off[j]:in_off[j + 1]].contiguous(), dst=peer, group=group))
            if out_splits[j]:
                recv_bufs[j] = torch.empty((out_splits[j], *out.shape[1:]), dtype=out.dtype)
                reqs.append(dist.irecv(recv_bufs[j], src=peer, group=group))
        for r in reqs:
            r.wait()
        for j, buf in recv_bufs.items():
            out[out_off[j]:out_off[j + 1]].copy_(buf)
        return
    dist.all_to_all_single(out, inp, out_splits, in_splits, group=group)


class AllToAllDispatcher:
    def __init__(self, group_name: str, num_experts: int):
        self.group_name = group_name
        self.num_experts = num_experts
        self.world = PM.size_of(group_name)
        self.rank = PM.rank_in(group_name)
        self.per_rank = num_experts // self.world
        self._state = None

    def dispatch(self, x, expert_ids, weights):
        """x ``[T,H]``, expert_ids ``[T,k]`` global, weights ``[T,k]`` -> rows received by this rank:
        ``(x' [R,H], local ids [R,k] with -1 for foreign experts, weights' [R,k])``."""
        group = PM.group_of(self.group_name)
        T, K = expert_ids.shape
        dest_rank = expert_ids // self.per_rank                                      # [T,k]
        hits = torch.zeros((T, self.world), dtype=torch.bool, device=x.device)
        hits.scatter_(1, dest_rank.clamp(0, self.world - 1), expert_ids >= 0)
        send_counts_t = hits.sum(0)
        # rows ordered by destination rank, token order inside a rank (stable)
        tok = hits.t().nonzero(as_tuple=False)                                     # [(rank, token)]
        token_of_row = tok[:, 1]
        rank_of_row = tok[:, 0]
        counts = torch.empty(self.world, dtype=torch.int64, device=x.device)
        _a2a(counts, send_counts_t.to(torch.int64), [1] * self.world, [1] * self.world, group)
        send_counts = send_counts_t.tolist()   # host sync: sizes of the variable all-to-all
        recv_counts = counts.tolist()
        xs = x.index_select(0, token_of_row)
        ids_s = expert_ids.index_select(0, token_of_row)
        w_s = weights.index_select(0, token_of_row)
        local = ids_s - rank_of_row.unsqueeze(1) * self.per_rank
        foreign = (local < 0) | (local >= self.per_rank) | (ids_s < 0)
        local = torch.where(foreign, torch.full_like(local, -1), local)
        w_s = torch.where(foreign, torch.zeros_like(w_s), w_s)
        xr = _AllToAllRows.apply(xs, send_counts, recv_counts, group)
        wr = _AllToAllRows.apply(w_s, send_counts, recv_counts, group)
        ids_r = torch.empty((sum(recv_counts), K), dtype=local.dtype, device=x.device)
        _a2a(ids_r, local.contiguous(), recv_counts, send_counts, group)
        self._state = (token_of_row, send_counts, recv_counts, T)
        return xr, ids_r, wr

    def combine(self, y):
        """Partial outputs ``[R,H]`` back to their source ranks, summed per token -> ``[T,H]``."""
        token_of_row, send_counts, recv_counts, T = self._state
        group = PM.group_of(self.group_name)
        back = _AllToAllRows.apply(y, recv_counts, send_counts, group)
        out = torch.zeros((T, y.shape[1]), dtype=torch.float32, device=y.device)
        out = out.index_add(0, token_of_row, back.float())
        return out.to(y.dtype)


def _peer_token_dispatcher(parallel: str, num_experts: int):
    from .peer_dispatcher import PeerMemoryDispatcher

    return PeerMemoryDispatcher(parallel, num_experts)


@optimizable({"deep_ep": _peer_token_dispatcher, "peer": _peer_token_dispatcher})
def TokenDispatcher(parallel: str, num_experts: int):
    """The dispatcher of the expert-parallel family ``parallel`` under the reference's name and constructor
    (model/ep_dispatcher/token_dispatcher.py:14-25): ``dispatch(hidden, expert_ids, weights)`` /
    ``combine(hidden)`` over all-to-alls.  ``set_optimization(TokenDispatcher="deep_ep")`` - the reference's switch to
    its NVLink dispatcher - returns the peer-memory dispatcher instead; ``MoEConfig.dispatcher`` set to anything but
    the default overrides the switch."""
    return AllToAllDispatcher(parallel, num_experts)


PEER_KINDS = ("peer", "deepep", "nvlink")           # "deepep": the reference's name for its NVLink dispatcher
ALLTOALL_KINDS = ("alltoall", "token", "nccl")      # "token": the reference's baseline TokenDispatcher


def build_dispatcher(kind: str, group_name: str, num_experts: int, capacity_factor: float | None = None):
    kind = str(kind).lower()
    if kind not in PEER_KINDS + ALLTOALL_KINDS:
        raise ValueError(f"unknown MoE dispatcher {kind!r}; choose from {PEER_KINDS + ALLTOALL_KINDS}")
    if kind in PEER_KINDS:
        from .peer_dispatcher import PeerMemoryDispatcher

        return PeerMemoryDispatcher(group_name, num_experts, capacity_factor)
    if kind == "alltoall":          # the default: the registry switch of the reference's experiment files applies
        return TokenDispatcher(group_name, num_experts)
    return AllToAllDispatcher(group_name, num_experts)
