"""Mixture-of-experts token routing ops.

Semantics of the reference ops (``steptronoss/model/utils/moe_utils.py:85-453``): ``histogram``
(ids equal to -1 are ignored), ``index_compute`` (stable expert-major position of every
(token, k) slot), ``moe_scatter`` (copy rows into expert-major order), ``moe_weighted_gather``
(``out[t] = sum_k w[t,k] * y[pos[t,k]]``) and their composition ``routed_grouped_ffn``.

Differences that follow from the grouped tcgen05 GEMM: every expert's segment starts at a multiple
of 128 rows and padding rows are zero (one row tile = one expert, whole 64-row reduction blocks),
and all sizes stay on the device: the expert-major buffer has a static worst-case row count, so no
``.item()`` / ``batch_sizes.tolist()`` synchronisation remains.
"""
from __future__ import annotations

import itertools

import torch

from ..utils.optimizable import optimizable
from . import native
from .fused import swiglu
from .gemm import count_launch
from .grouped import SEGMENT_ALIGNMENT, grouped_gemm_reduce, grouped_gemm_rows, tile_groups_from_offsets


@optimizable(native_names=("triton",))
def histogram(ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Count of every expert id in ``ids``; entries equal to -1 (foreign experts) are ignored."""
    flat = ids.reshape(-1)
    valid = flat >= 0
    return torch.bincount(torch.where(valid, flat, torch.zeros_like(flat)), weights=valid.to(torch.float32),
                          minlength=num_experts)[:num_experts].to(torch.int32)


def padded_rows(num_slots: int, num_experts: int) -> int:
    """Static upper bound of the expert-major buffer height (multiple of 128)."""
    worst = num_slots + num_experts * (SEGMENT_ALIGNMENT - 1)
    return (worst + SEGMENT_ALIGNMENT - 1) // SEGMENT_ALIGNMENT * SEGMENT_ALIGNMENT


@optimizable(native_names=("triton",))
def index_compute(ids: torch.Tensor, num_experts: int):
    """Destination row of every (token, k) slot in the expert-major buffer.

    Returns ``(dest [T,k] int64 with -1 for ignored slots, offsets [E+1] int32 aligned segment
    starts, counts [E] int32)``.  Inside an expert the slots keep their token order (stable)."""
    T, K = ids.shape
    flat = ids.reshape(-1).to(torch.int64)
    valid = flat >= 0
    key = torch.where(valid, flat, torch.full_like(flat, num_experts))
    order = torch.sort(key, stable=True).indices
    counts = torch.bincount(key, minlength=num_experts + 1)[:num_experts]
    aligned = (counts + SEGMENT_ALIGNMENT - 1) // SEGMENT_ALIGNMENT * SEGMENT_ALIGNMENT
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=ids.device)
    offsets[1:] = torch.cumsum(aligned, 0)
    starts_sorted = torch.zeros(num_experts + 1, dtype=torch.int64, device=ids.device)
    starts_sorted[1:] = torch.cumsum(counts, 0)
    sorted_key = key[order]
    rank = torch.arange(flat.numel(), device=ids.device) - starts_sorted[sorted_key.clamp(max=num_experts)]
    dest_sorted = torch.where(sorted_key < num_experts, offsets[sorted_key.clamp(max=num_experts - 1)] + rank,
                              torch.full_like(rank, -1))
    dest = torch.empty_like(dest_sorted)
    dest[order] = dest_sorted
    return dest.view(T, K), offsets.to(torch.int32), counts.to(torch.int32)


def _native_rows(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.shape[1] % 8 == 0 and native.available()


class RoutePlan:
    """Everything the routed FFN needs about one routing decision, computed by three small launches (chunk
    histograms, scan, stable ranks) without a sort or a host synchronisation.

    ``dest [T,k]`` int64 (-1 = ignored slot), ``offsets [E+1]`` int32 (128-aligned segment starts),
    ``counts [E]`` int32, ``tile_group [rows/128]`` int32 (expert of every 128-row tile, -1 past the last
    segment), ``slot_of_row [rows]`` int32 (flat slot index ``t*k + j`` held by every row, -1 = padding)."""

    __slots__ = ("dest", "offsets", "counts", "tile_group", "slot_of_row", "rows", "num_experts")

    def __init__(self, ids: torch.Tensor, num_experts: int, rows: int | None = None):
        T, K = ids.shape
        self.num_experts = num_experts
        self.rows = padded_rows(T * K, num_experts) if rows is None else rows
        dev = ids.device
        if ids.is_cuda and num_experts <= 1024 and native.available():
            lib = native.load()
            ids64 = ids.to(torch.int64).contiguous()
            n_tiles = self.rows // SEGMENT_ALIGNMENT
            self.dest = torch.empty((T, K), dtype=torch.int64, device=dev)
            meta = torch.empty(2 * num_experts + 1 + n_tiles + self.rows, dtype=torch.int32, device=dev)
            self.offsets, self.counts, self.tile_group, self.slot_of_row = meta.split(
                [num_experts + 1, num_experts, n_tiles, self.rows])
            scratch = torch.empty(max(lib.stb_moe_index_chunks(T * K), 1) * num_experts, dtype=torch.int32, device=dev)
            rc = lib.stb_moe_index(ids64.data_ptr(), T * K, num_experts, self.rows, self.dest.data_ptr(),
                                   self.offsets.data_ptr(), self.counts.data_ptr(), self.tile_group.data_ptr(), n_tiles,
                                   self.slot_of_row.data_ptr(), scratch.data_ptr(),
                                   native.status_word(dev).data_ptr(), native.stream())
            native.check(rc, "moe_index")
            count_launch(3)
        else:
            self.dest, self.offsets, self.counts = index_compute(ids, num_experts)
            self.tile_group = tile_groups_from_offsets(self.offsets, self.rows) if ids.is_cuda else None
            self.slot_of_row = slot_of_row_from_dest(self.dest, self.rows)


def slot_of_row_from_dest(dest: torch.Tensor, rows: int) -> torch.Tensor:
    """Inverse of ``dest``: flat slot index held by every expert-major row, -1 for padding rows."""
    d = dest.reshape(-1)
    inv = torch.full((rows + 1,), -1, dtype=torch.int32, device=dest.device)
    inv.scatter_(0, torch.where(d >= 0, d, torch.full_like(d, rows)),
                 torch.where(d >= 0, torch.arange(d.numel(), device=d.device, dtype=torch.int32),
                             torch.full((d.numel(),), -1, dtype=torch.int32, device=d.device)))
    return inv[:rows]


class _ScatterFn(torch.autograd.Function):
    """rows of x copied to ``dest`` (one copy per slot); backward sums the k copies of each token."""

    @staticmethod
    def forward(ctx, x, dest, rows, plan=None):
        T, K = dest.shape
        if plan is not None and _native_rows(x):
            x = x.contiguous()
            out = torch.empty((rows, x.shape[1]), dtype=x.dtype, device=x.device)
            rc = native.load().stb_moe_scatter(x.data_ptr(), plan.slot_of_row.data_ptr(), plan.offsets.data_ptr(),
                                               plan.num_experts, K, x.shape[1], rows, out.data_ptr(), native.stream())
            native.check(rc, "moe_scatter")
            count_launch()
            ctx.save_for_backward(dest)
            ctx.t, ctx.native = T, True
            return out
        ctx.native = False
        out = torch.zeros((rows, x.shape[1]), dtype=x.dtype, device=x.device)
        d = dest.reshape(-1)
        valid = d >= 0
        src = torch.arange(T, device=x.device).repeat_interleave(K)
        out.index_copy_(0, d[valid], x.index_select(0, src[valid]))
        ctx.save_for_backward(dest)
        ctx.t = T
        return out

    @staticmethod
    def backward(ctx, g):
        (dest,) = ctx.saved_tensors
        T, K = dest.shape
        if ctx.native:
            g = g.contiguous()
            dx = torch.empty((T, g.shape[1]), dtype=g.dtype, device=g.device)
            rc = native.load().stb_moe_gather(g.data_ptr(), dest.data_ptr(), None, T, K, g.shape[1], dx.data_ptr(),
                                              native.stream())
            native.check(rc, "moe_scatter_bwd")
            count_launch()
            return dx, None, None, None
        d = dest.reshape(-1)
        valid = (d >= 0).unsqueeze(-1)
        picked = g.index_select(0, d.clamp(min=0)).float() * valid
        return picked.view(T, K, -1).sum(1).to(g.dtype), None, None, None


def _moe_scatter_reference_alt(x, dest, rows, plan=None):
    return _ScatterFn.apply(x, dest, rows, None)


@optimizable({"reference": _moe_scatter_reference_alt}, native_names=("triton",))
def moe_scatter(x, dest, rows, plan: RoutePlan | None = None):
    """Copy the rows of ``x`` into expert-major order.  With a ``plan`` (bf16 on the GPU) one kernel writes
    every used row exactly once, padding rows as zeros; rows past the last segment stay unwritten."""
    return _ScatterFn.apply(x, dest, rows, plan)


class _WeightedGatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, dest, weights, plan=None):
        T, K = dest.shape
        ctx.plan = None
        if plan is not None and _native_rows(y) and K <= 16:
            y = y.contiguous()
            w32 = weights.to(torch.float32).contiguous()
            out = torch.empty((T, y.shape[1]), dtype=y.dtype, device=y.device)
            rc = native.load().stb_moe_gather(y.data_ptr(), dest.data_ptr(), w32.data_ptr(), T, K, y.shape[1],
                                              out.data_ptr(), native.stream())
            native.check(rc, "moe_gather")
            count_launch()
            ctx.save_for_backward(y, dest, w32)
            ctx.plan, ctx.w_dtype = plan, weights.dtype
            return out
        d = dest.reshape(-1)
        valid = (d >= 0).view(T, K, 1)
        picked = y.index_select(0, d.clamp(min=0)).view(T, K, -1).float() * valid
        out = (picked * weights.float().unsqueeze(-1)).sum(1).to(y.dtype)
        ctx.save_for_backward(y, dest, weights)
        return out

    @staticmethod
    def backward(ctx, g):
        y, dest, weights = ctx.saved_tensors
        T, K = dest.shape
        if ctx.plan is not None:
            plan, g = ctx.plan, g.contiguous()
            gy = torch.empty_like(y)
            gw = torch.empty((T, K), dtype=torch.float32, device=y.device)
            rc = native.load().stb_moe_gather_bwd(g.data_ptr(), y.data_ptr(), dest.data_ptr(), weights.data_ptr(),
                                                  plan.slot_of_row.data_ptr(), plan.offsets.data_ptr(),
                                                  plan.num_experts, T, K, y.shape[1], y.shape[0], gy.data_ptr(),
                                                  gw.data_ptr(), native.stream())
            native.check(rc, "moe_gather_bwd")
            count_launch()
            return gy, None, gw.to(ctx.w_dtype), None
        d = dest.reshape(-1)
        validf = (d >= 0)
        gy = torch.zeros_like(y)
        contrib = (g.float().unsqueeze(1) * weights.float().unsqueeze(-1)).view(T * K, -1)
        gy.index_copy_(0, d[validf], contrib[validf].to(y.dtype))
        picked = y.index_select(0, d.clamp(min=0)).view(T, K, -1).float() * validf.view(T, K, 1)
        gw = (picked * g.float().unsqueeze(1)).sum(-1).to(weights.dtype)
        return gy, None, gw, None


def _moe_gather_reference_alt(y, dest, weights, plan=None):
    return _WeightedGatherFn.apply(y, dest, weights, None)


@optimizable({"reference": _moe_gather_reference_alt}, native_names=("triton",))
def moe_weighted_gather(y, dest, weights, plan: RoutePlan | None = None):
    """``out[t] = sum_k weights[t,k] * y[dest[t,k]]`` (ignored slots contribute nothing)."""
    return _WeightedGatherFn.apply(y, dest, weights, plan)


class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, top_k, sigmoid, norm_topk, eps):
        lib = native.load()
        logits = logits.contiguous()
        T, E = logits.shape
        dev = logits.device
        grid = lib.stb_router_grid(T)
        ids = torch.empty((T, top_k), dtype=torch.int64, device=dev)
        weights = torch.empty((T, top_k), dtype=torch.float32, device=dev)
        part_prob = torch.empty((grid, E), dtype=torch.float32, device=dev)
        part_hist = torch.empty((grid, E), dtype=torch.int32, device=dev)
        part_stats = torch.empty((grid, 2), dtype=torch.float32, device=dev)
        b = None if bias is None else bias.to(torch.float32).contiguous()
        rc = lib.stb_router_fwd(logits.data_ptr(), native.ptr(b), T, E, top_k, int(sigmoid), int(norm_topk), float(eps),
                                ids.data_ptr(), weights.data_ptr(), part_prob.data_ptr(), part_hist.data_ptr(),
                                part_stats.data_ptr(), native.stream())
        native.check(rc, "router_fwd")
        count_launch()
        ctx.save_for_backward(logits, ids)
        ctx.cfg = (top_k, int(sigmoid), int(norm_topk), float(eps))
        # one launch adds up the per-CTA partials; stats also carries the busiest expert's share of the slots
        prob_sum = torch.empty(E, dtype=torch.float32, device=dev)
        hist = torch.empty(E, dtype=torch.int32, device=dev)
        hist_f = torch.empty(E, dtype=torch.float32, device=dev)
        stats = torch.empty(3, dtype=torch.float32, device=dev)
        rc = lib.stb_router_finalize(part_prob.data_ptr(), part_hist.data_ptr(), part_stats.data_ptr(), grid, E, T,
                                     prob_sum.data_ptr(), hist.data_ptr(), hist_f.data_ptr(), stats.data_ptr(),
                                     native.stream())
        native.check(rc, "router_finalize")
        count_launch()
        ctx.mark_non_differentiable(ids, hist, stats)
        return ids, weights, prob_sum, hist, stats

    @staticmethod
    def backward(ctx, _g_ids, g_w, g_ps, _g_hist, _g_stats):
        logits, ids = ctx.saved_tensors
        top_k, sigmoid, norm_topk, eps = ctx.cfg
        T, E = logits.shape
        g_w = torch.zeros((T, top_k), dtype=torch.float32, device=logits.device) if g_w is None else g_w.float().contiguous()
        g_ps = None if g_ps is None else g_ps.float().contiguous()
        dlogits = torch.empty_like(logits)
        rc = native.load().stb_router_bwd(logits.data_ptr(), T, E, top_k, sigmoid, norm_topk, eps, ids.data_ptr(),
                                          g_w.data_ptr(), native.ptr(g_ps), dlogits.data_ptr(), native.stream())
        native.check(rc, "router_bwd")
        count_launch()
        return dlogits, None, None, None, None, None


def router_native_ok(logits: torch.Tensor, top_k: int) -> bool:
    return (logits.is_cuda and logits.dim() == 2 and logits.shape[1] <= 512 and top_k <= min(32, logits.shape[1])
            and native.available())


def _router_reference_alt(*a, **k):
    return router_reference(*a, **k)


@optimizable({"reference": _router_reference_alt})
def fused_router(logits, bias, top_k: int, sigmoid: bool, norm_topk: bool, eps: float):
    """Scores, top-k and the per-expert sums of the auxiliary loss in one kernel (one warp per token).

    ``logits [T,E]`` fp32.  Returns ``ids [T,k]`` int64 (order and tie-break of a stable descending sort of
    ``prob + bias``), ``weights [T,k]`` fp32, ``prob_sum [E]`` (sum over tokens of the probabilities, for sigmoid
    scores of the probabilities renormalised per token), ``hist [E]`` int32 and ``stats = [max |logit|,
    mean over tokens of the largest probability, share of the busiest expert in the routed slots]``.  ``weights`` and ``prob_sum`` are differentiable."""
    return _RouterFn.apply(logits.float(), bias, top_k, sigmoid, norm_topk, eps)


def router_reference(logits, bias, top_k: int, sigmoid: bool, norm_topk: bool, eps: float):
    """The same quantities with plain tensor ops (oracle and CPU path)."""
    logits = logits.float()
    prob = torch.sigmoid(logits) if sigmoid else torch.softmax(logits, dim=1)
    select = prob + bias.float().unsqueeze(0) if bias is not None else prob
    ids = torch.sort(select, dim=1, descending=True, stable=True).indices[:, :top_k].contiguous()
    top = prob.gather(1, ids)
    weights = top
    if sigmoid:
        weights = top / (top.sum(-1, keepdim=True) + eps)
        prob = prob / (prob.sum(-1, keepdim=True) + eps)
    elif norm_topk:
        weights = top / (top.sum(-1, keepdim=True) + eps)
    hist = histogram(ids, logits.shape[1])
    stats = torch.stack([logits.detach().abs().max(), (torch.sigmoid(logits) if sigmoid else torch.softmax(logits, 1))
                         .detach().max(1).values.mean(), hist.max().float() / hist.sum().clamp_min(1).float()])
    return ids, weights, prob.sum(0), hist, stats


class _GroupedLinearFn(torch.autograd.Function):
    """Per-expert ``x_g @ w[g].T`` over expert-major rows; wgrad accumulates into ``w.main_grad``."""

    @staticmethod
    def forward(ctx, x, w, offsets, tile_group=None, fp8=False):
        if tile_group is None and x.is_cuda:
            tile_group = tile_groups_from_offsets(offsets, x.shape[0])
        if fp8 and x.is_cuda and x.shape[1] % 128 == 0 and w.shape[1] % 128 == 0 and x.dtype == torch.bfloat16:
            # forward product in block-scaled e4m3 (1 x 128 activation, 128 x 128 weight scales); the backward
            # products below stay in bf16 on the saved bf16 operands
            from . import fp8 as fp8_ops

            xq, sx = fp8_ops.quantize_rows_1x128(x)
            wq, sw = fp8_ops.quantize_blocks_128x128(w.reshape(w.shape[0] * w.shape[1], w.shape[2]))
            y = fp8_ops.grouped_gemm_fp8(xq, sx, wq, sw, offsets, w.shape[0], tile_group=tile_group)
        else:
            y = grouped_gemm_rows(x, w, offsets, trans_b=True, tile_group=tile_group)
        ctx.save_for_backward(x, w, offsets, tile_group if tile_group is not None else offsets)
        ctx.w_ref = w
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w, offsets, tile_group = ctx.saved_tensors
        gy = gy.contiguous()
        G = w.shape[0]
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = grouped_gemm_rows(gy, w, offsets, trans_b=False, tile_group=tile_group if x.is_cuda else None)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(ctx.w_ref, "main_grad", None)
            if main_grad is not None and x.is_cuda:
                grouped_gemm_reduce(gy, x, offsets, G, out=main_grad, accumulate=True)
                ctx.w_ref.grad_added_to_main_grad = True
            else:
                dw = grouped_gemm_reduce(gy, x, offsets, G)
        return dx, dw, None, None, None


def grouped_linear(x, w, offsets, tile_group=None, fp8: bool = False):
    return _GroupedLinearFn.apply(x, w, offsets, tile_group, fp8)


def _grouped_gemm_loop(mat_a_flat, mat_b, batch_sizes, trans_b: bool = False):
    outs, start = [], 0
    for g, n in enumerate(int(b) for b in batch_sizes.tolist()):
        rhs = mat_b[g].t() if trans_b else mat_b[g]
        outs.append(mat_a_flat[start:start + n] @ rhs)
        start += n
    if not outs:
        return mat_a_flat.new_zeros((0, mat_b.shape[1] if trans_b else mat_b.shape[2]))
    return torch.cat(outs, 0)


@optimizable({"function_imple": _grouped_gemm_loop, "reference": _grouped_gemm_loop},
             native_names=("nv_grouped_gemm", "triton_grouped_gemm"))
def grouped_gemm(mat_a_flat, mat_b, batch_sizes, trans_b: bool = False):
    """The reference's grouped-GEMM entry (model/utils/moe_utils.py:435-453): rows of ``mat_a_flat [sum, K]`` in
    consecutive groups of ``batch_sizes[g]`` rows, ``mat_b [G, N, K]`` (``trans_b``) or ``[G, K, N]``.

    The sizes are read on the host, as the reference's back-ends do.  Groups whose sizes are all multiples of 128
    with ``trans_b``, an output width that is a multiple of 128 and bf16 operands on the GPU run as one grouped tcgen05 GEMM (differentiable, weight gradient
    by the grouped reduce kernel); anything else runs one product per group.  The model path does not come through
    here: ``routed_grouped_ffn`` keeps its offsets on the device."""
    sizes = [int(b) for b in batch_sizes.tolist()]
    if (trans_b and sizes and _native_rows(mat_a_flat) and mat_b.dtype == torch.bfloat16 and mat_b.is_contiguous()
            and all(n % SEGMENT_ALIGNMENT == 0 for n in sizes) and mat_a_flat.shape[1] % 8 == 0
            and mat_b.shape[1] % 128 == 0):        # an output tile must not run into the next group's weights
        offsets = torch.tensor([0] + list(itertools.accumulate(sizes)), dtype=torch.int32, device=mat_a_flat.device)
        return grouped_linear(mat_a_flat.contiguous(), mat_b, offsets)
    return _grouped_gemm_loop(mat_a_flat, mat_b, batch_sizes, trans_b)


def _routed_ffn_reference_alt(x, expert_ids, weights, w1, w2, limit: float = 0.0, max_slots: int | None = None,
                              fp8: bool = False):
    return routed_grouped_ffn_reference(x, expert_ids, weights, w1, w2, limit)


@optimizable({"reference": _routed_ffn_reference_alt})
def routed_grouped_ffn(x, expert_ids, weights, w1, w2, limit: float = 0.0, max_slots: int | None = None,
                       fp8: bool = False):
    """Top-k routed SwiGLU experts on one rank.

    ``x [T,H]``, ``expert_ids [T,k]`` (local expert index or -1), ``weights [T,k]``,
    ``w1 [E, 2F, H]`` (gate | up), ``w2 [E, H, F]``.  Returns ``[T,H]``.  ``max_slots``: an upper bound of the
    slots with an id >= 0 when the caller knows one (rows of a sparse receive buffer); it sizes the expert-major
    buffers, which otherwise take the worst case ``T*k``.  ``fp8``: forward products of both expert GEMMs in
    block-scaled e4m3 (``ops/fp8.py``), backward in bf16."""
    E = w1.shape[0]
    T, K = expert_ids.shape
    if _native_rows(x) and K <= 16:
        plan = RoutePlan(expert_ids, E, None if max_slots is None else padded_rows(min(max_slots, T * K), E))
        xe = moe_scatter(x, plan.dest, plan.rows, plan)
        h = grouped_linear(xe, w1, plan.offsets, plan.tile_group, fp8)
        a = swiglu(h, limit)
        y = grouped_linear(a, w2, plan.offsets, plan.tile_group, fp8)
        return moe_weighted_gather(y, plan.dest, weights, plan)
    dest, offsets, _ = index_compute(expert_ids, E)
    rows = padded_rows(T * K, E)
    xe = moe_scatter(x, dest, rows)
    h = grouped_linear(xe, w1, offsets)
    a = swiglu(h, limit)
    y = grouped_linear(a, w2, offsets)
    return moe_weighted_gather(y, dest, weights)


def routed_grouped_ffn_reference(x, expert_ids, weights, w1, w2, limit: float = 0.0):
    """Plain loop over experts (oracle)."""
    from .fused import swiglu_reference

    out = torch.zeros_like(x, dtype=torch.float32)
    E = w1.shape[0]
    for e in range(E):
        tok, slot = (expert_ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = x[tok].float() @ w1[e].float().t()
        a = swiglu_reference(h, limit)
        y = a @ w2[e].float().t()
        out.index_add_(0, tok, y * weights[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)


# the reference's names for the autograd functions behind the three movers (model/utils/moe_utils.py)
MoEGateFunction, MoEScatter, MoEWeightedGather = _RouterFn, _ScatterFn, _WeightedGatherFn
