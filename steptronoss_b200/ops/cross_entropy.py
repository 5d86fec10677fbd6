"""Vocab-parallel cross-entropy, standalone and fused with the LM-head projection.

Semantics of the reference (``steptronoss/core/tensor_parallel/cross_entropy.py:28-166``): logits
are sharded over the vocabulary across the TP group; the row max, the target logit and the sum of
exponentials are reduced over the group; the per-token loss and the arg-max accuracy are returned.

The fused form never materialises fp32 logits: for each block of tokens the bf16 logits shard is
produced by the tcgen05 GEMM, reduced to ``(max, sumexp, target)`` by one kernel, turned in place
into its own gradient by a second kernel, and immediately consumed by the dgrad and wgrad GEMMs.
The loss therefore comes out of the forward pass together with ``dL/dh`` and ``dL/dW``; backward
only rescales them by the incoming gradient.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import native
from .gemm import count_launch, gemm


def _all_reduce(t, op, group):
    if group is not None and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=op, group=group)
    return t


class _VocabParallelCEFn(torch.autograd.Function):
    """PyTorch statement (any device): per-token loss from a vocab shard of logits."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_start, group, label_smoothing=0.0):
        lf = logits.float()
        V = lf.shape[-1]
        m = _all_reduce(lf.max(dim=-1).values, dist.ReduceOp.MAX, group)
        lf = lf - m.unsqueeze(-1)
        local = labels - vocab_start
        inside = (local >= 0) & (local < V)
        safe = local.masked_fill(~inside, 0)
        tgt = lf.gather(-1, safe.unsqueeze(-1)).squeeze(-1).masked_fill(~inside, 0.0)
        tgt = _all_reduce(tgt, dist.ReduceOp.SUM, group)
        ex = lf.exp()
        se = _all_reduce(ex.sum(-1), dist.ReduceOp.SUM, group)
        loss = se.log() - tgt
        softmax = ex / se.unsqueeze(-1)
        ctx.smoothing, ctx.vocab = 0.0, V
        if label_smoothing > 0:
            # (1 - a) on the label and a / (K - 1) on every other class, K = the whole vocabulary:
            # loss = (1 - s) * nll - s * mean_i log p_i  with  s = a * K / (K - 1)
            if not label_smoothing < 1.0:
                raise ValueError("label_smoothing must be in [0, 1)")
            K = V * (dist.get_world_size(group) if group is not None else 1)
            s = label_smoothing * K / (K - 1)
            mean_logp = _all_reduce(lf.sum(-1), dist.ReduceOp.SUM, group) / K - se.log()
            loss = (1.0 - s) * loss - s * mean_logp
            ctx.smoothing, ctx.vocab = s, K
        ctx.save_for_backward(softmax, inside, safe)
        ctx.in_dtype = logits.dtype
        # accuracy: global arg-max equals the label
        lmax, larg = lf.max(dim=-1)
        best = _all_reduce(lmax.clone(), dist.ReduceOp.MAX, group)
        cand = torch.where(lmax == best, larg + vocab_start, torch.full_like(larg, 2**62))
        cand = _all_reduce(cand, dist.ReduceOp.MIN, group)
        ctx.mark_non_differentiable(cand)
        return loss, cand

    @staticmethod
    def backward(ctx, gloss, _gc):
        softmax, inside, safe = ctx.saved_tensors
        grad = softmax.clone()
        onehot = torch.zeros_like(grad)
        onehot.scatter_(-1, safe.unsqueeze(-1), inside.unsqueeze(-1).to(grad.dtype))
        if ctx.smoothing:
            grad = grad - (1.0 - ctx.smoothing) * onehot - ctx.smoothing / ctx.vocab
        else:
            grad = grad - onehot
        grad = grad * gloss.unsqueeze(-1)
        return grad.to(ctx.in_dtype), None, None, None, None


def vocab_parallel_cross_entropy(logits, labels, vocab_start: int = 0, group=None, label_smoothing: float = 0.0):
    """Per-token loss ``[...]`` and arg-max prediction from (a vocab shard of) ``logits [..., V_local]``.

    ``label_smoothing`` spreads that much probability over the other classes of the WHOLE vocabulary (the
    reference counts only the classes of the local shard, ``cross_entropy.py:91-108``; the two agree at TP=1)."""
    return _VocabParallelCEFn.apply(logits, labels, vocab_start, group, label_smoothing)


class _FusedLinearCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels, weights, vocab_start, group, chunk):
        lib = native.load()
        T, H = h.shape
        V = w.shape[0]
        dev = h.device
        need_dh = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        loss_tok = torch.empty(T, dtype=torch.float32, device=dev)
        pred = torch.empty(T, dtype=torch.int64, device=dev)
        dh = torch.empty((T, H), dtype=torch.float32, device=dev) if need_dh else None
        main_grad = getattr(w, "main_grad", None)
        if need_dw:
            dw = main_grad if main_grad is not None else torch.zeros((V, H), dtype=torch.float32, device=dev)
        else:
            dw = None
        multi = group is not None and dist.get_world_size(group) > 1
        st = native.stream()
        for t0 in range(0, T, chunk):
            t1 = min(T, t0 + chunk)
            n = t1 - t0
            hc = h[t0:t1]
            lab = labels[t0:t1].contiguous()
            logits = gemm(hc, w)  # [n, V] bf16
            stats = torch.empty((n, 4), dtype=torch.float32, device=dev)
            amax = torch.empty(n, dtype=torch.int64, device=dev)
            native.check(lib.stb_ce_stats(logits.data_ptr(), lab.data_ptr(), stats.data_ptr(), amax.data_ptr(), n, V,
                                          logits.stride(0), vocab_start, st), "ce_stats")
            count_launch()
            lmax, lsum, ltgt = stats[:, 0], stats[:, 1], stats[:, 2]
            if multi:
                gmax = lmax.clone()
                dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
                pack = torch.stack([lsum * torch.exp(lmax - gmax), ltgt])
                dist.all_reduce(pack, op=dist.ReduceOp.SUM, group=group)
                gsum, gtgt = pack[0].contiguous(), pack[1]
                cand = torch.where(lmax == gmax, amax, torch.full_like(amax, 2**62))
                dist.all_reduce(cand, op=dist.ReduceOp.MIN, group=group)
                amax = cand
            else:
                gmax, gsum, gtgt = lmax.contiguous(), lsum.contiguous(), ltgt
            loss_tok[t0:t1] = torch.log(gsum) + gmax - gtgt
            pred[t0:t1] = amax
            if need_dh or need_dw:
                wt = weights[t0:t1].contiguous()
                native.check(lib.stb_ce_grad(logits.data_ptr(), lab.data_ptr(), gmax.data_ptr(), gsum.data_ptr(),
                                             wt.data_ptr(), n, V, logits.stride(0), vocab_start, st), "ce_grad")
                count_launch()
                if need_dh:
                    gemm(logits, w, b_mn_major=True, out=dh[t0:t1])
                if need_dw:
                    gemm(logits, hc, a_mn_major=True, b_mn_major=True, out=dw, accumulate=True)
        loss = (loss_tok * weights).sum()
        ctx.save_for_backward(dh if dh is not None else torch.empty(0, device=dev))
        ctx.dw = None if (dw is None or main_grad is not None) else dw
        ctx.w_ref = w
        ctx.used_main_grad = need_dw and main_grad is not None
        ctx.h_dtype = h.dtype
        ctx.mark_non_differentiable(loss_tok, pred)
        return loss, loss_tok, pred

    @staticmethod
    def backward(ctx, gloss, _g1, _g2):
        (dh,) = ctx.saved_tensors
        gh = gw = None
        if ctx.needs_input_grad[0]:
            gh = (dh * gloss).to(ctx.h_dtype)
        if ctx.needs_input_grad[1]:
            if ctx.used_main_grad:
                # dW already sits in main_grad with unit upstream gradient: the loss returned by this
                # function has to be the quantity that backward() is called on.
                ctx.w_ref.grad_added_to_main_grad = True
            else:
                gw = (ctx.dw * gloss).to(ctx.w_ref.dtype)
        return gh, gw, None, None, None, None, None


def fused_linear_cross_entropy(h, w, labels, weights, vocab_start: int = 0, group=None, chunk_tokens: int = 2048):
    """``sum_t weights[t] * CE(h[t] @ w.T, labels[t])`` with vocab-parallel ``w``.

    Returns ``(weighted loss sum, per-token loss, arg-max prediction)``; the last two carry no
    gradient.  ``weights`` holds the loss mask already divided by its normaliser (and by the number
    of micro-batches), so the returned scalar is what ``backward()`` is called on.
    """
    if not h.is_cuda:
        logits = torch.nn.functional.linear(h, w)
        loss_tok, pred = vocab_parallel_cross_entropy(logits, labels, vocab_start, group)
        return (loss_tok * weights).sum(), loss_tok.detach(), pred
    return _FusedLinearCEFn.apply(h, w, labels, weights, vocab_start, group, chunk_tokens)
