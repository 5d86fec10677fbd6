"""RMSNorm, QK-norm + RoPE, SwiGLU, embedding: autograd functions over the native kernels with
PyTorch restatements for CPU tensors (the restatements are also the oracles of the GPU tests).

Reference math: ``steptronoss/model/common/rms_norm.py:5-62``, ``rope.py:220-250``,
``feed_forward.py:20-26``, ``core/tensor_parallel/layers.py:120-139``.
"""
from __future__ import annotations

import torch

from . import native
from .gemm import count_launch


# --------------------------------------------------------------------------- RMSNorm
def rmsnorm_reference(x, weight, eps: float = 1e-6, zero_centered: bool = False):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    w = weight.float() + 1.0 if zero_centered else weight.float()
    return (xf * rstd * w).to(x.dtype)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, zero_centered):
        lib = native.load()
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty((rows, H), dtype=x.dtype, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        native.check(
            lib.stb_rmsnorm_fwd(x2.data_ptr(), weight.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, H,
                                x2.stride(0), y.stride(0), float(eps), int(zero_centered), native.stream()),
            "rmsnorm_fwd")
        count_launch()
        ctx.save_for_backward(x2, weight, rstd)
        ctx.weight_ref = weight
        ctx.zero_centered = zero_centered
        ctx.in_shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        lib = native.load()
        x2, weight, rstd = ctx.saved_tensors
        rows, H = x2.shape
        g2 = gy.reshape(rows, H)
        if g2.stride(-1) != 1:
            g2 = g2.contiguous()
        dx = torch.empty_like(x2)
        grid = lib.stb_rmsnorm_bwd_grid(rows)
        partial = torch.empty((grid, H), dtype=torch.float32, device=x2.device)
        main_grad = getattr(ctx.weight_ref, "main_grad", None)
        if main_grad is not None:
            dw_buf, acc = main_grad, 1
        else:
            dw_buf, acc = torch.empty(H, dtype=torch.float32, device=x2.device), 0
        native.check(
            lib.stb_rmsnorm_bwd(x2.data_ptr(), weight.data_ptr(), g2.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                dw_buf.data_ptr(), partial.data_ptr(), rows, H, x2.stride(0), g2.stride(0),
                                dx.stride(0), int(ctx.zero_centered), 0, acc, native.stream()),
            "rmsnorm_bwd")
        count_launch(2)
        dw = None
        if main_grad is None:
            dw = dw_buf.to(weight.dtype)
        else:
            ctx.weight_ref.grad_added_to_main_grad = True
        return dx.view(ctx.in_shape), dw, None, None


def rmsnorm(x, weight, eps: float = 1e-6, zero_centered: bool = False):
    if not x.is_cuda:
        return rmsnorm_reference(x, weight, eps, zero_centered)
    return _RMSNormFn.apply(x, weight, eps, zero_centered)


class _AddRMSNormFn(torch.autograd.Function):
    """``s = x + delta`` and ``y = rmsnorm(s)`` in one kernel (the residual add of a pre-norm block and the norm
    that follows it); backward adds the residual-stream gradient inside the norm's backward kernel."""

    @staticmethod
    def forward(ctx, x, delta, weight, eps, zero_centered):
        lib = native.load()
        H = x.shape[-1]
        x2, d2 = x.reshape(-1, H), delta.reshape(-1, H)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        if d2.stride(-1) != 1:
            d2 = d2.contiguous()
        rows = x2.shape[0]
        y = torch.empty((rows, H), dtype=x.dtype, device=x.device)
        s = torch.empty((rows, H), dtype=x.dtype, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        native.check(
            lib.stb_add_rmsnorm_fwd(x2.data_ptr(), d2.data_ptr(), weight.data_ptr(), y.data_ptr(), s.data_ptr(),
                                    rstd.data_ptr(), rows, H, x2.stride(0), d2.stride(0), y.stride(0), s.stride(0),
                                    float(eps), int(zero_centered), native.stream()),
            "add_rmsnorm_fwd")
        count_launch()
        ctx.save_for_backward(s, weight, rstd)
        ctx.weight_ref = weight
        ctx.zero_centered = zero_centered
        ctx.in_shape = x.shape
        return s.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, gs, gy):
        lib = native.load()
        s, weight, rstd = ctx.saved_tensors
        rows, H = s.shape
        g2, r2 = gy.reshape(rows, H), gs.reshape(rows, H)
        if g2.stride(-1) != 1:
            g2 = g2.contiguous()
        if r2.stride(-1) != 1:
            r2 = r2.contiguous()
        ds = torch.empty_like(s)
        grid = lib.stb_rmsnorm_bwd_grid(rows)
        partial = torch.empty((grid, H), dtype=torch.float32, device=s.device)
        main_grad = getattr(ctx.weight_ref, "main_grad", None)
        if main_grad is not None:
            dw_buf, acc = main_grad, 1
        else:
            dw_buf, acc = torch.empty(H, dtype=torch.float32, device=s.device), 0
        native.check(
            lib.stb_add_rmsnorm_bwd(s.data_ptr(), weight.data_ptr(), g2.data_ptr(), r2.data_ptr(), rstd.data_ptr(),
                                    ds.data_ptr(), dw_buf.data_ptr(), partial.data_ptr(), rows, H, s.stride(0),
                                    g2.stride(0), r2.stride(0), ds.stride(0), int(ctx.zero_centered), acc,
                                    native.stream()),
            "add_rmsnorm_bwd")
        count_launch(2)
        dw = None
        if main_grad is None:
            dw = dw_buf.to(weight.dtype)
        else:
            ctx.weight_ref.grad_added_to_main_grad = True
        ds = ds.view(ctx.in_shape)
        return ds, ds, dw, None, None


def add_rmsnorm(x, delta, weight, eps: float = 1e-6, zero_centered: bool = False):
    """``(x + delta, rmsnorm(x + delta))``: the residual stream and the input of the next sub-block."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or delta.dtype != x.dtype or delta.shape != x.shape:
        s = x + delta
        return s, rmsnorm(s, weight, eps, zero_centered)
    return _AddRMSNormFn.apply(x, delta, weight, eps, zero_centered)


class _AddFn(torch.autograd.Function):
    """bf16 ``a + b`` on the native kernel (the residual add that has no norm behind it)."""

    @staticmethod
    def forward(ctx, a, b):
        lib = native.load()
        a2, b2 = a.contiguous(), b.contiguous()
        out = torch.empty_like(a2)
        native.check(lib.stb_add_bf16(a2.data_ptr(), b2.data_ptr(), out.data_ptr(), a2.numel(), native.stream()), "add")
        count_launch()
        return out

    @staticmethod
    def backward(ctx, g):
        return g, g


def residual_add(a, b):
    if not a.is_cuda or a.dtype != torch.bfloat16 or b.dtype != a.dtype or a.shape != b.shape or a.numel() % 8:
        return a + b
    return _AddFn.apply(a, b)


# --------------------------------------------------------------------------- QK-norm + RoPE
def rope_tables(max_pos: int, rot_dim: int, theta: float, device, scaling=None):
    """fp32 cos/sin tables ``[max_pos, rot_dim/2]`` (kept fp32 whatever the model dtype, as the
    reference keeps its caches, ``rope.py:38-120``)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    if scaling is not None:
        inv_freq = scaling(inv_freq)
    t = torch.arange(max_pos, dtype=torch.float64)
    ang = torch.outer(t, inv_freq)
    return ang.cos().float().to(device), ang.sin().float().to(device)


def qknorm_rope_reference(qkv, q_weight, k_weight, cos, sin, pos, hq, hkv, head_dim, rot_dim=None,
                          eps=1e-6, use_norm=True, zero_centered=False):
    """qkv ``[T, (hq+2*hkv)*D]`` laid out ``[q | k | v]`` -> (q ``[T,hq,D]``, k ``[T,hkv,D]``, v view)."""
    T = qkv.shape[0]
    D = head_dim
    rot = rot_dim or D
    q = qkv[:, : hq * D].reshape(T, hq, D)
    k = qkv[:, hq * D : (hq + hkv) * D].reshape(T, hkv, D)
    v = qkv[:, (hq + hkv) * D :].reshape(T, hkv, D)

    def norm(x, w):
        if not use_norm:
            return x.float()
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        wf = w.float() + 1.0 if zero_centered else w.float()
        return xf * rstd * wf

    def rotate(x):
        c = cos[pos.long()].unsqueeze(1)  # [T,1,rot/2]
        s = sin[pos.long()].unsqueeze(1)
        x1, x2, rest = x[..., : rot // 2], x[..., rot // 2 : rot], x[..., rot:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)

    qo = rotate(norm(q, q_weight)).to(qkv.dtype)
    ko = rotate(norm(k, k_weight)).to(qkv.dtype)
    return qo, ko, v


class _QKNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, q_weight, k_weight, cos, sin, pos, hq, hkv, head_dim, rot, eps, use_norm, zero_centered):
        lib = native.load()
        T = qkv.shape[0]
        q = torch.empty((T, hq, head_dim), dtype=qkv.dtype, device=qkv.device)
        k = torch.empty((T, hkv, head_dim), dtype=qkv.dtype, device=qkv.device)
        rstd = torch.empty(T * (hq + hkv), dtype=torch.float32, device=qkv.device) if use_norm else None
        native.check(
            lib.stb_qknorm_rope_fwd(qkv.data_ptr(), native.ptr(q_weight), native.ptr(k_weight), cos.data_ptr(),
                                    sin.data_ptr(), pos.data_ptr(), q.data_ptr(), k.data_ptr(), native.ptr(rstd), T,
                                    hq, hkv, head_dim, qkv.stride(0), rot, float(eps), int(use_norm),
                                    int(zero_centered), native.stream()),
            "qknorm_rope_fwd")
        count_launch()
        v = qkv[:, (hq + hkv) * head_dim :].view(T, hkv, head_dim)
        ctx.save_for_backward(qkv, q_weight, k_weight, cos, sin, pos, rstd)
        ctx.params = (q_weight, k_weight)
        ctx.cfg = (hq, hkv, head_dim, rot, use_norm, zero_centered)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        lib = native.load()
        qkv, q_weight, k_weight, cos, sin, pos, rstd = ctx.saved_tensors
        hq, hkv, D, rot, use_norm, zero_centered = ctx.cfg
        T = qkv.shape[0]
        dqkv = torch.empty((T, (hq + 2 * hkv) * D), dtype=qkv.dtype, device=qkv.device)
        if dv is not None:
            dqkv[:, (hq + hkv) * D :].copy_(dv.reshape(T, hkv * D))
        else:
            dqkv[:, (hq + hkv) * D :].zero_()
        dq = dq.contiguous() if dq is not None else torch.zeros((T, hq, D), dtype=qkv.dtype, device=qkv.device)
        dk = dk.contiguous() if dk is not None else torch.zeros((T, hkv, D), dtype=qkv.dtype, device=qkv.device)
        grid = lib.stb_qknorm_rope_bwd_grid()
        partial = torch.empty((grid, 2, D), dtype=torch.float32, device=qkv.device)
        qp, kp = ctx.params
        dwq = dwk = None
        acc = 0
        if use_norm:
            mq, mk = getattr(qp, "main_grad", None), getattr(kp, "main_grad", None)
            if mq is not None and mk is not None:
                dwq, dwk, acc = mq, mk, 1
            else:
                dwq = torch.empty(D, dtype=torch.float32, device=qkv.device)
                dwk = torch.empty(D, dtype=torch.float32, device=qkv.device)
        native.check(
            lib.stb_qknorm_rope_bwd(qkv.data_ptr(), native.ptr(q_weight), native.ptr(k_weight), cos.data_ptr(),
                                    sin.data_ptr(), pos.data_ptr(), dq.data_ptr(), dk.data_ptr(), native.ptr(rstd),
                                    dqkv.data_ptr(), native.ptr(dwq), native.ptr(dwk), partial.data_ptr(), T, hq, hkv,
                                    D, qkv.stride(0), dqkv.stride(0), rot, int(use_norm), int(zero_centered), acc,
                                    native.stream()),
            "qknorm_rope_bwd")
        count_launch(3)
        gq = gk = None
        if use_norm:
            if acc:
                qp.grad_added_to_main_grad = True
                kp.grad_added_to_main_grad = True
            else:
                gq, gk = dwq.to(q_weight.dtype), dwk.to(k_weight.dtype)
        return dqkv, gq, gk, None, None, None, None, None, None, None, None, None, None


def qknorm_rope(qkv, q_weight, k_weight, cos, sin, pos, hq, hkv, head_dim, rot_dim=None, eps=1e-6,
                use_norm=True, zero_centered=False):
    """Split a packed qkv projection, RMS-normalise q and k per head, rotate them by position.

    Returns ``q [T,hq,D]``, ``k [T,hkv,D]`` and ``v [T,hkv,D]`` (a strided view of ``qkv``)."""
    rot = rot_dim or head_dim
    if not qkv.is_cuda or head_dim != 128:
        return qknorm_rope_reference(qkv, q_weight, k_weight, cos, sin, pos, hq, hkv, head_dim, rot, eps,
                                     use_norm, zero_centered)
    if pos.dtype != torch.int32:
        pos = pos.to(torch.int32)
    return _QKNormRopeFn.apply(qkv, q_weight, k_weight, cos, sin, pos, hq, hkv, head_dim, rot, eps, use_norm,
                               zero_centered)


# --------------------------------------------------------------------------- SwiGLU
def swiglu_reference(x, limit: float = 0.0):
    F = x.shape[-1] // 2
    g, u = x[..., :F].float(), x[..., F:].float()
    act = torch.nn.functional.silu(g)
    if limit and limit > 0:      # the activated gate is clamped from above, the up branch on both sides
        act = act.clamp(max=limit)                       # (reference: model/common/feed_forward.py:20-26)
        u = u.clamp(min=-limit, max=limit)
    return (act * u).to(x.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, limit):
        lib = native.load()
        F = x.shape[-1] // 2
        x2 = x.reshape(-1, 2 * F)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        out = torch.empty((x2.shape[0], F), dtype=x.dtype, device=x.device)
        native.check(lib.stb_swiglu_fwd(x2.data_ptr(), out.data_ptr(), x2.shape[0], F, x2.stride(0), out.stride(0),
                                        float(limit), native.stream()), "swiglu_fwd")
        count_launch()
        ctx.save_for_backward(x2)
        ctx.limit = limit
        ctx.in_shape = x.shape
        return out.view(*x.shape[:-1], F)

    @staticmethod
    def backward(ctx, gy):
        lib = native.load()
        (x2,) = ctx.saved_tensors
        F = x2.shape[-1] // 2
        g2 = gy.reshape(-1, F)
        if g2.stride(-1) != 1:
            g2 = g2.contiguous()
        dx = torch.empty_like(x2)
        native.check(lib.stb_swiglu_bwd(x2.data_ptr(), g2.data_ptr(), dx.data_ptr(), x2.shape[0], F, x2.stride(0),
                                        g2.stride(0), dx.stride(0), float(ctx.limit), native.stream()), "swiglu_bwd")
        count_launch()
        return dx.view(ctx.in_shape), None


def swiglu(x, limit: float = 0.0):
    """``silu(gate) * up`` for ``x = [gate | up]`` on the last dimension (optional clamps)."""
    if not x.is_cuda:
        return swiglu_reference(x, limit)
    return _SwiGLUFn.apply(x, limit or 0.0)


# --------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, vocab_start, vocab_end):
        lib = native.load()
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        H = table.shape[1]
        out = torch.empty((flat.numel(), H), dtype=table.dtype, device=table.device)
        native.check(lib.stb_embedding_fwd(flat.data_ptr(), table.data_ptr(), out.data_ptr(), flat.numel(), H,
                                           vocab_start, vocab_end, native.stream()), "embedding_fwd")
        count_launch()
        ctx.save_for_backward(flat)
        ctx.table_ref = table
        ctx.range = (vocab_start, vocab_end)
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, gy):
        lib = native.load()
        (flat,) = ctx.saved_tensors
        table = ctx.table_ref
        H = table.shape[1]
        g2 = gy.reshape(-1, H).contiguous()
        main_grad = getattr(table, "main_grad", None)
        buf = main_grad if main_grad is not None else torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        native.check(lib.stb_embedding_bwd(flat.data_ptr(), g2.data_ptr(), buf.data_ptr(), flat.numel(), H,
                                           ctx.range[0], ctx.range[1], native.stream()), "embedding_bwd")
        count_launch()
        if main_grad is not None:
            table.grad_added_to_main_grad = True
            return None, None, None, None
        return None, buf.to(table.dtype), None, None


def embedding(ids, table, vocab_start: int = 0, vocab_end: int | None = None):
    """Rows of a (vocab-sharded) table; ids outside ``[vocab_start, vocab_end)`` give zero rows."""
    vocab_end = vocab_start + table.shape[0] if vocab_end is None else vocab_end
    if not table.is_cuda:
        mask = (ids < vocab_start) | (ids >= vocab_end)
        local = (ids - vocab_start).masked_fill(mask, 0)
        out = torch.nn.functional.embedding(local, table)
        return out.masked_fill(mask.unsqueeze(-1), 0.0)
    return _EmbeddingFn.apply(ids, table, vocab_start, vocab_end)


# --------------------------------------------------------------------------- SwiGLU fused into the down projection
class _SwiGLULinearFn(torch.autograd.Function):
    """``swiglu(h) @ w.T`` that keeps only ``h``: the activation is recomputed in backward instead of being
    stored (the role of the reference's pre-function linear, ``core/tensor_parallel/layers.py:349-524``)."""

    @staticmethod
    def forward(ctx, h, w, limit):
        from .gemm import gemm

        lib = native.load()
        F = h.shape[-1] // 2
        h2 = h.reshape(-1, 2 * F)
        a = torch.empty((h2.shape[0], F), dtype=h.dtype, device=h.device)
        native.check(lib.stb_swiglu_fwd(h2.data_ptr(), a.data_ptr(), h2.shape[0], F, h2.stride(0), a.stride(0),
                                        float(limit), native.stream()), "swiglu_fwd")
        count_launch()
        y = gemm(a, w)
        ctx.save_for_backward(h2, w)
        ctx.w_ref, ctx.limit, ctx.in_shape = w, limit, h.shape
        return y.view(*h.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        from .gemm import gemm

        lib = native.load()
        h2, w = ctx.saved_tensors
        F = h2.shape[-1] // 2
        g2 = gy.reshape(-1, gy.shape[-1]).contiguous()
        a = torch.empty((h2.shape[0], F), dtype=h2.dtype, device=h2.device)
        native.check(lib.stb_swiglu_fwd(h2.data_ptr(), a.data_ptr(), h2.shape[0], F, h2.stride(0), a.stride(0),
                                        float(ctx.limit), native.stream()), "swiglu_fwd")
        dw = None
        main_grad = getattr(ctx.w_ref, "main_grad", None)
        if ctx.needs_input_grad[1]:
            if main_grad is not None:
                gemm(g2, a, a_mn_major=True, b_mn_major=True, out=main_grad, accumulate=True)
                ctx.w_ref.grad_added_to_main_grad = True
            else:
                dw = gemm(g2, a, a_mn_major=True, b_mn_major=True, out_dtype=w.dtype)
        da = gemm(g2, w, b_mn_major=True, out=a)  # reuse the activation buffer for its gradient
        dh = torch.empty_like(h2)
        native.check(lib.stb_swiglu_bwd(h2.data_ptr(), da.data_ptr(), dh.data_ptr(), h2.shape[0], F, h2.stride(0),
                                        da.stride(0), dh.stride(0), float(ctx.limit), native.stream()), "swiglu_bwd")
        count_launch(2)
        return dh.view(ctx.in_shape), dw, None


def swiglu_linear(h, w, limit: float = 0.0):
    """``swiglu(h) @ w.T`` without storing the activation (recomputed in backward)."""
    if not h.is_cuda:
        return torch.nn.functional.linear(swiglu_reference(h, limit), w)
    return _SwiGLULinearFn.apply(h, w, limit or 0.0)
