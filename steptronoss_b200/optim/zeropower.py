"""Matrix orthogonalisation routines for Muon.

``zeropower`` is the quintic Newton-Schulz iteration ``X <- a X + (b A + c A^2) X`` with
``A = X X^T`` on the spectrally-normalised input; the coefficient sets are the ones the reference
ships (``steptronoss/optimizer/_helpers.py:36-98``) together with its non-orthogonalising
alternatives (SVD, double normalisation, Sinkhorn-Knopp, dualisations).

On CUDA the three products of an iteration are tcgen05 GEMMs (``A`` and ``A^2`` are symmetric, so
both are plain ``X X^T``-type products without a transposed copy, computed on the upper triangle of
tiles only, with the scaled adds of the polynomial in the epilogue); the iteration runs in bf16.  The
reference casts to fp16 for the same step ("run_ns_in_fp16"); bf16 is what the sm_100a kernel takes
and has the wider exponent range.
"""
from __future__ import annotations

from functools import partial

import torch

from ..ops.gemm import gemm

_PE = [
    (8.28721201814563, -23.595886519098837, 17.300387312530933),
    (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
    (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
    (3.3184196573706015, -2.488488024314874, 0.51004894012372),
    (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
    (1.891301407787398, -1.2679958271945868, 0.37680408948524835),
    (1.8750014808534479, -1.2500016453999487, 0.3750001645474248),
    (1.875, -1.25, 0.375),
]
_PE_SLOW = [
    (2.6708353888008127, -3.2853566190584504, 1.6385678673837945),
    (1.8756101482892078, -1.25067777555517, 0.3750677840207064),
    (1.8750001724801866, -1.2500003448894914, 0.37500017240930517),
    (1.875, -1.25, 0.375),
]


def _with_safety(table):
    """All but the last polynomial are deflated by 1.01 per odd power for numerical headroom."""
    return [(a / 1.01, b / 1.01 ** 3, c / 1.01 ** 5) for a, b, c in table[:-1]] + [table[-1]]


ZEROPOWER_COEFFS = {
    "default": (3.4445, -4.7750, 2.0315),
    "youjc_250416": [(4.0848, -6.8946, 2.9270), (3.9505, -6.3029, 2.6377), (3.7418, -5.5913, 2.3037),
                     (2.8769, -3.1427, 1.2046), (2.8366, -3.0525, 1.2012)],
    "youjc_6": [(3955 / 1024, -8306 / 1024, 5008 / 1024), (3735 / 1024, -6681 / 1024, 3463 / 1024),
                (3799 / 1024, -6499 / 1024, 3211 / 1024), (4019 / 1024, -6385 / 1024, 2906 / 1024),
                (2677 / 1024, -3029 / 1024, 1162 / 1024), (2172 / 1024, -1833 / 1024, 682 / 1024)],
    "sujl_6": [(4140 / 1024, -7553 / 1024, 3571 / 1024), (3892 / 1024, -6637 / 1024, 2973 / 1024),
               (3668 / 1024, -6456 / 1024, 3021 / 1024), (3248 / 1024, -6211 / 1024, 3292 / 1024),
               (2792 / 1024, -5759 / 1024, 3796 / 1024), (3176 / 1024, -5507 / 1024, 4048 / 1024)],
    "polar_express": _with_safety(_PE),
    "polar_express_slow_convergence": _with_safety(_PE_SLOW),
}


def _schedule(coeffs, steps: int):
    table = [tuple(coeffs)] if isinstance(coeffs[0], (int, float)) else [tuple(c) for c in coeffs]
    if len(table) < steps:
        table = table + [table[-1]] * (steps - len(table))
    return table[:steps]


def _ns_native_2d(X: torch.Tensor, table) -> torch.Tensor:
    """X ``[m, n]`` bf16 CUDA with ``m <= n`` and both multiples of 8.

    ``A = X X^T`` and ``b A + c A^2`` are symmetric: their products compute only the tiles that reach the diagonal
    (44 % of the tiles of a 4096 x 4096 result lie below it) and a small kernel mirrors the rest; the scaled adds
    ``b A + ...`` and ``a X + ...`` run in the epilogue of the products."""
    upper = _upper_triangle_pays(X.shape[0])
    for a, b, c in table:
        A = gemm(X, X, upper_only=upper)                                  # X X^T                 [m, m]
        B = gemm(A, A, alpha=c, addend=A, beta=b, upper_only=upper)       # c A A^T + b A  (A symmetric)
        X = gemm(B, X, b_mn_major=True, addend=X, beta=a)                 # B X + a X             [m, n]
    return X


def _upper_triangle_pays(m: int) -> bool:
    """Skipping the tiles below the diagonal only helps when it saves a wave of the persistent grid (a 3072-wide
    result has 288 tiles of 128 x 256, 156 of them on or above the diagonal: two waves of 148 SMs either way)."""
    from ..ops import native

    sms = native.load().stb_sm_count() or 148
    num_m, block_n = -(-m // 128), 256 if m > 128 else 128
    num_n = -(-m // block_n)
    full = num_m * num_n
    upper = sum(num_n - (i * 128) // block_n for i in range(num_m))
    return -(-upper // sms) < -(-full // sms)


def zeropower(G: torch.Tensor, steps: int = 5, run_ns_in_fp16: bool = True, coeffs=ZEROPOWER_COEFFS["default"]):
    """Approximate ``U V^T`` of ``G = U S V^T`` (last two dims; leading dims are a batch)."""
    assert G.ndim >= 2
    tall = G.size(-2) > G.size(-1)
    X = G.mT if tall else G
    X = X / (X.float().norm(dim=(-2, -1), keepdim=True) * 1.01 + 1e-7).to(X.dtype)
    table = _schedule(coeffs, steps)
    native_ok = X.is_cuda and run_ns_in_fp16 and X.size(-1) % 8 == 0 and X.size(-2) % 8 == 0
    if native_ok:
        Xb = X.to(torch.bfloat16).contiguous()
        if Xb.dim() == 2:
            out = _ns_native_2d(Xb, table)
        else:
            flat = Xb.reshape(-1, Xb.size(-2), Xb.size(-1))
            out = torch.stack([_ns_native_2d(m.contiguous(), table) for m in flat]).view(Xb.shape)
        X = out
    else:
        if run_ns_in_fp16:
            X = X.to(torch.bfloat16 if not X.is_cuda else torch.float16)
        for a, b, c in table:
            A = X @ X.mT
            B = b * A + c * (A @ A)
            X = a * X + B @ X
    return X.mT.contiguous() if tall else X


def zeropower_via_svd(G, steps=None):
    U, _, Vh = torch.linalg.svd(G.float(), full_matrices=False)
    return U @ Vh


def double_normalize(G, steps):
    order = [-2, -1] if G.shape[-2] < G.shape[-1] else [-1, -2]
    for _ in range(steps):
        for dim in order:
            G = G / (G.norm(dim=dim, keepdim=True, p=2) + 1e-7)
    return G


def sinkhorn_knopp(G, steps):
    order = [-2, -1] if G.shape[-2] < G.shape[-1] else [-1, -2]
    for _ in range(steps):
        for dim in order:
            G = G / (G.norm(dim=dim, keepdim=True, p=1) + 1e-7)
    return G * G.shape[order[-1]] ** 0.5


def dualize_1_to_p(G, steps=None, p=1):
    return G / (torch.linalg.vector_norm(G, dim=-2, keepdim=True, ord=p) + 1e-7) * G.shape[-2] ** 0.5


def dualize_p_to_infinity(G, steps=None, p=1):
    q = 1 if p == float("inf") else p / (p - 1)
    return G / (torch.linalg.vector_norm(G, dim=-1, keepdim=True, ord=q) + 1e-7) * (G.shape[-1] / G.shape[-2] ** 0.5)


def dualize_schatten_2_norm(G, steps=None):
    return G / (torch.linalg.matrix_norm(G, ord="fro", dim=(-2, -1), keepdim=True) + 1e-7) * min(G.shape[-2:]) ** 0.5


def get_zeropower_fn(name: str, run_ns_in_fp16: bool = True):
    table = {
        "svd": zeropower_via_svd,
        "double_normalize": double_normalize,
        "sinkhorn_knopp": sinkhorn_knopp,
        "dualize_1_to_1": partial(dualize_1_to_p, p=1),
        "dualize_inf_to_inf": partial(dualize_p_to_infinity, p=float("inf")),
        "dualize_schatten_2_norm": dualize_schatten_2_norm,
    }
    if name in table:
        return table[name]
    return partial(zeropower, run_ns_in_fp16=run_ns_in_fp16, coeffs=ZEROPOWER_COEFFS[name])


def adjust_ratio_for_muon(matched_adamw_rms: float, shape) -> float:
    """Scale that gives an orthogonalised update the RMS of an AdamW update: ``rms * sqrt(max(m, n))``."""
    return matched_adamw_rms * (max(shape[-2], shape[-1]) ** 0.5)


# ---------------------------------------------------------------------------------------------------------------
# Spectral tools built on an orthogonaliser ``fn(G, steps) ~ U V^T`` (reference: optimizer/_helpers.py:176-247)
# ---------------------------------------------------------------------------------------------------------------
def get_step_fun(fn, threshold: float, steps: int = 5):
    """``G = U diag(s) V^T  ->  U diag(step(s - threshold)) V^T``: singular directions above ``threshold`` are kept
    with value 1, those below are removed.  Two orthogonalisations: ``sign(s)`` and ``sign(s - threshold)`` share
    the singular vectors, so their mean is the step."""

    @torch.no_grad()
    def step_fun(G):
        first = fn(G, steps)
        return 0.5 * (first + fn(G - threshold * first, steps))

    return step_fun


def get_clip_fun(fn, threshold: float, steps: int = 5):
    """``M = U diag(s) V^T  ->  U diag(min(s, threshold)) V^T`` without an SVD.  With ``P = fn(M)`` and
    ``Q = fn(M - threshold P)`` (signs of ``s`` and of ``s - threshold``):
    ``min(s, t) = (s + t - |s - t|) / 2`` and ``U diag(|s - t|) V^T = (M P^T - t I) Q``."""

    @torch.no_grad()
    def clip_fun(M):
        P = fn(M, steps)
        Q = fn(M - threshold * P, steps)
        eye = torch.eye(M.shape[-2], device=M.device, dtype=M.dtype)
        return 0.5 * (M + threshold * P - (M @ P.mT - threshold * eye) @ Q)

    return clip_fun


def get_max_singular_value(M):
    return torch.linalg.svdvals(M.float()).max()


@torch.no_grad()
def weight_decay_in_spectral_norm(M, steps: int = 10, pre_iters: int = 3):
    """Gradient of the spectral norm, ``u1 v1^T`` of the leading singular pair, for ``[m, n]`` or a batch
    ``[B, m, n]``, by power iteration.  The matrix is first scaled to a spectral norm a little below one and
    multiplied ``pre_iters`` times by ``M^T M``: that raises every singular value to the power ``2 pre_iters + 1``
    and so widens the gap that the ``steps`` power iterations then work with."""
    single = M.dim() == 2
    X = M.unsqueeze(0) if single else M
    wide = X.shape[-1] > X.shape[-2]
    if wide:                                                       # work on the tall orientation
        X = X.mT
    X = X / ((X.norm(dim=(-2, -1), keepdim=True) + 1e-7) / X.shape[-1] ** 0.5)
    gram = X.mT @ X
    for _ in range(pre_iters):
        X = X @ gram
    gram = X.mT @ X
    v = torch.randn((X.shape[0], X.shape[-1], 1), device=X.device, dtype=X.dtype)
    for _ in range(steps):
        v = torch.nn.functional.normalize(gram @ v, dim=1)
    u = torch.nn.functional.normalize(X @ v, dim=1)
    grad = u @ v.mT
    if wide:
        grad = grad.mT.contiguous()
    return grad[0] if single else grad
