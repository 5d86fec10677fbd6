"""tcgen05 GEMM against an fp32 PyTorch product, all operand layouts, output types and tails."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    am = a.float().t() if a_mn else a.float()
    bm = b.float() if b_mn else b.float().t()
    return am @ bm


def _check(out, ref, K):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < 1.6e-2, f"max err {err} vs scale {scale}"
    # tighter statistical check: bf16 rounding of inputs only
    rel = (out.float() - ref).norm() / (ref.norm() + 1e-6)
    assert rel < 5e-3, f"relative Frobenius error {rel}"


SHAPES = [(128, 256, 64), (256, 512, 128), (384, 768, 256), (200, 264, 136), (1024, 1024, 1024), (130, 8, 72),
          (4096, 6144, 4096)]


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    from steptronoss_b200.ops import gemm
    from steptronoss_b200.ops import native

    if a_mn and M % 8:
        pytest.skip("MN-major A needs M % 8 == 0 (row pitch multiple of 16 bytes)")
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn)
    torch.cuda.synchronize()
    native.raise_if_kernel_error()
    _check(out, _ref(a, b, a_mn, b_mn), K)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_accumulate_and_alpha(out_dtype):
    from steptronoss_b200.ops import gemm

    torch.manual_seed(1)
    M, N, K = 512, 384, 320
    a = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    c0 = torch.randn(M, N, device="cuda", dtype=torch.float32).to(out_dtype)
    c = c0.clone()
    gemm(a, b, a_mn_major=True, b_mn_major=True, out=c, accumulate=True, alpha=0.5)
    ref = c0.float() + 0.5 * _ref(a, b, True, True)
    tol = 2e-2 if out_dtype == torch.bfloat16 else 1.6e-2
    assert ((c.float() - ref).abs().max() / ref.abs().max()).item() < tol


def test_gemm_strided_views():
    from steptronoss_b200.ops import gemm

    torch.manual_seed(2)
    big_a = torch.randn(300, 512, device="cuda", dtype=torch.bfloat16)
    big_b = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    a, b = big_a[:, 64:320], big_b[:, 128:384]   # row pitch 512, 256 columns
    out_big = torch.zeros(300, 512, device="cuda", dtype=torch.bfloat16)
    out = out_big[:, 256:512]
    gemm(a, b, out=out)
    _check(out, a.float() @ b.float().t(), 256)
    assert out_big[:, :256].abs().max().item() == 0


def test_linear_autograd_matches_pytorch():
    from steptronoss_b200.ops import linear

    torch.manual_seed(3)
    x = torch.randn(1024, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(768, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(1024, 768, device="cuda", dtype=torch.bfloat16)
    y = linear(x, w)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())
    _check(y, yr.detach(), 512)
    _check(x.grad, xr.grad, 768)
    _check(w.grad, wr.grad, 1024)
    # fused accumulation into an fp32 main_grad
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.ones(768, 512, device="cuda", dtype=torch.float32)
    linear(x.detach(), w2).backward(g)
    assert w2.grad is None
    _check(w2.main_grad - 1.0, wr.grad, 1024)


def test_grouped_gemm_rows_and_reduce():
    from steptronoss_b200.ops.grouped import grouped_gemm_reduce, grouped_gemm_rows

    torch.manual_seed(4)
    G, K, N = 4, 256, 512
    rows = [256, 128, 0, 384]
    offs = [0]
    for r in rows:
        offs.append(offs[-1] + r)
    M = offs[-1]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(G, N, K, device="cuda", dtype=torch.bfloat16)
    offsets = torch.tensor(offs, device="cuda", dtype=torch.int32)
    y = grouped_gemm_rows(x, w, offsets, trans_b=True)
    ref = torch.cat([x[offs[g]:offs[g + 1]].float() @ w[g].float().t() for g in range(G)])
    _check(y, ref, K)
    w2 = torch.randn(G, K, N, device="cuda", dtype=torch.bfloat16)
    y2 = grouped_gemm_rows(x, w2, offsets, trans_b=False)
    ref2 = torch.cat([x[offs[g]:offs[g + 1]].float() @ w2[g].float() for g in range(G)])
    _check(y2, ref2, K)
    g_out = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    dw = grouped_gemm_reduce(g_out, x, offsets, G)   # [G, N, K]
    refw = torch.stack([g_out[offs[g]:offs[g + 1]].float().t() @ x[offs[g]:offs[g + 1]].float() for g in range(G)])
    _check(dw, refw, 384)


@pytest.mark.parametrize("n,k", [(256, 128), (1024, 384), (2304, 512), (520, 256)])
def test_symmetric_product_with_scaled_addend_on_the_upper_triangle(n, k):
    """``alpha X X^T + beta D`` with only the tiles that reach the diagonal computed and the rest mirrored."""
    from steptronoss_b200.ops.gemm import gemm

    torch.manual_seed(n)
    x = (torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16)
    d = torch.randn(n, n, device="cuda")
    d = ((d + d.t()) * 0.5).to(torch.bfloat16)
    want = 0.75 * (x.float() @ x.float().t()) + (-1.5) * d.float()
    full = gemm(x, x, alpha=0.75, addend=d, beta=-1.5)
    upper = gemm(x, x, alpha=0.75, addend=d, beta=-1.5, upper_only=True)
    torch.cuda.synchronize()
    assert (full.float() - want).abs().max() < 3e-2 * want.abs().max()
    assert torch.equal(upper, upper.t().contiguous())
    assert (upper.float() - want).abs().max() < 3e-2 * want.abs().max()
    iu = torch.triu_indices(n, n, device="cuda")
    assert torch.equal(upper[iu[0], iu[1]], full[iu[0], iu[1]])     # the computed triangle is the same product


def test_newton_schulz_on_the_gpu_matches_the_fp32_iteration():
    from steptronoss_b200.optim.zeropower import ZEROPOWER_COEFFS, zeropower

    torch.manual_seed(0)
    for shape in ((512, 768), (1280, 512)):
        g = torch.randn(*shape, device="cuda", dtype=torch.bfloat16)
        got = zeropower(g, 5, True, ZEROPOWER_COEFFS["default"]).float()
        want = zeropower(g.float().cpu(), 5, False, ZEROPOWER_COEFFS["default"]).to("cuda")
        assert ((got - want).norm() / want.norm()).item() < 5e-2
        s = torch.linalg.svdvals(got)
        assert s.max() < 1.3 and s.min() > 0.5


def test_weight_gradient_product_with_the_reduction_split_over_ctas():
    """fp32 accumulate-into-C products with few output tiles cut their reduction extent into parts that several
    CTAs add into C (8 tiles x 4 parts here); the sum must still be the product."""
    from steptronoss_b200.ops import gemm

    torch.manual_seed(5)
    M, N, K = 512, 512, 4096
    a = (torch.randn(K, M, device="cuda") * 0.1).to(torch.bfloat16)
    b = (torch.randn(K, N, device="cuda") * 0.1).to(torch.bfloat16)
    c0 = torch.randn(M, N, device="cuda", dtype=torch.float32)
    c = c0.clone()
    gemm(a, b, a_mn_major=True, b_mn_major=True, out=c, accumulate=True)
    torch.cuda.synchronize()
    ref = c0 + _ref(a, b, True, True)
    assert ((c - ref).abs().max() / ref.abs().max()).item() < 2e-3
