"""Block-scaled fp8 products: the quantisation statements on CPU, the sm_100a kernels against them on a GPU."""
import pytest
import torch


def test_block_quantisation_round_trip_and_scales():
    from steptronoss_b200.ops import fp8

    torch.manual_seed(0)
    x = torch.randn(64, 256) * torch.logspace(-2, 2, 64).unsqueeze(1)
    q, s = fp8.quantize_rows_1x128_reference(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (64, 2)
    back = fp8.dequantize_rows(q, s)
    assert ((back - x).abs() <= x.abs() * 0.07 + s.repeat_interleave(128, dim=1) * 2e-3 + 1e-12).all()
    assert torch.allclose(s, x.view(64, 2, 128).abs().amax(-1) / 448.0)
    w = torch.randn(256, 384)
    qw, sw = fp8.quantize_blocks_128x128_reference(w)
    assert sw.shape == (2, 3)
    assert ((fp8.dequantize_blocks(qw, sw) - w).abs() <= w.abs() * 0.07 + 0.02).all()
    z, sz = fp8.quantize_rows_1x128_reference(torch.zeros(2, 128))
    assert sz.eq(1).all() and z.float().eq(0).all()


def test_grouped_product_statement_follows_the_segments():
    from steptronoss_b200.ops import fp8

    torch.manual_seed(1)
    G, N, K = 3, 128, 256
    offsets = torch.tensor([0, 128, 128, 384], dtype=torch.int32)     # group 1 is empty
    x = torch.randn(384, K)
    w = torch.randn(G * N, K) * 0.05
    xq, sx = fp8.quantize_rows_1x128(x)
    wq, sw = fp8.quantize_blocks_128x128(w)
    y = fp8.grouped_gemm_fp8(xq, sx, wq, sw, offsets, G).float()
    want = torch.zeros(384, N)
    want[:128] = x[:128] @ w[:N].t()
    want[128:] = x[128:] @ w[2 * N:].t()
    assert (y - want).norm() / want.norm() < 0.06     # two e4m3 roundings of ~2^-4 relative each, averaged over K


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K,G", [(128, 128, 128, 1), (300, 256, 512, 1), (1024, 1536, 2048, 4), (640, 768, 4096, 3)])
def test_fp8_kernels_match_the_dequantised_fp32_statement(M, N, K, G):
    from steptronoss_b200.ops import fp8, native

    torch.manual_seed(2)
    dev = "cuda"
    x = (torch.randn(M, K, device=dev) * torch.rand(M, 1, device=dev).mul(4).exp()).to(torch.bfloat16)
    w = (torch.randn(G * N, K, device=dev) * 0.05).to(torch.bfloat16)
    xq, sx = fp8.quantize_rows_1x128(x)
    wq, sw = fp8.quantize_blocks_128x128(w)
    # the quantisation kernels against their statements: same scales, values that differ by rounding of x / scale at most
    xq_ref, sx_ref = fp8.quantize_rows_1x128_reference(x)
    wq_ref, sw_ref = fp8.quantize_blocks_128x128_reference(w)
    assert torch.allclose(sx, sx_ref, rtol=1e-6) and torch.allclose(sw, sw_ref, rtol=1e-6)
    assert (fp8.dequantize_rows(xq, sx) - fp8.dequantize_rows(xq_ref, sx_ref)).abs().max() <= x.float().abs().max() * 0.07
    assert (xq.float() != xq_ref.float()).float().mean() < 0.02
    assert (wq.float() != wq_ref.float()).float().mean() < 0.02
    if G == 1:
        offsets = None
    else:
        per = (M // 128) // G * 128          # rows of every group but the last; segment starts on 128-row tiles
        offsets = torch.tensor([min(g * per, M) for g in range(G)] + [M], dtype=torch.int32, device=dev)
    y = fp8.grouped_gemm_fp8(xq, sx, wq, sw, offsets, G)
    torch.cuda.synchronize()
    native.raise_if_kernel_error()
    off_ref = offsets if offsets is not None else torch.tensor([0, M], dtype=torch.int32)
    want = fp8.grouped_gemm_fp8_reference(xq, sx, wq, sw, off_ref.cpu(), G).float()
    err = (y.float() - want).abs().max() / want.abs().max()
    assert err < 1e-2, err                    # same operands: only the order of the fp32 sums and bf16 rounding differ


@pytest.mark.gpu
def test_routed_ffn_with_fp8_forward_stays_close_to_bf16_and_keeps_bf16_gradients():
    from steptronoss_b200.ops import moe as moe_ops
    from steptronoss_b200.ops import native

    torch.manual_seed(3)
    dev = "cuda"
    T, H, F, E, K = 512, 256, 128, 4, 2
    x = torch.randn(T, H, device=dev).to(torch.bfloat16).requires_grad_()
    w1 = (torch.randn(E, 2 * F, H, device=dev) * 0.05).to(torch.bfloat16).requires_grad_()
    w2 = (torch.randn(E, H, F, device=dev) * 0.05).to(torch.bfloat16).requires_grad_()
    ids = torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)])
    wts = torch.rand(T, K, device=dev)
    g = torch.randn(T, H, device=dev).to(torch.bfloat16)
    outs = {}
    for fp8 in (False, True):
        for t in (x, w1, w2):
            t.grad = None
        y = moe_ops.routed_grouped_ffn(x, ids, wts, w1, w2, fp8=fp8)
        y.backward(g)
        outs[fp8] = [y.detach().float(), x.grad.float().clone(), w1.grad.float().clone()]
    torch.cuda.synchronize()
    native.raise_if_kernel_error()
    rel = lambda a, b: float((a - b).norm() / b.norm())
    assert 1e-4 < rel(outs[True][0], outs[False][0]) < 0.08       # fp8 was really used, and stays close
    assert rel(outs[True][1], outs[False][1]) < 0.08 and rel(outs[True][2], outs[False][2]) < 0.08
