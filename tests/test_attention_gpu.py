"""tcgen05 flash attention (forward and backward) against the fp32 PyTorch restatement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()


CASES = [
    # lens_q, lens_k (None = same), hq, hkv, causal, window
    ([128], None, 2, 2, True, 0),
    ([256], None, 4, 1, True, 0),
    ([100, 300, 57], None, 4, 2, True, 0),
    ([1000, 24, 512, 200], None, 8, 2, True, 0),
    ([384, 129], None, 4, 2, False, 0),
    ([700, 300], None, 4, 2, True, 128),
    ([700, 300, 77], None, 4, 2, True, 65),     # odd windows: a sliding_window_size of w shows w + 1 keys
    ([1100], None, 4, 4, True, 513),
    ([200, 100], [500, 228], 4, 2, True, 0),   # q rows are the tail of longer key segments
    ([2048], None, 4, 4, True, 0),
]


@pytest.mark.parametrize("lens_q,lens_k,hq,hkv,causal,window", CASES)
def test_flash_attention_fwd_bwd(lens_q, lens_k, hq, hkv, causal, window):
    from steptronoss_b200.ops import native
    from steptronoss_b200.ops.attention import attention, attention_reference

    torch.manual_seed(0)
    lens_k = lens_k or lens_q
    Tq, Tk, D = sum(lens_q), sum(lens_k), 128
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device="cuda")
    q = torch.randn(Tq, hq, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(Tk, hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    # v as a strided view of a wider buffer, like the v slice of a packed qkv projection
    vbuf = torch.randn(Tk, 3 * hkv * D, device="cuda", dtype=torch.bfloat16)
    v = vbuf[:, hkv * D: 2 * hkv * D].view(Tk, hkv, D).detach().requires_grad_()
    g = torch.randn(Tq, hq, D, device="cuda", dtype=torch.bfloat16)
    o = attention(q, k, v, cu_q, cu_k, max(lens_q), causal=causal, window=window)
    o.backward(g)
    torch.cuda.synchronize()
    native.raise_if_kernel_error()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    oref = attention_reference(qr, kr, vr, cu_q.cpu(), cu_k.cpu(), causal, window)
    oref.backward(g.float())
    assert _rel(o, oref) < 1e-2, f"fwd rel err {_rel(o, oref)}"
    assert _rel(q.grad, qr.grad) < 2e-2, f"dq rel err {_rel(q.grad, qr.grad)}"
    assert _rel(k.grad, kr.grad) < 2e-2, f"dk rel err {_rel(k.grad, kr.grad)}"
    assert _rel(v.grad, vr.grad) < 2e-2, f"dv rel err {_rel(v.grad, vr.grad)}"


def test_flash_attention_is_deterministic():
    from steptronoss_b200.ops.attention import attention

    torch.manual_seed(1)
    q = torch.randn(640, 4, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(640, 2, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(640, 2, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cu = torch.tensor([0, 300, 640], dtype=torch.int32, device="cuda")
    outs = []
    for _ in range(2):
        for t in (q, k, v):
            t.grad = None
        o = attention(q, k, v, cu, cu, 340)
        o.sum().backward()
        outs.append((o.detach().clone(), q.grad.clone(), k.grad.clone(), v.grad.clone()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("splits", [1, 2, 4, 8])
def test_dkv_pass_split_over_the_q_heads_of_a_group(splits):
    """hq=16 / hkv=2 (group of 8): the dK/dV pass with the group on one CTA and split over 2, 4 and 8 CTAs gives the
    gradients of the fp32 restatement, and each split count is bitwise reproducible."""
    from steptronoss_b200.ops import attention_native, native
    from steptronoss_b200.ops.attention import attention, attention_reference

    torch.manual_seed(3)
    lens = [700, 324, 129]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    q = torch.randn(T, 16, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, 2, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, 2, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(T, 16, 128, device="cuda", dtype=torch.bfloat16)
    old = attention_native._FORCE_SPLITS
    attention_native._FORCE_SPLITS = splits
    try:
        runs = []
        for _ in range(2):
            for t in (q, k, v):
                t.grad = None
            attention(q, k, v, cu, cu, max(lens)).backward(g)
            runs.append((k.grad.clone(), v.grad.clone(), q.grad.clone()))
        torch.cuda.synchronize()
        native.raise_if_kernel_error()
    finally:
        attention_native._FORCE_SPLITS = old
    for a, b in zip(*runs):
        assert torch.equal(a, b)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    attention_reference(qr, kr, vr, cu.cpu(), cu.cpu(), True, 0).backward(g.float())
    assert _rel(runs[0][0], kr.grad) < 2e-2 and _rel(runs[0][1], vr.grad) < 2e-2 and _rel(runs[0][2], qr.grad) < 2e-2
