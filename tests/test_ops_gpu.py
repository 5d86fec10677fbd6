"""Native fused kernels against their PyTorch restatements (fp32 math on the same inputs)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol=2e-2):
    a, b = a.float(), b.float()
    denom = b.abs().max().item() + 1e-6
    assert ((a - b).abs().max().item() / denom) < tol, f"{(a - b).abs().max().item()} / {denom}"


@pytest.mark.parametrize("rows,H,zc", [(64, 256, False), (1000, 4096, False), (333, 2048, True), (8, 8192, False)])
def test_rmsnorm_fwd_bwd(rows, H, zc):
    from steptronoss_b200.ops import rmsnorm, rmsnorm_reference

    torch.manual_seed(0)
    x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(H, device="cuda") * 0.1 + (0.0 if zc else 1.0)).to(torch.bfloat16).requires_grad_()
    g = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
    y = rmsnorm(x, w, 1e-6, zc)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = rmsnorm_reference(xr, wr, 1e-6, zc)
    yr.backward(g.float())
    _close(y, yr.detach(), 1e-2)
    _close(x.grad, xr.grad, 2e-2)
    _close(w.grad, wr.grad, 2e-2)


@pytest.mark.parametrize("rot,use_norm", [(128, True), (64, True), (128, False)])
def test_qknorm_rope_fwd_bwd(rot, use_norm):
    from steptronoss_b200.ops import qknorm_rope, qknorm_rope_reference, rope_tables

    torch.manual_seed(1)
    T, hq, hkv, D = 777, 8, 2, 128
    qkv = torch.randn(T, (hq + 2 * hkv) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    qw = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_()
    kw = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_()
    cos, sin = rope_tables(1024, rot, 1e6, "cuda")
    pos = torch.randint(0, 1024, (T,), device="cuda", dtype=torch.int32)
    q, k, v = qknorm_rope(qkv, qw, kw, cos, sin, pos, hq, hkv, D, rot, 1e-6, use_norm)
    gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    qkv_r = qkv.detach().float().requires_grad_()
    qw_r, kw_r = qw.detach().float().requires_grad_(), kw.detach().float().requires_grad_()
    q2, k2, v2 = qknorm_rope_reference(qkv_r, qw_r, kw_r, cos, sin, pos, hq, hkv, D, rot, 1e-6, use_norm)
    torch.autograd.backward([q2, k2, v2], [gq.float(), gk.float(), gv.float()])
    _close(q, q2.detach(), 1e-2)
    _close(k, k2.detach(), 1e-2)
    assert torch.equal(v, qkv.detach()[:, (hq + hkv) * D:].view(T, hkv, D))
    _close(qkv.grad, qkv_r.grad, 2e-2)
    if use_norm:
        _close(qw.grad, qw_r.grad, 3e-2)
        _close(kw.grad, kw_r.grad, 3e-2)


@pytest.mark.parametrize("limit", [0.0, 1.5])
def test_swiglu_fwd_bwd(limit):
    from steptronoss_b200.ops import swiglu, swiglu_reference

    torch.manual_seed(2)
    x = (2 * torch.randn(513, 2 * 768, device="cuda")).to(torch.bfloat16).requires_grad_()
    g = torch.randn(513, 768, device="cuda", dtype=torch.bfloat16)
    y = swiglu(x, limit)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = swiglu_reference(xr, limit)
    yr.backward(g.float())
    _close(y, yr.detach(), 1e-2)
    _close(x.grad, xr.grad, 2e-2)


def test_swiglu_linear_recomputes_activation():
    from steptronoss_b200.ops.fused import swiglu_linear, swiglu_reference

    torch.manual_seed(7)
    h = torch.randn(640, 2 * 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.1 * torch.randn(384, 256, device="cuda")).to(torch.bfloat16).requires_grad_()
    g = torch.randn(640, 384, device="cuda", dtype=torch.bfloat16)
    y = swiglu_linear(h, w, 0.0)
    y.backward(g)
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = swiglu_reference(hr, 0.0) @ wr.t()
    yr.backward(g.float())
    _close(y, yr.detach(), 2e-2)
    _close(h.grad, hr.grad, 3e-2)
    _close(w.grad, wr.grad, 3e-2)


def test_embedding_fwd_bwd_sharded():
    from steptronoss_b200.ops import embedding

    torch.manual_seed(3)
    V, H = 1000, 256
    table = torch.randn(500, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, V, (4, 300), device="cuda")
    out = embedding(ids, table, 250, 750)
    g = torch.randn_like(out)
    out.backward(g)
    mask = (ids >= 250) & (ids < 750)
    ref = torch.where(mask.unsqueeze(-1), table.detach()[(ids - 250).clamp(0, 499)], torch.zeros_like(out))
    assert torch.equal(out, ref)
    gref = torch.zeros(500, H, device="cuda")
    gref.index_add_(0, (ids - 250).clamp(0, 499)[mask], g.float()[mask])
    _close(table.grad, gref, 2e-2)


@pytest.mark.parametrize("T,V,chunk", [(300, 1024, 128), (1000, 5000 // 8 * 8, 512)])
def test_fused_linear_cross_entropy(T, V, chunk):
    from steptronoss_b200.ops import fused_linear_cross_entropy

    torch.manual_seed(4)
    H = 256
    h = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(V, H, device="cuda")).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    weights = (torch.rand(T, device="cuda") > 0.3).float()
    weights = weights / weights.sum()
    loss, loss_tok, pred = fused_linear_cross_entropy(h, w, labels, weights, chunk_tokens=chunk)
    loss.backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    logits = (hr @ wr.t()).to(torch.bfloat16).float() if False else hr @ wr.t()
    lt = torch.nn.functional.cross_entropy(logits, labels, reduction="none")
    lr = (lt * weights).sum()
    lr.backward()
    assert abs(loss.item() - lr.item()) < 2e-2 * abs(lr.item())
    _close(loss_tok, lt.detach(), 2e-2)
    assert (pred == logits.argmax(-1)).float().mean().item() > 0.97
    _close(h.grad, hr.grad, 3e-2)
    _close(w.grad, wr.grad, 3e-2)


def test_adam_matches_torch_and_clip_scalars():
    from steptronoss_b200.ops import native
    lib = native.load()
    torch.manual_seed(5)
    n = 100_000 + 37
    p0 = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    ref_p = p0.clone().requires_grad_()
    opt = torch.optim.Adam([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    from steptronoss_b200.optim.adam import FlatAdamShard

    class B:
        pass

    b = B()
    b.param_buf = p0.to(torch.bfloat16)
    b.grad_buf = torch.zeros(n, device="cuda")
    sh = FlatAdamShard(b, 0, n, [(0, n, 1.0, 1.0)], "adam")
    sh.master.copy_(p0)
    scal = torch.tensor([0.0, 0.0, 0.5, 1.0], device="cuda")
    for step in range(1, 4):
        b.grad_buf.copy_(g * step)
        ref_p.grad = (g * step) * 0.25 * 0.5   # grad_scale 0.25, clip 0.5
        opt.step()
        sh.step(step, 1e-2, 0.1, 0.9, 0.95, 1e-8, 0.25, scal)
    assert (sh.master - ref_p.detach()).abs().max().item() < 1e-5
    assert torch.equal(b.param_buf, sh.master.to(torch.bfloat16))
    # squared norm + clip coefficient
    part = torch.empty(lib.stb_sqnorm_grid(), device="cuda")
    out = torch.zeros(4, device="cuda")
    native.check(lib.stb_sqnorm(g.data_ptr(), n, part.data_ptr(), out.data_ptr(), 0, native.stream()), "sqnorm")
    native.check(lib.stb_clip_coef(out.data_ptr(), 1.0, native.stream()), "clip")
    nrm = g.double().norm().item()
    assert abs(out[1].item() - nrm) / nrm < 1e-5
    assert abs(out[2].item() - 1.0 / (nrm + 1e-6)) < 1e-6 and out[3].item() == 1.0


def test_tiny_model_on_gpu_matches_the_cpu_fp32_loss_curve_and_gradient_norms():
    """The whole model through the native kernels (bf16) against the same experiment trained in fp32 on the CPU
    through the PyTorch restatements: same seed, same data, same optimizer; three steps.  Losses and gradient
    norms must agree within bf16 tolerance."""
    import json
    import os
    import subprocess
    import sys

    from steptronoss_b200.ops import native
    from tests.tiny_exp import make_tiny_exp

    kw = dict(hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048, layers=2, seq=512, gbs=2, iters=3,
              min_doc=32, max_doc=256)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK"):
        env.pop(k, None)
    cpu = subprocess.run([sys.executable, os.path.join(root, "tests", "mp_gpu_worker.py"), json.dumps(kw), "3", "cpu_fp32"],
                         capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert cpu.returncode == 0, cpu.stdout[-2000:] + cpu.stderr[-2000:]
    oracle = json.loads([l for l in cpu.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])

    exp = make_tiny_exp(dtype=torch.bfloat16, **kw)
    exp.seed = 0
    tr = exp.trainer_cfg.get_trainer_cls()(exp=exp)
    tr.before_train()
    for _ in range(3):
        tr.train_step()
        tr.iteration += 1
        tr.training_log()
    native.raise_if_kernel_error()
    losses = [h["lm_loss"] for h in tr.history]
    norms = [h["grad_norm"] for h in tr.history]
    assert all(math.isfinite(l) for l in losses)
    assert abs(losses[0] - math.log(2048)) < 0.5
    for a, b in zip(losses, oracle["losses"]):
        assert abs(a - b) < 2e-2 * abs(b), (losses, oracle["losses"])
    for a, b in zip(norms, oracle["grad_norms"]):
        assert abs(a - b) < 5e-2 * abs(b), (norms, oracle["grad_norms"])


@pytest.mark.parametrize("M,N,K", [(256, 4, 256), (130, 772, 64)])
def test_gemm_with_unaligned_row_pitch_uses_the_library(M, N, K):
    from steptronoss_b200.ops.gemm import gemm

    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    out = gemm(a, b)
    ref = a.float() @ b.float().t()
    assert out.shape == (M, N) and float((out.float() - ref).abs().max() / ref.abs().max()) < 2e-2


@pytest.mark.parametrize("rows,H", [(37, 512), (300, 4096), (5, 8192)])
def test_add_rmsnorm_matches_the_unfused_statement(rows, H):
    """x + delta and its RMSNorm in one kernel: forward and backward against fp32 PyTorch on the bf16-rounded sum."""
    from steptronoss_b200.ops import add_rmsnorm, residual_add

    torch.manual_seed(0)
    x = torch.randn(rows, H, device="cuda").to(torch.bfloat16).requires_grad_()
    d = torch.randn(rows, H, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_()
    s, y = add_rmsnorm(x, d, w, 1e-6, False)
    s_ref = (x.detach() + d.detach())                                        # bf16 add
    assert torch.equal(s, s_ref)
    xs = s_ref.float().requires_grad_()
    wf = w.detach().float().requires_grad_()
    y_ref = xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    assert float((y.float() - y_ref).abs().max()) < 3e-2
    gs = torch.randn_like(s)
    gy = torch.randn_like(y)
    torch.autograd.backward([s, y], [gs, gy])
    y_ref.backward(gy.float())
    ds_ref = xs.grad + gs.float()
    assert torch.equal(x.grad, d.grad)
    assert float((x.grad.float() - ds_ref).abs().max() / ds_ref.abs().max()) < 2e-2
    assert float((w.grad.float() - wf.grad).abs().max() / wf.grad.abs().max()) < 2e-2
    a = torch.randn(64, 256, device="cuda").to(torch.bfloat16).requires_grad_()
    b = torch.randn(64, 256, device="cuda").to(torch.bfloat16).requires_grad_()
    out = residual_add(a, b)
    assert torch.equal(out, a.detach() + b.detach())
    out.sum().backward()
    assert torch.equal(a.grad, torch.ones_like(a)) and torch.equal(b.grad, torch.ones_like(b))
