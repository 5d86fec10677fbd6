"""Muon: orthogonalisation quality, the stand-alone optimizer step, and the gradient-manager path."""
import pytest
import torch

from steptronoss_b200.optim.muon import Muon
from steptronoss_b200.optim.zeropower import ZEROPOWER_COEFFS, get_zeropower_fn, zeropower


def test_newton_schulz_pushes_singular_values_towards_one():
    torch.manual_seed(0)
    for shape in [(32, 64), (64, 32), (3, 16, 48)]:
        G = torch.randn(shape)
        X = zeropower(G, steps=5, run_ns_in_fp16=False)
        s = torch.linalg.svdvals(X.float())
        assert s.max() < 1.3 and s.min() > 0.4, (shape, s.min(), s.max())
        assert X.shape == G.shape


def test_polar_express_schedule_has_safety_factor_and_converges():
    tab = ZEROPOWER_COEFFS["polar_express"]
    assert abs(tab[0][0] - 8.28721201814563 / 1.01) < 1e-12 and tab[-1] == (1.875, -1.25, 0.375)
    torch.manual_seed(1)
    G = torch.randn(24, 40)
    X = get_zeropower_fn("polar_express", run_ns_in_fp16=False)(G, steps=8)
    s = torch.linalg.svdvals(X)
    assert (s - 1).abs().max() < 0.05
    U = get_zeropower_fn("svd")(G)
    assert torch.allclose(X, U, atol=0.05)


def test_muon_step_matches_manual_rule_and_state_restores():
    torch.manual_seed(2)
    w = torch.nn.Parameter(torch.randn(8, 16))
    b = torch.nn.Parameter(torch.randn(16))
    groups = [{"params": [w], "is_muon_param": True}, {"params": [b], "is_muon_param": False}]
    opt = Muon(groups, lr=0.1, weight_decay=0.01, run_ns_in_fp16=False, adamw_betas=(0.9, 0.95))
    w0, b0 = w.detach().clone(), b.detach().clone()
    gw, gb = torch.randn(8, 16), torch.randn(16)
    w.grad, b.grad = gw.clone(), gb.clone()
    opt.step()
    buf = gw.clone()
    g = gw + 0.95 * buf
    upd = zeropower(g, 5, False) * 0.2 * (16 ** 0.5)
    assert torch.allclose(w.detach(), w0 * (1 - 0.1 * 0.01) - 0.1 * upd, atol=1e-5)
    m1, m2 = 0.1 * gb, 0.05 * gb * gb
    step = m1 / (1e-8 + m2.sqrt()) * ((1 - 0.95) ** 0.5 / (1 - 0.9))
    assert torch.allclose(b.detach(), b0 * (1 - 0.1 * 0.01) - 0.1 * step, atol=1e-5)
    sd = opt.state_dict()
    opt2 = Muon([{"params": [w], "is_muon_param": True}, {"params": [b], "is_muon_param": False}], lr=0.1,
                weight_decay=0.01, run_ns_in_fp16=False, adamw_betas=(0.9, 0.95))
    opt2.load_state_dict(sd)
    assert torch.equal(opt2.state[w]["muon_buffer"], opt.state[w]["muon_buffer"])


def test_gradient_manager_with_muon_trains():
    from steptronoss_b200.exp.optimizer import MuonConfig
    from tests.tiny_exp import make_tiny_exp

    e = make_tiny_exp(gbs=2, seq=128, iters=3, layers=1, hidden=64, heads=2, kv_heads=1, head_dim=32, ffn=128, vocab=256)
    e.optimizer_cfg.optimizer_cfg = MuonConfig
    e.optimizer_cfg.optimizer_cfg.muon_run_ns_in_fp16 = False
    tr = e.trainer_cfg.get_trainer_cls()(exp=e)
    tr.before_train()
    gm = tr.grad_manager
    assert gm.muon is not None and len(gm.muon.entries) == 4   # wqkv, wo, w1, w2 (embeddings / head / norms -> AdamW)
    names = {en["slot"].name.split(".")[-2] for en in gm.muon.entries}
    assert names == {"wqkv", "wo", "w1", "w2"}
    before = {n: p.detach().clone() for n, p in tr.models[0].named_parameters()}
    tr.train_step()
    changed = [n for n, p in tr.models[0].named_parameters() if not torch.equal(p, before[n])]
    assert len(changed) == len(before)


def test_update_shaping_alternatives_have_their_stated_norms():
    """The choices of ``get_zeropower_fn`` that do not orthogonalise: each fixes a different norm of the update."""
    import torch

    from steptronoss_b200.optim.zeropower import get_zeropower_fn

    torch.manual_seed(0)
    G = torch.randn(2, 6, 10)                                             # a batch of two wide matrices
    m, n = 6, 10
    U = get_zeropower_fn("svd")(G[0], None)
    assert torch.allclose(U @ U.T, torch.eye(m), atol=1e-5)
    D = get_zeropower_fn("double_normalize")(G, 3)
    assert torch.allclose(D.norm(dim=-1), torch.ones(2, m), atol=1e-5)     # wide: columns first, rows last, so the rows end at norm 1
    S = get_zeropower_fn("sinkhorn_knopp")(G.abs(), 20)
    assert torch.allclose(S.abs().sum(-1), torch.full((2, m), n ** 0.5), rtol=1e-4)
    assert torch.allclose(S.abs().sum(-2), torch.full((2, n), m / n * n ** 0.5), rtol=2e-2)   # doubly scaled after enough rounds
    A = get_zeropower_fn("dualize_1_to_1")(G)
    assert torch.allclose(A.abs().sum(-2), torch.full((2, n), m ** 0.5), rtol=1e-5)
    B = get_zeropower_fn("dualize_inf_to_inf")(G)
    assert torch.allclose(B.abs().sum(-1), torch.full((2, m), n / m ** 0.5), rtol=1e-5)
    F = get_zeropower_fn("dualize_schatten_2_norm")(G)
    assert torch.allclose(torch.linalg.matrix_norm(F), torch.full((2,), m ** 0.5), rtol=1e-5)
    tall = get_zeropower_fn("double_normalize")(G.mT, 2)
    assert torch.allclose(tall.norm(dim=-2), torch.ones(2, m), atol=1e-5)
    ns = get_zeropower_fn("polar_express", run_ns_in_fp16=False)(G[0], steps=8)
    assert torch.allclose(ns @ ns.T, torch.eye(m), atol=2e-2)


def test_spectral_step_clip_and_norm_gradient_against_the_svd():
    from steptronoss_b200.optim.zeropower import (get_clip_fun, get_max_singular_value, get_step_fun,
                                                  weight_decay_in_spectral_norm, zeropower_via_svd)

    torch.manual_seed(0)
    U, _ = torch.linalg.qr(torch.randn(6, 4, dtype=torch.float64))
    V, _ = torch.linalg.qr(torch.randn(4, 4, dtype=torch.float64))
    s = torch.tensor([3.0, 1.5, 0.7, 0.2], dtype=torch.float64)
    M = U @ torch.diag(s) @ V.mT
    exact = lambda G, steps: zeropower_via_svd(G).to(G.dtype)
    assert torch.allclose(get_step_fun(exact, 1.0)(M), U @ torch.diag((s > 1.0).double()) @ V.mT, atol=1e-5)
    assert torch.allclose(get_clip_fun(exact, 1.0)(M), U @ torch.diag(s.clamp(max=1.0)) @ V.mT, atol=1e-5)
    assert float(get_max_singular_value(M)) == pytest.approx(3.0, rel=1e-5)
    lead = U[:, :1] @ V[:, :1].mT
    for mat in (M, M.mT.contiguous(), torch.stack([M, 2 * M])):
        g = weight_decay_in_spectral_norm(mat.clone(), steps=20)
        want = lead if mat.shape == M.shape else (lead.mT if mat.dim() == 2 else torch.stack([lead, lead]))
        sign = torch.sign((g * want).sum())                              # the pair is defined up to a common sign
        assert torch.allclose(g * sign, want, atol=1e-4)
