"""MoE routing ops on CPU: histogram with ignored ids, stable aligned index computation,
scatter / weighted gather with gradients, and the routed FFN against a per-expert loop."""
import pytest
import torch

from steptronoss_b200.ops import moe


def test_histogram_ignores_minus_one():
    ids = torch.tensor([[0, 2], [2, -1], [-1, -1], [3, 2]])
    assert moe.histogram(ids, 4).tolist() == [1, 0, 3, 1]


def test_index_compute_is_stable_and_aligned():
    ids = torch.tensor([[1, 0], [1, -1], [0, 1], [2, 1]])
    dest, offsets, counts = moe.index_compute(ids, 3)
    assert counts.tolist() == [2, 4, 1]
    assert offsets.tolist() == [0, 128, 256, 384]
    # expert 1 slots in token order: (0,0) (1,0) (2,1) (3,1)
    assert dest[0, 0] == 128 and dest[1, 0] == 129 and dest[2, 1] == 130 and dest[3, 1] == 131
    assert dest[0, 1] == 0 and dest[2, 0] == 1 and dest[3, 0] == 256 and dest[1, 1] == -1


def test_scatter_gather_roundtrip_and_grads():
    torch.manual_seed(0)
    T, K, H, E = 20, 2, 8, 4
    x = torch.randn(T, H, requires_grad=True)
    ids = torch.randint(-1, E, (T, K))
    w = torch.rand(T, K, requires_grad=True)
    dest, offsets, _ = moe.index_compute(ids, E)
    xe = moe.moe_scatter(x, dest, moe.padded_rows(T * K, E))
    out = moe.moe_weighted_gather(xe, dest, w)
    ref = x * (w * (ids >= 0)).sum(1, keepdim=True)
    assert torch.allclose(out, ref, atol=1e-6)
    g = torch.randn(T, H)
    out.backward(g)
    gx, gw = torch.autograd.grad((ref * g).sum(), [x, w])
    assert torch.allclose(x.grad, gx, atol=1e-5) and torch.allclose(w.grad, gw, atol=1e-5)


def test_routed_ffn_matches_expert_loop_with_grads():
    torch.manual_seed(1)
    T, K, H, F, E = 64, 2, 16, 24, 5
    x = torch.randn(T, H, requires_grad=True)
    w1 = (0.3 * torch.randn(E, 2 * F, H)).requires_grad_()
    w2 = (0.3 * torch.randn(E, H, F)).requires_grad_()
    ids = torch.stack([torch.randperm(E)[:K] for _ in range(T)])
    ids[3, 1] = -1
    wt = torch.rand(T, K, requires_grad=True)
    out = moe.routed_grouped_ffn(x, ids, wt, w1, w2)
    g = torch.randn(T, H)
    grads = torch.autograd.grad((out * g).sum(), [x, w1, w2, wt])
    ref = moe.routed_grouped_ffn_reference(x, ids, wt, w1, w2)
    rgrads = torch.autograd.grad((ref * g).sum(), [x, w1, w2, wt])
    assert torch.allclose(out, ref, atol=1e-4)
    for a, b in zip(grads, rgrads):
        assert torch.allclose(a, b, atol=1e-4)


def test_permute_unpermute_round_trip_mask_and_index():
    import torch

    from steptronoss_b200.ops.permute import (moe_permute, moe_permute_with_probs, moe_sort_chunks_by_index,
                                              moe_unpermute)

    torch.manual_seed(0)
    T, E, K, H = 6, 4, 2, 3
    x = torch.randn(T, H)
    ids = torch.stack([torch.randperm(E)[:K] for _ in range(T)])
    probs_k = torch.rand(T, K)
    mask = torch.zeros(T, E, dtype=torch.bool).scatter_(1, ids, True)
    probs_e = torch.zeros(T, E).scatter_(1, ids, probs_k)
    out, pp, rmap = moe_permute_with_probs(x, probs_e, mask)
    assert out.shape == (T * K, H)
    experts = rmap // T
    assert torch.all(experts[1:] >= experts[:-1])                      # expert-major
    assert torch.equal(out, x[rmap % T]) and torch.allclose(pp, probs_e.t().reshape(-1)[rmap])
    back = moe_unpermute(out, rmap, merging_probs=probs_e)
    want = x * probs_k.sum(1, keepdim=True)
    assert torch.allclose(back, want, atol=1e-6)
    out_i, rmap_i = moe_permute(x, ids, map_type="index")
    assert torch.equal(out_i, x[rmap_i // K])
    back_i = moe_unpermute(out_i, rmap_i, merging_probs=probs_k, map_type="index")
    assert torch.allclose(back_i, want, atol=1e-6)
    padded, rmap_p = moe_permute(x, mask, num_out_tokens=T * K + 3)
    assert padded.shape[0] == T * K + 3 and int((rmap_p < 0).sum()) == 3 and float(padded[-3:].abs().sum()) == 0
    chunks = moe_sort_chunks_by_index(torch.arange(6).unsqueeze(1), torch.tensor([1, 2, 3]), torch.tensor([2, 0, 1]))
    assert chunks.flatten().tolist() == [3, 4, 5, 0, 1, 2]


def test_route_plan_matches_index_compute_and_inverts_dest():
    torch.manual_seed(4)
    T, K, E = 200, 3, 7
    ids = torch.stack([torch.randperm(E)[:K] for _ in range(T)])
    ids[::5, 2] = -1
    plan = moe.RoutePlan(ids, E)
    dest, offsets, counts = moe.index_compute(ids, E)
    assert torch.equal(plan.dest, dest) and torch.equal(plan.offsets, offsets) and torch.equal(plan.counts, counts)
    assert plan.rows == moe.padded_rows(T * K, E) and plan.slot_of_row.shape == (plan.rows,)
    d = dest.reshape(-1)
    valid = d >= 0
    assert torch.equal(plan.slot_of_row[d[valid]].long(), torch.arange(T * K)[valid])
    assert int((plan.slot_of_row >= 0).sum()) == int(valid.sum())


def test_router_reference_gives_sorted_top_k_and_normalised_weights():
    torch.manual_seed(2)
    logits = torch.randn(50, 12)
    bias = torch.randn(12) * 0.1
    ids, w, ps, hist, stats = moe.router_reference(logits, bias, 3, True, True, 1e-20)
    assert ids.shape == (50, 3) and torch.allclose(w.sum(1), torch.ones(50), atol=1e-5)
    assert torch.allclose(ps.sum(), torch.tensor(50.0), atol=1e-3) and int(hist.sum()) == 150
    sel = torch.sigmoid(logits) + bias
    assert torch.equal(ids, sel.topk(3, dim=1).indices)
    assert float(stats[0]) == float(logits.abs().max())


def test_expert_parallel_moe_block_on_two_gloo_ranks():
    """The worker of the 2-GPU test also runs on CPU ranks: there both dispatcher names resolve to the
    all-to-all path, which checks the expert-parallel block end to end (router, dispatch, experts, combine)."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29743", os.path.join(root, "tests", "mp_moe_worker.py")]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=root)
    assert out.returncode == 0, out.stderr[-3000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    assert len(res) == 24 and max(res.values()) < 1e-6


def test_set_optimization_switches_registered_ops_to_their_reference_statement():
    from steptronoss_b200.utils.optimizable import OPTIMIZABLE_REGISTER, set_optimization

    name = moe.routed_grouped_ffn.__optimizable_name__
    assert name.endswith("ops.moe.routed_grouped_ffn") and "reference" in OPTIMIZABLE_REGISTER[name]["alternatives"]
    torch.manual_seed(0)
    x, w1, w2 = torch.randn(16, 8), torch.randn(3, 12, 8) * 0.3, torch.randn(3, 8, 6) * 0.3
    ids = torch.randint(0, 3, (16, 2))
    wt = torch.rand(16, 2)
    base = moe.routed_grouped_ffn(x, ids, wt, w1, w2)
    calls = []
    OPTIMIZABLE_REGISTER[name]["alternatives"]["spy"] = lambda *a, **k: calls.append(1) or moe.routed_grouped_ffn_reference(*a[:5])
    try:
        assert set_optimization(routed_grouped_ffn="spy") == {name: "spy"}        # short name
        assert torch.allclose(moe.routed_grouped_ffn(x, ids, wt, w1, w2), base, atol=1e-5) and calls == [1]
        assert set_optimization(routed_grouped_ffn="no-such-backend") == {}          # unknown: kept, with a warning
        assert OPTIMIZABLE_REGISTER[name]["use_optimize"] == "spy"
        assert set_optimization(default="reference")[name] == "reference"           # every op that has one
        assert set_optimization(**{name: "native"}) == {name: "native"}             # full name, back to the kernel path
        assert OPTIMIZABLE_REGISTER[name]["use_optimize"] is None
    finally:
        set_optimization(routed_grouped_ffn=None, fused_router=None)
        OPTIMIZABLE_REGISTER[name]["alternatives"].pop("spy", None)


def test_reference_experiment_switches_select_what_exists_here():
    """An experiment file written for the reference calls ``set_optimization`` with its own operator and back-end
    names; every one of them maps to an entry here, accelerated back-ends mean the kernel path."""
    import importlib

    from steptronoss_b200.parallel import ep_dispatcher

    attn_ops = importlib.import_module("steptronoss_b200.ops.attention")      # the package also exports the function
    from steptronoss_b200.utils.optimizable import current_optimization, set_optimization

    chosen = set_optimization(routed_grouped_ffn="fused", moe_weighted_gather="triton", moe_scatter="triton",
                              histogram="triton", index_compute="triton", TokenDispatcher="deep_ep",
                              grouped_gemm="nv_grouped_gemm", AttentionCore="flash-attn-3")
    try:
        assert chosen[ep_dispatcher.TokenDispatcher.__optimizable_name__] == "deep_ep"
        assert chosen[attn_ops.attention.__optimizable_name__] == "flash-attn-3"
        assert current_optimization("AttentionCore") is None and current_optimization("grouped_gemm") is None
        assert current_optimization("TokenDispatcher") == "deep_ep"
        set_optimization(AttentionCore="sdpa", grouped_gemm="function_imple")
        assert current_optimization("attention") == "sdpa" and current_optimization("grouped_gemm") == "function_imple"
        q = torch.randn(12, 4, 8)
        cu = torch.tensor([0, 5, 12], dtype=torch.int32)
        assert torch.equal(attn_ops.attention(q, q[:, :2], q[:, :2], cu, cu, 7),
                           attn_ops.attention_reference(q, q[:, :2], q[:, :2], cu, cu))
    finally:
        set_optimization(AttentionCore=None, grouped_gemm=None, TokenDispatcher=None)
    assert current_optimization("TokenDispatcher") is None


def test_grouped_gemm_entry_with_the_reference_signature():
    a = torch.randn(9, 6, dtype=torch.float64, requires_grad=True)
    w = torch.randn(3, 4, 6, dtype=torch.float64, requires_grad=True)
    sizes = torch.tensor([2, 0, 7])
    y = moe.grouped_gemm(a, w, sizes, trans_b=True)
    want = torch.cat([a[:2] @ w[0].t(), a[2:] @ w[2].t()])
    assert torch.allclose(y, want)
    y.sum().backward()
    assert torch.allclose(w.grad[1], torch.zeros(4, 6, dtype=torch.float64)) and a.grad is not None
    y2 = moe.grouped_gemm(a.detach(), w.detach().transpose(1, 2).contiguous(), sizes)          # [G, K, N]
    assert torch.allclose(y2, want)
    assert moe.grouped_gemm(a[:0].detach(), w.detach(), torch.tensor([0, 0, 0]), trans_b=True).shape == (0, 4)


def test_attention_core_module_follows_the_reference_call_surface():
    from steptronoss_b200.ops.attention import AttentionCore, FlashAttention, parse_cu_seqlens

    torch.manual_seed(0)
    q, k, v = torch.randn(2, 10, 4, 8), torch.randn(2, 10, 2, 8), torch.randn(2, 10, 2, 8)
    qi, kj = torch.arange(10)[:, None], torch.arange(10)[None]
    kk, vv = (t.transpose(1, 2).repeat_interleave(2, 1) for t in (k, v))
    for w, mask in ((-1, kj <= qi), (3, (kj <= qi) & (kj >= qi - 3))):           # w keys to the left and the query itself
        out = AttentionCore(sliding_window=w).eval()(q, k, v)
        want = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), kk, vv, attn_mask=mask).transpose(1, 2)
        assert torch.allclose(out, want, atol=1e-5)
    # packed stream: 20 rows cut at 7; the second table form names queries and keys separately
    cu = torch.tensor([0, 7, 20])
    packed = FlashAttention()(q, k, v, cu_seqlens=cu)
    assert torch.allclose(packed.reshape(20, 4, 8)[:7], AttentionCore()(q[:, :7][:1], k[:, :7][:1], v[:, :7][:1])[0], atol=1e-5)
    cq, ck, mq, mk = parse_cu_seqlens({"q": torch.tensor([0, 3]), "k": torch.tensor([0, 10])})
    assert (cq.dtype, mq, mk) == (torch.int32, 3, 10)
    tail = AttentionCore()(q[:1, 7:], k[:1], v[:1], cu_seqlens={"q": torch.tensor([0, 3]), "k": torch.tensor([0, 10])})
    assert torch.allclose(tail, AttentionCore()(q[:1], k[:1], v[:1])[:, 7:], atol=1e-5)    # causality aligned to the key end
    m = AttentionCore(attention_dropout=0.5).train()
    torch.manual_seed(1)
    a = m(q, k, v)
    assert not torch.allclose(a, m.eval()(q, k, v)) and torch.isfinite(a).all()
    with pytest.raises(ValueError):
        AttentionCore(causal=False, sliding_window=4)
