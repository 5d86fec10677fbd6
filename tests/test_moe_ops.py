"""MoE routing ops on CPU: histogram with ignored ids, stable aligned index computation,
scatter / weighted gather with gradients, and the routed FFN against a per-expert loop."""
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
