"""Tensor / sequence / context / pipeline parallel training on gloo ranks reproduces the single-process run."""
import pytest
import torch

from tests.dist_helpers import run_ranks, run_single

BASE = dict(gbs=2, seq=128, iters=3, layers=2, hidden=64, heads=4, kv_heads=2, head_dim=16, ffn=128, vocab=256,
            min_doc=16, max_doc=64)


def _close(a, b, tol):
    return all(abs(x - y) <= tol * max(1.0, abs(y)) for x, y in zip(a, b))


@pytest.fixture(scope="module")
def single():
    torch.set_num_threads(1)
    return run_single(dict(BASE))


@pytest.mark.parametrize("sp", [False, True])
def test_tp2(single, sp):
    res = run_ranks(2, dict(BASE, tp=2, sp=sp))
    for rank, losses, norms, _ in res:
        assert _close(losses, single[0], 2e-5), (rank, losses, single[0])
        assert _close(norms, single[1], 1e-4), (rank, norms, single[1])


def test_cp2(single):
    res = run_ranks(2, dict(BASE, cp=2))
    for rank, losses, norms, _ in res:
        assert _close(losses, single[0], 2e-5), (rank, losses, single[0])
        assert _close(norms, single[1], 1e-4), (rank, norms, single[1])


def test_pp2(single):
    res = run_ranks(2, dict(BASE, pp=2))
    last = res[-1]
    assert _close(last[1], single[0], 2e-5), (last[1], single[0])


def test_pp2_interleaved(single):
    """Two stages x two virtual chunks (4 layers, one per virtual stage), 2 and 4 micro-batches."""
    base4 = dict(BASE, layers=4)
    ref = run_single(dict(base4))
    res = run_ranks(2, dict(base4, pp=2, vpp=2))
    assert _close(res[-1][1], ref[0], 2e-5), (res[-1][1], ref[0])
    ref8 = run_single(dict(base4, gbs=4))
    res8 = run_ranks(2, dict(base4, pp=2, vpp=2, gbs=4))
    assert _close(res8[-1][1], ref8[0], 2e-5), (res8[-1][1], ref8[0])


def test_pp2_with_activations_kept_on_the_host_and_tp2_with_split_saved_inputs(single):
    """Two memory options that must not change the numbers: pipeline stages park saved activations on the host
    (``pipeline_activation_cpu_offload``); recomputed blocks keep 1/TP of their input per rank
    (``distribute_saved_activations``, tensor parallel without sequence parallel)."""
    res = run_ranks(2, dict(BASE, pp=2, set={"model_cfg.pipeline_activation_cpu_offload": True}))
    assert _close(res[-1][1], single[0], 2e-5), (res[-1][1], single[0])
    res = run_ranks(2, dict(BASE, tp=2, sp=False, recompute=True, set={"model_cfg.tp_cfg.distribute_saved_activations": True}))
    for rank, losses, norms, _ in res:
        assert _close(losses, single[0], 2e-5), (rank, losses, single[0])
        assert _close(norms, single[1], 1e-4), (rank, norms, single[1])


def test_uneven_layer_map_with_an_empty_chunk_and_a_placeholder_layer():
    """Three layers over 2 stages x 2 virtual chunks: the last chunk holds no layer at all, or one placeholder that
    passes its input through; both reproduce the three-layer single-process run."""
    base3 = dict(BASE, layers=3)
    ref = run_single(dict(base3))
    res = run_ranks(2, dict(base3, pp=2, vpp=2, set={"model_cfg.chunk_lengths": [1, 1, 1, 0]}))
    assert _close(res[-1][1], ref[0], 2e-5), (res[-1][1], ref[0])
    res = run_ranks(2, dict(base3, pp=2, vpp=2, set={"model_cfg.chunk_lengths": [1, 1, 1, 1], "model_cfg.noop_chunks": [3]}))
    assert _close(res[-1][1], ref[0], 2e-5), (res[-1][1], ref[0])


@pytest.mark.parametrize("layout", [dict(pp=2), dict(), dict(tp=2, sp=True), dict(zero1=False)], ids=["pp2", "dp2_zero1", "tp2_sp", "dp2_allreduce"])
def test_detailed_gradient_norms_agree_on_every_rank_and_add_up(layout):
    """Per-part gradient norms: every rank reports the same numbers, each element is counted once whatever the
    layout (pipeline stages hold different parts, ZeRO owners different parameters, TP ranks different shards)."""
    res = run_ranks(2, dict(BASE, **layout, set={"trainer_cfg.log_detailed_grad_norms": True}))
    parts0 = res[0][2]["parts"]
    assert set(parts0) == {"layer0", "layer1", "tok_embeddings", "output"}
    for rank, _, norms, _ in res:
        assert norms["parts"] == pytest.approx(parts0, rel=1e-6)
        total = norms["total"][-1]
        assert sum(v * v for v in norms["parts"].values()) ** 0.5 == pytest.approx(total, rel=1e-4)


def test_tp2_cp2_pp2_with_muon_on_eight_ranks_matches_one_process():
    """The layout of the long-context configuration (TP=2 x CP=2 x PP=2, 1F1B with 4 micro-batches) with Muon on the
    2-D hidden matrices: the last pipeline stage reports the loss curve of the single-process run."""
    from steptronoss_b200.exp.optimizer import MuonConfig

    muon = {"optimizer_cfg.optimizer_cfg": MuonConfig, "optimizer_cfg.optimizer_cfg.muon_run_ns_in_fp16": False}
    base = dict(BASE, gbs=4, layers=4, seq=256, max_doc=256, lr=2e-3)
    ref = run_single(dict(base, set=dict(muon)))
    res = run_ranks(8, dict(base, tp=2, sp=True, cp=2, pp=2, set=dict(muon)), timeout=600)
    last = res[-1]
    assert _close(last[1], ref[0], 5e-5), (last[1], ref[0])
