"""End-to-end training on CPU: single process, and 2 gloo ranks of data parallelism that must
reproduce the single-process loss curve and parameters."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from steptronoss_b200.exp.base_exp import DataConfig
from tests.tiny_exp import make_tiny_exp


class FixedDocsLoader:
    """Each sample packs two documents of 128 tokens; ids uniform in [0, vocab) from seed 0; labels are
    the inputs shifted by one; the loss mask covers the last 64 positions of each document."""

    def __init__(self, dp_rank, dp_size, vocab=1024, n=40):
        g = torch.Generator().manual_seed(0)
        self.all = torch.randint(0, vocab, (n, 2, 129), generator=g)
        self.i, self.dp_rank, self.dp_size = 0, dp_rank, dp_size

    def __iter__(self):
        return self

    def __len__(self):
        return len(self.all)

    def __next__(self):
        docs = self.all[self.i * self.dp_size + self.dp_rank]
        self.i += 1
        ids = docs[:, :-1].reshape(1, -1)
        labels = docs[:, 1:].reshape(1, -1)
        mask = torch.zeros(2, 128)
        mask[:, 64:] = 1.0
        pos = torch.arange(128, dtype=torch.int32).repeat(2)
        return {"input_ids": ids, "labels": labels, "loss_masks": mask.reshape(1, -1),
                "cu_seqlens": torch.tensor([0, 128, 256], dtype=torch.int32),
                "max_seq_len": torch.tensor(128, dtype=torch.int32), "position_id": pos}


class FixedDataConfig(DataConfig):
    global_data_keys = ["cu_seqlens", "position_id", "max_seq_len"]

    def build_dataloader(self, dp_rank=0, dp_size=1):
        return FixedDocsLoader(dp_rank, dp_size)

    def preprocess(self, batch):
        return batch


def _run(exp, steps=10):
    exp.data_cfg = FixedDataConfig
    tr = exp.trainer_cfg.get_trainer_cls()(exp=exp)
    tr.before_train()
    losses = []
    for _ in range(steps):
        tr.train_step()
        tr.iteration += 1
        tr.training_log()
        losses.append(tr.history[-1]["lm_loss"])
    params = {n: p.detach().clone() for n, p in tr.models[0].named_parameters()}
    return losses, params, tr


def _make(zero1=True, **kw):
    e = make_tiny_exp(gbs=2, seq=256, iters=10, lr=1e-3, wd=0.1, clip=1.0, zero1=zero1, **kw)
    e.seed = 0
    e.optimizer_cfg.optimizer_cfg.adam_beta1, e.optimizer_cfg.optimizer_cfg.adam_beta2 = 0.9, 0.95
    return e


def test_single_process_loss_decreases_on_repeated_batch():
    e = _make()
    losses, _, _ = _run(e, steps=10)
    assert all(l == l for l in losses)
    assert 6.5 < losses[0] < 7.5


def _worker(rank, world, port, zero1, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    from steptronoss_b200.parallel.state import PM

    PM.initialize(backend="gloo")
    losses, params, _ = _run(_make(zero1=zero1))
    q.put((rank, losses, {k: v.numpy() for k, v in params.items()}))
    torch.distributed.barrier()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("zero1", [True, False])
def test_dp2_gloo_matches_single_process_exactly(zero1):
    torch.set_num_threads(1)
    os.environ.pop("WORLD_SIZE", None)
    ref_losses, ref_params, _ = _run(_make(zero1=zero1))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, zero1, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, losses, params in results:
        assert losses == ref_losses, f"rank {rank}: {losses} vs {ref_losses}"
        for k, v in ref_params.items():
            assert torch.equal(torch.from_numpy(params[k]), v), f"rank {rank}: parameter {k} differs"


def test_optimizer_state_offload_and_zero_count_do_not_change_the_run(monkeypatch):
    """``offload_optimizer_state`` moves masters and moments off the device around forward/backward and back for
    the update: the loss curve and the parameters stay bit-identical; the memory marks appear in order."""
    from steptronoss_b200.utils.memory_tracker import CMT

    base_losses, base_params, _ = _run(_make(), steps=4)
    e = _make()
    e.trainer_cfg.offload_optimizer_state = True
    e.trainer_cfg.log_num_zeros_in_grad = True
    monkeypatch.setattr(CMT, "enabled", True)
    monkeypatch.setattr(CMT, "marks", [])
    moved = []
    losses, params, tr = _run(e, steps=4)
    gm = tr.grad_manager
    real_off, real_on = gm.offload_state, gm.reload_state
    monkeypatch.setattr(gm, "offload_state", lambda: (moved.append("off"), real_off())[1])
    monkeypatch.setattr(gm, "reload_state", lambda: (moved.append("on"), real_on())[1])
    tr.train_step()
    assert moved == ["off", "on"]
    gm.to_device("cpu")                                   # the reference's spellings take the same paths
    gm.to_device("cuda:0")                                # any non-host device means: back to where the manager lives
    assert moved == ["off", "on", "off", "on"]
    shard = next(iter(gm.shards.values()))
    shard.master.add_(1.0)
    gm.reload_model_params()                              # masters follow the parameters again
    assert torch.equal(shard.master, shard.bucket.param_buf[shard.lo:shard.hi].float())
    assert losses == base_losses
    for k in base_params:
        assert torch.equal(params[k], base_params[k]), k
    names = [m.name for m in CMT.marks][:5]
    assert names == ["before_cpu_offload_optimizer_state", "after_cpu_offload_optimizer_state", "after_forward_backward",
                     "after_cpu_backload_optimizer_state", "after_optimizer_step"]


def test_detailed_gradient_norms_add_up_to_the_global_norm():
    from steptronoss_b200.utils.metrics import GlobalMetrics

    e = _make()
    e.trainer_cfg.log_detailed_grad_norms = True
    tr = e.trainer_cfg.get_trainer_cls()(exp=e)
    tr.before_train()
    tr.train_step()
    parts = GlobalMetrics.grad_norms.reduce()
    total = float(GlobalMetrics.grad_norm.reduce())
    assert set(parts) == {"layer0", "layer1", "tok_embeddings", "output"}
    assert all(float(v) > 0 for v in parts.values())
    assert sum(float(v) ** 2 for v in parts.values()) ** 0.5 == pytest.approx(total, rel=1e-4)


def test_check_nan_names_the_stage_whose_output_went_bad():
    e = _make()
    e.model_cfg.check_nan = True
    tr = e.trainer_cfg.get_trainer_cls()(exp=e)
    tr.before_train()
    tr.train_step()                                              # finite: nothing happens
    with torch.no_grad():
        next(tr.models[0].parameters()).fill_(float("nan"))
    with pytest.raises(FloatingPointError, match="pipeline stage 0"):
        tr.train_step()


def test_step_with_a_non_finite_gradient_is_skipped_and_counted():
    e = _make()
    e.data_cfg = FixedDataConfig
    tr = e.trainer_cfg.get_trainer_cls()(exp=e)
    tr.before_train()
    tr.train_step()
    gm = tr.grad_manager
    assert gm.skipped_steps() == 0
    before = [p.detach().clone() for p in tr.models[0].parameters()]
    hook = next(tr.models[0].parameters()).register_hook(lambda g: torch.full_like(g, float("inf")))
    tr.train_step()
    hook.remove()
    assert gm.skipped_steps() == 1
    assert all(torch.equal(a, b) for a, b in zip(before, tr.models[0].parameters()))    # no update was applied
    tr.train_step()                                                                     # and training goes on
    assert gm.skipped_steps() == 1
    assert not all(torch.equal(a, b) for a, b in zip(before, tr.models[0].parameters()))
    tr.iteration += 1
    tr.training_log()
    assert tr.last_metrics["N-skipped"] == 1


@pytest.mark.parametrize("change", [
    {"model_cfg.recompute": ["attention", "ffn_norm"]},
    {"model_cfg.recompute": True, "model_cfg.recompute_num_layers": 1},
    {"model_cfg.ffn_cfg.swiglu_recompute_silu_out_proj": True},
], ids=["recompute_parts", "recompute_first_layer", "swiglu_in_down_projection"])
def test_memory_options_leave_the_loss_curve_unchanged(change):
    base, _, _ = _run(_make(), steps=3)
    e = _make()
    for path, value in change.items():
        node = e
        *parents, leaf = path.split(".")
        for part in parents:
            node = getattr(node, part)
        setattr(node, leaf, value)
    got, _, _ = _run(e, steps=3)
    assert got == pytest.approx(base, rel=1e-6)


def test_hooks_built_by_the_trainer_config_run_at_their_points():
    from steptronoss_b200.exp.ntp import NTPTrainerConfig

    calls = []

    class HookedTrainer(NTPTrainerConfig):
        def build_after_init_hooks(self):
            return super().build_after_init_hooks() + [lambda tr: calls.append(("after_init", bool(getattr(tr, "models", None))))]

        def build_before_train_hooks(self):
            return [lambda tr: calls.append(("before_train", None))]

        def build_before_step_hooks(self):
            return [lambda tr: calls.append(("before_step", tr.iteration))]

        def build_after_step_hooks(self):
            return [lambda tr: calls.append(("after_step", tr.iteration))]

        def build_after_train_hooks(self):
            return [lambda tr: calls.append(("after_train", tr.iteration))]

    e = _make()
    e.data_cfg = FixedDataConfig
    old = e.trainer_cfg
    e.trainer_cfg = HookedTrainer
    for k in ("global_batch_size", "global_seq_length", "micro_batch_size", "train_iters", "writer_backend", "log_interval"):
        setattr(e.trainer_cfg, k, getattr(old, k))
    e.trainer_cfg.train_iters = 2
    tr = e.trainer_cfg.get_trainer_cls()(exp=e)
    tr.train()
    names = [c[0] for c in calls]
    assert names[:2] == ["after_init", "before_train"] and names[-1] == "after_train"
    assert names.count("before_step") == names.count("after_step") == 2
    assert calls[0] == ("after_init", False)                                       # runs before the models exist
    tr.build_hooks(e.trainer_cfg)                                                  # a second call adds nothing
    assert len(tr._hooks["before_step"]) == 1
    assert [c for c in calls if c[0].endswith("_step")] == [("before_step", 0), ("after_step", 0), ("before_step", 1),
                                                             ("after_step", 1)]    # both inside the step
    tr.train_step()                                                                # driven by hand: hooks still run
    assert [c[0] for c in calls][-2:] == ["before_step", "after_step"]


def test_experiment_hook_selects_operator_back_ends_before_training(monkeypatch, tmp_path):
    import sys

    from steptronoss_b200.utils.optimizable import current_optimization, set_optimization

    e = _make()
    e.data_cfg = FixedDataConfig
    e.trainer_cfg.train_iters = 1
    e.log_dir = str(tmp_path)                          # Exp.train() opens a log file under log_dir / exp_name
    seen = []

    def configure():
        seen.append(set_optimization(AttentionCore="sdpa", grouped_gemm="nv_grouped_gemm"))

    object.__setattr__(e, "configure_optimizable", configure)
    monkeypatch.setattr(sys, "argv", ["exp.py"])
    try:
        e.train()
        assert len(seen) == 1 and current_optimization("AttentionCore") == "sdpa"
    finally:
        set_optimization(AttentionCore=None)
