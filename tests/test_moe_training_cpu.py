"""Whole-model expert parallelism on CPU ranks: EP=2 training follows the single-process run, and a checkpoint
written under EP=2 restores every rank's own experts."""
import os

import pytest
import torch
import torch.multiprocessing as mp

from tests.dist_helpers import free_port


def _exp(save_dir=None, iters=4, interval=None, ep=1):
    from steptronoss_b200.exp.checkpointing import CheckpointConfig
    from tests.test_step3p5_cpu import _make

    e = _make()
    e.seed = 0
    e.trainer_cfg.train_iters = iters
    e.model_cfg.parallel_cfg.expert_model_parallel_size = ep
    e.model_cfg.moe_cfg.router_bias_update_rate = 0.0
    if save_dir is not None:
        e._allow_set_new_attr = True
        e.checkpoint_cfg = CheckpointConfig
        e.checkpoint_cfg.save_dir, e.checkpoint_cfg.exp_name = str(save_dir), "moe_ckpt"
        e.checkpoint_cfg.save_interval, e.checkpoint_cfg.async_save = interval, False
    return e


def _run(e):
    tr = e.trainer_cfg.get_trainer_cls()(exp=e)
    tr.train()
    return tr


def _worker(rank, world, port, save_dir, iters, interval, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    try:
        from steptronoss_b200.parallel.state import PM

        PM.initialize(backend="gloo")
        tr = _run(_exp(save_dir, iters, interval, ep=2))
        experts = {k: v.detach().clone() for k, v in tr.models[0].named_parameters() if ".experts." in k}
        q.put((rank, [h["lm_loss"] for h in tr.history], {k: v.numpy() for k, v in experts.items()}, None))
        torch.distributed.barrier()
    except BaseException:
        import traceback

        q.put((rank, None, None, traceback.format_exc()))
        raise


def _ranks(save_dir, iters, interval):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, save_dir, iters, interval, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(2):
            rank, losses, experts, err = q.get(timeout=300)
            assert err is None, err
            res[rank] = (losses, experts)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    return res


def test_ep2_follows_the_single_process_run_and_resumes_with_each_ranks_own_experts(tmp_path):
    single = _run(_exp(iters=4))
    want = [h["lm_loss"] for h in single.history]
    full = _ranks(str(tmp_path / "full"), 4, None)
    for rank in (0, 1):
        assert full[rank][0] == pytest.approx(want, rel=2e-4), (rank, full[rank][0], want)
    _ranks(str(tmp_path / "cut"), 2, 2)                               # two iterations, checkpoint, stop
    it = open(tmp_path / "cut" / "moe_ckpt" / "latest_ckpt").read().strip()
    assert it.endswith("it2") and os.path.exists(os.path.join(it, "TP00_PP000_DP001.pt"))
    resumed = _ranks(str(tmp_path / "cut"), 4, None)                  # picks the checkpoint up, runs iterations 3 and 4
    for rank in (0, 1):
        assert resumed[rank][0] == pytest.approx(full[rank][0], rel=1e-5)   # the history of the first half is restored too
        for k, v in full[rank][1].items():
            assert abs(resumed[rank][1][k] - v).max() < 1e-5, (rank, k)
    # the two ranks hold different experts: a resume that handed rank 0's experts to rank 1 would not pass the above
    k = next(iter(full[0][1]))
    assert abs(full[0][1][k] - full[1][1][k]).max() > 1e-3
