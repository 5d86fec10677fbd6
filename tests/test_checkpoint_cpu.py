"""Native checkpoint: save, resume bit-exactly, refuse incomplete directories."""
import os

import torch

from tests.tiny_exp import make_tiny_exp


def _exp(tmp, iters, interval, qwen=False):
    from steptronoss_b200.exp.checkpointing import CheckpointConfig

    e = make_tiny_exp(gbs=2, seq=128, iters=iters, layers=1, hidden=64, heads=2, kv_heads=1, head_dim=32, ffn=128, vocab=256)
    e._allow_set_new_attr = True
    e.checkpoint_cfg = CheckpointConfig
    e.checkpoint_cfg.save_dir = str(tmp)
    e.checkpoint_cfg.exp_name = "ckpt_test"
    e.checkpoint_cfg.save_interval = interval
    e.checkpoint_cfg.async_save = False
    if qwen:  # the Qwen model class carries the HF <-> native weight mapping
        from steptronoss_b200.models.qwen_dense import QwenModel

        cfg = e.model_cfg
        object.__setattr__(cfg, "build_model", lambda vpp_rank=None: QwenModel(cfg=cfg, layer_map=cfg.build_layer_map(),
                                                                                vpp_rank=vpp_rank))
    return e


def _train(e):
    tr = e.trainer_cfg.get_trainer_cls()(exp=e)
    tr.train()
    return tr


def test_resume_reproduces_uninterrupted_run(tmp_path):
    full = _train(_exp(tmp_path / "a", 6, None))
    ref = {k: v.detach().clone() for k, v in full.models[0].named_parameters()}
    part = _train(_exp(tmp_path / "b", 3, 3))
    latest = open(tmp_path / "b" / "ckpt_test" / "latest_ckpt").read().strip()
    assert latest.endswith("it3") and os.path.exists(os.path.join(latest, "0.success"))
    assert os.path.exists(os.path.join(latest, "TP00_PP000_DP000.pt")) and os.path.exists(os.path.join(latest, "TP00_PP000_DP000_OPT.pt"))
    assert os.path.exists(os.path.join(latest, "data.pkl"))
    resumed = _train(_exp(tmp_path / "b", 6, None))
    assert resumed.iteration == 6
    for k, v in resumed.models[0].named_parameters():
        assert torch.equal(v, ref[k]), k


def test_incomplete_checkpoint_is_ignored(tmp_path):
    e = _exp(tmp_path / "c", 2, 2)
    _train(e)
    d = tmp_path / "c" / "ckpt_test"
    latest = open(d / "latest_ckpt").read().strip()
    os.remove(os.path.join(latest, "0.success"))     # simulate a rank that died before finishing its write
    ck = e.checkpoint_cfg.build_checkpointer()
    assert ck.latest() is None


def test_checkpoint_config_reference_names_aliases_and_save_options():
    from steptronoss_b200.exp.checkpointing import CheckpointConfig

    c = CheckpointConfig()
    c.load_option.none(but=["model"])
    assert c.load_option.model and not c.load_option.optimizer and c.load_options is c.load_option
    c.save_option.all(but=["optimizer"])
    assert c.save_option.model and not c.save_option.optimizer
    c.async_save = False
    assert c.async_dump is False
    c.load_path, c.load_safetensors = "/x", "/y"
    import pytest
    with pytest.raises(AssertionError):
        c.sanity_check()


def test_hf_view_beside_the_checkpoint_starts_a_new_run_and_save_options_drop_parts(tmp_path):
    """``save_safetensors`` writes ``it<N>/hf``; a second run that loads it (weights only) starts from those weights
    with fresh optimizer state and fp32 masters that follow them; ``save_option`` leaves the optimizer file out."""
    e = _exp(tmp_path / "a", 2, 2, qwen=True)
    e.checkpoint_cfg.save_safetensors = True
    e.checkpoint_cfg.save_option.all(but=["optimizer", "data"])
    first = _train(e)
    it = open(tmp_path / "a" / "ckpt_test" / "latest_ckpt").read().strip()
    assert os.path.exists(os.path.join(it, "hf", "model.safetensors.index.json"))
    assert os.path.exists(os.path.join(it, "TP00_PP000_DP000.pt"))
    assert not os.path.exists(os.path.join(it, "TP00_PP000_DP000_OPT.pt")) and not os.path.exists(os.path.join(it, "data.pkl"))
    trained = {k: v.detach().clone() for k, v in first.models[0].named_parameters()}

    e2 = _exp(tmp_path / "b", 1, None, qwen=True)
    e2.checkpoint_cfg.load_safetensors = os.path.join(it, "hf")
    e2.checkpoint_cfg.load_option.none(but=["model"])
    tr = e2.trainer_cfg.get_trainer_cls()(exp=e2)
    tr.before_train()
    assert tr.iteration == 0
    for k, v in tr.models[0].named_parameters():
        assert torch.equal(v, trained[k]), k
    for shard in tr.grad_manager.shards.values():          # masters were refreshed from the loaded weights
        assert torch.equal(shard.master, shard.bucket.param_buf[shard.lo:shard.hi].float())
        assert float(shard.exp_avg.abs().sum()) == 0.0
    before = {k: v.detach().clone() for k, v in tr.models[0].named_parameters()}
    tr.train_step()
    moved = max(float((v - before[k]).abs().max()) for k, v in tr.models[0].named_parameters())
    assert 0 < moved < 0.05                               # one small step away from the loaded weights, not a jump back to the initialisation


def _dp2_save_worker(rank, world, port, save_dir, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    try:
        from steptronoss_b200.parallel.state import PM

        PM.initialize(backend="gloo")
        tr = _train(_exp(save_dir, 3, 3))
        q.put((rank, [h["lm_loss"] for h in tr.history], None))
        torch.distributed.barrier()
    except BaseException:
        import traceback

        q.put((rank, None, traceback.format_exc()))
        raise


def test_optimizer_shards_are_recut_when_the_data_parallel_size_changes(tmp_path):
    """Two ZeRO-1 ranks write a checkpoint; one process resumes from it.  Without ``reshard_optimizer_state`` the
    loader says what to do; with it the run continues exactly like an uninterrupted single-process run."""
    import pytest
    import torch.multiprocessing as mp

    from tests.dist_helpers import free_port

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_dp2_save_worker, args=(r, 2, port, str(tmp_path / "two"), q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        for _ in range(2):
            rank, losses, err = q.get(timeout=300)
            assert err is None, err
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    it = open(tmp_path / "two" / "ckpt_test" / "latest_ckpt").read().strip()
    assert sorted(f for f in os.listdir(it) if f.endswith("_OPT.pt")) == ["TP00_PP000_DP000_OPT.pt", "TP00_PP000_DP001_OPT.pt"]

    full = _train(_exp(tmp_path / "one", 6, None))
    ref = {k: v.detach().clone() for k, v in full.models[0].named_parameters()}

    e = _exp(tmp_path / "two", 6, None)
    with pytest.raises(RuntimeError, match="reshard_optimizer_state"):
        e.trainer_cfg.get_trainer_cls()(exp=e).before_train()
    e = _exp(tmp_path / "two", 6, None)
    e.checkpoint_cfg.reshard_optimizer_state = True
    resumed = _train(e)
    assert resumed.iteration == 6
    for k, v in resumed.models[0].named_parameters():
        assert torch.allclose(v, ref[k], atol=1e-6), k


def test_auto_resume_loads_everything_whatever_the_start_options_say(tmp_path):
    """A job configured to START from foreign weights without their optimizer still RESUMES its own optimizer."""
    full = _train(_exp(tmp_path / "a", 6, None))
    ref = {k: v.detach().clone() for k, v in full.models[0].named_parameters()}
    _train(_exp(tmp_path / "b", 3, 3))
    e = _exp(tmp_path / "b", 6, None)
    e.checkpoint_cfg.load_path = "/somewhere/pretrained"              # what a first start would load ...
    e.checkpoint_cfg.load_option.none(but=["model"])                  # ... weights only
    resumed = _train(e)
    ck = e.checkpoint_cfg
    assert ck.load_path.endswith("it3") and ck.load_option.optimizer and ck.load_option.data and ck.load_safetensors is None
    assert resumed.iteration == 6
    for k, v in resumed.models[0].named_parameters():
        assert torch.equal(v, ref[k]), k
    fresh = _exp(tmp_path / "c", 1, None)                             # nothing to resume: configuration untouched
    fresh.checkpoint_cfg.load_option.none(but=["model"])
    tr = _train(fresh)
    assert not tr.set_autoresume() and not fresh.checkpoint_cfg.load_option.optimizer
