"""Native checkpoint: save, resume bit-exactly, refuse incomplete directories."""
import os

import torch

from tests.tiny_exp import make_tiny_exp


def _exp(tmp, iters, interval):
    from steptronoss_b200.exp.checkpointing import CheckpointConfig

    e = make_tiny_exp(gbs=2, seq=128, iters=iters, layers=1, hidden=64, heads=2, kv_heads=1, head_dim=32, ffn=128, vocab=256)
    e._allow_set_new_attr = True
    e.checkpoint_cfg = CheckpointConfig
    e.checkpoint_cfg.save_dir = str(tmp)
    e.checkpoint_cfg.exp_name = "ckpt_test"
    e.checkpoint_cfg.save_interval = interval
    e.checkpoint_cfg.async_save = False
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
