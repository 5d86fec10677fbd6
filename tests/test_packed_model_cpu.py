"""PackedModel: forward/backward + optimizer step through the bundle, and host offload of each part."""
import torch

from tests.tiny_exp import make_tiny_exp


def _packed(training=True):
    from steptronoss_b200.parallel.state import PM, set_mpu_random_seed
    from steptronoss_b200.trainers.packed_model import PackedModel

    exp = make_tiny_exp(hidden=64, heads=2, kv_heads=1, head_dim=32, ffn=128, vocab=128, layers=2, seq=64, gbs=2)
    PM.initialize()
    PM.set_mesh(exp.model_cfg.parallel_cfg)
    set_mpu_random_seed(0)
    pm = PackedModel(exp.trainer_cfg, exp.model_cfg, exp.optimizer_cfg, exp.scheduler_cfg, training=training, seed=3)
    return exp, pm


def _batches(exp, n):
    loader = exp.data_cfg.build_dataloader(0, 1)
    it = iter(loader)
    return [next(it) for _ in range(n)]


def test_packed_model_trains_and_offloads_each_part():
    exp, pm = _packed()
    tc = exp.trainer_cfg
    data = _batches(exp, 6)
    losses = []

    def loss_fn(d, out, scale):
        loss = tc.loss_func(d, out, scale)
        losses.append(float(out["lm_loss"]) if isinstance(out, dict) and "lm_loss" in out else None)
        return loss

    for step in range(3):
        pm.forward_backward(data[2 * step: 2 * step + 2], exp.data_cfg.preprocess, loss_fn=tc.loss_func)
        ok, grad_norm, _ = pm.optimizer_step()
        assert ok
    before = {n: p.detach().clone() for n, p in pm.models.named_parameters()}
    # every part goes to the host and comes back unchanged
    pm.offload_model()
    assert all(p.device.type == "cpu" for p in pm.models.parameters())
    pm.offload_state()
    assert all(p.main_grad is None for p in pm.models.parameters())
    pm.backload_model()
    pm.backload_state()
    for n, p in pm.models.named_parameters():
        assert torch.equal(p, before[n]) and p.main_grad is not None and float(p.main_grad.abs().sum()) == 0.0
    with pm.on_gpu():
        pm.forward_backward(data[:2], exp.data_cfg.preprocess, loss_fn=tc.loss_func)
        pm.optimizer_step()
    moved = sum(float((p - before[n]).abs().sum()) for n, p in pm.models.named_parameters())
    assert moved > 0


def test_packed_model_hydrates_from_state_dicts_and_runs_forward_only():
    from steptronoss_b200.trainers.packed_model import PackedModel

    exp, pm = _packed()
    sd = pm.state_dicts()
    ref = PackedModel(exp.trainer_cfg, exp.model_cfg, training=False, state_dicts={"model": sd["model"]}, seed=99)
    for (n, a), (_, b) in zip(pm.models.named_parameters(), ref.models.named_parameters()):
        assert torch.equal(a, b), n
    data = _batches(exp, 2)
    outs = ref.forward_backward(data, exp.data_cfg.preprocess, collect_output=True)
    assert len(outs) == 2
