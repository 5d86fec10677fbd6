"""Learning-rate shapes, the cosine schedule with a second warm-up, and the scheduler's writes and state."""
import math

import pytest
import torch


def test_shapes_after_linear_warmup():
    from steptronoss_b200.optim import hparam_scheduler as hs

    for make in (hs.FuncConstant, hs.FuncLinear, hs.FuncCosineDecr, hs.FuncCosineIncr, hs.FuncInvSqrt):
        f = make(n=110, warmup=10, min_scale=0.1)
        assert f(0) == 0.0 and f(5) == 0.5 and f(10) == 1.0          # warm-up is the same for every shape
    assert hs.FuncConstant(n=110, warmup=10)(70) == 1.0
    lin = hs.FuncLinear(n=110, warmup=10, min_scale=0.1)
    assert lin(60) == pytest.approx(0.1 + 0.9 * 0.5) and lin(110) == pytest.approx(0.1) and lin(500) == 0.0   # clip_min
    cos = hs.FuncCosineDecr(n=110, warmup=10, min_scale=0.1)
    assert cos(60) == pytest.approx(0.1 + 0.9 * 0.5) and cos(110) == pytest.approx(0.1) == cos(10_000)
    up = hs.FuncCosineIncr(n=110, warmup=10)
    assert up(11) < 0.01 and up(60) == pytest.approx(0.5) and up(110) == pytest.approx(1.0)
    inv = hs.FuncInvSqrt(n=10_000, warmup=100)
    assert inv(150) == 1.0 and inv(200) == pytest.approx(1.0) and inv(500) == pytest.approx(math.sqrt(100 / 400))
    with pytest.raises(AssertionError):
        hs.FuncLinear(n=10, warmup=10)


def test_cosine_with_second_warmup():
    from steptronoss_b200.optim.hparam_scheduler import CosineFuncWithReWarmup

    plain = CosineFuncWithReWarmup(n=1000, warmup=100, clip_min=0.1)
    assert plain(0) == 0.0 and plain(50) == 0.5 and plain(100) == pytest.approx(1.0)
    assert plain(550) == pytest.approx(0.1 + 0.9 * 0.5) and plain(1000) == pytest.approx(0.1) == plain(5000)
    re = CosineFuncWithReWarmup(n=1000, warmup=100, clip_min=0.1, re_warmup=50, start_token=400, re_warmup_min=0.2)
    assert re(399) == pytest.approx(plain(399))
    assert re(400) == pytest.approx(0.2) and re(425) == pytest.approx((0.2 + plain(450)) / 2)
    assert re(450) == pytest.approx(plain(450)) and re(700) == pytest.approx(plain(700))   # joins the cosine again
    capped = CosineFuncWithReWarmup(n=1000, warmup=100, re_warmup=50, start_token=400, re_warmup_max=0.3)
    assert capped(449.999) == pytest.approx(0.3, abs=1e-3)
    late = CosineFuncWithReWarmup(n=1000, warmup=100, start_bias=200)
    assert late(150) == 0.0 and late(250) == pytest.approx(0.5) and late(300) == pytest.approx(1.0)
    with pytest.raises(AssertionError):
        CosineFuncWithReWarmup(n=1000, re_warmup=10, start_token=5, start_bias=5)


def test_scheduler_writes_groups_and_restores():
    from steptronoss_b200.exp.lr_schedulers import CosineSchedulerConfig, CosineWithReWarmupSchedulerConfig
    from steptronoss_b200.optim.hparam_scheduler import Scheduler

    w = torch.nn.Parameter(torch.zeros(2))
    opt = torch.optim.SGD([{"params": [w], "lr_mult": 0.5, "wd_mult": 0.0}, {"params": [torch.nn.Parameter(torch.zeros(1))]}], lr=1.0)
    cfg = CosineSchedulerConfig()
    cfg.lr, cfg.min_lr, cfg.weight_decay, cfg.total_schedule, cfg.warmup_schedule, cfg.scheduler_unit = 2e-3, 2e-4, 0.1, 110, 10, "sample"
    cfg.sanity_check()
    assert cfg.increment(global_batch_size=8, tokens=4096) == 8
    s = cfg.build_scheduler(opt)
    assert s.cur_lr == 0.0
    s.step(5)
    assert [g["lr"] for g in opt.param_groups] == [pytest.approx(0.5e-3), pytest.approx(1e-3)]
    assert [g["weight_decay"] for g in opt.param_groups] == [0.0, pytest.approx(0.1)]
    s.step(55)                                                       # half of the decay span
    assert s.cur_lr == pytest.approx(2e-4 + (2e-3 - 2e-4) * 0.5)
    state = s.state_dict()
    assert state["num_tokens"] == 60
    fresh = cfg.build_scheduler(opt)
    fresh.load_state_dict(state)
    assert fresh.cur_lr == pytest.approx(s.cur_lr) and opt.param_groups[1]["lr"] == pytest.approx(s.cur_lr)
    keep = Scheduler(opt, 9.0, 0.0, lambda x: 1.0, lambda x: 1.0, use_checkpointed=True)
    keep.load_state_dict(state)
    assert keep.base_lr == 2e-3                                       # the checkpointed base wins when asked for
    rw = CosineWithReWarmupSchedulerConfig()
    rw.lr, rw.min_lr, rw.total_schedule, rw.warmup_schedule, rw.re_warmup, rw.start_token = 1.0, 0.1, 1000, 100, 50, 400
    r = rw.build_scheduler(None)
    r.step(400)
    assert r.cur_lr == 0.0                                            # the second warm-up starts from re_warmup_min
    with pytest.raises(AssertionError):
        Scheduler(None, 1.0, 0.0, 1.0, lambda x: 1.0)


def test_custom_shape_by_overriding_get():
    from steptronoss_b200.optim.hparam_scheduler import FuncLinear, ScaleFnWithWarmUpAndClip, ScaleFunction

    class Quadratic(ScaleFnWithWarmUpAndClip):
        def get(self, x):
            return (1 - min(x, self.n) / self.n) ** 2

    f = Quadratic(n=110, warmup=10, min_scale=0.1, clip_min=0.15)
    assert isinstance(f, ScaleFunction) and f.n == 100
    assert f(5) == 0.5 and f(10) == 1.0                                   # linear warm-up, then the shape from its start
    assert f(60) == pytest.approx(0.9 * 0.25 + 0.1) and f(110) == 0.15 and f(500) == 0.15     # floor, then the clip
    base = ScaleFnWithWarmUpAndClip(n=20, warmup=0)
    assert base(7) == 1.0
    lin, mine = FuncLinear(n=50, warmup=5, min_scale=0.2), type("L", (ScaleFnWithWarmUpAndClip,), {"get": lambda s, x: 1 - x / s.n})(50, 5, 0.2)
    assert all(lin(x) == pytest.approx(mine(x)) for x in (0, 3, 5, 20, 50))
    with pytest.raises(NotImplementedError):
        ScaleFunction(3)(1)
