"""Scheduler configurations (reference ``steptronoss/exp/lr_schedulers.py:8-134``)."""
from __future__ import annotations

from .abstract import SchedulerConfig as AbstractSchedulerConfig


class SchedulerConfig(AbstractSchedulerConfig):
    lr: float = 1e-4
    min_lr: float = 0.0
    weight_decay: float = 0.01
    total_schedule: float = 1000
    warmup_schedule: float = 100
    scheduler_unit: str = "iter"
    shape: str = "constant"

    def sanity_check(self) -> None:
        super().sanity_check()
        assert self.min_lr <= self.lr
        assert self.scheduler_unit in ("iter", "sample", "token")

    def increment(self, global_batch_size: int, tokens: int) -> int:
        """Progress added by one optimizer step in this scheduler's unit."""
        return {"iter": 1, "sample": global_batch_size, "token": tokens}[self.scheduler_unit]

    def build_scheduler(self, optimizer, *args):
        from ..optim.hparam_scheduler import Scheduler, WarmupShape

        return Scheduler(optimizer=optimizer, base_lr=self.lr, base_wd=self.weight_decay,
                         lr_func=WarmupShape(self.shape, self.total_schedule, self.warmup_schedule,
                                             self.min_lr / self.lr if self.lr else 0.0),
                         wd_func=lambda x: 1.0)


class ConstantSchedulerConfig(SchedulerConfig):
    shape = "constant"


class LinearSchedulerConfig(SchedulerConfig):
    shape = "linear"


class CosineSchedulerConfig(SchedulerConfig):
    shape = "cosine"


class InvSqrtSchedulerConfig(SchedulerConfig):
    shape = "inv_sqrt"


class CosineWithReWarmupSchedulerConfig(SchedulerConfig):
    re_warmup: float = 0
    start_token: float = 0
    re_warmup_min: float = 0.0
    re_warmup_max: float | None = None
    start_bias: float = 0

    def build_scheduler(self, optimizer, *args):
        from ..optim.hparam_scheduler import CosineFuncWithReWarmup, Scheduler

        fn = CosineFuncWithReWarmup(self.total_schedule, self.warmup_schedule, self.min_lr / self.lr, self.re_warmup,
                                    self.start_token, self.re_warmup_min, self.re_warmup_max, self.start_bias)
        return Scheduler(optimizer=optimizer, base_lr=self.lr, base_wd=self.weight_decay, lr_func=fn,
                         wd_func=lambda x: 1.0)
