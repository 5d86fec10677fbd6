"""Learning-rate / weight-decay schedules driven by a progress counter (iterations, samples or
tokens).  Behaviour of the reference (``steptronoss/optimizer/hparam_scheduler.py:14-236``): linear
warm-up, a shape function on the remaining span scaled into ``[min_scale, 1]`` and clipped; a
cosine schedule with a second warm-up; state = the counter (named ``num_tokens`` in checkpoints).
"""
from __future__ import annotations

import math
from typing import Callable

_SHAPES: dict[str, Callable[[float, float, float], float]] = {
    # (x after warm-up, span, warm-up length) -> value in [0, 1] before min-scale mapping
    "constant": lambda x, n, w: 1.0,
    "linear": lambda x, n, w: 1.0 - x / n,
    "cosine": lambda x, n, w: 0.5 * (math.cos(math.pi * min(x, n) / n) + 1.0),
    "cosine_incr": lambda x, n, w: 0.5 * (math.cos(math.pi * (1.0 - min(x, n) / n)) + 1.0),
    # the reference's rule: sqrt(warmup / steps since the warm-up ended); above 1 (hence clipped) until 2 x warmup
    "inv_sqrt": lambda x, n, w: (w ** 0.5) / (x ** 0.5) if x > 0 else 1.0,
}


class WarmupShape:
    """``f(progress) -> scale``: ``progress/warmup`` during warm-up, then the named shape."""

    def __init__(self, shape: str, n: float = 0, warmup: float = 0, min_scale: float = 0.0, clip_max: float = 1.0,
                 clip_min: float = 0.0):
        if not warmup < n:
            raise AssertionError("Warmup should less than total!")
        self.shape, self.span, self.warmup = shape, n - warmup, warmup
        self.min_scale, self.clip_max, self.clip_min = min_scale, clip_max, clip_min

    def __call__(self, x: float) -> float:
        if self.warmup and x <= self.warmup:
            return x / self.warmup
        v = _SHAPES[self.shape](x - self.warmup, self.span, self.warmup)
        v = (1.0 - self.min_scale) * v + self.min_scale
        return min(max(v, self.clip_min), self.clip_max)


class ScaleFunction:
    """Base of user-written schedules: ``__call__(progress) -> scale`` with the horizon in ``self.n``."""

    def __init__(self, n: float):
        self.n = n

    def __call__(self, x: float) -> float:
        raise NotImplementedError


class ScaleFnWithWarmUpAndClip(WarmupShape, ScaleFunction):
    """A schedule of one's own with the stock warm-up, floor and clipping: override ``get(x)``, the shape after
    warm-up as a function of the progress since warm-up ended (``self.n`` is the horizon without the warm-up, as in
    the reference: optimizer/hparam_scheduler.py:29-62)::

        class Quadratic(ScaleFnWithWarmUpAndClip):
            def get(self, x):
                return (1 - min(x, self.n) / self.n) ** 2
    """

    def __init__(self, n: float = 0, warmup: float = 0, min_scale: float = 0.0, clip_max: float = 1.0, clip_min: float = 0.0):
        WarmupShape.__init__(self, "constant", n, warmup, min_scale, clip_max, clip_min)
        self.n = self.span

    def get(self, x: float) -> float:
        return 1.0

    def __call__(self, x: float) -> float:
        if self.warmup and x <= self.warmup:
            return x / self.warmup
        v = (1.0 - self.min_scale) * self.get(x - self.warmup) + self.min_scale
        return min(max(v, self.clip_min), self.clip_max)


def FuncConstant(n=0, warmup=0, min_scale=0, **kw):  # noqa: N802
    return WarmupShape("constant", n, warmup, min_scale, **kw)


def FuncLinear(n=0, warmup=0, min_scale=0, **kw):  # noqa: N802
    return WarmupShape("linear", n, warmup, min_scale, **kw)


def FuncCosineDecr(n=0, warmup=0, min_scale=0, **kw):  # noqa: N802
    return WarmupShape("cosine", n, warmup, min_scale, **kw)


def FuncCosineIncr(n=0, warmup=0, min_scale=0, **kw):  # noqa: N802
    return WarmupShape("cosine_incr", n, warmup, min_scale, **kw)


def FuncInvSqrt(n=0, warmup=0, min_scale=0, **kw):  # noqa: N802
    return WarmupShape("inv_sqrt", n, warmup, min_scale, **kw)


class CosineFuncWithReWarmup:
    """Cosine decay to ``clip_min`` at ``n`` after a warm-up that may start at ``start_bias``; between
    ``start_token`` and ``start_token + re_warmup`` the scale ramps linearly from ``re_warmup_min`` up to
    the value the cosine has at the end of the ramp (or ``re_warmup_max``)."""

    def __init__(self, n, warmup=0, clip_min: float = 0, re_warmup=0, start_token=0, re_warmup_min: float = 0,
                 re_warmup_max: float | None = None, start_bias: float = 0):
        self.end, self.warmup = n, warmup + start_bias
        self.clip_min, self.re_warmup, self.start_bias = clip_min, re_warmup, start_bias
        if re_warmup > 0:
            if not start_token > start_bias:
                raise AssertionError("start_token must be greater than start_bias")
            self.start_token = start_token
            self.re_end = re_warmup + start_token
            top = self._decay(self.re_end) if re_warmup_max is None else re_warmup_max
            self.re_max, self.re_min = max(top, 0), max(re_warmup_min, 0)

    def _decay(self, x: float) -> float:
        if self.warmup and x < self.warmup:
            if self.warmup <= self.start_bias:
                return 0.0
            return max(0.0, (x - self.start_bias) / (self.warmup - self.start_bias))
        prog = min((x - self.warmup) / (self.end - self.warmup), 1.0)
        return max(self.clip_min + (1.0 - self.clip_min) * 0.5 * (1.0 + math.cos(math.pi * prog)), 0.0)

    def __call__(self, x: float) -> float:
        if self.re_warmup > 0 and self.start_token <= x < self.re_end:
            t = min(max((x - self.start_token) / self.re_warmup, 0.0), 1.0)
            return (1 - t) * self.re_min + t * self.re_max
        return self._decay(x)


class Scheduler:
    """Writes ``lr`` / ``weight_decay`` into ``optimizer.param_groups`` from a progress counter."""

    def __init__(self, optimizer, base_lr: float, base_wd: float, lr_func: Callable, wd_func: Callable,
                 use_checkpointed: bool = False):
        if not callable(lr_func) or not callable(wd_func):
            raise AssertionError("lr_func and wd_func must be callables f(progress) -> scale")
        self.optimizer = optimizer
        self.base_lr, self.base_wd = base_lr, base_wd
        self.lr_func, self.wd_func = lr_func, wd_func
        self.num_tokens = 0
        self.cur_lr = self.cur_wd = None
        self.use_checkpointed = use_checkpointed
        self.step(0)

    def get_lr(self) -> float:
        return self.base_lr * self.lr_func(self.num_tokens)

    def get_wd(self) -> float:
        return self.base_wd * self.wd_func(self.num_tokens)

    def step(self, increment) -> None:
        self.num_tokens += increment
        self.cur_lr, self.cur_wd = self.get_lr(), self.get_wd()
        try:
            from ..utils.metrics import GlobalMetrics

            if "learning_rate" in GlobalMetrics.metrics:
                GlobalMetrics.learning_rate.add(self.cur_lr)
        except Exception:
            pass
        if self.optimizer is not None:
            for g in self.optimizer.param_groups:
                g["lr"] = self.cur_lr * g.get("lr_mult", 1.0)
                g["weight_decay"] = self.cur_wd * g.get("wd_mult", 1.0)

    def state_dict(self) -> dict:
        return {"base_lr": self.base_lr, "cur_lr": self.cur_lr, "base_wd": self.base_wd, "cur_wd": self.cur_wd,
                "num_tokens": self.num_tokens}

    def load_state_dict(self, sd: dict) -> None:
        self.num_tokens = sd.get("num_tokens", self.num_tokens)
        if self.use_checkpointed:
            self.base_lr = sd.get("base_lr", self.base_lr)
            self.base_wd = sd.get("base_wd", self.base_wd)
        self.step(0)
