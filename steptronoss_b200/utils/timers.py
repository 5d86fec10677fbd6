"""Named timers with log levels (reference ``steptronoss/timers.py:17-327``): CUDA-event or wall
clock timing, ``timeit`` decorator / context manager, per-interval report."""
from __future__ import annotations

import functools
import time

import torch


class Timer:
    def __init__(self, name: str, use_event: bool = True):
        self.name = name
        self.use_event = use_event and torch.cuda.is_available()
        self.elapsed_ms = 0.0
        self.count = 0
        self._pending: list = []
        self._t0 = None
        self._ev0 = None
        self.started = False

    def start(self):
        if self.started:
            return
        if self.use_event:
            self._ev0 = torch.cuda.Event(enable_timing=True)
            self._ev0.record()
        else:
            self._t0 = time.perf_counter()
        self.started = True

    def stop(self):
        if not self.started:
            return
        if self.use_event:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            self._pending.append((self._ev0, ev1))
        else:
            self.elapsed_ms += (time.perf_counter() - self._t0) * 1e3
        self.count += 1
        self.started = False

    def elapsed(self, reset: bool = True) -> float:
        """Accumulated milliseconds (synchronises on the recorded events)."""
        was = self.started
        if was:
            self.stop()
        for a, b in self._pending:
            b.synchronize()
            self.elapsed_ms += a.elapsed_time(b)
        self._pending = []
        out = self.elapsed_ms
        if reset:
            self.elapsed_ms, self.count = 0.0, 0
        if was:
            self.start()
        return out


class _Noop:
    """Stands in for a timer whose level is above the configured one: every call is free."""

    name = "noop"

    def start(self, *a, **k): pass   # noqa: E704
    def stop(self, *a, **k): pass    # noqa: E704
    def reset(self): pass            # noqa: E704
    def elapsed(self, *a, **k): return 0.0   # noqa: E704
    def __enter__(self): return self   # noqa: E704
    def __exit__(self, *a): return False   # noqa: E704


class _Scope:
    """Times a region; with ``nvtx`` also brackets it with an NVTX range of the timer's name, so the regions show
    up by name on a profiler's timeline."""

    def __init__(self, timer, nvtx: bool = False):
        self.timer, self.nvtx = timer, nvtx and torch.cuda.is_available()

    def __enter__(self):
        if self.nvtx:
            torch.cuda.nvtx.range_push(self.timer.name)
        self.timer.start()
        return self.timer

    def __exit__(self, *a):
        self.timer.stop()
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
        return False


class Timers:
    """Levels: 0 always, 1 coarse (forward-backward, optimizer-step, dataloader-next), 2 fine."""

    def __init__(self, log_level: int = 0, use_event: bool = True, nvtx: bool = False):
        self.log_level = log_level
        self.use_event = use_event
        self.nvtx = nvtx
        self.timers: dict[str, Timer] = {}
        self._noop = _Noop()

    def __call__(self, name: str, log_level: int = 0):
        if log_level > self.log_level:
            return self._noop
        if name not in self.timers:
            self.timers[name] = Timer(name, self.use_event)
        return self.timers[name]

    def record(self, name: str, log_level: int = 0):
        t = self(name, log_level)
        return t if isinstance(t, _Noop) else _Scope(t, self.nvtx)

    def report(self, names=None, normalizer: float = 1.0, reset: bool = True) -> dict:
        names = names or list(self.timers)
        return {n: self.timers[n].elapsed(reset) / normalizer for n in names if n in self.timers}

    def log_string(self, normalizer: float = 1.0, reset: bool = True) -> str:
        rep = self.report(normalizer=normalizer, reset=reset)
        return "time (ms) | " + " | ".join(f"{k}: {v:.2f}" for k, v in rep.items())

    def write(self, writer, iteration: int, normalizer: float = 1.0, reset: bool = False) -> dict:
        """One ``Timers/<name>`` scalar per timer that ran, in seconds per ``normalizer`` calls (this rank's times;
        reference: timers.py:241-254).  Returns what was written."""
        if normalizer <= 0:
            raise ValueError("normalizer must be positive")
        rep = {n: ms / 1e3 for n, ms in self.report(normalizer=normalizer, reset=reset).items() if ms > 0}
        if writer is not None:
            for name, seconds in rep.items():
                writer.add_scalar("Timers/" + name, seconds, iteration)
        return rep

    def log(self, iteration: int, normalizer: float = 1.0, reset: bool = True, prefix: str = "") -> str:
        """Log the timers that ran, one per line, in seconds (reference: timers.py:256-266)."""
        rep = {n: ms / 1e3 for n, ms in self.report(normalizer=normalizer, reset=reset).items() if ms > 0}
        if not rep:
            return ""
        from .logger import logger

        text = f"{prefix or f'iteration {iteration}'} | Activated Timers:\n" + "".join(
            f"{name}".ljust(48, ".") + f"{seconds:.4e} s\n" for name, seconds in rep.items())
        logger.info(text, at=0)
        return text

    def reload(self, new_log_level: int, new_use_event: bool) -> None:
        """Change level and clock at run time (a profiler window that wants finer timers for some iterations).
        Timers that exist keep their accumulated time and take the new clock from their next ``start``."""
        self.log_level = min(int(new_log_level), 2)
        self.use_event = bool(new_use_event)
        for t in self.timers.values():
            if not t.started:
                t.use_event = self.use_event and torch.cuda.is_available()


# the reference's class names: its code checks ``isinstance(timers, DummyTimers)`` and annotates with ``LocalTimers``
LocalTimers = Timers
TimerBase = Timer
DummyTimer = _Noop


class DummyTimers(Timers):
    """Timers that time nothing (log level below every timer's level)."""

    def __init__(self):
        super().__init__(log_level=-(10 ** 6))


_GLOBAL = Timers()


def init_timers(log_level: int = 0, use_event: bool = True, nvtx: bool = False) -> Timers:
    global _GLOBAL
    _GLOBAL = Timers(log_level, use_event, nvtx)
    return _GLOBAL


def get_timers() -> Timers:
    return _GLOBAL


class timeit:  # noqa: N801
    """``@timeit("name", log_level=1)``, ``@timeit()`` (the function's name) or ``with timeit("name"):``.

    ``barrier`` joins the ranks and ``sync_device`` drains the GPU before the clock starts and before it stops, for
    numbers that compare across ranks (both cost time: measurements only).  ``level`` is accepted as another
    spelling of ``log_level`` (the reference's, ``steptronoss/timers.py:284-315``)."""

    def __init__(self, name: str | None = None, log_level: int | None = None, level: int | None = None,
                 barrier: bool = False, sync_device: bool = False):
        self.name = name
        self.log_level = log_level if log_level is not None else (level if level is not None else 2)
        self.barrier, self.sync_device = barrier, sync_device

    def _fence(self):
        if self.sync_device:
            import torch

            if torch.cuda.is_available():
                torch.cuda.synchronize()
        if self.barrier:
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized():
                dist.barrier()

    def clone(self) -> "timeit":
        return type(self)(self.name, self.log_level, None, self.barrier, self.sync_device)

    def __call__(self, fn):
        scope = self.clone()
        if scope.name is None:
            scope.name = fn.__name__

        @functools.wraps(fn)
        def wrapper(*a, **k):
            with scope.clone():
                return fn(*a, **k)
        return wrapper

    def __enter__(self):
        if self.name is None:
            raise ValueError("timeit used as a context needs a name")
        self._fence()
        self._scope = get_timers().record(self.name, self.log_level)
        return self._scope.__enter__()

    def __exit__(self, *a):
        self._fence()
        return self._scope.__exit__(*a)
