"""Run a function in a side process with a deadline (reference ``steptronoss/text_processing/utils.py:6-61``):
symbolic answer comparison can take unbounded time on adversarial model output."""
from __future__ import annotations

from concurrent.futures import ProcessPoolExecutor
from concurrent.futures import TimeoutError as FutureTimeout
from concurrent.futures.process import BrokenProcessPool


class TimedRunner:
    def __init__(self):
        self.executor = ProcessPoolExecutor(max_workers=1)

    def reset(self) -> None:
        """Kill the worker (it may be stuck in native code) and start a fresh one."""
        try:
            for proc in list(getattr(self.executor, "_processes", {}).values()):
                try:
                    proc.kill()
                except Exception:
                    pass
            self.executor.shutdown(wait=False, cancel_futures=True)
        finally:
            self.executor = ProcessPoolExecutor(max_workers=1)

    def __call__(self, func, *args, timeout: float = 10, **kwargs):
        try:
            future = self.executor.submit(func, *args, **kwargs)
        except (BrokenProcessPool, RuntimeError):
            self.reset()
            future = self.executor.submit(func, *args, **kwargs)
        try:
            return future.result(timeout=timeout)
        except FutureTimeout:
            self.reset()
            raise TimeoutError(f"Runner timeout after {timeout} seconds") from None
        except BrokenProcessPool:
            self.reset()
            raise

    def __del__(self):
        try:
            self.executor.shutdown(wait=False)
        except Exception:
            pass


_RUNNER: TimedRunner | None = None


def get_runner() -> TimedRunner:
    global _RUNNER
    if _RUNNER is None:
        _RUNNER = TimedRunner()
    return _RUNNER
