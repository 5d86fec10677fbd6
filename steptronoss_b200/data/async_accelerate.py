"""Turn a :class:`SlowFastNextable` into a multi-process, prefetching, pinned-memory loader.

Reference: ``steptronoss/data/nextable/async_accelerate.py:21-274``.  ``num_workers`` forked processes each
hold a copy of the iterator; worker ``w`` builds items ``w, w + N, w + 2N ...`` (``next``) and skips the rest
(``fast_step``), so the merged round-robin stream is exactly the serial stream.  A thread in the consumer
drains the worker queues in that order, pins the tensors and keeps a short queue ready.

State: the consumer's own copy of the iterator never produces items; it is advanced with ``fast_step`` once
per delivered item, so ``state_dict`` is answered locally and points at the next undelivered item
(work the workers did ahead is simply redone after a resume).
"""
from __future__ import annotations

import multiprocessing as mp
import queue
import threading
import time
from typing import Any

import torch

from ..utils.logger import logger
from .nextable import SlowFastNextable

PREFETCH_QUEUE_SIZE = 10
WARN_INTERVAL_S = 60.0


def _stop_process(p, timeout: float = 2.0) -> None:
    p.terminate()
    p.join(timeout=timeout)
    if p.is_alive():
        p.kill()


def _pin(obj):
    if torch.is_tensor(obj):
        return obj.pin_memory() if torch.cuda.is_available() and not obj.is_cuda else obj
    if isinstance(obj, dict):
        return {k: _pin(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_pin(v) for v in obj)
    return obj


def _worker(nextable: SlowFastNextable, out_q, wid: int, n_workers: int) -> None:
    torch.set_num_threads(1)
    i = 0
    try:
        while True:
            if i % n_workers == wid:
                out_q.put(next(nextable))
            else:
                nextable.fast_step()
            i += 1
    except StopIteration:
        out_q.put(StopIteration())
    except Exception as e:  # delivered to the consumer, which re-raises it
        out_q.put(RuntimeError(f"data worker {wid}: {type(e).__name__}: {e}"))


def soft_kill_process(process, timeout: float = 2) -> None:
    """Ask a worker process to stop (SIGTERM), give it ``timeout`` seconds, then kill it if it is still alive."""
    process.terminate()
    process.join(timeout=timeout)
    if process.is_alive():
        process.kill()
        process.join(timeout=timeout)


class _RoundRobinPrefetcher:
    """Multi-in / single-out: take from the worker queues in turn, pin, keep a few items ready."""

    def __init__(self, queues: list, pin_memory: bool):
        self.queues, self.pin_memory = queues, pin_memory
        self.out: queue.Queue = queue.Queue(PREFETCH_QUEUE_SIZE)
        self.stop = False
        self._warned = 0.0
        self.thread = threading.Thread(target=self._loop, name="PrefetchLoop", daemon=True)
        self.thread.start()

    def _loop(self):
        idx = 0
        while not self.stop:
            q = self.queues[idx % len(self.queues)]
            t0 = time.time()
            while not self.stop:
                try:
                    item = q.get(timeout=0.2)
                    break
                except queue.Empty:
                    if time.time() - t0 > 10 and time.time() - self._warned > WARN_INTERVAL_S:
                        logger.warning(f"data worker queue {idx % len(self.queues)} empty for {time.time() - t0:.0f} s")
                        self._warned = time.time()
            else:
                return
            if self.pin_memory and not isinstance(item, Exception):
                item = _pin(item)
            while not self.stop:
                try:
                    self.out.put(item, timeout=0.2)
                    break
                except queue.Full:
                    pass
            if isinstance(item, Exception):
                return
            idx += 1

    def get(self, timeout: float | None = None):
        return self.out.get(timeout=timeout)

    def close(self):
        self.stop = True


class AsyncAcceleratedSlowFast(SlowFastNextable):
    def __init__(self, slowfast: SlowFastNextable, queue_size: int = 100, num_workers: int = 2,
                 pin_memory: bool = False, start_method: str = "fork"):
        self.nextable, self.queue_size, self.num_workers = slowfast, queue_size, num_workers
        self.pin_memory, self.start_method = pin_memory, start_method
        self._procs: list | None = None
        self._prefetch: _RoundRobinPrefetcher | None = None

    def _reset(self) -> None:
        self.close()
        ctx = mp.get_context(self.start_method)
        per = max(1, self.queue_size // self.num_workers)
        queues = [ctx.Queue(per) for _ in range(self.num_workers)]
        # every worker starts from the consumer's current state (forked copy)
        self._procs = [ctx.Process(target=_worker, args=(self.nextable, queues[w], w, self.num_workers), daemon=True)
                       for w in range(self.num_workers)]
        for p in self._procs:
            p.start()
        self._prefetch = _RoundRobinPrefetcher(queues, self.pin_memory)

    def __next__(self) -> Any:
        if self._procs is None:
            self._reset()
        item = self._prefetch.get()
        if isinstance(item, StopIteration):
            raise StopIteration
        if isinstance(item, Exception):
            raise item
        self.nextable.fast_step()  # the local copy shadows what has been delivered
        return item

    def fast_step(self) -> None:
        next(self)

    def __len__(self) -> int:
        return len(self.nextable)

    def __repr__(self) -> str:
        return "Asynced " + repr(self.nextable)

    def state_dict(self) -> dict:
        return self.nextable.state_dict()

    def load_state_dict(self, state: dict) -> None:
        self.nextable.load_state_dict(state)
        self._reset()

    def close(self) -> None:
        if self._prefetch is not None:
            self._prefetch.close()
            self._prefetch = None
        if self._procs is not None:
            for p in self._procs:
                _stop_process(p)
            self._procs = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def async_accelerate_slowfast(slowfast: SlowFastNextable, queue_size: int = 100, num_workers: int = 8,
                              pin_memory: bool = True) -> AsyncAcceleratedSlowFast:
    assert isinstance(slowfast, SlowFastNextable), "Only SlowFastNextable can be accelerated."
    return AsyncAcceleratedSlowFast(slowfast, queue_size, num_workers, pin_memory)


async_accelearte_slowfast = async_accelerate_slowfast  # spelling used by the reference's callers
