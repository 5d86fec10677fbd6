"""Concurrent execution of generatable items (rollouts, evaluation prompts).

Contract, shared with the reference's module of the same name
(``steptronoss/generation/async_generation.py:18-273``):

* an item is a ``GenableItem`` whose ``generate()`` (or, for training, a ``TrainableItem``'s
  ``generate_for_train()``) is a coroutine that talks to an inference server;
* ``SingleGenerationController`` runs every submitted item concurrently inside one process;
  ``GenerationController`` spreads items over ``num_workers`` processes and admits at most
  ``max_concurrent_genables`` of them at a time, the rest wait in submission order;
* results are handed to a callback ``callback(item, result)`` in the submitting process, or yielded in
  completion order by ``generate(items)``;
* an item that raises comes back with a ``RuntimeError`` *value* as its result (a plain exception, so that it
  survives pickling); nothing is raised inside a worker.

Design.  Inside a process the items are tasks of one asyncio event loop that lives on its own thread; a
submission is handed to the loop with ``run_coroutine_threadsafe`` (no polling).  Across processes the parent
numbers every submission with a ticket, keeps the callbacks by ticket, and a collector thread feeds the
results back and admits the next waiting items.
"""
from __future__ import annotations

import asyncio
import itertools
import multiprocessing as mp
import queue
import threading
import traceback
from collections import deque
from collections.abc import Callable, Iterator
from functools import partial
from typing import Any

from ..utils.logger import logger
from .base_generatable import GenableItem, TrainableItem


async def _produce(item: GenableItem, for_train: bool):
    if not for_train:
        return await item.generate()
    if not isinstance(item, TrainableItem):
        raise TypeError(f"generation for training needs a TrainableItem, not a {type(item).__name__}")
    return await item.generate_for_train()


async def _run_item(item: GenableItem, for_train: bool, deliver: Callable) -> None:
    """One item from start to delivery; a failure becomes the item's result."""
    try:
        result = await _produce(item, for_train)
    except Exception as exc:                     # noqa: BLE001 - whatever the item raised is reported as its result
        logger.error("generation item failed:\n" + "".join(traceback.format_exception(exc)))
        result = RuntimeError(f"{type(exc).__name__}: {exc}")
    deliver(item, result)


class _LoopThread:
    """An asyncio event loop on a daemon thread."""

    def __init__(self, name: str = "generation-loop"):
        self.loop = asyncio.new_event_loop()
        self._thread = threading.Thread(target=self._serve, name=name, daemon=True)
        self._thread.start()

    def _serve(self) -> None:
        asyncio.set_event_loop(self.loop)
        try:
            self.loop.run_forever()
        finally:
            for task in asyncio.all_tasks(self.loop):
                task.cancel()
            self.loop.run_until_complete(self.loop.shutdown_asyncgens())
            self.loop.close()

    def spawn(self, coro) -> None:
        asyncio.run_coroutine_threadsafe(coro, self.loop)

    def stop(self, timeout: float = 2.0) -> None:
        if self.loop.is_running():
            self.loop.call_soon_threadsafe(self.loop.stop)
        self._thread.join(timeout=timeout)


class SingleGenerationController:
    """All submitted items run concurrently on one event loop of this process."""

    def __init__(self):
        self._runner = _LoopThread()

    @staticmethod
    async def work_on_item(item: GenableItem, callback: Callable, for_train: bool) -> None:
        """One item from start to ``callback(item, result)``; a failure is delivered as a ``RuntimeError`` result.
        The coroutine a subclass with its own event loop schedules (the reference's name and argument order)."""
        await _run_item(item, for_train, callback)

    def submit_with_callback(self, genable: GenableItem, for_train: bool = False, callback: Callable | None = None,
                             task_meta: dict | None = None) -> None:
        if task_meta:
            genable.meta.update(task_meta)
        self._runner.spawn(_run_item(genable, for_train, callback or print))

    def generate(self, gen_items: list, for_train: bool = False) -> Iterator:
        finished: queue.SimpleQueue = queue.SimpleQueue()
        for item in gen_items:
            self.submit_with_callback(item, for_train, callback=lambda it, res: finished.put((it, res)))
        for _ in range(len(gen_items)):
            yield finished.get()

    def shutdown(self) -> None:
        self._runner.stop()


def _report(outbox, ticket, item: GenableItem, result) -> None:
    outbox.put((ticket, item, result))


def _worker_main(inbox, outbox) -> None:
    """Body of a worker process: items arrive as ``(ticket, item, for_train)``, ``None`` ends the process."""
    runner = SingleGenerationController()
    while True:
        try:
            message = inbox.get()
        except (EOFError, OSError):
            break
        except Exception as exc:                 # noqa: BLE001 - e.g. an item that cannot be unpickled here
            logger.error(f"generation worker could not read a submission: {exc}")
            continue
        if message is None:
            break
        ticket, item, for_train = message
        runner.submit_with_callback(item, for_train, callback=partial(_report, outbox, ticket))
    runner.shutdown()


class GenerationController:
    """Items run in ``num_workers`` processes; at most ``max_concurrent_genables`` are admitted at a time."""

    def __init__(self, num_workers: int | None = None, max_concurrent_genables: int | None = None,
                 start_method: str | None = None):
        if max_concurrent_genables is not None and max_concurrent_genables < 1:
            raise ValueError("max_concurrent_genables must be >= 1")
        self.num_workers = num_workers or min(mp.cpu_count(), 16)
        self.max_concurrent_genables = max_concurrent_genables
        ctx = mp.get_context(start_method) if start_method else mp
        self._inbox, self._outbox = ctx.Queue(), ctx.Queue()
        self._tickets = itertools.count()
        self._waiting: deque = deque()           # (ticket, item, for_train) not yet admitted
        self._callbacks: dict = {}               # ticket -> callback, for every submission that has not finished
        self._admitted: set = set()
        self._lock = threading.Lock()
        self._completed = 0
        self._closing = threading.Event()
        self._bar = None                         # progress over completed items; configured by ``set_tqdm``
        self._bar_cfg = {"disabled": True, "total": None, "desc": "Cumulative Completed"}
        self.worker_processes = [ctx.Process(target=_worker_main, args=(self._inbox, self._outbox), daemon=True)
                                 for _ in range(self.num_workers)]
        for proc in self.worker_processes:
            proc.start()
        self._collector = threading.Thread(target=self._collect, name="generation-collector", daemon=True)
        self._collector.start()

    # ------------------------------------------------------------------ bookkeeping
    @property
    def completed_count(self) -> int:
        return self._completed

    @property
    def inflight_count(self) -> int:
        with self._lock:
            return len(self._admitted)

    def set_tqdm(self, disabled: bool, total: int, desc: str) -> None:
        """Show (or hide) a progress bar that advances with every finished item: ``total`` items expected, ``desc`` as
        its label.  A bar that is already open is closed; the next finished item opens the new one.  Off until called
        (reference: generation/async_generation.py:159-201, where the bar is on by default)."""
        if total < 0:
            raise ValueError(f"Expected total >= 0, got {total}")
        with self._lock:
            self._bar_cfg = {"disabled": bool(disabled), "total": total, "desc": desc}
            self._close_bar()

    def _close_bar(self) -> None:
        """Caller holds the lock."""
        if self._bar is not None:
            self._bar.close()
            self._bar = None

    def _tick_bar(self) -> None:
        """Caller holds the lock."""
        if self._bar_cfg["disabled"]:
            return
        if self._bar is None:
            from tqdm import tqdm

            self._bar = tqdm(total=self._bar_cfg["total"], desc=self._bar_cfg["desc"], dynamic_ncols=True)
        self._bar.update(1)

    def _admit_waiting(self) -> None:
        """Caller holds the lock."""
        cap = self.max_concurrent_genables
        while self._waiting and (cap is None or len(self._admitted) < cap):
            entry = self._waiting.popleft()
            self._admitted.add(entry[0])
            self._inbox.put(entry)

    def _collect(self) -> None:
        while not self._closing.is_set():
            try:
                ticket, item, result = self._outbox.get(timeout=0.2)
            except queue.Empty:
                continue
            except (EOFError, OSError):
                return
            with self._lock:
                callback = self._callbacks.pop(ticket, None)
                self._admitted.discard(ticket)
                self._admit_waiting()
            if callback is not None:
                try:
                    callback(item, result)
                except Exception as exc:         # noqa: BLE001 - a user callback must not stop the collector
                    logger.error(f"generation callback raised: {exc}")
            with self._lock:
                self._completed += 1
                self._tick_bar()

    # ------------------------------------------------------------------ public API
    def submit_with_callback(self, genable: GenableItem, for_train: bool = False, callback: Callable | None = None,
                             task_id: Any = None) -> None:
        ticket = next(self._tickets) if task_id is None else task_id
        with self._lock:
            self._callbacks[ticket] = callback or print
            self._waiting.append((ticket, genable, for_train))
            self._admit_waiting()

    def generate(self, gen_items: list, for_train: bool = False) -> Iterator:
        finished: queue.SimpleQueue = queue.SimpleQueue()
        for item in gen_items:
            self.submit_with_callback(item, for_train, callback=lambda it, res: finished.put((it, res)))
        for _ in range(len(gen_items)):
            yield finished.get()

    def shutdown(self) -> None:
        self._closing.set()
        with self._lock:
            self._close_bar()
        for _ in self.worker_processes:
            self._inbox.put(None)
        for proc in self.worker_processes:
            proc.join(timeout=1)
            if proc.is_alive():
                proc.terminate()
        self._collector.join(timeout=0.5)
