"""Run generatable items concurrently: one asyncio loop per worker, several worker processes, one
controller-wide cap on items in flight.

Reference: ``steptronoss/generation/async_generation.py:18-273``.  ``SingleGenerationController`` owns a
thread with an event loop that starts a task per submitted item; ``GenerationController`` spreads items
over ``num_workers`` such processes, keeps a FIFO of submissions beyond ``max_concurrent_genables`` and
invokes the callbacks in the submitting process.  A failing item comes back as a ``RuntimeError`` value
(plain, so that it pickles), never as a raised exception in a worker.
"""
from __future__ import annotations

import asyncio
import multiprocessing as mp
import threading
import traceback
from collections import deque
from collections.abc import Callable, Iterable
from queue import Empty, Queue
from typing import Any
from uuid import uuid4

from ..utils.general import run_async
from ..utils.logger import logger
from .base_generatable import GenableItem, TrainableItem


class SingleGenerationController:
    def __init__(self):
        self.input_queue: Queue = Queue()
        self._alive = True
        self._worker = threading.Thread(target=lambda: run_async(self._generate_loop()), daemon=True)
        self._worker.start()

    @staticmethod
    async def work_on_item(item: GenableItem, callback, for_train: bool) -> None:
        try:
            if for_train:
                if not isinstance(item, TrainableItem):
                    raise TypeError(f"Expected TrainableItem for training generation, got {type(item).__name__}")
                result = await item.generate_for_train()
            else:
                result = await item.generate()
        except Exception as e:
            logger.error("".join(traceback.format_exception(e)))
            result = RuntimeError(f"{type(e).__name__}: {e}")
        callback(item, result)

    def generate(self, gen_items: list, for_train: bool = False) -> Iterable:
        out: Queue = Queue()
        for item in gen_items:
            self.input_queue.put((item, lambda a, b: out.put((a, b)), for_train))
        for _ in gen_items:
            yield out.get()

    def submit_with_callback(self, genable: GenableItem, for_train: bool = False, callback: Callable | None = None,
                             task_meta: dict | None = None) -> None:
        if task_meta:
            genable.meta.update(task_meta)
        self.input_queue.put((genable, callback or print, for_train))

    async def _generate_loop(self):
        tasks: list = []
        while self._alive:
            while True:
                try:
                    tasks.append(asyncio.create_task(self.work_on_item(*self.input_queue.get_nowait())))
                except Empty:
                    break
            if tasks:
                done, pending = await asyncio.wait(tasks, timeout=0.05, return_when=asyncio.FIRST_COMPLETED)
                for t in done:
                    await t
                tasks = list(pending)
            else:
                await asyncio.sleep(0.02)
        for t in tasks:
            t.cancel()

    def shutdown(self):
        self._alive = False
        self._worker.join(timeout=2)


def _generation_worker_process(input_queue, result_queue) -> None:
    worker = SingleGenerationController()
    while True:
        try:
            task = input_queue.get()
            if task is None:
                break
            item, task_id, for_train = task
            item.meta["_gc_task_id"] = task_id
            worker.submit_with_callback(
                item, for_train=for_train,
                callback=lambda x, r, q=result_queue: q.put((x.meta.pop("_gc_task_id"), x, r)))
        except Exception as e:  # keep the worker alive: the controller is waiting on its queue
            logger.error(f"Worker process error: {e}")
    worker.shutdown()


class GenerationController:
    def __init__(self, num_workers: int | None = None, max_concurrent_genables: int | None = None,
                 start_method: str | None = None):
        if max_concurrent_genables is not None and max_concurrent_genables < 1:
            raise ValueError("max_concurrent_genables must be >= 1")
        self.num_workers = num_workers or min(mp.cpu_count(), 16)
        self.max_concurrent_genables = max_concurrent_genables
        ctx = mp.get_context(start_method) if start_method else mp
        self.input_queue, self.result_queue = ctx.Queue(), ctx.Queue()
        self.callback_map: dict = {}
        self._pending: deque = deque()
        self._inflight: set = set()
        self._lock = threading.Lock()
        self._completed = 0
        self._alive = True
        self.worker_processes = []
        for _ in range(self.num_workers):
            p = ctx.Process(target=_generation_worker_process, args=(self.input_queue, self.result_queue), daemon=True)
            p.start()
            self.worker_processes.append(p)
        self.callback_thread = threading.Thread(target=self._callback_loop, daemon=True)
        self.callback_thread.start()

    @property
    def completed_count(self) -> int:
        return self._completed

    @property
    def inflight_count(self) -> int:
        with self._lock:
            return len(self._inflight)

    def _callback_loop(self):
        while self._alive:
            try:
                task_id, item, result = self.result_queue.get(timeout=0.2)
            except Empty:
                continue
            except (EOFError, OSError):
                return
            with self._lock:
                callback = self.callback_map.pop(task_id)
                self._inflight.discard(task_id)
                self._dispatch_locked()
            try:
                callback(item, result)
            except Exception as e:
                logger.error(f"generation callback failed: {e}")
            self._completed += 1

    def _dispatch_locked(self) -> None:
        while self._pending and (self.max_concurrent_genables is None
                                 or len(self._inflight) < self.max_concurrent_genables):
            genable, task_id, for_train = self._pending.popleft()
            self._inflight.add(task_id)
            self.input_queue.put((genable, task_id, for_train))

    def generate(self, gen_items: list, for_train: bool = False) -> Iterable:
        out: Queue = Queue()
        for item in gen_items:
            self.submit_with_callback(item, for_train, lambda it, res, q=out: q.put((it, res)))
        for _ in gen_items:
            yield out.get()

    def submit_with_callback(self, genable: GenableItem, for_train: bool = False, callback: Callable | None = None,
                             task_id: Any = None) -> None:
        task_id = str(uuid4()) if task_id is None else task_id
        with self._lock:
            self.callback_map[task_id] = callback or print
            self._pending.append((genable, task_id, for_train))
            self._dispatch_locked()

    def shutdown(self):
        self._alive = False
        for _ in self.worker_processes:
            self.input_queue.put(None)
        for p in self.worker_processes:
            p.join(timeout=1)
            if p.is_alive():
                p.terminate()
        self.callback_thread.join(timeout=0.5)
