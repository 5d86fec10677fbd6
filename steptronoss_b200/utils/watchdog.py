"""A thread that watches the kernels' status word and a heartbeat of the training loop.

Kernels of the native library never spin forever: a wait that runs out records a code in a per-device status word
and the kernel returns (``ops/native.py``).  The trainer reads that word when it logs; this watchdog reads it every
``interval_s`` seconds from a side stream (without waiting for the work queued on the training stream), so that a
peer that never arrived or a pipeline wait that ran out turns into a Python exception within seconds instead of at
the next log line.  It also notices a loop that stopped calling :meth:`beat` for ``stall_s`` seconds (a rank stuck in
a collective, a starved data loader) and reports where the main thread is.

On an error the watchdog logs it, stores it (``error``), sets ``tripped`` and calls ``on_error(message)``; the default
handler interrupts the main thread (``KeyboardInterrupt`` there ends ``train()`` through its normal ``finally``
blocks, so checkpoints in flight are joined and process groups destroyed).
"""
from __future__ import annotations

import faulthandler
import sys
import threading
import time

import torch

from .logger import logger


def _interrupt_main(message: str) -> None:
    import _thread

    _thread.interrupt_main()


class KernelWatchdog:
    def __init__(self, interval_s: float = 2.0, stall_s: float | None = None, on_error=_interrupt_main,
                 read_status=None):
        """``read_status() -> {device index: code}``; the default reads the native library's status words."""
        self.interval_s, self.stall_s, self.on_error = interval_s, stall_s, on_error
        self._read = read_status or self._read_native
        self._stop = threading.Event()
        self.tripped = threading.Event()
        self.error: str | None = None
        self._last_beat = time.monotonic()
        self._thread: threading.Thread | None = None
        self._streams: dict = {}
        self._host: dict = {}

    # ------------------------------------------------------------------ status sources
    def _read_native(self) -> dict:
        from ..ops import native

        out = {}
        for idx, word in list(native._STATUS.items()):
            if not word.is_cuda:
                out[idx] = int(word.item())
                continue
            if idx not in self._streams:
                self._streams[idx] = torch.cuda.Stream(device=idx)
                self._host[idx] = torch.zeros(1, dtype=torch.int32).pin_memory()
            s = self._streams[idx]
            with torch.cuda.stream(s):
                self._host[idx].copy_(word, non_blocking=True)
            s.synchronize()
            out[idx] = int(self._host[idx][0])
        return out

    # ------------------------------------------------------------------ life cycle
    def start(self) -> "KernelWatchdog":
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name="stb200-kernel-watchdog", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.interval_s + 5)
            self._thread = None

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
        return False

    def beat(self) -> None:
        """Called by the training loop once per step."""
        self._last_beat = time.monotonic()

    def raise_if_tripped(self) -> None:
        if self.tripped.is_set():
            raise RuntimeError(self.error)

    # ------------------------------------------------------------------ the loop
    def _trip(self, message: str) -> None:
        self.error = message
        logger.error(message, at=None)
        try:
            self.on_error(message)
        except Exception as e:  # a handler must not kill the watchdog silently
            logger.error(f"watchdog handler failed: {e}", at=None)
        self.tripped.set()

    def _run(self) -> None:
        from ..ops.native import _ERRORS

        while not self._stop.wait(self.interval_s):
            try:
                codes = self._read()
            except Exception as e:
                logger.warning(f"watchdog could not read the kernel status: {e}", at=None)
                continue
            bad = {i: c for i, c in codes.items() if c}
            if bad:
                what = ", ".join(f"device {i}: {_ERRORS.get(c, c)}" for i, c in sorted(bad.items()))
                self._trip(f"kernel status reports an error ({what})")
                return
            if self.stall_s is not None and time.monotonic() - self._last_beat > self.stall_s:
                faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
                self._trip(f"no training step finished for {self.stall_s:.0f} s (stacks of all threads are on stderr)")
                return
