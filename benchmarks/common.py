"""Timing helpers for the kernel micro-benchmarks: CUDA events on the launching stream, warm-up,
an L2 flush between timed launches, best and median of the timed iterations."""
from __future__ import annotations

import json
import os
import statistics

import torch

_FLUSH = None


def flush_l2() -> None:
    """Overwrite a buffer larger than the 126 MB L2 so that the next launch starts cold."""
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def time_cuda(fn, warmup: int = 3, iters: int = 10, flush: bool = True) -> dict:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return {"best_ms": min(times), "median_ms": statistics.median(times)}


def measured_peaks() -> dict:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return json.load(open(path))
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "fallback": True}
