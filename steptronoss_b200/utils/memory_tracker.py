"""Memory marks (reference ``steptronoss/utils/memory_tracker.py:74-350``): ``CMT.mark(name)`` records GPU
allocated / reserved / peak and host RSS when ``MEM_DIAGNOSE`` is set; ``report`` ranks the largest peaks
and deltas and can gather every rank's table."""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass, field
from typing import TypedDict

import torch


def _rss_bytes() -> int:
    try:
        import psutil

        return psutil.Process().memory_info().rss
    except Exception:
        try:
            with open("/proc/self/statm") as f:
                return int(f.read().split()[1]) * os.sysconf("SC_PAGE_SIZE")
        except Exception:
            return 0


def get_caller_name(depth: int = 0) -> str:
    """Module name of the code that called this function (``depth`` 0), of its caller (1), and so on; "<unknown>"
    past the outermost frame."""
    frame = sys._getframe(1)
    for _ in range(depth):
        frame = frame.f_back if frame is not None else None
    return "<unknown>" if frame is None else frame.f_globals.get("__name__", "<unknown>")


class MemoryRecord(TypedDict):
    """One mark as a plain mapping (what ``MemoryTracker.records`` returns): bytes and a wall-clock time."""

    mark: str
    time: float
    allocated: float
    reserved: float
    cpu_rss: float


@dataclass
class Mark:
    name: str
    allocated: int
    reserved: int
    peak: int
    rss: int
    time: float = field(default_factory=time.time)


class MemoryTracker:
    def __init__(self, enabled: bool | None = None):
        self.enabled = bool(os.environ.get("MEM_DIAGNOSE")) if enabled is None else enabled
        self.marks: list[Mark] = []

    def mark(self, name: str | None = None) -> Mark | None:
        """Record a mark; without a name the calling module and line name it."""
        if not self.enabled:
            return None
        if name is None:
            f = sys._getframe(1)
            name = f"{f.f_globals.get('__name__', '<unknown>')}:{f.f_lineno}"
        if torch.cuda.is_available():
            a, r, p = torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.max_memory_allocated()
            torch.cuda.reset_peak_memory_stats()
        else:
            a = r = p = 0
        m = Mark(name, a, r, p, _rss_bytes())
        self.marks.append(m)
        return m

    def deltas(self) -> list[tuple[str, int, int]]:
        out = []
        for prev, cur in zip(self.marks[:-1], self.marks[1:]):
            out.append((f"{prev.name} -> {cur.name}", cur.allocated - prev.allocated, cur.rss - prev.rss))
        return out

    def top_peaks(self, k: int = 5) -> list[Mark]:
        return sorted(self.marks, key=lambda m: -m.peak)[:k]

    def report(self, k: int = 5, all_ranks: bool = False) -> str:
        gb = 1024 ** 3
        lines = ["memory marks (GB): name | allocated | reserved | peak-since-last | host rss"]
        for m in self.marks:
            lines.append(f"  {m.name:32s} {m.allocated / gb:8.2f} {m.reserved / gb:8.2f} {m.peak / gb:8.2f} {m.rss / gb:8.2f}")
        lines.append("largest peaks: " + ", ".join(f"{m.name}={m.peak / gb:.2f}" for m in self.top_peaks(k)))
        big = sorted(self.deltas(), key=lambda d: -abs(d[1]))[:k]
        lines.append("largest deltas: " + ", ".join(f"{n}={d / gb:+.2f}" for n, d, _ in big))
        text = "\n".join(lines)
        if all_ranks and torch.distributed.is_initialized():
            from .dist_utils import all_gather_object

            return "\n".join(f"[rank {i}]\n{t}" for i, t in enumerate(all_gather_object(text)))
        return text

    def records(self) -> list[MemoryRecord]:
        return [MemoryRecord(mark=m.name, time=m.time, allocated=float(m.allocated), reserved=float(m.reserved),
                             cpu_rss=float(m.rss)) for m in self.marks]

    def report_over_world(self, topk: int = 3, topk_ranks: int = 1) -> str:
        """This rank's report plus, gathered over all ranks, the ``topk_ranks`` ranks with the highest and the lowest
        peak and the marks at which they reached it.  Collective (one object all-gather): every rank calls it.
        Reference: utils/memory_tracker.py:189-331."""
        if not self.enabled:
            return ""
        text = self.report(max(1, topk))
        if not (torch.distributed.is_available() and torch.distributed.is_initialized()):
            return text
        from .dist_utils import all_gather_object

        top = self.top_peaks(1)
        mine = (top[0].peak if top else 0, top[0].name if top else "-", max((m.rss for m in self.marks), default=0))
        table = sorted(enumerate(all_gather_object(mine)), key=lambda kv: -kv[1][0])
        n, gb = max(1, topk_ranks), 1024 ** 3
        fmt = lambda rows: ", ".join(f"rank {r}: {p / gb:.2f} GB at {name!r} (host {rss / gb:.2f} GB)" for r, (p, name, rss) in rows)
        return text + f"\nhighest peaks: {fmt(table[:n])}\nlowest peaks: {fmt(table[-n:][::-1])}"

    def reset(self) -> None:
        self.marks = []


CudaMemoryTracker = MemoryTracker      # the reference's class name
CMT = MemoryTracker()
