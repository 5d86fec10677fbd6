"""Memory marks (reference ``steptronoss/utils/memory_tracker.py:74-350``): ``CMT.mark(name)`` records GPU
allocated / reserved / peak and host RSS when ``MEM_DIAGNOSE`` is set; ``report`` ranks the largest peaks
and deltas and can gather every rank's table."""
from __future__ import annotations

import os
from dataclasses import dataclass

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


@dataclass
class Mark:
    name: str
    allocated: int
    reserved: int
    peak: int
    rss: int


class MemoryTracker:
    def __init__(self, enabled: bool | None = None):
        self.enabled = bool(os.environ.get("MEM_DIAGNOSE")) if enabled is None else enabled
        self.marks: list[Mark] = []

    def mark(self, name: str) -> Mark | None:
        if not self.enabled:
            return None
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

    def reset(self) -> None:
        self.marks = []


CMT = MemoryTracker()
