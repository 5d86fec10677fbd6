"""Greedy non-truncating packing (reference ``steptronoss/data/packing/non_truncation.py``): consecutive
samples are packed while they fit into ``max_len``; a sample longer than ``max_len`` is dropped or becomes a
packed sample of its own (``extend``)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class PackingResult:
    num_packed_samples: int
    num_droped: int
    packed_sample_ranges: list
    """``(first sample index, number of samples)`` of every packed sample."""


def pack(sizes: list[int], max_len: int, oversize_policy: str = "drop") -> PackingResult:
    if oversize_policy not in ("drop", "extend"):
        raise ValueError(oversize_policy)
    ranges: list = []
    dropped = 0
    start, count, used = None, 0, 0

    def close():
        nonlocal start, count, used
        if count:
            ranges.append((start, count))
        start, count, used = None, 0, 0

    for i, n in enumerate(sizes):
        if n > max_len:
            close()
            if oversize_policy == "extend":
                ranges.append((i, 1))
            else:
                dropped += 1
            continue
        if used + n > max_len:
            close()
        if count == 0:
            start = i
        count += 1
        used += n
        if used == max_len:
            close()
    close()
    return PackingResult(len(ranges), dropped, ranges)
