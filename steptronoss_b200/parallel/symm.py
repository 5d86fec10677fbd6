"""Symmetric peer memory for fused compute+collective kernels (filled in by ``enable``)."""
from __future__ import annotations

_ENABLED = False


def enabled() -> bool:
    return _ENABLED
