"""Registry of functions that have a PyTorch restatement next to their native kernel.

The reference uses ``@optimizable`` / ``set_optimization`` to choose at run time between several
back-ends of an op (``steptronoss/utils/optimizable.py:19-103``).  This framework has exactly one
production path per op (the sm_100a kernel); the registry survives as a test and debugging switch
between ``"native"`` and ``"reference"`` (the PyTorch restatement), with the same call surface so that
ported experiment files keep working.
"""
from __future__ import annotations

from functools import wraps
from typing import Callable

from .logger import logger

OPTIMIZABLE_REGISTER: dict = {}


def optimizable(alternatives: dict | None = None):
    """Register ``func`` under ``module.qualname`` with named alternatives (same arguments, allclose output)."""

    def wrapper(func: Callable):
        reg = f"{getattr(func, '__module__', 'unknown')}.{getattr(func, '__qualname__', func.__name__)}"
        OPTIMIZABLE_REGISTER[reg] = {"alternatives": dict(alternatives or {}), "use_optimize": None, "base": func}

        @wraps(func)
        def wrapped(*a, **k):
            meta = OPTIMIZABLE_REGISTER[reg]
            alt = meta["use_optimize"]
            if alt:
                return meta["alternatives"][alt](*a, **k)
            return func(*a, **k)

        wrapped.__optimizable_name__ = reg
        return wrapped

    return wrapper


def set_optimization(default: str | None = None, **kwargs) -> dict:
    """Select alternatives by function name (short or full). Unknown alternative names are ignored with a
    warning (experiment files written for the reference name back-ends that do not exist here)."""
    short = {}
    for k in OPTIMIZABLE_REGISTER:
        short.setdefault(k.split(".")[-1], []).append(k)
    chosen = {}
    for reg, meta in OPTIMIZABLE_REGISTER.items():
        if default and default in meta["alternatives"]:
            meta["use_optimize"] = default
            chosen[reg] = default
    for name, alt in kwargs.items():
        targets = [name] if name in OPTIMIZABLE_REGISTER else short.get(name, [])
        if not targets:
            logger.warning(f"set_optimization: no optimizable function named {name!r}", at=0)
            continue
        for reg in targets:
            meta = OPTIMIZABLE_REGISTER[reg]
            if alt in (None, "native", "default"):
                meta["use_optimize"] = None
            elif alt in meta["alternatives"]:
                meta["use_optimize"] = alt
            else:
                logger.warning(f"set_optimization: {reg} has no alternative {alt!r}; keeping the native path", at=0)
                continue
            chosen[reg] = alt
    return chosen
