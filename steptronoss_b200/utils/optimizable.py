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


def optimizable(alternatives: dict | None = None, aliases: tuple = (), native_names: tuple = ()):
    """Register ``func`` under ``module.qualname`` with named alternatives (same arguments, allclose output).

    ``aliases``: further short names that ``set_optimization`` accepts for this entry (the name the reference
    registers the same operator under, e.g. ``AttentionCore`` for the attention function).  ``native_names``:
    back-end names of the reference that all mean the kernel path here (``"flash-attn-3"``, ``"triton"``,
    ``"nv_grouped_gemm"`` ...), so that an experiment file written for the reference selects it without a warning."""

    def wrapper(func: Callable):
        reg = f"{getattr(func, '__module__', 'unknown')}.{getattr(func, '__qualname__', func.__name__)}"
        OPTIMIZABLE_REGISTER[reg] = {"alternatives": dict(alternatives or {}), "use_optimize": None, "base": func,
                                     "aliases": tuple(aliases), "native_names": tuple(native_names)}

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
    for k, meta in OPTIMIZABLE_REGISTER.items():
        for nick in (k.split(".")[-1],) + tuple(meta.get("aliases", ())):
            if k not in short.setdefault(nick, []):
                short[nick].append(k)
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
            if alt in (None, "native", "default") or alt in meta.get("native_names", ()):
                meta["use_optimize"] = None
            elif alt in meta["alternatives"]:
                meta["use_optimize"] = alt
            else:
                logger.warning(f"set_optimization: {reg} has no alternative {alt!r}; keeping the native path", at=0)
                continue
            chosen[reg] = alt
    return chosen


def current_optimization(name: str) -> str | None:
    """The alternative selected for ``name`` (full name, short name or alias); None = the kernel path."""
    for reg, meta in OPTIMIZABLE_REGISTER.items():
        if name == reg or name == reg.split(".")[-1] or name in meta.get("aliases", ()):
            return meta["use_optimize"]
    raise KeyError(name)
