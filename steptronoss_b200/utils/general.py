"""Small framework-independent helpers (reference ``steptronoss/utils/general.py``)."""
from __future__ import annotations

import asyncio
import contextlib
import functools
import importlib
import random
import socket
import subprocess
import time
import weakref
from collections import OrderedDict
from typing import Any, Callable, Sequence

import torch


def safediv(n: int, d: int) -> int:
    q, r = divmod(n, d)
    if r:
        raise AssertionError(f"{n} is not divisible by {d}")
    return q


def make_divisible(number: int, divisible_by: int) -> int:
    return -(-number // divisible_by) * divisible_by


def shift_left(t: torch.Tensor, pad=0, shift: int = 1) -> torch.Tensor:
    """[1, 2, 3] -> [2, 3, pad] along the first dimension."""
    out = torch.full_like(t, pad)
    out[:-shift] = t[shift:]
    return out


def shift_right(t: torch.Tensor, pad=0, shift: int = 1) -> torch.Tensor:
    """[1, 2, 3] -> [pad, 1, 2] along the first dimension."""
    out = torch.full_like(t, pad)
    out[shift:] = t[:-shift]
    return out


def get_position_id_from_cu_seqlens(cu_seqlens: torch.Tensor) -> torch.Tensor:
    """[0, 3, 5] -> [0, 1, 2, 0, 1]: position of every token inside its document."""
    total = int(cu_seqlens[-1])
    idx = torch.arange(total, device=cu_seqlens.device, dtype=cu_seqlens.dtype)
    lens = cu_seqlens[1:] - cu_seqlens[:-1]
    starts = torch.repeat_interleave(cu_seqlens[:-1], lens.long(), output_size=total)
    return idx - starts


def lens_to_cum_len(sizes, dtype=torch.int32, device=None) -> torch.Tensor:
    sizes = torch.as_tensor(sizes, dtype=torch.int64)
    out = torch.zeros(len(sizes) + 1, dtype=torch.int64)
    out[1:] = torch.cumsum(sizes, 0)
    return out.to(dtype=dtype, device=device)


def convert_num(num: float, nfp: int = 3, G: bool = False) -> str:  # noqa: N803
    units = [("T", 1e12), ("G" if G else "B", 1e9), ("M", 1e6), ("K", 1e3)]
    for u, s in units:
        if abs(num) >= s:
            return f"{num / s:.{nfp}f}{u}"
    return f"{num:.{nfp}f}" if isinstance(num, float) else str(num)


def pad_tensor(t: torch.Tensor, dim: int, to: int, value=0) -> torch.Tensor:
    cur = t.shape[dim]
    if cur >= to:
        return t
    shape = list(t.shape)
    shape[dim] = to - cur
    return torch.cat([t, torch.full(shape, value, dtype=t.dtype, device=t.device)], dim=dim)


def list_split(data: Sequence, split: int) -> list[list]:
    """Contiguous split into ``split`` parts, earlier parts take the remainder: [0,1,2] x2 -> [0,1],[2]."""
    n, r = divmod(len(data), split)
    out, pos = [], 0
    for i in range(split):
        k = n + (1 if i < r else 0)
        out.append(list(data[pos : pos + k]))
        pos += k
    return out


def list_split_T(data: Sequence, split: int) -> list[list]:  # noqa: N802
    """Strided split: element i goes to part i % split."""
    return [list(data[i::split]) for i in range(split)]


def list_chunk(data: Sequence, chunk_size: int) -> list[list]:
    return [list(data[i : i + chunk_size]) for i in range(0, len(data), chunk_size)]


def balanced_list_split(data: Sequence, sizes: Sequence[int], split: int, number_balance: bool = False) -> list[list]:
    """Greedy size-balanced partition (largest first onto the lightest part). With
    ``number_balance`` the parts also receive (almost) equal item counts."""
    order = sorted(range(len(data)), key=lambda i: (-sizes[i], i))
    parts: list[list] = [[] for _ in range(split)]
    load = [0] * split
    cap = -(-len(data) // split) if number_balance else None
    for i in order:
        cands = [q for q in range(split) if cap is None or len(parts[q]) < cap]
        q = min(cands, key=lambda j: (load[j], j))
        parts[q].append(data[i])
        load[q] += sizes[i]
    return parts


def balanced_list_split_keep_order(data: Sequence, sizes: Sequence[int], k: int) -> list[list]:
    """Split into ``k`` contiguous runs minimising the largest run sum (binary search on the bound)."""
    if k <= 0:
        raise ValueError("k must be positive")
    lo, hi = max(sizes, default=0), sum(sizes)

    def runs_needed(bound):
        cnt, cur = 1, 0
        for s in sizes:
            if cur + s > bound:
                cnt, cur = cnt + 1, 0
            cur += s
        return cnt

    while lo < hi:
        mid = (lo + hi) // 2
        if runs_needed(mid) <= k:
            hi = mid
        else:
            lo = mid + 1
    out, cur, acc = [], [], 0
    for item, s in zip(data, sizes):
        if cur and acc + s > lo:
            out.append(cur)
            cur, acc = [], 0
        cur.append(item)
        acc += s
    out.append(cur)
    while len(out) < k:
        out.append([])
    return out


def recur_to(sample: Any, to="cpu"):
    """Move every tensor of a nested container (dict / list / tuple / DataClass) to a device."""
    from ..config import DataClass

    if torch.is_tensor(sample):
        return sample.to(to, non_blocking=True)
    if isinstance(sample, dict):
        return {k: recur_to(v, to) for k, v in sample.items()}
    if isinstance(sample, DataClass):
        for k, v in sample.items():
            sample[k] = recur_to(v, to)
        return sample
    if isinstance(sample, (list, tuple)):
        return type(sample)(recur_to(v, to) for v in sample)
    return sample


@contextlib.contextmanager
def fork_rng_state(seed: int = 2718):
    py, tc = random.getstate(), torch.get_rng_state()
    random.seed(seed)
    torch.manual_seed(seed)
    try:
        yield
    finally:
        random.setstate(py)
        torch.set_rng_state(tc)


def cache_with_tensor(is_tensor: list, maxsize: int = 128):
    """LRU cache whose key uses tensor *identity* (``id`` + version) for the flagged positional
    arguments; entries die with their tensors."""

    def deco(fn):
        cache: OrderedDict = OrderedDict()

        @functools.wraps(fn)
        def wrapper(*args):
            key = []
            for i, a in enumerate(args):
                if i < len(is_tensor) and is_tensor[i] and torch.is_tensor(a):
                    key.append(("T", id(a), a._version, tuple(a.shape)))
                else:
                    key.append(("V", a))
            key = tuple(key)
            hit = cache.get(key)
            if hit is not None:
                refs, val = hit
                if all(r() is not None for r in refs):
                    cache.move_to_end(key)
                    return val
                del cache[key]
            val = fn(*args)
            refs = [weakref.ref(a) for i, a in enumerate(args) if i < len(is_tensor) and is_tensor[i] and torch.is_tensor(a)]
            cache[key] = (refs, val)
            while len(cache) > maxsize:
                cache.popitem(last=False)
            return val

        wrapper.cache = cache
        return wrapper

    return deco


def run_async(coro):
    try:
        loop = asyncio.get_running_loop()
    except RuntimeError:
        return asyncio.run(coro)
    return loop.run_until_complete(coro)


def retry_on(exceptions=(Exception,), retries: int = 3, delay: float = 1.0, backoff: float = 2.0,
             max_delay: float = 60.0, on_retry: Callable | None = None):
    """Retry decorator for sync and async callables with exponential back-off."""

    def deco(fn):
        if asyncio.iscoroutinefunction(fn):
            @functools.wraps(fn)
            async def awrap(*a, **k):
                d = delay
                for attempt in range(retries + 1):
                    try:
                        return await fn(*a, **k)
                    except exceptions as e:
                        if attempt == retries:
                            raise
                        if on_retry:
                            on_retry(e, attempt)
                        await asyncio.sleep(d)
                        d = min(d * backoff, max_delay)
            return awrap

        @functools.wraps(fn)
        def wrap(*a, **k):
            d = delay
            for attempt in range(retries + 1):
                try:
                    return fn(*a, **k)
                except exceptions as e:
                    if attempt == retries:
                        raise
                    if on_retry:
                        on_retry(e, attempt)
                    time.sleep(d)
                    d = min(d * backoff, max_delay)
        return wrap

    return deco


def get_git_revision_hash() -> str:
    try:
        return subprocess.check_output(["git", "rev-parse", "HEAD"], stderr=subprocess.DEVNULL).decode().strip()
    except Exception:
        return "unknown"


def require_package(package: str):
    try:
        return importlib.import_module(package)
    except ImportError as e:
        raise ImportError(f"package '{package}' is required for this feature") from e


def get_my_ip() -> str:
    try:
        return socket.gethostbyname(socket.gethostname())
    except OSError:
        return "127.0.0.1"


def get_free_port() -> int:
    with socket.socket() as s:
        s.bind(("", 0))
        return s.getsockname()[1]


def sync_point(text: str = "") -> None:
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()


def load(path: str, mode: str | None = None, **kwargs):
    """Read a file by its extension (or ``mode``): ``json``, ``jsonl`` (list of records), ``hjson``, ``torch``
    (``.pt`` / ``.pth``, on the CPU), ``pickle`` (``.pkl``), ``yaml``, ``npy`` / ``npz``, ``safetensors`` (dict of
    tensors), ``text`` (``.txt``); reference ``steptronoss/utils/utils.py:546-590``."""
    import json
    import pickle

    def is_(ext: tuple, name: str) -> bool:
        return mode == name or (mode is None and path.endswith(ext))

    if is_((".json",), "json"):
        with open(path, "rb") as f:
            return json.load(f, **kwargs)
    if is_((".jsonl",), "jsonl"):
        with open(path, encoding="utf-8") as f:
            return [json.loads(line, **kwargs) for line in f if line.strip()]
    if is_((".hjson",), "hjson"):
        import hjson

        with open(path, "rb") as f:
            return hjson.load(f, **kwargs)
    if is_((".pt", ".pth"), "torch"):
        return torch.load(path, weights_only=False, map_location="cpu", **kwargs)
    if is_((".pkl", ".pickle"), "pickle"):
        with open(path, "rb") as f:
            return pickle.load(f, **kwargs)
    if is_((".yaml", ".yml"), "yaml"):
        import yaml

        with open(path, "rb") as f:
            return yaml.safe_load(f)
    if is_((".npy", ".npz"), "numpy"):
        import numpy as np

        return np.load(path, **kwargs)
    if is_((".safetensors",), "safetensors"):
        from safetensors.torch import load_file

        return load_file(path, **kwargs)
    if is_((".txt",), "text"):
        with open(path, encoding="utf-8") as f:
            return f.read()
    raise ValueError(f"cannot tell how to load {path!r}: pass mode=json|jsonl|hjson|torch|pickle|yaml|numpy|safetensors|text")


# ---- files, modules, pickles ---------------------------------------------------------------------------------------
def check_and_link(src: str, dst: str) -> None:
    """Symlink ``dst -> src``; an existing link to the same target is fine, anything else in the way raises."""
    import os

    src, dst = src.rstrip("/"), dst.rstrip("/")
    try:
        os.symlink(src, dst)
    except OSError:
        if not os.path.islink(dst) or os.readlink(dst) != src:
            raise


def try_save(*args, **kwargs):
    """``torch.save`` that logs a failure instead of raising (a side dump must not end a job)."""
    from .logger import logger

    try:
        return torch.save(*args, **kwargs)
    except Exception as e:
        logger.error(f"torch.save failed: {e}")
        return None


def get_object_from_file(file: str, name: str = "Exp"):
    """``name`` from the python file ``file`` given as a path relative to an import root (``playground/x/y.py`` ->
    module ``playground.x.y``), e.g. the experiment class of an experiment file."""
    import os

    stem, _ = os.path.splitext(file)
    module = ".".join(p for p in stem.replace(os.sep, "/").split("/") if p not in ("", "."))
    return getattr(importlib.import_module(module), name)


def hack_pickle_load() -> None:
    """Let ``pickle.load`` get past classes that cannot be imported any more (an old dump naming a module that
    moved): such objects come back as inert placeholders.  Process-wide; for inspection tools, not for training."""
    import pickle

    class LoadFailure:
        def __init__(self, *a, **k):
            pass

        def __setstate__(self, state):
            self.state = state

    pickle.Unpickler = pickle._Unpickler                     # the pure-python unpickler can be patched
    if getattr(pickle._Unpickler.find_class, "_tolerant", False):
        return
    find = pickle._Unpickler.find_class

    def find_class(self, module, name):
        try:
            return find(self, module, name)
        except Exception:
            print(f"Cannot Load {module}.{name}: replaced by a placeholder.")
            return LoadFailure

    find_class._tolerant = True
    pickle._Unpickler.find_class = find_class


def deprecated(message: str = "This function is deprecated."):
    """Decorator: warn (once per function) when a deprecated function is called."""

    def decorate(fn):
        warned = []

        @functools.wraps(fn)
        def wrapper(*a, **k):
            if not warned:
                from .logger import logger

                logger.warning(f"{fn.__qualname__}: {message}")
                warned.append(True)
            return fn(*a, **k)

        return wrapper

    return decorate


class GroupedProgressBar:
    """One progress bar over everything plus one per named group (``totals``: name -> count)."""

    def __init__(self, totals: dict):
        from tqdm import tqdm

        self.total_bar = tqdm(total=sum(totals.values()), desc="All Groups", position=0, dynamic_ncols=True)
        self.group_bars = {name: tqdm(total=n, desc=name, position=i, dynamic_ncols=True)
                           for i, (name, n) in enumerate(totals.items(), start=1)}

    def update(self, name: str, n: int = 1) -> None:
        self.total_bar.update(n)
        self.group_bars[name].update(n)

    def close(self) -> None:
        for bar in [self.total_bar, *self.group_bars.values()]:
            bar.close()
