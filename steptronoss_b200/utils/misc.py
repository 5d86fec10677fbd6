"""Assorted helpers of the reference's ``utils/utils.py`` and ``utils/general.py`` that the rest of the framework
does not depend on but experiment files and notebooks use: parameter norm, memory one-liners, layer-map and path-tree
rendering, jsonl / msgpack files, device-moving iteration, a multi-valued dictionary, grouped progress bars,
``deprecated``."""
from __future__ import annotations

import functools
import gc
import json
import os

import torch
import torch.distributed as dist

from .logger import logger


# ------------------------------------------------------------------------------------------------ tensors / memory
def calc_params_l2_norm(models) -> float:
    """L2 norm of all parameters of the job, every parameter counted once: tensor-parallel replicas (norms, router)
    only on TP rank 0, expert replicas only on the first rank of their replica group, the sum taken over the
    model-parallel group (reference ``utils/utils.py:36-73``)."""
    from ..parallel.state import PM

    models = models if isinstance(models, (list, tuple)) else [models]
    total = None
    seen = set()
    for m in models:
        for p in m.parameters():
            if id(p) in seen:
                continue
            seen.add(id(p))
            expert = bool(getattr(p, "expert_model_parallel", False))
            sharded = bool(getattr(p, "tensor_model_parallel", False))
            fam = "ETP" if expert else "TP"
            if not sharded and PM.has(fam) and PM.rank_in(fam) != 0:
                continue
            sq = p.detach().float().pow(2).sum()
            total = sq if total is None else total + sq
    if total is None:
        total = torch.zeros(())
    fam = "MP" if PM.has("MP") else None
    if fam and dist.is_initialized() and PM.size_of(fam) > 1:
        dist.all_reduce(total, group=PM.group_of(fam))
    return float(total) ** 0.5


def cos_sim(a: torch.Tensor, b: torch.Tensor) -> float:
    return float(torch.nn.functional.cosine_similarity(a.flatten().float(), b.to(a.device).flatten().float(), dim=0))


def get_mem_brief(name: str = "", unit: str = "G") -> str:
    div = 1024 ** 2 if unit == "M" else 1024 ** 3
    if not torch.cuda.is_available():
        return f"{name} MemReport (no GPU)"
    c = torch.cuda
    return (f"{name} MemReport Allocated: {c.memory_allocated() / div:.1f} (max: {c.max_memory_allocated() / div:.1f}) {unit} | "
            f"Reserved: {c.memory_reserved() / div:.1f} (max: {c.max_memory_reserved() / div:.1f}) {unit} | ")


def force_clear_mem() -> None:
    """Collect garbage and hand cached blocks back to the driver."""
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()


def moving_iter(data, active="cuda", default="cpu"):
    """Iterate ``data`` with the current item on ``active`` and every other item on ``default``.  Items are moved
    with ``recur_to`` (nested containers of tensors); the item is moved back when the consumer asks for the next."""
    from .general import recur_to

    for i, item in enumerate(data):
        item = recur_to(item, active)
        yield item
        moved = recur_to(item, default)
        try:
            data[i] = moved
        except TypeError:  # not an indexable container: nothing to write back to
            pass


# ------------------------------------------------------------------------------------------------ rendering
def _runs(keys: list, value_of) -> list:
    """Maximal runs of consecutive integer keys with equal values: ``[(first, last, value), ...]``."""
    out = []
    for k in keys:
        v = value_of(k)
        if out and out[-1][1] + 1 == k and out[-1][2] == v:
            out[-1] = (out[-1][0], k, v)
        else:
            out.append((k, k, v))
    return out


def format_layermap(layer_map: dict) -> str:
    """``{pp: {vp: {layer: options}}}`` as text, one line per virtual stage, equal consecutive layers collapsed to
    ``first-last``."""
    lines = []
    for pp in sorted(layer_map):
        for vp in sorted(layer_map[pp]):
            chunk = layer_map[pp][vp]
            parts = []
            for a, b, v in _runs(sorted(chunk), lambda k: chunk[k]):
                name = f"{a}" if a == b else f"{a}-{b}"
                opts = ", ".join(f"{k}={v[k]!r}" for k in sorted(v)) if isinstance(v, dict) else repr(v)
                parts.append(f"{name}: {{{opts}}}")
            lines.append(f"pp{pp}/vp{vp}: " + "; ".join(parts))
    return "\n".join(lines)


def print_layer_map(layer_map: dict) -> None:
    logger.info("layer map\n" + format_layermap(layer_map), at=0)


def get_path_tree_repr(paths: list) -> str:
    """File paths as an indented tree (directories first-seen order kept, ``|--`` / ``+--`` branches)."""
    tree: dict = {}
    for p in paths:
        node = tree
        for part in [x for x in p.strip("/").split("/") if x]:
            node = node.setdefault(part, {})
    lines = []

    def walk(node: dict, prefix: str) -> None:
        names = list(node)
        for i, name in enumerate(names):
            last = i == len(names) - 1
            lines.append(prefix + ("+-- " if last else "|-- ") + name)
            walk(node[name], prefix + ("    " if last else "|   "))

    walk(tree, "")
    return "\n".join(lines)


# ------------------------------------------------------------------------------------------------ files
def safe_dump_jsonl(records: list, path: str) -> bool:
    """Write one JSON object per line; an error is logged, not raised (metrics dumps must not end a run)."""
    try:
        with open(path, "w", encoding="utf-8") as f:
            for r in records:
                f.write(json.dumps(r, ensure_ascii=False) + "\n")
        return True
    except Exception as e:
        logger.error(f"could not write {path}: {e}", at=None)
        return False


def load_jsonl(path: str) -> list:
    with open(path, encoding="utf-8") as f:
        return [json.loads(line) for line in f if line.strip()]


def safe_dump_msgpack(obj, path: str) -> bool:
    try:
        import msgpack

        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(msgpack.packb(obj, use_bin_type=True))
        os.replace(tmp, path)
        return True
    except Exception as e:
        logger.error(f"could not write {path}: {e}", at=None)
        return False


def load_msgpack(path: str):
    import msgpack

    with open(path, "rb") as f:
        return msgpack.unpackb(f.read(), raw=False)


def check_and_link(src: str, dst: str) -> None:
    """Symlink ``dst -> src``; an existing link that already points there is fine, anything else raises."""
    src, dst = src.rstrip("/"), dst.rstrip("/")
    try:
        os.symlink(src, dst)
    except OSError:
        if not os.path.islink(dst) or os.readlink(dst) != src:
            raise


def try_save(*args, **kwargs):
    try:
        return torch.save(*args, **kwargs)
    except Exception as e:
        logger.error(f"torch.save failed: {e}", at=None)
        return None


# ------------------------------------------------------------------------------------------------ containers / misc
class RepeatedDict:
    """A dictionary whose keys hold a queue of values: ``d[k] = v`` appends, ``d[k]`` reads the oldest, ``pop(k)``
    removes it (``None`` when absent); ``update(other, repeat=n)`` enqueues every value ``n`` times."""

    def __init__(self):
        self.dict: dict = {}

    def pop(self, key):
        q = self.dict.get(key)
        if not q:
            return None
        v = q.pop(0)
        if not q:
            del self.dict[key]
        return v

    def update(self, other: dict, repeat: int = 1) -> None:
        for k, v in other.items():
            self.dict.setdefault(k, []).extend([v] * repeat)

    def clear(self) -> None:
        self.dict.clear()

    def __len__(self) -> int:
        return sum(len(q) for q in self.dict.values())

    def __contains__(self, key) -> bool:
        return key in self.dict

    def __getitem__(self, key):
        return self.dict[key][0]

    def __setitem__(self, key, value) -> None:
        self.dict.setdefault(key, []).append(value)

    def __delitem__(self, key):
        raise NotImplementedError("RepeatedDict does not support del; use pop()")

    def state_dict(self) -> dict:
        return self.dict

    def load_state_dict(self, states: dict | None) -> None:
        self.dict = {} if states is None else states


class GroupedProgressBar:
    """One overall ``tqdm`` bar plus one per named group."""

    def __init__(self, totals: dict):
        from tqdm import tqdm

        self.total_bar = tqdm(total=sum(totals.values()), desc="All Groups", position=0, dynamic_ncols=True)
        self.group_bars = {name: tqdm(total=n, desc=name, position=pos, dynamic_ncols=True)
                           for pos, (name, n) in enumerate(totals.items(), start=1)}

    def update(self, name: str, n: int = 1) -> None:
        self.total_bar.update(n)
        self.group_bars[name].update(n)

    def close(self) -> None:
        self.total_bar.close()
        for b in self.group_bars.values():
            b.close()


def deprecated(message: str = "This function is deprecated."):
    """Log ``message`` the first time the decorated function is called."""

    def deco(fn):
        warned = []

        @functools.wraps(fn)
        def wrapper(*a, **k):
            if not warned:
                warned.append(True)
                logger.warning(f"{fn.__qualname__}: {message}", at=None)
            return fn(*a, **k)

        return wrapper

    return deco
