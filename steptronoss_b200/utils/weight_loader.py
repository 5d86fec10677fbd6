"""Rename / slice / concatenate rules over a HF safetensors checkpoint, and a sharded writer.

Surface of the reference's ``utils/weight_loader.py:34-364`` (``HFWeights``, ``export`` with its small rule
language, ``write_safetensors_to``).  Tensors are read lazily, one at a time, from the shard that holds them
(:class:`~steptronoss_b200.checkpointing.hf_checkpoint.HFWeights`), so exporting a checkpoint never holds more
than the rule's operands in memory; the reference loads every shard up front.

Rule language (one rule per line, or a ``{target: Is | Cat}`` dict):

``new.*.name: old.*.name``
    rename; every ``*`` of the source captures a piece of the key and fills the ``*`` of the target in order
    (``$1``, ``$2`` ... may be written instead of ``*`` in the target).
``new.*: old.*|TP@0``
    rename and keep this rank's slice of dimension 0 under the parallel family ``TP``.
``*wqkv* CAT(0) *q_proj* *k_proj* *v_proj*``  (also written ``*wqkv*: CAT(0) *q_proj* ...``)
    concatenate, along the given dimension, the tensors whose (already renamed) keys match the components; the
    captures of the first component name the others and the target.

Keys that no rename rule matches keep their name.
"""
from __future__ import annotations

import json
import os
import re

import torch

from ..checkpointing.hf_checkpoint import HFWeights as _LazyWeights
from ..parallel.state import PM

__all__ = ["HFWeights", "Is", "Cat", "parse_rules", "key_pattern", "fill_target", "translate", "apply_match",
           "parse_indicator_from_str"]


def key_pattern(glob: str) -> re.Pattern:
    """``*`` captures any run of characters (runs of ``*`` count once), ``?`` one character; the rest is literal."""
    out, prev_star = [], False
    for ch in glob:
        if ch == "*":
            if not prev_star:
                out.append("(.*)")
            prev_star = True
            continue
        prev_star = False
        out.append("." if ch == "?" else re.escape(ch))
    return re.compile("(?s:" + "".join(out) + r")\Z")


def fill_target(match: re.Match, target: str) -> str:
    """Put the captures of ``match`` into ``target`` (``*`` in order, or ``$n``)."""
    groups = match.groups()
    if "*" in target:
        if "$" in target:
            raise ValueError(f"target {target!r} mixes * and $n")
        pieces = target.split("*")
        if len(pieces) - 1 > len(groups):
            raise ValueError(f"target {target!r} has more * than its source captured")
        return "".join(p + (groups[i] if i < len(pieces) - 1 else "") for i, p in enumerate(pieces))
    for i in sorted(range(len(groups)), reverse=True):   # $10 before $1
        target = target.replace(f"${i + 1}", groups[i])
    return target


def translate(pat: str) -> str:
    """The regular expression (as text) that ``key_pattern`` compiles: the reference's name for the glob translation."""
    return key_pattern(pat).pattern


apply_match = fill_target                  # the reference's names for the same two steps of the rule language
parse_indicator_from_str = None            # bound below, once parse_rules exists


class Is:
    """Source key pattern of a rename, with an optional ``|FAMILY@dim`` slice."""

    def __init__(self, source: str):
        self.slice = None
        if "|" in source:
            source, op = source.split("|", 1)
            fam, dim = op.split("@")
            self.slice = (fam.strip(), int(dim))
        self.source = source.strip()
        self.pattern = key_pattern(self.source)


class Cat:
    """Concatenation of the tensors matching ``components`` along ``dim``; ``pop`` removes the operands."""

    def __init__(self, *components: str, dim: int = 0, pop: bool = True):
        if not components:
            raise ValueError("Cat needs at least one component")
        self.components, self.dim, self.pop = components, dim, pop


_CAT = re.compile(r"CAT\((-?\d+)\)")


def parse_rules(rules) -> dict:
    if isinstance(rules, dict):
        return rules
    lines = rules.splitlines() if isinstance(rules, str) else list(rules)
    out: dict = {}
    for line in lines:
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        words = line.replace(":", " ", 1).split() if ":" in line.split("CAT(")[0] else line.split()
        target, rest = words[0], words[1:]
        if not rest:
            raise ValueError(f"rule without a source: {line!r}")
        m = _CAT.fullmatch(rest[0])
        if m:
            out[target] = Cat(*rest[1:], dim=int(m.group(1)))
        elif len(rest) == 1:
            out[target] = Is(rest[0])
        else:
            raise ValueError(f"unknown operation in rule {line!r}")
    return out


parse_indicator_from_str = parse_rules


def _rank_slice(t: torch.Tensor, family: str, dim: int) -> torch.Tensor:
    n, r = PM.size_of(family), PM.rank_in(family)
    if t.shape[dim] % n:
        raise ValueError(f"dimension {dim} of size {t.shape[dim]} does not split over {family}={n}")
    step = t.shape[dim] // n
    return t.narrow(dim, r * step, step)


class HFWeights(_LazyWeights):
    """Checkpoint directory as a read-only mapping ``name -> tensor`` (read on access)."""

    def get(self, k, default=None):
        return self[k] if k in self else default

    def export(self, rules) -> dict:
        """Apply rename / slice rules to every key, then the concatenations; returns ``{new name: tensor}``."""
        rules = parse_rules(rules)
        renames = [(t, r) for t, r in rules.items() if isinstance(r, Is)]
        cats = [(t, r) for t, r in rules.items() if isinstance(r, Cat)]
        # plan first (names only), read afterwards: a tensor is loaded when its output is assembled
        plan: dict = {}
        for k in self.keys():
            name, sl = k, None
            for target, rule in renames:
                m = rule.pattern.match(k)
                if m:
                    name, sl = fill_target(m, target), rule.slice
                    break
            plan[name] = (k, sl)

        def read(name):
            src, sl = plan[name]
            t = self[src]
            return _rank_slice(t, *sl) if sl else t

        out: dict = {}
        consumed: set = set()
        for target, rule in cats:
            lead = key_pattern(rule.components[0])
            for name in list(plan):
                m = lead.match(name)
                if not m or name in consumed:
                    continue
                parts = [fill_target(m, c) for c in rule.components]
                missing = [p for p in parts if p not in plan]
                if missing:
                    raise KeyError(f"CAT rule for {target!r}: no tensor named {missing[0]!r}")
                out[fill_target(m, target)] = torch.cat([read(p) for p in parts], dim=rule.dim)
                if rule.pop:
                    consumed.update(parts)
        for name in plan:
            if name not in consumed and name not in out:
                out[name] = read(name)
        return out

    def write_safetensors_to(self, path: str, shard_max_size: float = 10e9, tensors: dict | None = None) -> dict:
        """Write ``tensors`` (default: this checkpoint) as ``model-%05d.safetensors`` shards of at most
        ``shard_max_size`` bytes plus ``model.safetensors.index.json``; returns the weight map."""
        return write_safetensors(tensors if tensors is not None else self, path, shard_max_size)


def write_safetensors(tensors, path: str, shard_max_size: float = 10e9) -> dict:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    weight_map, total = {}, 0
    shard, shard_bytes, index = {}, 0, 1

    def flush():
        nonlocal shard, shard_bytes, index
        if shard:
            save_file(shard, os.path.join(path, f"model-{index:05d}.safetensors"))
            shard, shard_bytes, index = {}, 0, index + 1

    for k, v in tensors.items():
        v = v.detach().cpu().contiguous()
        size = v.numel() * v.element_size()
        if shard and shard_bytes + size > shard_max_size:
            flush()
        weight_map[k] = f"model-{index:05d}.safetensors"
        shard[k] = v
        shard_bytes += size
        total += size
    flush()
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f)
    return weight_map
