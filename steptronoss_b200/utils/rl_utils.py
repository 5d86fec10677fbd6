"""Reinforcement-learning helpers: running moments, generalised advantage estimation, sample dumping and
the acknowledged ("persistent") queues behind the rollout flow controllers.

Reference: ``steptronoss/utils/rl_utils.py:25-404``.
"""
from __future__ import annotations

import contextlib
import os
import re
import threading
import time
from collections import OrderedDict, defaultdict, deque
from typing import Any
from uuid import uuid4

import torch

from .dist_utils import all_gather_object


class RunningMoments:
    """Running mean / std of a stream whose batches are spread over the DP group."""

    def __init__(self):
        self.mean, self.std, self.var, self.count = 0.0, 1.0, 1.0, 1e-24

    def update(self, xs: torch.Tensor):
        from ..parallel.state import PM

        group = PM.group_of("DP")
        stats = torch.stack([torch.as_tensor(float(xs.numel()), device=xs.device), xs.float().sum()])
        if group is not None:
            torch.distributed.all_reduce(stats, group=group)
        n, mean = stats[0], stats[1] / stats[0]
        var = ((xs.float() - mean) ** 2).sum()
        if group is not None:
            torch.distributed.all_reduce(var, group=group)
        var = var / n
        delta = mean - self.mean
        tot = self.count + n
        tot_sum = self.var * self.count + delta ** 2 * self.count * n / tot + var * n
        self.mean = self.mean + delta * n / tot
        self.var = tot_sum / tot
        self.std = (self.var * tot / (tot - 1)).sqrt()
        self.count = tot
        return mean, (var * n / (n - 1)).sqrt()


class DistributedDictList:
    """``dict[str, list]`` filled locally inside ``in_local()`` and merged over the group on exit."""

    def __init__(self, dist_group=None):
        self.local_data, self.global_data = defaultdict(list), defaultdict(list)
        self._in_local, self.group = False, dist_group

    @contextlib.contextmanager
    def in_local(self):
        self._in_local = True
        yield
        self.synchronize()
        self._in_local = False

    def __setitem__(self, key, value):
        (self.local_data if self._in_local else self.global_data)[key] = value

    def __getitem__(self, key):
        return (self.local_data if self._in_local else self.global_data)[key]

    def synchronize(self):
        gathered = all_gather_object(self.local_data, group=self.group)
        self.local_data = defaultdict(list)
        for d in gathered:
            for k, v in d.items():
                self.global_data[k] += v


def compute_gae(values: torch.Tensor, rewards: torch.Tensor, lambd: float = 0.95, gamma: float = 1.0,
                cu_seqlens: torch.Tensor | None = None):
    """Advantages and returns along the last dimension (``cu_seqlens`` restarts the recursion per packed
    segment of a 1-D input).  On CUDA one kernel walks every segment backwards in parallel; no host loop."""
    if values.is_cuda and values.dim() == 1:
        from ..ops import native

        v, r = values.float().contiguous(), rewards.float().contiguous()
        if cu_seqlens is None:
            cu_seqlens = torch.tensor([0, v.numel()], dtype=torch.int32, device=v.device)
        cu = cu_seqlens.to(device=v.device, dtype=torch.int32).contiguous()
        adv, ret = torch.empty_like(v), torch.empty_like(v)
        rc = native.load().stb_gae(v.data_ptr(), r.data_ptr(), cu.data_ptr(), cu.numel() - 1, float(gamma),
                                   float(lambd), adv.data_ptr(), ret.data_ptr(), native.stream())
        native.check(rc, "gae")
        return adv, ret
    if cu_seqlens is not None and values.dim() == 1:
        adv, ret = torch.empty_like(values, dtype=torch.float32), torch.empty_like(values, dtype=torch.float32)
        bounds = [int(x) for x in cu_seqlens.tolist()]
        for b, e in zip(bounds[:-1], bounds[1:]):
            if e > b:
                adv[b:e], ret[b:e] = compute_gae(values[b:e], rewards[b:e], lambd, gamma)
        return adv, ret
    v, r = values.float(), rewards.float()
    T = v.shape[-1]
    nxt = torch.cat([v[..., 1:], torch.zeros_like(v[..., :1])], dim=-1)
    delta = r + gamma * nxt - v
    adv = torch.empty_like(delta)
    run = torch.zeros_like(delta[..., 0])
    for t in reversed(range(T)):
        run = delta[..., t] + gamma * lambd * run
        adv[..., t] = run
    return adv, adv + v


def gae_coefficients(T: int, lambd: float = 0.95, gamma: float = 1.0, device=None) -> torch.Tensor:
    """``C[s, t] = (gamma * lambd) ** (s - t)`` for ``s >= t``, else 0: ``advantages = delta @ C``."""
    idx = torch.arange(T, device=device)
    power = (idx[:, None] - idx[None, :]).float()
    return torch.where(power >= 0, torch.tensor(float(gamma * lambd), device=device) ** power.clamp_min(0), torch.zeros((), device=device))


def compute_gae_opt(values, rewards, lambd: float = 0.95, gamma: float = 1.0, gae_coeff: torch.Tensor | None = None):
    """``compute_gae`` with the reference's signature (utils/rl_utils.py:195-210).  With a precomputed coefficient
    matrix (``gae_coefficients``; its top-left ``T x T`` corner is used) the recursion becomes one product, which
    is how batches of equal-length rows are best done; without it this is ``compute_gae`` (one kernel on CUDA)."""
    if gae_coeff is None:
        return compute_gae(values, rewards, lambd, gamma)
    v, r = values.float(), rewards.float()
    T = v.shape[-1]
    nxt = torch.cat([v[..., 1:], torch.zeros_like(v[..., :1])], dim=-1)
    adv = (r + gamma * nxt - v) @ gae_coeff[:T, :T].to(device=v.device, dtype=v.dtype)
    return adv, adv + v


class RaggedPPOSampleDumper:
    """Unpack ``PackedPPOSamples`` into per-sample dicts holding the requested keys (for ``torch.save``)."""

    packed_keys = ("ref_logprobs", "actor_logprobs", "advantages", "returns", "values")

    def _unpack(self, packed, keys: list) -> list:
        samples = packed.samples or []
        wanted = [k for k in keys if k in self.packed_keys]
        if not samples or not wanted:
            return samples
        cu = [int(x) for x in packed.cu_seqlens.tolist()]
        mask = packed.is_gen_mask.reshape(-1)
        lens = [int(mask[b:e].sum()) for b, e in zip(cu[:-1], cu[1:])]
        for key in wanted:
            flat = getattr(packed, key, None)
            if flat is None:
                continue
            off = 0
            for sample, n in zip(samples, lens):
                setattr(sample, key, flat[off:off + n])
                off += n
        return samples

    def __call__(self, samples: list, dump_sample_keys: list) -> list:
        out = []
        for packed in samples:
            for s in self._unpack(packed, dump_sample_keys):
                item = {k: getattr(s, k) for k in dump_sample_keys}
                item["meta"] = s.meta
                out.append(item)
        return out


class PersistentQueue:
    """FIFO whose consumers acknowledge what they took: ``get`` moves an item to *pending* under a fresh id,
    ``ack(id)`` forgets it; a snapshot (``state_dict``) puts unacknowledged items back in front, in order."""

    def __init__(self):
        self.data: deque = deque()
        self.pending: OrderedDict = OrderedDict()

    def __repr__(self):
        def runs(items):
            out, last, n = [], None, 0
            for it in list(items) + [None]:
                if type(it) is not last:
                    if n:
                        out.append(f"{last.__name__} x{n}")
                    last, n = type(it), 0
                n += 1
            return ", ".join(out)

        return f"{type(self).__name__}[{runs(self.data)}]~[{runs(reversed(self.pending.values()))}]~>"

    def pop(self) -> Any:
        while not self.data:
            time.sleep(0.05)
        return self.data.pop()

    def get(self) -> tuple[str, Any]:
        item = self.pop()
        key = str(uuid4())
        self.pending[key] = item
        return key, item

    def put(self, *items) -> None:
        self.data.extendleft(items)

    def ack(self, key) -> None:
        self.pending.pop(key, None)

    def state_dict(self):
        return list(self.data) + list(self.pending.values())[::-1]

    def load_state_dict(self, state) -> None:
        self.data = deque(state)
        self.pending = OrderedDict()

    @classmethod
    def from_state_dict(cls, state):
        q = cls()
        q.load_state_dict(state)
        return q

    def __len__(self):
        return len(self.data)

    def empty(self) -> bool:
        return len(self) == 0

    def all_done(self) -> bool:
        return not (self.data or self.pending)


class PersistentSource(PersistentQueue):
    """Queue fed by a state-dict iterator; restored items are served before new ones."""

    def __init__(self, nextable):
        super().__init__()
        self._source = nextable

    def pop(self):
        return self.data.pop() if self.data else next(self._source)

    def put(self, *items):
        raise RuntimeError("Cannot put to Source!")

    def state_dict(self):
        return {"source": self._source.state_dict(), "data": super().state_dict()}

    def load_state_dict(self, state):
        self._source.load_state_dict(state["source"])
        super().load_state_dict(state["data"])


class PersistentDumper(PersistentQueue):
    """Sink that writes every ``dump_interval`` items to ``pdump_<n>.pt`` in ``dump_dir``."""

    def __init__(self, dump_dir: str = "./", dump_interval: int = 1024):
        super().__init__()
        self.dump_dir, self.dump_interval, self.dump_counter = dump_dir, dump_interval, 0
        if os.path.exists(dump_dir):
            ids = [int(m.group(1)) for m in (re.search(r"pdump_(\d+)\.pt", x) for x in os.listdir(dump_dir)) if m]
            if ids:
                self.dump_counter = max(ids) + 1

    def get(self):
        raise RuntimeError("Cannot get from Dumper!")

    def ack(self, key):
        raise RuntimeError("Cannot ack sample to Dumper!")

    def put(self, item):
        self.data.appendleft(item)
        if len(self.data) >= self.dump_interval:
            os.makedirs(self.dump_dir, exist_ok=True)
            torch.save(list(self.data), os.path.join(self.dump_dir, f"pdump_{self.dump_counter}.pt"))
            self.dump_counter += 1
            self.data.clear()

    def state_dict(self):
        return list(self.data)


class PersistentFlow(dict):
    """Named stages of :class:`PersistentQueue` plus a lock and a free-form ``meta`` dict, checkpointable as
    one unit.  Moving an item between stages under ``flow.lock`` (put downstream, then ack upstream) makes
    a snapshot taken at any time lose nothing and duplicate nothing."""

    class Signal(dict):
        def __init__(self, name: str, **data):
            super().__init__(**data)
            self.name = self["name"] = name

    def __init__(self, meta: dict | None = None, **stages):
        super().__init__(**stages)
        self.lock = threading.Lock()
        self.meta = meta or {}

    def state_dict(self):
        return {k: self[k].state_dict() for k in self} | {"meta": self.meta}

    def load_state_dict(self, state: dict):
        state = dict(state)
        self.meta = state.pop("meta", {})
        for k, v in state.items():
            self[k].load_state_dict(v)
