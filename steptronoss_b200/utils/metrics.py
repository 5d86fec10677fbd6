"""Chainable metrics: ``Metric().mean("time").mean("dp").sum("pp")``.

Reference: ``steptronoss/utils/metrics.py:20-782``.  A metric collects values between two log
points (the ``time`` axis) and is then reduced along the declared chain; each non-``time`` link is
one collective over the process-group family of that name (``dp``, ``tp``, ``pp``, ``ep``, ``cp``,
``mp``, ``world``).  Unlike the reference, values added as device tensors stay on the device until
the reduction (no host synchronisation per ``add``).
"""
from __future__ import annotations

import contextlib
from typing import Any

import torch
import torch.distributed as dist

_OPS = ("mean", "sum", "max", "min", "last", "first")


class ROps:
    """Names of the reductions a metric chain takes (``Metric()._link(ROps.mean, RDims.dp)`` = ``.mean("dp")``)."""

    sum, mean, max, min, gather, last, first, std = "sum", "mean", "max", "min", "gather", "last", "first", "std"


class RDims:
    """Names of the axes a metric reduces over: ``time`` (the values of one log interval) and the parallel families."""

    time, tp, pp, dp, ep, mp, cp, world = "time", "tp", "pp", "dp", "ep", "mp", "cp", "world"

    @classmethod
    def _get_group(cls, dim: str):
        """The process group of an axis (None for ``world``, as ``torch.distributed`` spells the default group)."""
        return None if dim == cls.world else _group_for(dim)[0]


def _group_for(axis: str):
    from ..parallel.state import PM

    if axis == "world":
        return dist.group.WORLD if dist.is_initialized() else None, PM.world_size
    name = axis.upper()
    if not PM.has(name):
        return None, 1
    return PM.group_of(name), PM.size_of(name)


def _reduce_time(vals: list, op: str):
    if not vals:
        return None
    if op == "last":
        return vals[-1]
    if op == "first":
        return vals[0]
    ts = [v if torch.is_tensor(v) else torch.tensor(float(v)) for v in vals]
    dev = next((t.device for t in ts if t.is_cuda), ts[0].device)
    st = torch.stack([t.detach().float().to(dev) for t in ts])
    return {"mean": st.mean(0), "sum": st.sum(0), "max": st.amax(0), "min": st.amin(0)}[op]


def _reduce_group(val: torch.Tensor, axis: str, op: str):
    group, size = _group_for(axis)
    if size == 1 or not dist.is_initialized():
        return val
    if dist.get_backend(group) == "nccl" and not val.is_cuda:
        val = val.cuda()
    val = val.clone()
    red = {"mean": dist.ReduceOp.SUM, "sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op]
    dist.all_reduce(val, op=red, group=group)
    if op == "mean":
        val = val / size
    return val


class Metric:
    """``Metric(is_group=True)`` gives a :class:`GroupMetric` (the reference spells grouped metrics this way)."""

    def __new__(cls, *args, is_group: bool = False, **kwargs):
        if is_group and cls is Metric:
            return object.__new__(GroupMetric)
        return object.__new__(cls)

    def __init__(self, name: str | None = None, reductions=None, sample_interval: int = 1,
                 is_group: bool = False) -> None:
        self.chain: list[tuple[str, str]] = list(reductions or [])
        self.values: list = []
        self.enabled = True
        self.name: str | None = name
        self.sample_interval = sample_interval

    def _link(self, op: str, axis: str):
        self.chain.append((op, axis.lower()))
        return self

    def mean(self, axis: str): return self._link("mean", axis)      # noqa: E704
    def sum(self, axis: str): return self._link("sum", axis)        # noqa: E704
    def max(self, axis: str): return self._link("max", axis)        # noqa: E704
    def min(self, axis: str): return self._link("min", axis)        # noqa: E704
    def last(self, axis: str = "time"): return self._link("last", axis)    # noqa: E704
    def first(self, axis: str = "time"): return self._link("first", axis)  # noqa: E704
    def gather(self, axis: str = "world"): return self._link("gather", axis)  # noqa: E704

    def enable(self):
        self.enabled = True
        return self

    def disable(self):
        self.enabled = False
        return self

    def add(self, value, subname: str | None = None, iop: str | None = None) -> None:
        """Record one value. ``iop`` (``"sum"``/``"max"``/...) merges into the last recorded value
        instead of appending (in-place accumulation inside one iteration)."""
        if not self.enabled:
            return
        if callable(iop):  # an input transform such as torch.mean / torch.max / torch.detach
            value, iop = iop(value), None
        if torch.is_tensor(value):
            value = value.detach()
        if iop and self.values:
            prev = self.values[-1]
            self.values[-1] = {"sum": lambda a, b: a + b, "max": lambda a, b: torch.maximum(torch.as_tensor(a), torch.as_tensor(b)),
                               "min": lambda a, b: torch.minimum(torch.as_tensor(a), torch.as_tensor(b)),
                               "mean": lambda a, b: (a + b) / 2}[iop](prev, value)
        else:
            self.values.append(value)

    def reduce(self):
        chain = self.chain or [("mean", "time")]
        val: Any = None
        time_done = False
        for op, axis in chain:
            if axis == "time":
                val = _reduce_time(self.values, op)
                time_done = True
            else:
                if not time_done:
                    val = _reduce_time(self.values, "mean")
                    time_done = True
                if val is None:
                    val = torch.zeros(())
                val = _reduce_group(torch.as_tensor(val, dtype=torch.float32), axis, op)
        if not time_done:
            val = _reduce_time(self.values, "mean")
        return val

    def reset(self) -> None:
        self.values = []

    def __repr__(self) -> str:
        return f"{type(self).__name__}({'.'.join(f'{o}({a})' for o, a in self.chain)})"


class GroupMetric(Metric):
    """A family of metrics sharing one chain, keyed by ``subname``; reduces to ``{name/sub: value}``."""

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        self.sub: dict[str, list] = {}

    def add(self, value, subname: str | None = None, iop: str | None = None) -> None:
        if not self.enabled:
            return
        key = subname or "_"
        self.values = self.sub.setdefault(key, [])
        super().add(value, iop=iop)
        self.sub[key] = self.values

    def reduce(self):
        out = {}
        for key in sorted(self.sub):
            self.values = self.sub[key]
            out[key] = Metric.reduce(self)
        return out

    def reset(self) -> None:
        self.sub, self.values = {}, []


class ModelLayerMetric(GroupMetric):
    """Per-layer values (``subname`` = layer id) gathered along the pipeline by the ``pp`` link."""


class GradNormMetric(GroupMetric):
    """Gradient norms per named part of the model (``layer3``, ``tok_embeddings``, ``output`` ...).

    ``add(squared_norm, subname=part)`` records what THIS rank contributes (its shards, its pipeline stage); ``reduce``
    adds the contributions of all ranks and takes the root.  Ranks may hold different parts: the names are agreed on
    first, so every rank joins the same all-reduce.  The last recorded step of the interval is reported."""

    def __init__(self) -> None:
        super().__init__()
        self.chain = [("last", "time")]
        self.armed = False
        """set by the producer on EVERY rank of a job that records detailed norms, also on ranks that contribute
        nothing: only then does ``reduce`` talk to the other ranks (no collective in jobs that do not use this)"""

    def reduce(self):
        if not self.armed:
            return {}
        local = {}
        for key, vals in self.sub.items():
            if vals:
                local[key] = float(torch.as_tensor(vals[-1]))
        keys = sorted(local)
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
        if multi:
            every = [None] * dist.get_world_size()
            dist.all_gather_object(every, keys)
            keys = sorted(set().union(*every))
        if not keys:
            return {}
        vec = torch.tensor([local.get(k, 0.0) for k in keys], dtype=torch.float64)
        if multi:
            on_gpu = dist.get_backend() == "nccl"
            buf = vec.cuda() if on_gpu else vec
            dist.all_reduce(buf)
            vec = buf.cpu()
        return {k: vec[i].sqrt().float() for i, k in enumerate(keys)}


class AvgMetric(Metric):
    """Statistic of the pooled samples: every value recorded in the interval on every rank of the group goes into one
    list, and ``mean`` / ``max`` / ``min`` / ``std`` is taken over that list - a true per-sample statistic, where a
    plain ``Metric`` would average per-rank means whatever the number of samples behind each.  One reduction
    (``AvgMetric().mean("world")``; the last one chained wins), over ``dp`` or ``world``; values are python numbers.
    Reference: utils/metrics.py:268-336."""

    def std(self, axis: str):
        return self._link("std", axis)

    def add(self, value, subname=None, iop=None) -> None:  # type: ignore[override]
        if not self.enabled:
            return
        if callable(iop):
            value = iop(value)
        self.values.append(float(value))

    def reduce(self):
        pairs = [(op, ax) for op, ax in self.chain if ax != "time"]
        op, axis = pairs[-1] if pairs else ("mean", "world")
        if op not in ("mean", "max", "min", "std"):
            raise ValueError(f"AvgMetric reduces with mean, max, min or std, not {op!r}")
        pooled = list(self.values)
        group, size = _group_for(axis)
        if size > 1 and dist.is_initialized():
            from .dist_utils import all_gather_object

            pooled = [v for part in all_gather_object(pooled, group=group) for v in part]
        if not pooled:
            return None
        data = torch.tensor(pooled, dtype=torch.float32)
        if op == "std":
            return data.std() if data.numel() > 1 else torch.zeros(())
        return {"mean": data.mean, "max": data.max, "min": data.min}[op]()


class PercentageMetric(Metric):
    """``add(numerator, denominator)`` pairs reduce to one ratio; ``add(count, subname=category)`` entries
    reduce to ``{category: share of the total}``."""

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        self.cats: dict[str, float] = {}

    def add(self, value, total=None, subname=None, iop=None) -> None:  # type: ignore[override]
        if not self.enabled:
            return
        if subname is not None:
            self.cats[subname] = self.cats.get(subname, 0.0) + float(value)
            return
        v = torch.as_tensor(value, dtype=torch.float32).detach()
        t = torch.as_tensor(1.0 if total is None else total, dtype=torch.float32).detach()
        if t.device != v.device:
            t = t.to(v.device)
        self.values.append(torch.stack([v.reshape(()), t.reshape(())]))

    def reset(self) -> None:
        super().reset()
        self.cats = {}

    def _reduce_categories(self):
        cats = dict(self.cats)
        axes = [ax for _, ax in self.chain if ax != "time"]
        if axes and dist.is_available() and dist.is_initialized():
            group, _ = _group_for(axes[0])
            gathered = [None] * dist.get_world_size(group)
            dist.all_gather_object(gathered, cats, group=group)
            cats = {}
            for d in gathered:
                for k, v in d.items():
                    cats[k] = cats.get(k, 0.0) + v
        tot = sum(cats.values())
        return {k: torch.tensor(v / tot if tot else 0.0) for k, v in sorted(cats.items())}

    def reduce(self):
        if self.cats:
            return self._reduce_categories()
        if not self.values:
            return None
        saved_chain = self.chain
        self.chain = [(("sum" if op == "mean" else op), ax) for op, ax in (saved_chain or [("sum", "time")])]
        try:
            pair = Metric.reduce(self)
        finally:
            self.chain = saved_chain
        return pair[0] / pair[1].clamp_min(1e-12)


class HistogramMetric(Metric):
    def reduce(self):
        if not self.values:
            return None
        return torch.cat([torch.as_tensor(v).detach().float().flatten().cpu() for v in self.values])


class TextMetric(Metric):
    """Keeps up to ``max_items`` strings per interval (sample generations for qualitative inspection)."""

    def __init__(self, max_items: int | None = None, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        self.max_items = max_items

    def add(self, value, subname=None, iop=None) -> None:
        if self.enabled and (self.max_items is None or len(self.values) < self.max_items):
            self.values.append(str(value))

    def reduce(self):
        vals = list(self.values)
        if any(op == "gather" for op, _ in self.chain) and dist.is_available() and dist.is_initialized():
            axis = next(ax for op, ax in self.chain if op == "gather")
            group, _ = _group_for(axis)
            out = [None] * dist.get_world_size(group)
            dist.all_gather_object(out, vals, group=group)
            vals = [v for part in out for v in part]
        return vals[: self.max_items] if self.max_items else vals


class WithDataDumpOutlierMetric(Metric):
    """Counts, and keeps the evidence of, values that stand out against the recent past (e.g. a loss spike).

    ``add({"real_value": v, "data": payload})`` records one observation together with whatever is needed to
    reproduce it (typically the micro-batch).  At reduction time the mean of the observations since the last
    reduction joins a sliding window (``max_window_size`` reductions); once the window is full every observation
    above the window's mean is an outlier: its payload is written to ``<outlier_data_dump_dir>/outlier_losses/``
    and the metric's value is the number of outliers summed over the data-parallel ranks.  Counterpart of the
    reference's metric of the same name (``steptronoss/utils/metrics.py:617-693``)."""

    def __init__(self, name: str | None = None, reductions=None, sample_interval: int = 1, is_group: bool = False,
                 max_window_size: int = 100, outlier_data_dump_dir: str | None = None) -> None:
        super().__init__(name=name, reductions=reductions, sample_interval=sample_interval)
        import collections
        import os

        if outlier_data_dump_dir is None:
            raise ValueError("WithDataDumpOutlierMetric needs outlier_data_dump_dir")
        self.window = collections.deque(maxlen=max_window_size)
        self.pending: list = []          # (value, payload) since the last reduction
        self.output_dir = os.path.join(outlier_data_dump_dir, "outlier_losses")
        self.dumped: list = []           # paths written so far
        os.makedirs(self.output_dir, exist_ok=True)

    def add(self, value, subname: str | None = None, iop=None) -> None:  # type: ignore[override]
        if not self.enabled:
            return
        if subname is not None:
            raise ValueError("WithDataDumpOutlierMetric has no sub-metrics")
        if callable(iop):
            value = iop(value)
        if not (isinstance(value, dict) and {"real_value", "data"} <= set(value)):
            raise ValueError("expected {'real_value': number, 'data': payload}")
        self.pending.append((float(value["real_value"]), value["data"]))

    def _count_local_outliers(self) -> float:
        import os

        if not self.pending:
            return 0.0
        mean_now = sum(v for v, _ in self.pending) / len(self.pending)
        if len(self.window) < self.window.maxlen:       # still learning what "normal" is
            self.window.append(mean_now)
            return 0.0
        baseline = sum(self.window) / len(self.window)
        count = 0
        for i, (v, payload) in enumerate(self.pending):
            if v > baseline:
                path = os.path.join(self.output_dir, f"value{v:.6g}_n{len(self.dumped)}.pt")
                torch.save({"real_value": v, "baseline": baseline, "data": payload}, path)
                self.dumped.append(path)
                count += 1
        self.window.append(mean_now)
        return float(count)

    def reduce(self):
        local = torch.tensor(self._count_local_outliers())
        return _reduce_group(local, "dp", "sum")

    def reset(self) -> None:
        self.pending = []


class DummyMetric:
    """Accepts and forgets: what ``GlobalMetrics.<unregistered name>`` resolves to."""

    enabled = False

    def add(self, *args, **kwargs) -> None:
        pass

    def reduce(self):
        return None

    def reset(self) -> None:
        pass


dummy_metric = DummyMetric()


class MetricHolder:
    """Registry reachable as ``GlobalMetrics.<name>``; unknown names resolve to a disabled sink so
    that model code can record metrics that an experiment did not register."""

    def __init__(self) -> None:
        object.__setattr__(self, "metrics", {})
        object.__setattr__(self, "_disabled", False)
        object.__setattr__(self, "_sink", dummy_metric)

    def register(self, name: str, metric: Metric) -> None:
        metric.name = name
        self.metrics[name] = metric

    def __setattr__(self, name: str, value) -> None:
        if isinstance(value, Metric):           # ``holder.loss = Metric().mean("time")`` registers, like ``register``
            self.register(name, value)
        else:
            object.__setattr__(self, name, value)

    def batch_register(self, cfg) -> None:
        for k, v in cfg.items():
            if isinstance(v, Metric):
                self.register(k, v)

    def __getattr__(self, name: str):
        m = self.metrics.get(name)
        if m is None or self._disabled:
            return self._sink
        return m

    def __contains__(self, name: str) -> bool:
        return name in self.metrics

    def reduce_all(self, reset: bool = True) -> dict:
        out = {}
        for name, m in self.metrics.items():
            val = m.reduce()
            if isinstance(val, dict):
                for k, v in val.items():
                    if v is not None:
                        out[f"{name}/{k}" if k != "_" else name] = v
            elif val is not None:
                out[name] = val
            if reset:
                m.reset()
        return out

    def reset(self) -> None:
        for m in self.metrics.values():
            m.reset()

    def clear(self) -> None:
        self.metrics.clear()

    @contextlib.contextmanager
    def disable(self):
        prev = self._disabled
        object.__setattr__(self, "_disabled", True)
        try:
            yield
        finally:
            object.__setattr__(self, "_disabled", prev)

    @contextlib.contextmanager
    def fork(self):
        """Temporarily collect into fresh copies (e.g. an evaluation pass); yields the holder."""
        saved = {k: list(getattr(m, "values", [])) for k, m in self.metrics.items()}
        saved_sub = {k: dict(m.sub) for k, m in self.metrics.items() if isinstance(m, GroupMetric)}
        self.reset()
        try:
            yield self
        finally:
            for k, m in self.metrics.items():
                m.values = saved.get(k, [])
                if isinstance(m, GroupMetric):
                    m.sub = saved_sub.get(k, {})


GlobalMetrics = MetricHolder()
