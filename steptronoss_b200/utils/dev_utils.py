"""Developer aids (reference ``steptronoss/utils/dev_utils.py:10-202``, ``utils/utils.py:377-453``):
profiler window around a module's forward/backward, collective bandwidth probe, parameter table."""
from __future__ import annotations

import functools
import os
import time

import torch
import torch.distributed as dist

from .logger import logger


def capture_trace(at: int = 0, fw_file: str = "fw_trace.json", bw_file: str | None = None, rank: int = 0,
                  warmup: int = 1):
    """Decorator for a module ``forward``: on call number ``warmup + at`` (on global rank ``rank``) open a
    ``torch.profiler`` window that covers the forward pass and, through a tensor hook, the matching backward
    pass; export chrome traces (forward and backward separately when ``bw_file`` is given)."""

    def deco(forward):
        state = {"calls": 0}

        @functools.wraps(forward)
        def wrapped(*a, **k):
            state["calls"] += 1
            if state["calls"] != warmup + at + 1 or int(os.getenv("RANK", "0")) != rank:
                return forward(*a, **k)
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            prof = torch.profiler.profile(activities=acts, record_shapes=False)
            prof.__enter__()
            with torch.profiler.record_function("FW"):
                out = forward(*a, **k)
            first = out if torch.is_tensor(out) else next((o for o in (out.values() if isinstance(out, dict) else out)
                                                         if torch.is_tensor(o) and o.requires_grad), None)

            def finish():
                if torch.cuda.is_available():
                    torch.cuda.synchronize()
                prof.__exit__(None, None, None)
                prof.export_chrome_trace(bw_file or fw_file)
                logger.info(f"trace written to {bw_file or fw_file}", at=None)

            if first is not None and first.requires_grad and torch.is_grad_enabled():
                if bw_file:
                    # close the forward window now, open a second one that ends when backward has run
                    if torch.cuda.is_available():
                        torch.cuda.synchronize()
                    prof.__exit__(None, None, None)
                    prof.export_chrome_trace(fw_file)
                    prof2 = torch.profiler.profile(activities=acts)
                    prof2.__enter__()

                    def done_bw():
                        if torch.cuda.is_available():
                            torch.cuda.synchronize()
                        prof2.__exit__(None, None, None)
                        prof2.export_chrome_trace(bw_file)

                    first.register_hook(lambda g: (torch.autograd.Variable._execution_engine.queue_callback(done_bw), g)[1])
                else:
                    first.register_hook(lambda g: (torch.autograd.Variable._execution_engine.queue_callback(finish), g)[1])
            else:
                finish()
            return out

        return wrapped

    return deco


def profile_allreduce(size_bytes: int = 1 << 30, iters: int = 10, groups: dict | None = None) -> dict:
    """All-reduce bandwidth (GB/s, bus bandwidth) of the world group and of every named family, measured
    with CUDA events; also warms the communicators up (reference start-up probe, ``utils/utils.py:377-433``)."""
    from ..parallel.state import PM

    if not dist.is_initialized() or not torch.cuda.is_available():
        return {}
    out = {}
    buf = torch.empty(size_bytes // 4, dtype=torch.float32, device="cuda")
    targets = {"world": dist.group.WORLD}
    for name in (groups or PM.parallels):
        g = PM.group_of(name)
        if g is not None and PM.size_of(name) > 1:
            targets[name] = g
    for name, g in targets.items():
        n = dist.get_world_size(g)
        dist.all_reduce(buf, group=g)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            dist.all_reduce(buf, group=g)
        b.record()
        torch.cuda.synchronize()
        sec = a.elapsed_time(b) / 1e3 / iters
        out[name] = size_bytes / sec / 1e9 * 2 * (n - 1) / n
    logger.info("all-reduce bus bandwidth (GB/s): " + ", ".join(f"{k}={v:.0f}" for k, v in out.items()), at=0)
    return out


def print_n_params(models) -> dict:
    """Parameter counts of this rank's model chunks, split into expert / non-expert."""
    tot = exp = 0
    for m in models if isinstance(models, (list, tuple, torch.nn.ModuleList)) else [models]:
        for n, p in m.named_parameters():
            tot += p.numel()
            if getattr(p, "expert_model_parallel", False) or ".experts." in n:
                exp += p.numel()
    info = {"total": tot, "expert": exp, "dense": tot - exp}
    logger.info(f"parameters on this rank: total {tot / 1e9:.3f} B (expert {exp / 1e9:.3f} B)", at=None)
    return info


def check_nan(tensor, flag: torch.Tensor | None = None):
    """Device-side finite check: ORs 1 into ``flag`` (int32 on the device) when ``tensor`` holds a NaN/Inf.
    Returns the flag without synchronising."""
    if flag is None:
        flag = torch.zeros(1, dtype=torch.int32, device=tensor.device)
    if tensor.is_cuda and tensor.dtype == torch.bfloat16:
        from ..ops import native

        native.check(native.load().stb_nonfinite_flag(tensor.data_ptr(), tensor.numel(), flag.data_ptr(), native.stream()),
                     "nonfinite_flag")
    else:
        flag |= (~torch.isfinite(tensor)).any().to(torch.int32)
    return flag


_NONFINITE_FLAGS: dict = {}


def nonfinite_flag(device) -> torch.Tensor:
    """The job-wide "a checked tensor held NaN/Inf" flag of a device (int32, lives on that device)."""
    device = torch.device(device)
    if device not in _NONFINITE_FLAGS:
        _NONFINITE_FLAGS[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _NONFINITE_FLAGS[device]


def note_nonfinite(obj, where: str = "") -> None:
    """Check every floating tensor in ``obj`` (tensor, dict, list).  On the GPU the result goes into the device flag
    without a host synchronisation (read it later with :func:`raise_if_nonfinite`); on the CPU a bad value raises at
    once, naming ``where``."""
    if torch.is_tensor(obj):
        if not obj.is_floating_point():
            return
        if obj.is_cuda:
            check_nan(obj.detach(), nonfinite_flag(obj.device))
        elif not bool(torch.isfinite(obj).all()):
            raise FloatingPointError(f"non-finite values in {where or 'a checked tensor'}")
    elif isinstance(obj, dict):
        for k, v in obj.items():
            note_nonfinite(v, f"{where}[{k!r}]" if where else repr(k))
    elif isinstance(obj, (list, tuple)):
        for i, v in enumerate(obj):
            note_nonfinite(v, f"{where}[{i}]")


def raise_if_nonfinite() -> None:
    """Read the device flags (a host read: call where the device is synchronised anyway) and raise if one is set."""
    for dev, flag in _NONFINITE_FLAGS.items():
        if int(flag) != 0:
            flag.zero_()
            raise FloatingPointError(f"a checked tensor on {dev} held NaN or Inf since the last check "
                                     f"(model_cfg.check_nan); the stage outputs of this interval are suspect")


class Stopwatch:
    def __enter__(self):
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *a):
        self.dt = time.perf_counter() - self.t0
        return False


def text_chart(values, height: int = 18, width: int = 100, fmt: str = "{:.3e}") -> str:
    """A line chart drawn with characters: one column per (down-sampled) value, the y axis labelled on the left."""
    vals = [float(v) for v in values if v == v]
    if not vals:
        return "(no values)"
    if len(vals) > width:                      # mean of equal slices, so that spikes do not vanish entirely
        edges = [round(i * len(vals) / width) for i in range(width + 1)]
        vals = [sum(vals[a:b]) / (b - a) for a, b in zip(edges[:-1], edges[1:]) if b > a]
    lo, hi = min(vals), max(vals)
    span = (hi - lo) or 1.0
    rows = max(int(height), 2)
    level = [round((v - lo) / span * (rows - 1)) for v in vals]
    grid = [[" "] * len(vals) for _ in range(rows)]
    for x, y in enumerate(level):
        if x and level[x - 1] != y:            # join to the previous column
            a, b = sorted((level[x - 1], y))
            for yy in range(a + 1, b):
                grid[yy][x] = "|"
        grid[y][x] = "*"
    labels = [fmt.format(lo + span * r / (rows - 1)) for r in range(rows)]
    pad = max(len(s) for s in labels)
    return "\n".join(f"{labels[r].rjust(pad)} |{''.join(grid[r])}" for r in reversed(range(rows)))


class TBRecord(dict):
    """The scalars of a TensorBoard run directory, read back: ``"train/loss" in rec``, ``rec["train/loss"]`` (a list
    of events with ``.step`` / ``.value`` / ``.wall_time``, re-read on every access so a live run can be followed)
    and ``rec.asciichart(key)`` for a look at a curve in a terminal (reference
    ``steptronoss/utils/dev_utils.py:205-240``)."""

    def __init__(self, path: str = ""):
        super().__init__()
        from tensorboard.backend.event_processing.event_accumulator import EventAccumulator

        self.ea = EventAccumulator(path, size_guidance={"scalars": 0})
        self.refresh()

    def refresh(self):
        self.ea.Reload()
        self._keys = list(self.ea.Tags()["scalars"])

    def keys(self):
        return self._keys

    def __iter__(self):
        return iter(self._keys)

    def __len__(self):
        return len(self._keys)

    def __contains__(self, key) -> bool:
        return key in self._keys

    def __getitem__(self, key):
        self.refresh()
        return self.ea.Scalars(key)

    def values(self, key) -> list:
        return [e.value for e in self[key]]

    def asciichart(self, scalar_key: str, height: int = 18):
        class _Shown(str):
            def __repr__(self):
                return str(self)

        return _Shown(text_chart(self.values(scalar_key), height))
