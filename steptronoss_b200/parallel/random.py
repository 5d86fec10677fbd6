"""Named RNG streams for model-parallel regions and activation recomputation.

Counterpart of ``steptronoss/core/tensor_parallel/random.py:59-381``: a tracker of named
generator states (``model-parallel-rng`` differs across TP ranks, the default stream does not),
and ``checkpoint`` which drops a function's intermediate activations and recomputes them in
backward under the RNG states recorded in forward.  ``RECOMPUTE_SANITY_CHECK=1`` compares the
recomputed output with the original one.
"""
from __future__ import annotations

import contextlib
import os

import torch


def _device_rng_get():
    return torch.cuda.get_rng_state() if torch.cuda.is_available() else torch.get_rng_state()


def _device_rng_set(state) -> None:
    if torch.cuda.is_available():
        torch.cuda.set_rng_state(state)
    else:
        torch.set_rng_state(state)


class RNGStatesTracker:
    def __init__(self) -> None:
        self.states: dict[str, torch.Tensor] = {}
        self.seeds: set[int] = set()

    def reset(self) -> None:
        self.states, self.seeds = {}, set()

    def get_states(self) -> dict[str, torch.Tensor]:
        return dict(self.states)

    def set_states(self, states: dict[str, torch.Tensor]) -> None:
        self.states = dict(states)

    def add(self, name: str, seed: int) -> None:
        if seed in self.seeds:
            raise RuntimeError(f"seed {seed} already present")
        if name in self.states:
            raise RuntimeError(f"rng state {name} already present")
        self.seeds.add(seed)
        orig = _device_rng_get()
        if torch.cuda.is_available():
            torch.cuda.manual_seed(seed)
        else:
            torch.manual_seed(seed)
        self.states[name] = _device_rng_get()
        _device_rng_set(orig)

    @contextlib.contextmanager
    def fork(self, name: str = "model-parallel-rng"):
        if name not in self.states:
            yield
            return
        orig = _device_rng_get()
        _device_rng_set(self.states[name])
        try:
            yield
        finally:
            self.states[name] = _device_rng_get()
            _device_rng_set(orig)


_TRACKER = RNGStatesTracker()


def get_rng_tracker() -> RNGStatesTracker:
    return _TRACKER


def _detach(args):
    out = []
    for a in args:
        if torch.is_tensor(a):
            d = a.detach()
            d.requires_grad_(a.requires_grad)
            out.append(d)
        else:
            out.append(a)
    return tuple(out)


class _CheckpointFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_function, n_tensor_args, *args):
        ctx.run_function = run_function
        ctx.cpu_rng = torch.get_rng_state()
        ctx.dev_rng = _device_rng_get()
        ctx.tracker_states = get_rng_tracker().get_states()
        with torch.no_grad():
            outputs = run_function(*args)
        tensors = [a for a in args if torch.is_tensor(a)]
        ctx.arg_is_tensor = [torch.is_tensor(a) for a in args]
        ctx.non_tensors = [a for a in args if not torch.is_tensor(a)]
        ctx.save_for_backward(*tensors)
        if os.environ.get("RECOMPUTE_SANITY_CHECK", "0") == "1":
            ctx.sanity = outputs.detach().clone() if torch.is_tensor(outputs) else [o.detach().clone() for o in outputs]
        return outputs

    @staticmethod
    def backward(ctx, *grads):
        tensors = list(ctx.saved_tensors)
        nts = list(ctx.non_tensors)
        args = [tensors.pop(0) if is_t else nts.pop(0) for is_t in ctx.arg_is_tensor]
        cpu_rng, dev_rng = torch.get_rng_state(), _device_rng_get()
        tracker_now = get_rng_tracker().get_states()
        torch.set_rng_state(ctx.cpu_rng)
        _device_rng_set(ctx.dev_rng)
        get_rng_tracker().set_states(ctx.tracker_states)
        detached = _detach(args)
        with torch.enable_grad():
            outputs = ctx.run_function(*detached)
        torch.set_rng_state(cpu_rng)
        _device_rng_set(dev_rng)
        get_rng_tracker().set_states(tracker_now)
        if torch.is_tensor(outputs):
            outputs = (outputs,)
        if hasattr(ctx, "sanity"):
            ref = ctx.sanity if isinstance(ctx.sanity, list) else [ctx.sanity]
            for a, b in zip(ref, outputs):
                if not torch.equal(a, b.detach()):
                    raise RuntimeError("recomputed activation differs from the forward pass")
        pairs = [(o, g) for o, g in zip(outputs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([p[0] for p in pairs], [p[1] for p in pairs])
        in_grads = tuple(a.grad if torch.is_tensor(a) else None for a in detached)
        return (None, None) + in_grads


def checkpoint(function, *args):
    """Run ``function(*args)`` without keeping its intermediate activations; recompute in backward."""
    return _CheckpointFn.apply(function, len(args), *args)
