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


CudaRNGStatesTracker = RNGStatesTracker          # the reference's names (core/tensor_parallel/random.py)


def get_cuda_rng_tracker() -> RNGStatesTracker:
    return get_rng_tracker()


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
    def forward(ctx, run_function, distribute, *args):
        ctx.run_function = run_function
        ctx.cpu_rng = torch.get_rng_state()
        ctx.dev_rng = _device_rng_get()
        ctx.tracker_states = get_rng_tracker().get_states()
        with torch.no_grad():
            outputs = run_function(*args)
        tensors = [a for a in args if torch.is_tensor(a)]
        ctx.arg_is_tensor = [torch.is_tensor(a) for a in args]
        ctx.non_tensors = [a for a in args if not torch.is_tensor(a)]
        ctx.full_shape = None
        if distribute and tensors:
            # keep 1/TP of the first tensor on every rank; backward gathers it again (for inputs that are equal on
            # all TP ranks, i.e. without sequence parallelism)
            from .state import PM

            tp, r = PM.size_of("TP"), PM.rank_in("TP")
            if tp > 1 and tensors[0].numel() % tp == 0:
                ctx.full_shape = tensors[0].shape
                tensors[0] = tensors[0].detach().reshape(-1).chunk(tp)[r].clone().requires_grad_(tensors[0].requires_grad)
        ctx.save_for_backward(*tensors)
        if os.environ.get("RECOMPUTE_SANITY_CHECK", "0") == "1":
            ctx.sanity = outputs.detach().clone() if torch.is_tensor(outputs) else [o.detach().clone() for o in outputs]
        return outputs

    @staticmethod
    def backward(ctx, *grads):
        tensors = list(ctx.saved_tensors)
        if ctx.full_shape is not None:
            from .state import PM

            shard = tensors[0]
            full = torch.empty(shard.numel() * PM.size_of("TP"), dtype=shard.dtype, device=shard.device)
            torch.distributed.all_gather_into_tensor(full, shard.detach().contiguous(), group=PM.group_of("TP"))
            tensors[0] = full.view(ctx.full_shape).requires_grad_(shard.requires_grad)
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


CheckpointFunction = CheckpointFunctionWithSanityCheck = _CheckpointFn      # one class does both (env switch)


def checkpoint(function, *args, distribute_saved_activations: bool = False):
    """Run ``function(*args)`` without keeping its intermediate activations; recompute in backward.
    ``distribute_saved_activations``: every TP rank keeps only its 1/TP of the first tensor argument."""
    return _CheckpointFn.apply(function, bool(distribute_saved_activations), *args)


class _RngSnapshot:
    """CPU, device and tracker generator states at one point, to replay a function under the same randomness."""

    def __init__(self):
        self.cpu, self.dev, self.tracker = torch.get_rng_state(), _device_rng_get(), get_rng_tracker().get_states()

    @contextlib.contextmanager
    def replay(self):
        now = _RngSnapshot()
        torch.set_rng_state(self.cpu)
        _device_rng_set(self.dev)
        get_rng_tracker().set_states(self.tracker)
        try:
            yield
        finally:
            torch.set_rng_state(now.cpu)
            _device_rng_set(now.dev)
            get_rng_tracker().set_states(now.tracker)


class _DiscardableFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, owner, run_function, *args):
        with torch.no_grad():
            outputs = run_function(*args)
        ctx.arg_is_tensor = [torch.is_tensor(a) for a in args]
        ctx.non_tensors = [a for a in args if not torch.is_tensor(a)]
        ctx.save_for_backward(*[a for a in args if torch.is_tensor(a)])
        ctx.recomputed = None
        owner._ctx = ctx
        return outputs

    @staticmethod
    def backward(ctx, *grads):
        if ctx.recomputed is None:
            raise RuntimeError("the output was never recomputed: call discard_output_and_register_recompute(t) with a "
                               "tensor t computed from the output, and run backward through t")
        outputs, inputs = ctx.recomputed
        ctx.recomputed = None
        pairs = [(o, g) for o, g in zip(outputs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([p[0] for p in pairs], [p[1] for p in pairs])
        return (None, None) + tuple(a.grad if torch.is_tensor(a) else None for a in inputs)


class CheckpointWithoutOutput:
    """Recompute that also gives up the function's OUTPUT between forward and backward.

    ``checkpoint`` keeps the output alive because the next operator saved it.  Here the caller says when the output
    has been consumed; its storage is released then and filled again, by running the function a second time, just
    before the consumer's backward reads it (a hook on the consumer's result)::

        ck = CheckpointWithoutOutput()
        h = ck.checkpoint(norm, x)            # cheap to recompute, large to keep
        y = linear(h)
        ck.discard_output_and_register_recompute(y)

    Reference: ``steptronoss/core/tensor_parallel/random.py:311-381``.
    """

    def __init__(self):
        self._fn = self._ctx = self._rng = self._outputs = None

    def checkpoint(self, run_function, *args):
        self._fn, self._rng = run_function, _RngSnapshot()
        out = _DiscardableFn.apply(self, run_function, *args)
        self._outputs = out if isinstance(out, tuple) else (out,)
        return out

    def discard_output_and_register_recompute(self, hook_tensor: torch.Tensor) -> None:
        if self._outputs is None:
            return
        for o in self._outputs:
            if torch.is_tensor(o):
                o.untyped_storage().resize_(0)
        if hook_tensor.requires_grad:
            hook_tensor.register_hook(self._refill)

    def _refill(self, grad):
        ctx = self._ctx
        tensors, nts = list(ctx.saved_tensors), list(ctx.non_tensors)
        args = _detach([tensors.pop(0) if is_t else nts.pop(0) for is_t in ctx.arg_is_tensor])
        with self._rng.replay(), torch.enable_grad():
            again = self._fn(*args)
        again = again if isinstance(again, tuple) else (again,)
        with torch.no_grad():
            for old, new in zip(self._outputs, again):
                if torch.is_tensor(old):
                    st = old.untyped_storage()
                    st.resize_(new.untyped_storage().size())
                    st.copy_(new.untyped_storage())
        ctx.recomputed = (again, args)
        self._fn = self._ctx = self._rng = self._outputs = None
        return grad
