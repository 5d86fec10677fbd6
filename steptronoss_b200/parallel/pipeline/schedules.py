"""Micro-batch schedules: plain forward/backward, 1F1B pipeline, interleaved (virtual) 1F1B.

Reference: ``steptronoss/core/pipeline_parallel/schedules.py:127-693``.  A schedule is configured
with the model chunks, the data iterators, ``data_sync_fn`` (fetch + broadcast one micro-batch),
``data_proc_fn`` (pre-process) and ``loss_fn``; ``run(n)`` executes ``n`` micro-batches and leaves the
gradients accumulated in the parameters' ``main_grad``.

1F1B: stage ``r`` of ``P`` runs ``min(P - r - 1, n)`` warm-up forwards, then alternates one forward and
one backward, then drains the remaining backwards.  Interleaved: ``n % P == 0`` is required; the
warm-up is ``(P - r - 1)·2 + (chunks - 1)·P`` micro-steps (all of them when ``n == P``).
"""
from __future__ import annotations

from typing import Callable, Iterator

import torch

from ...utils.timers import get_timers
from ..state import PM
from .p2p import P2P


def _unwrap(m):
    from ...models.module import unwrap_model

    return unwrap_model(m)


def backward_step(input_tensor, output_tensor, output_grad):
    """Back-propagate one micro-batch through a stage; returns the gradient w.r.t. its input."""
    if input_tensor is not None and input_tensor.requires_grad:
        input_tensor.retain_grad()
    if output_grad is None:
        output_tensor.backward()
    else:
        torch.autograd.backward(output_tensor, grad_tensors=output_grad)
    return input_tensor.grad if input_tensor is not None else None


def deallocate_output_tensor(out):
    """Free the activation that was sent downstream; only its ``grad_fn`` is needed for backward."""
    if out is not None and torch.is_tensor(out) and out.numel() > 1:
        out.data = torch.empty((1,), device=out.device, dtype=out.dtype)


def custom_backward(output, grad_output):
    """Backward through an output whose storage was released by ``deallocate_output_tensor``."""
    if grad_output is None:
        grad_output = torch.ones_like(output, memory_format=torch.preserve_format)
    torch.autograd.Variable._execution_engine.run_backward(
        tensors=(output,), grad_tensors=(grad_output,), keep_graph=False, create_graph=False, inputs=tuple(),
        allow_unreachable=True, accumulate_grad=True)


class FWBWScheduler:
    def __init__(self, config) -> None:
        self.config = config
        self._prefetched = None
        self._collected: list = []

    def configure(self, models, data_iterators, data_sync_fn: Callable[[Iterator], dict],
                  data_proc_fn: Callable[[dict], dict], collect_output: bool = False, loss_fn: Callable | None = None,
                  training: bool = True):
        self.models, self.data_iterators = list(models), list(data_iterators)
        self.data_sync_fn, self.data_proc_fn = data_sync_fn, data_proc_fn
        self.collect_output, self.loss_func, self.training = collect_output, loss_fn, training
        return self

    def _prefetch(self, n: int) -> None:
        with get_timers().record("batch-generator", 2):
            keep = PM.get_vpp_rank()
            self._prefetched = [[] for _ in self.models]
            live = [it for it in self.data_iterators if it is not None]
            if len(self.models) > 1 and len({id(it) for it in live}) <= 1:
                # one stream feeds every model chunk of this rank: fetch each micro-batch once and share it
                PM.set_vpp_rank(0)
                batches = [self.data_sync_fn(self.data_iterators[0]) for _ in range(n)]
                self._prefetched = [list(batches) for _ in self.models]
            else:
                for vp, it in enumerate(self.data_iterators):
                    PM.set_vpp_rank(vp)
                    for _ in range(n):
                        self._prefetched[vp].append(self.data_sync_fn(it))
            PM.set_vpp_rank(keep)

    def forward_chunk(self, vp_rank: int = 0, input_tensor=None, loss_scale: float = 1.0):
        PM.set_vpp_rank(vp_rank)
        model = self.models[vp_rank]
        _unwrap(model).set_input_tensor(input_tensor)
        data = self._prefetched[vp_rank].pop(0)
        with get_timers().record("data-preprocess", 1):
            data = self.data_proc_fn(data) if self.data_proc_fn is not None else data
        data = dict(data or {})
        data["loss_scale"] = loss_scale
        with get_timers().record("forward-step", 2):
            output = model(**data)
        if getattr(self.config, "check_nan", False):
            from ...utils.dev_utils import note_nonfinite

            note_nonfinite(output, f"output of pipeline stage {PM.rank_in('PP')} (chunk {vp_rank})")
        if _unwrap(model).is_last_stage:
            if self.collect_output:
                self._collected.append(output)
            if self.loss_func is not None:
                return self.loss_func(data, output, loss_scale)
            return output
        return output

    def run(self, forward_num: int = 1):
        self._collected.clear()
        assert len(self.models) == 1
        self._prefetch(forward_num)
        for _ in range(forward_num):
            out = self.forward_chunk(0, loss_scale=1.0 / forward_num)
            if self.training:
                with get_timers().record("backward-step", 2):
                    backward_step(None, out, None)
        self._prefetched = None
        return self._collected


class PPScheduler(FWBWScheduler):
    """Non-interleaved 1F1B."""

    def _p2p(self) -> P2P:
        c = self.config
        return P2P(tensor_shape=tuple(c.pp_comm_shape) if not c.variable_seq_lengths else None, dtype=c.params_dtype,
                   variable_seq_lengths=c.variable_seq_lengths, overlap=bool(getattr(c, "overlap_p2p_comm", False)))

    def run(self, forward_num: int = 1):
        self._collected.clear()
        assert len(self.models) == 1
        self._prefetch(forward_num)
        p2p = self._p2p()
        P, r = PM.size_of("PP"), PM.rank_in("PP")
        warmup = min(P - r - 1, forward_num)
        steady = forward_num - warmup
        scale = 1.0 / forward_num
        inputs, outputs = [], []
        ctx = (torch.autograd.graph.save_on_cpu(pin_memory=torch.cuda.is_available())
               if self.config.pipeline_activation_cpu_offload else None)

        def fwd(inp):
            if ctx is not None:
                with ctx:
                    return self.forward_chunk(0, inp, scale)
            return self.forward_chunk(0, inp, scale)

        for _ in range(warmup):
            inp = p2p.recv_forward()
            out = fwd(inp)
            p2p.send_forward(out)
            if self.training:
                inputs.append(inp)
                outputs.append(out)
                if not PM.is_pipeline_last_stage(True):
                    deallocate_output_tensor(out)
        inp = p2p.recv_forward() if steady > 0 else None
        for i in range(steady):
            last = i == steady - 1
            out = fwd(inp)
            if not self.training:
                p2p.send_forward(out)
                inp = p2p.recv_forward() if not last else None
                continue
            grad = p2p.send_forward_recv_backward(out)
            inputs.append(inp)
            outputs.append(out)
            if not PM.is_pipeline_last_stage(True):
                deallocate_output_tensor(out)
            i0, o0 = inputs.pop(0), outputs.pop(0)
            gin = self._backward(i0, o0, grad)
            if last:
                p2p.send_backward(gin)
                inp = None
            else:
                inp = p2p.send_backward_recv_forward(gin)
        if self.training:
            for _ in range(warmup):
                i0, o0 = inputs.pop(0), outputs.pop(0)
                grad = p2p.recv_backward()
                gin = self._backward(i0, o0, grad)
                p2p.send_backward(gin)
        p2p.drain()
        self._prefetched = None
        return self._collected

    @staticmethod
    def _backward(inp, out, grad):
        if inp is not None and inp.requires_grad:
            inp.retain_grad()
        if grad is None:
            out.backward()
        else:
            custom_backward(out, grad)
        return inp.grad if inp is not None else None


class VPPScheduler(PPScheduler):
    """Interleaved 1F1B: every rank holds ``C = len(models)`` model chunks; virtual stage ``v = c * P + r``.

    Micro-step ``k`` of the forward order works on chunk ``(k mod P*C) // P`` (backward: mirrored), i.e. ``P``
    micro-batches go through chunk 0, then the same ``P`` through chunk 1, and so on.  After a warm-up of
    ``2 (P - r - 1) + (C - 1) P`` forward steps every step runs one forward and one backward and exchanges both
    results with the neighbours in a single batch; the ring wraps from the last rank to the first between
    chunks.  Needs ``forward_num`` to be a multiple of ``P``.  This is the published Megatron-LM interleaved
    schedule (Narayanan et al., 2021), which the reference follows too
    (``steptronoss/core/pipeline_parallel/schedules.py:322-693``).
    """

    def run(self, forward_num: int = 1):
        self._collected.clear()
        P, r = PM.size_of("PP"), PM.rank_in("PP")
        C = len(self.models)
        if forward_num % P != 0:
            raise AssertionError("interleaved schedule needs the number of micro-batches to be a multiple of PP")
        self._prefetch(forward_num)
        p2p = self._p2p()
        total = forward_num * C
        scale = 1.0 / forward_num
        train = self.training
        all_warmup = forward_num == P or not train
        warmup = total if all_warmup else min((P - r - 1) * 2 + (C - 1) * P, total)
        remaining = total - warmup
        inputs = [[] for _ in range(C)]
        outputs = [[] for _ in range(C)]
        out_grads = [[] for _ in range(C)]
        first_rank, last_rank = r == 0, r == P - 1

        def chunk_of(k: int, forward: bool) -> int:
            c = (k % (P * C)) // P
            return c if forward else C - 1 - c

        def forward_step(k: int):
            c = chunk_of(k, True)
            PM.set_vpp_rank(c)
            if first_rank and c == 0 and len(inputs[c]) == len(outputs[c]):
                inputs[c].append(None)
            out = self.forward_chunk(c, inputs[c][-1], scale)
            if train:
                outputs[c].append(out)
            else:
                inputs[c].pop()
            return None if (last_rank and c == C - 1) else out  # the last virtual stage sends nothing on

        def backward_step(k: int):
            c = chunk_of(k, False)
            PM.set_vpp_rank(c)
            if last_rank and c == C - 1 and len(out_grads[c]) == 0:
                out_grads[c].append(None)
            gin = self._backward(inputs[c].pop(0), outputs[c].pop(0), out_grads[c].pop(0))
            return None if (first_rank and c == 0) else gin   # the first virtual stage sends nothing back

        PM.set_vpp_rank(0)
        inputs[0].append(p2p.recv_forward())
        for k in range(warmup):
            out = forward_step(k)
            nxt = chunk_of(k + 1, True)
            recv_prev = not (first_rank and nxt == 0) and k != total - 1
            if k == warmup - 1 and train and not all_warmup:
                got, grad = p2p.send_forward_backward_recv_forward_backward(out, None, recv_prev, not last_rank)
                out_grads[C - 1].append(grad)
            else:
                got = p2p.send_forward_recv_forward(out, recv_prev)
            if recv_prev or not (k == total - 1):
                inputs[nxt].append(got)
            if out is not None and train:
                deallocate_output_tensor(out)

        for k in range(remaining):
            fk = k + warmup
            out = forward_step(fk)
            gin = backward_step(k)
            # what arrives next: the first rank runs P-1 steps ahead of the last rank around the ring
            recv_prev = True
            if first_rank:
                nf = chunk_of(fk - (P - 1), True)
                if nf == C - 1:
                    recv_prev = False
                nf += 1
            else:
                nf = chunk_of(fk + 1, True)
            recv_next = True
            if last_rank:
                nb = chunk_of(k - (P - 1), False)
                if nb == 0:
                    recv_next = False
                nb -= 1
            else:
                nb = chunk_of(k + 1, False)
            if k == remaining - 1:
                recv_prev = False
            got, grad = p2p.send_forward_backward_recv_forward_backward(out, gin, recv_prev, recv_next)
            if out is not None:
                deallocate_output_tensor(out)
            if recv_prev:
                inputs[nf].append(got)
            if recv_next:
                out_grads[nb].append(grad)

        if train:
            if all_warmup:
                out_grads[C - 1].append(p2p.recv_backward())
            for k in range(remaining, total):
                gin = backward_step(k)
                nb = chunk_of(k + 1, False)
                recv_next = not (last_rank and nb == C - 1) and k != total - 1
                grad = p2p.send_backward_recv_backward(gin, recv_next)
                out_grads[nb].append(grad)
        p2p.drain()
        PM.set_vpp_rank(0)
        self._prefetched = None
        return self._collected
