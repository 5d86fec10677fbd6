"""Pipeline point-to-point exchange of activations and their gradients.

Reference: ``steptronoss/core/pipeline_parallel/p2p_communication.py:14-546``.  Pipeline traffic
stays on NCCL send/recv (it is latency-tolerant and overlaps with compute); the combined
operations post every send and receive of one step as a single batch.  With
``variable_seq_lengths`` the shape is exchanged first (three int64: ndim-padded dims).
Receives are posted on the current stream; the tensors are safe to use once ``wait`` returned.

``overlap`` (the reference's ``overlap_p2p_comm``): a batch that only *sends* is not waited for.  NCCL runs the
transfer on its own stream behind the kernel that produced the tensor, so without the wait the compute stream
goes straight on with the next micro-batch while the activation (or gradient) is on its way; the tensor is kept
alive until the transfer has finished (``P2P.drain`` at the end of a schedule, or as the list of transfers in
flight grows).  Batches that receive are always waited for, because their result is the next kernel's input,
and a send stays in the same batch as the receive it is paired with: NCCL matches the two directions between a
pair of ranks inside one group, and splitting them can deadlock.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..state import PM


def _device():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and PM.backend == "nccl" else torch.device("cpu")


def _exchange_shapes(send_next, send_prev, recv_prev: bool, recv_next: bool):
    dev = _device()
    ops, bufs = [], {}
    group = PM.group_of("PP")

    def enc(t):
        s = list(t.shape) + [0] * (3 - t.dim())
        return torch.tensor(s[:3], dtype=torch.int64, device=dev)

    prev, nxt = PM.pipeline_prev_rank(), PM.pipeline_next_rank()
    sends, recvs = [], []
    if send_prev is not None:
        sends.append(dist.P2POp(dist.isend, enc(send_prev), prev, group))
    if send_next is not None:
        sends.append(dist.P2POp(dist.isend, enc(send_next), nxt, group))
    if recv_prev:
        bufs["prev"] = torch.empty(3, dtype=torch.int64, device=dev)
        recvs.append(dist.P2POp(dist.irecv, bufs["prev"], prev, group))
    if recv_next:
        bufs["next"] = torch.empty(3, dtype=torch.int64, device=dev)
        recvs.append(dist.P2POp(dist.irecv, bufs["next"], nxt, group))
    if prev == nxt:
        recvs.reverse()  # see communicate(): one peer on both sides, messages match in issue order
    ops = sends + recvs
    if ops:
        for r in dist.batch_isend_irecv(ops):
            r.wait()
    def dec(t):
        return tuple(int(x) for x in t.tolist() if int(x) != 0)
    return dec(bufs["prev"]) if "prev" in bufs else None, dec(bufs["next"]) if "next" in bufs else None


def communicate(send_next=None, send_prev=None, recv_prev: bool = False, recv_next: bool = False,
                tensor_shape=None, dtype=torch.bfloat16, variable_seq_lengths: bool = False, wait: bool = True):
    """Post the requested sends/receives with the neighbouring stages as one batch.

    Returns ``(from_prev, from_next, requests)``; with ``wait=True`` the requests are already
    complete and ``requests`` is empty."""
    group = PM.group_of("PP")
    dev = _device()
    shape_prev = shape_next = tensor_shape
    if variable_seq_lengths:
        shape_prev, shape_next = _exchange_shapes(send_next, send_prev, recv_prev, recv_next)
    from_prev = from_next = None
    prev, nxt = PM.pipeline_prev_rank(), PM.pipeline_next_rank()
    sends, recvs = [], []
    if send_prev is not None:
        sends.append(dist.P2POp(dist.isend, send_prev.contiguous(), prev, group))
    if send_next is not None:
        sends.append(dist.P2POp(dist.isend, send_next.contiguous(), nxt, group))
    if recv_prev:
        from_prev = torch.empty(shape_prev, dtype=dtype, device=dev, requires_grad=True)
        recvs.append(dist.P2POp(dist.irecv, from_prev, prev, group))
    if recv_next:
        from_next = torch.empty(shape_next, dtype=dtype, device=dev)
        recvs.append(dist.P2POp(dist.irecv, from_next, nxt, group))
    if prev == nxt:
        # two stages: both neighbours are the same rank, and messages between one pair of ranks match in issue
        # order.  The peer issues (to-prev, to-next); its to-prev is what this rank receives "from next".
        recvs.reverse()
    ops = sends + recvs
    reqs = dist.batch_isend_irecv(ops) if ops else []
    if wait:
        for r in reqs:
            r.wait()
        reqs = []
    return from_prev, from_next, reqs


class P2P:
    """The nine send/recv combinations of the reference, bound to one shape/dtype policy."""

    MAX_IN_FLIGHT = 8

    def __init__(self, tensor_shape=None, dtype=torch.bfloat16, variable_seq_lengths=False, overlap: bool = False):
        self.kw = dict(tensor_shape=tensor_shape, dtype=dtype, variable_seq_lengths=variable_seq_lengths)
        self.overlap = bool(overlap)
        self._in_flight: list = []          # (requests, tensors kept alive) of sends nobody waited for yet

    def _send_only(self, **sends) -> None:
        if not self.overlap:
            communicate(**sends, **self.kw)
            return
        # an alias of its own: the schedule frees an output's storage right after sending it (by re-pointing
        # ``out.data``), which must not pull the buffer from under a transfer that is still running
        sends = {k: t.detach() for k, t in sends.items() if t is not None}
        _, _, reqs = communicate(wait=False, **sends, **self.kw)
        self._in_flight.append((reqs, list(sends.values())))
        if len(self._in_flight) > self.MAX_IN_FLIGHT:
            self._reap(len(self._in_flight) - self.MAX_IN_FLIGHT)

    def _reap(self, count: int) -> None:
        for reqs, _tensors in self._in_flight[:count]:
            for r in reqs:
                r.wait()
        del self._in_flight[:count]

    def drain(self) -> None:
        """Wait for every send that was left in flight (end of a schedule: buffers are about to be reused)."""
        self._reap(len(self._in_flight))

    def recv_forward(self):
        if PM.is_pipeline_first_stage(ignore_virtual=True):
            return None
        return communicate(recv_prev=True, **self.kw)[0]

    def recv_backward(self):
        if PM.is_pipeline_last_stage(ignore_virtual=True):
            return None
        return communicate(recv_next=True, **self.kw)[1]

    def send_forward(self, out):
        if not PM.is_pipeline_last_stage(ignore_virtual=True):
            self._send_only(send_next=out)

    def send_backward(self, grad):
        if not PM.is_pipeline_first_stage(ignore_virtual=True):
            self._send_only(send_prev=grad)

    def send_forward_recv_backward(self, out):
        if PM.is_pipeline_last_stage(ignore_virtual=True):
            return None
        return communicate(send_next=out, recv_next=True, **self.kw)[1]

    def send_backward_recv_forward(self, grad):
        if PM.is_pipeline_first_stage(ignore_virtual=True):
            return None
        return communicate(send_prev=grad, recv_prev=True, **self.kw)[0]

    def send_forward_recv_forward(self, out, recv_prev: bool, wait: bool = True):
        r = communicate(send_next=out, recv_prev=recv_prev, wait=wait, **self.kw)
        return r[0] if wait else (r[0], r[2])

    def send_backward_recv_backward(self, grad, recv_next: bool, wait: bool = True):
        r = communicate(send_prev=grad, recv_next=recv_next, wait=wait, **self.kw)
        return r[1] if wait else (r[1], r[2])

    def send_forward_backward_recv_forward_backward(self, out, grad, recv_prev: bool, recv_next: bool):
        r = communicate(send_next=out, send_prev=grad, recv_prev=recv_prev, recv_next=recv_next, **self.kw)
        return r[0], r[1]


# ---------------------------------------------------------------------------------------------------------------
# Free-function spellings (reference: core/pipeline_parallel/p2p_communication.py:327-560), for a schedule of one's
# own written against them: the first argument is the model config (``params_dtype`` / ``pipeline_dtype`` and
# ``variable_seq_lengths`` are read from it), ``tensor_shape`` the shape of the activation that travels.
# ---------------------------------------------------------------------------------------------------------------
def _bound(cfg, tensor_shape) -> P2P:
    dtype = getattr(cfg, "pipeline_dtype", None) or getattr(cfg, "params_dtype", None) or torch.bfloat16
    return P2P(tensor_shape, dtype, bool(getattr(cfg, "variable_seq_lengths", False)))


def recv_forward(cfg, tensor_shape=None):
    return _bound(cfg, tensor_shape).recv_forward()


def recv_backward(cfg, tensor_shape=None):
    return _bound(cfg, tensor_shape).recv_backward()


def send_forward(cfg, output_tensor, tensor_shape=None) -> None:
    _bound(cfg, tensor_shape).send_forward(output_tensor)


def send_backward(cfg, input_tensor_grad, tensor_shape=None) -> None:
    _bound(cfg, tensor_shape).send_backward(input_tensor_grad)


def send_forward_recv_backward(cfg, output_tensor, tensor_shape=None):
    return _bound(cfg, tensor_shape).send_forward_recv_backward(output_tensor)


def send_backward_recv_forward(cfg, input_tensor_grad, tensor_shape=None):
    return _bound(cfg, tensor_shape).send_backward_recv_forward(input_tensor_grad)


def send_forward_recv_forward(cfg, output_tensor, recv_prev: bool, tensor_shape=None, overlap_p2p_comm: bool = False):
    """With ``overlap_p2p_comm`` the transfer is left in flight: ``(tensor, requests to wait on)`` comes back."""
    return _bound(cfg, tensor_shape).send_forward_recv_forward(output_tensor, recv_prev, wait=not overlap_p2p_comm)


def send_backward_recv_backward(cfg, input_tensor_grad, recv_next: bool, tensor_shape=None, overlap_p2p_comm: bool = False):
    return _bound(cfg, tensor_shape).send_backward_recv_backward(input_tensor_grad, recv_next, wait=not overlap_p2p_comm)


def send_forward_backward_recv_forward_backward(cfg, output_tensor, input_tensor_grad, recv_prev: bool, recv_next: bool,
                                                tensor_shape=None):
    return _bound(cfg, tensor_shape).send_forward_backward_recv_forward_backward(output_tensor, input_tensor_grad,
                                                                                 recv_prev, recv_next)
