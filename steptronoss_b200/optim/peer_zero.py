"""ZeRO-1 reduction, Adam and parameter refresh over peer memory for data-parallel groups inside one node.

Stands where the reference calls ``reduce_scatter_tensor`` on the flat gradient buffer, takes the gradient norm in
another pass, steps torch Adam and all-gathers the bf16 parameters
(``steptronoss/optimizer/zero1_gradient_manager.py:164-228``).  With this module the flat gradient and parameter
buffers of a bucket live in memory that the other ranks of the reduce group have mapped (CUDA IPC), and a step is
three launches per bucket (``csrc/zero_peer.cu``):

1. ``stb_zero_reduce``: the owner of a shard sums that shard over all ranks' gradient buffers with peer loads, in
   rank order, applies the EDP correction factor, writes the result in place and leaves the shard's squared norm
   in a device scalar (no separate norm pass);
2. the clip coefficient is formed on the device as before (one small all-reduce of the norm);
3. ``stb_adam_push``: Adam on the owned shard; the new bf16 values are stored into the parameter buffer of every
   rank of the group, so no all-gather follows.

Two flag words per rank order the ranks: "gradients complete" (raised after backward, awaited inside the reduce
kernel) and "parameters delivered" (raised after the last push, awaited before the next step touches parameters
or clears gradients; it also tells a rank that every peer has finished reading its gradients).  Waits are bounded
(``STB200_PEER_WAIT_S``) and end in an error status, never in a hang.

Enabled for a bucket when its reduce group has 2 to 8 ranks on one node over NCCL and ``STB200_PEER_ZERO`` is not
``0``.  ``destroy_buffer`` / parameter offload (RL role swapping) drop back to the NCCL statement.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_void_p

import torch
import torch.distributed as dist

from ..ops import native
from ..ops.gemm import count_launch
from ..parallel.state import PM

P, I, L, F, U, ULL = c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_uint, ctypes.c_ulonglong
native.register_signature("stb_zero_reduce_blocks", [])
native.register_signature("stb_zero_publish", [P, I, I, I, U, P])
native.register_signature("stb_zero_reduce", [P, L, I, I, F, P, P, I, P, I, U, ULL, P, P])
native.register_signature("stb_adam_push", [P, P, P, P, P, I, P, I, P, F, F, F, F, F, F, F, I, P])
native.register_signature("stb_peer_wait_flags", [P, I, I, U, ULL, P, P])

_FLAG_GRADS, _FLAG_PARAMS = 0, 1
_DISABLED = os.environ.get("STB200_PEER_ZERO", "1") == "0"


def group_supported(group_name: str) -> bool:
    """Collective over the group: every rank gets the same answer."""
    from ..parallel import symm

    if _DISABLED or not torch.cuda.is_available() or not dist.is_initialized() or not PM.has(group_name):
        return False
    n = PM.size_of(group_name)
    group = PM.group_of(group_name)
    return 2 <= n <= 8 and dist.get_backend(group) == "nccl" and symm._same_node(group) and native.available()


class PeerZeroGroup:
    """Flag page and the symmetric gradient / parameter buffers of the buckets of one reduce group."""

    def __init__(self, group_name: str):
        from ..parallel.symm import _WAIT_NS, SymmetricBuffer

        self._SymmetricBuffer, self.wait_ns = SymmetricBuffer, _WAIT_NS
        self.group_name = group_name
        self.group = PM.group_of(group_name)
        self.rank, self.world = PM.rank_in(group_name), PM.size_of(group_name)
        self.lib = native.load()
        self.flags = SymmetricBuffer(2 * 8 * 4, self.group, self.lib)
        self.flags.own_tensor().zero_()
        self._flag_arr = self.flags.ptr_array()
        self.grad_mem: dict = {}
        self.param_mem: dict = {}
        self.partials = torch.empty(self.lib.stb_zero_reduce_blocks(), dtype=torch.float32, device="cuda")
        self.epoch = 0
        self.params_pending = False
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------ buffers
    def allocate(self, key, numel: int, dtype: torch.dtype, kind: str) -> torch.Tensor:
        """A zeroed flat buffer of the bucket in symmetric memory (collective over the group)."""
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        mem = self._SymmetricBuffer(max(nbytes, 16), self.group, self.lib)
        (self.grad_mem if kind == "grad" else self.param_mem)[key] = mem
        t = mem.own_tensor()[:nbytes].view(dtype)
        t.zero_()
        return t

    def finish_allocation(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def release(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for mem in list(self.grad_mem.values()) + list(self.param_mem.values()):
            mem.release()
        self.grad_mem, self.param_mem = {}, {}

    # ------------------------------------------------------------------ the step
    def begin_step(self) -> None:
        """After backward: tell the peers that this rank's gradients are complete."""
        self.epoch += 1
        rc = self.lib.stb_zero_publish(self._flag_arr, _FLAG_GRADS, self.world, self.rank, self.epoch & 0xFFFFFFFF,
                                       native.stream())
        native.check(rc, "zero publish")
        count_launch()

    def reduce(self, key, bucket, scale: float, sq_out: torch.Tensor, accumulate: bool) -> None:
        lo, hi = bucket.own_range()
        ptrs = self.grad_mem[key].ptr_array(lo * 4)
        rc = self.lib.stb_zero_reduce(ptrs, hi - lo, self.world, self.rank, float(scale), self.partials.data_ptr(),
                                      sq_out.data_ptr(), int(accumulate), self.flags.own, _FLAG_GRADS,
                                      self.epoch & 0xFFFFFFFF, self.wait_ns,
                                      native.status_word(bucket.grad_buf.device).data_ptr(), native.stream())
        native.check(rc, "zero reduce")
        count_launch(2)

    def param_ptrs(self, key, bucket):
        lo, _ = bucket.own_range()
        return self.param_mem[key].ptr_array(lo * bucket.param_buf.element_size())

    def end_step(self) -> None:
        """After the last push: tell the peers that this rank's parameter shards have landed."""
        rc = self.lib.stb_zero_publish(self._flag_arr, _FLAG_PARAMS, self.world, self.rank, self.epoch & 0xFFFFFFFF,
                                       native.stream())
        native.check(rc, "zero publish")
        count_launch()
        self.params_pending = True

    def wait_params(self) -> None:
        """Before parameters are read or gradients cleared again: every peer's shards are here, and every peer is
        done reading this rank's gradients."""
        if not self.params_pending:
            return
        rc = self.lib.stb_peer_wait_flags(self.flags.own, _FLAG_PARAMS, self.world, self.epoch & 0xFFFFFFFF,
                                          self.wait_ns, native.status_word(torch.device("cuda")).data_ptr(),
                                          native.stream())
        native.check(rc, "zero wait")
        count_launch()
        self.params_pending = False
