"""Gradient clipping and zero counting over a plain list of parameters.

The gradient managers clip on their flat buffers with device-resident scalars (``gradient_manager.py``); these two
functions serve code that holds ordinary ``param.grad`` tensors - a critic head, an adapter trained beside the
model, a test - with the call surface of the reference (optimizer/clip_grads.py:20-150).  Both read one number back
to the host, as the reference's do.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..parallel.tensor_utils import (param_is_not_expert_parallel_duplicate, param_is_not_shared,
                                     param_is_not_tensor_parallel_duplicate)


def _as_list(x):
    return [x] if isinstance(x, torch.Tensor) else list(x)


def _reduce(value: torch.Tensor, op, group) -> torch.Tensor:
    if dist.is_available() and dist.is_initialized() and (group is None or dist.get_world_size(group) > 1):
        dist.all_reduce(value, op=op, group=group)
    return value


def clip_grad_norm_fp32(parameters, grads_for_norm, max_norm: float, norm_type: float = 2, model_parallel_group=None) -> float:
    """Scale the gradients of ``parameters`` in place so that the norm of ``grads_for_norm`` - the gradients that
    count once over the model-parallel group, summed over that group - is at most ``max_norm``.  Returns the norm
    before clipping."""
    grads = [p.grad.detach() for p in _as_list(parameters) if p.grad is not None]
    counted = _as_list(grads_for_norm)
    device = (counted or grads or [torch.zeros(())])[0].device
    norm_type = float(norm_type)
    if math.isinf(norm_type):
        local = torch.stack([g.abs().max().float() for g in counted]).max() if counted else torch.zeros((), device=device)
        total = float(_reduce(local.reshape(1).clone(), dist.ReduceOp.MAX, model_parallel_group))
    else:
        if counted:
            per = torch._foreach_norm(counted, norm_type)
            local = torch.stack([n.float() for n in per]).pow(norm_type).sum()
        else:
            local = torch.zeros((), device=device)
        total = float(_reduce(local.reshape(1).clone(), dist.ReduceOp.SUM, model_parallel_group)) ** (1.0 / norm_type)
    coef = max_norm / (total + 1.0e-6)
    if coef < 1.0 and grads:
        torch._foreach_mul_(grads, coef)
    return total


def count_zeros_fp32(parameters, model_parallel_group=None) -> float:
    """Zero entries in the gradients, each parameter counted once over the model-parallel group: shared parameters
    are left out, expert parameters count where they are not an expert-parallel duplicate, the others where they
    are not a tensor-parallel duplicate."""
    total = None
    for p in _as_list(parameters):
        if p.grad is None or not param_is_not_shared(p):
            continue
        once = (param_is_not_expert_parallel_duplicate(p) if getattr(p, "expert_model_parallel", False)
                else param_is_not_tensor_parallel_duplicate(p))
        if not once:
            continue
        zeros = (p.grad.numel() - torch.count_nonzero(p.grad.detach())).float().reshape(1)
        total = zeros if total is None else total + zeros
    if total is None:
        dev = next((p.device for p in _as_list(parameters)), torch.device("cpu"))
        total = torch.zeros(1, device=dev)
    return float(_reduce(total, dist.ReduceOp.SUM, model_parallel_group))
