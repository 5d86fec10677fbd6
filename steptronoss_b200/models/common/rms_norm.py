"""RMSNorm module (reference ``steptronoss/model/common/rms_norm.py:5-62``).

The reference's fused kernel ignores its ``eps`` argument and always uses 1e-5; this module
honours ``eps`` and offers ``legacy_eps=True`` to reproduce the reference bit-for-bit.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ...ops import add_rmsnorm, rmsnorm


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, sequence_parallel: bool = False, use_zero_init: bool = False,
                 params_dtype=torch.bfloat16, legacy_eps: bool = False, device=None):
        super().__init__()
        self.eps = 1e-5 if legacy_eps else eps
        self.zero_centered = use_zero_init
        self.weight = nn.Parameter(torch.empty(dim, dtype=params_dtype, device=device))
        self.weight.init_kind = "zeros" if use_zero_init else "ones"
        # replicated over TP but fed with different tokens under sequence parallelism:
        # its gradient has to be summed over the TP group by the gradient manager
        self.weight.sequence_parallel = sequence_parallel

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return rmsnorm(x, self.weight, self.eps, self.zero_centered)

    def forward_with_residual(self, x: torch.Tensor, delta: torch.Tensor):
        """``(x + delta, norm(x + delta))`` in one kernel: the residual add in front of this norm fused into it."""
        return add_rmsnorm(x, delta, self.weight, self.eps, self.zero_centered)
