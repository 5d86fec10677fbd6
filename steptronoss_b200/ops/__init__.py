"""Hot operators. Each is one function with two bodies: the sm_100a kernel for CUDA tensors and a
PyTorch restatement for CPU tensors (used by the CPU test-suite and as the oracle of GPU tests)."""
from .attention import attention, attention_reference
from .cross_entropy import fused_linear_cross_entropy, vocab_parallel_cross_entropy
from .fused import (
    add_rmsnorm,
    embedding,
    qknorm_rope,
    qknorm_rope_reference,
    residual_add,
    rmsnorm,
    rmsnorm_reference,
    rope_tables,
    swiglu,
    swiglu_reference,
)
from .gemm import gemm, launch_count, linear

__all__ = [
    "attention", "attention_reference", "fused_linear_cross_entropy", "vocab_parallel_cross_entropy",
    "embedding", "qknorm_rope", "qknorm_rope_reference", "rmsnorm", "rmsnorm_reference", "rope_tables",
    "swiglu", "swiglu_reference", "gemm", "launch_count", "linear", "add_rmsnorm", "residual_add",
]
