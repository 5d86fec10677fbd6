"""ctypes binding of the sm_100a kernel library (``steptronoss_b200/_native/libstb200.so``).

The library exports plain C entry points that take device pointers, sizes and a CUDA stream and
return 0 or a negative error.  On a machine with a GPU the library is mandatory: if it is missing
and cannot be built, importing an op that needs it raises instead of falling back to another
implementation.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from pathlib import Path

import torch

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "_native" / "libstb200.so"


class NativeLibraryError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def load(build_if_missing: bool = True):
    """Load (building first when absent and nvcc is available) and return the ctypes handle."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists() and build_if_missing:
        from ..csrc.build import build

        build()
    if not _LIB_PATH.exists():
        raise NativeLibraryError(f"native kernel library not found at {_LIB_PATH}; run python -m steptronoss_b200.csrc.build")
    lib = ctypes.CDLL(str(_LIB_PATH))
    _declare(lib)
    _LIB = lib
    return lib


def available() -> bool:
    """True when the native library loads.  On a machine with a GPU a library that cannot be loaded is an error
    (the kernels are the only path there: nothing falls back to PyTorch silently); without a GPU the answer is
    simply False and callers take the PyTorch restatements."""
    try:
        load()
        return True
    except Exception:
        if torch.cuda.is_available():
            raise
        return False


P, I, L, F = c_void_p, c_int, c_longlong, c_float

_SIGNATURES = {
    "stb_sm_count": [],
    "stb_gemm_bf16": [P, P, P, I, I, I, I, I, I, I, I, I, I, F, P, P],
    "stb_gemm_bf16_ex": [P, P, P, I, I, I, I, I, I, I, I, F, P, L, F, I, P, P],
    "stb_mirror_upper_bf16": [P, I, L, P],
    "stb_gemm_bf16_grouped_rows": [P, P, P, P, I, I, I, I, I, I, I, I, I, I, P, P],
    "stb_gemm_bf16_grouped_reduce": [P, P, P, P, I, I, I, I, I, I, I, I, I, P, P],
    "stb_rmsnorm_fwd": [P, P, P, P, L, I, L, L, F, I, P],
    "stb_add_rmsnorm_fwd": [P, P, P, P, P, P, L, I, L, L, L, L, F, I, P],
    "stb_add_rmsnorm_bwd": [P, P, P, P, P, P, P, P, L, I, L, L, L, L, I, I, P],
    "stb_rmsnorm_bwd_grid": [L],
    "stb_rmsnorm_bwd": [P, P, P, P, P, P, P, L, I, L, L, L, I, I, I, P],
    "stb_qknorm_rope_fwd": [P, P, P, P, P, P, P, P, P, I, I, I, I, L, I, F, I, I, P],
    "stb_qknorm_rope_bwd_grid": [],
    "stb_qknorm_rope_bwd": [P, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, L, L, I, I, I, I, P],
    "stb_swiglu_fwd": [P, P, L, I, L, L, F, P],
    "stb_swiglu_bwd": [P, P, P, L, I, L, L, L, F, P],
    "stb_embedding_fwd": [P, P, P, L, I, L, L, P],
    "stb_embedding_bwd": [P, P, P, L, I, L, L, P],
    "stb_add_bf16": [P, P, P, L, P],
    "stb_ce_stats": [P, P, P, P, L, I, L, L, P],
    "stb_ce_grad": [P, P, P, P, P, L, I, L, L, P],
    "stb_moe_index_chunks": [I],
    "stb_moe_index": [P, I, I, I, P, P, P, P, I, P, P, P, P],
    "stb_moe_scatter": [P, P, P, I, I, I, I, P, P],
    "stb_moe_gather": [P, P, P, I, I, I, P, P],
    "stb_moe_gather_bwd": [P, P, P, P, P, P, I, I, I, I, I, P, P, P],
    "stb_router_grid": [I],
    "stb_router_fwd": [P, P, I, I, I, I, I, F, P, P, P, P, P, P],
    "stb_router_finalize": [P, P, P, I, I, I, P, P, P, P, P],
    "stb_router_bwd": [P, I, I, I, I, I, F, P, P, P, P, P],
    "stb_sqnorm_grid": [],
    "stb_sqnorm": [P, L, P, P, I, P],
    "stb_clip_coef": [P, F, P],
    "stb_adam": [P, P, P, P, P, P, I, P, F, F, F, F, F, F, F, I, P],
    "stb_cast_f32_bf16": [P, P, L, P],
    "stb_accumulate_bf16": [P, P, L, P],
    "stb_scale_f32": [P, L, F, P],
    "stb_nonfinite_flag": [P, L, P, P],
    "stb_gae": [P, P, P, I, F, F, P, P, P],
    "stb_attn_fwd": [P] * 9 + [I] * 6 + [L] * 3 + [I, I, F, P, P, P, I, I, P, P],
    "stb_attn_bwd": [P] * 14 + [I] + [P] * 2 + [I] * 6 + [L] * 4 + [I, I, F, P, I, P, P, P, I, I, P, P],
    "stb_attn_bwd_splits": [I, I, I],
}


def _declare(lib) -> None:
    for name, argtypes in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = argtypes
        fn.restype = I
    for name in dir(lib):
        pass


def register_signature(name: str, argtypes: list) -> None:
    """Declare one more exported function (used by optional kernel families)."""
    _SIGNATURES[name] = argtypes
    if _LIB is not None:
        fn = getattr(_LIB, name)
        fn.argtypes = argtypes
        fn.restype = I


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_DEVICE_INDEX: int | None = None


def stream() -> int:
    """The raw handle of the current CUDA stream.  Called once per kernel launch, so it avoids building a
    ``torch.cuda.Stream`` object (about 15 us each, a tenth of the host time of a launch-bound step): one process
    drives one device, whose index is looked up once."""
    global _DEVICE_INDEX
    if _RAW_STREAM is None:
        return torch.cuda.current_stream().cuda_stream
    if _DEVICE_INDEX is None:
        _DEVICE_INDEX = torch.cuda.current_device()
    return _RAW_STREAM(_DEVICE_INDEX)


_ERRORS = {
    1: "producer wait timed out",
    2: "MMA wait on operand stage timed out",
    3: "MMA wait on TMEM buffer timed out",
    4: "epilogue wait timed out",
    5: "peer flag wait timed out",
    6: "bad argument (alignment / shape)",
    7: "softmax wait timed out",
    8: "correction wait timed out",
    9: "MoE capacity exceeded: more routed slots than the expert-major buffers hold (raise moe capacity_factor)",
}


def check(rc: int, what: str) -> None:
    if rc != 0:
        code = -rc
        msg = _ERRORS.get(code, f"CUDA/driver error {code}")
        raise NativeLibraryError(f"{what} failed: {msg} (rc={rc})")


_STATUS: dict[int, torch.Tensor] = {}


def status_word(device: torch.device | None = None) -> torch.Tensor:
    """Per-device int32 word in which kernels record a bounded-wait timeout (0 = healthy)."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if idx not in _STATUS:
        _STATUS[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _STATUS[idx]


def raise_if_kernel_error() -> None:
    """Read the status word (synchronises) and raise when a kernel reported a timeout."""
    for idx, t in _STATUS.items():
        code = int(t.item())
        if code != 0:
            t.zero_()
            raise NativeLibraryError(f"device {idx}: kernel reported '{_ERRORS.get(code, code)}'")


def use_native(t: torch.Tensor) -> bool:
    """True when ``t`` lives on a GPU (the native kernels are then the only path)."""
    return t.is_cuda
