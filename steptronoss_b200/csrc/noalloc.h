// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference framework; it exists for embedders of this
// library whose code runs where cudaMalloc is off limits: inside a real-time or safety-partitioned
// process that fixed its memory budget at start-up, inside a host application that owns the whole
// device heap through its own pool, or from a plug-in interface that hands the library nothing but
// input and output pointers.  stb_rmsnorm_bwd needs `grid x H` floats of scratch from its caller (one
// row of weight-gradient partials per thread block); this variant keeps that scratch in a fixed 4 MiB
// array inside the library image instead, so the caller passes inputs and outputs only and neither
// this function nor anything it calls allocates or frees memory.
//
// Limits and rules
//   * H (hidden size) must be a multiple of 8 and at most stb_rmsnorm_bwd_noalloc_max_hidden() (4096);
//     larger sizes are rejected with an error message and a negative return value.  Any row count works.
//   * Every device that loads the library holds the 4 MiB array until the process exits.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress).  Make that
//     first call outside of any stream capture.
//   * All calls on a device share the one array.  It keeps whatever the previous call left there; that is
//     harmless because every call overwrites the part it later reads.  Two calls that may run on the GPU
//     at the same time (different streams) would overwrite each other's partials: serialise them.
//
// Arguments are those of stb_rmsnorm_bwd without the scratch pointer: x, w, g (upstream gradient) and dx
// are bf16, rstd is the fp32 per-row reciprocal RMS saved by the forward pass, dw is fp32 [H] (may be
// null), strides are in elements.  add_to_dx accumulates into dx, accumulate_dw into dw.
// Returns 0 on success, a negative code otherwise.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int stb_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* g, const float* rstd, void* dx, float* dw,
                            long long rows, int H, long long x_stride, long long g_stride, long long dx_stride,
                            int zero_centered, int add_to_dx, int accumulate_dw, cudaStream_t stream);

int stb_rmsnorm_bwd_noalloc_max_hidden(void);

#ifdef __cplusplus
}
#endif
