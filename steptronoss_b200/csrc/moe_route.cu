// Mixture-of-experts token routing on the device: slot -> expert-major row index, row scatter, weighted
// gather and their backward passes.  Semantics of the reference ops histogram / index_compute / moe_scatter /
// moe_weighted_gather (steptronoss/model/utils/moe_utils.py:85-453) with the layout the grouped tcgen05 GEMM
// wants: every expert's segment starts at a multiple of 128 rows, padding rows inside a segment are zero,
// rows past the last segment are never read (their row tiles carry group -1 and are skipped by the GEMM).
//
//   stb_moe_index       : ids [n_slots] (int64; < 0 or >= E = ignored) -> dest [n_slots] (int64, -1 = ignored),
//                         offsets [E+1], counts [E], tile_group [n_tiles], slot_of_row [rows] (-1 = padding).
//                         Stable: inside an expert the slots keep their order.  Three small launches
//                         (chunk histograms; scan over chunks and experts; ranks), no sort, no host sync.
//   stb_moe_scatter     : out[r] = x[slot_of_row[r] / K] or 0, one warp per expert-major row, each row written once
//   stb_moe_scatter_bwd : dx[t] = sum_k g[dest[t,k]]
//   stb_moe_gather      : out[t] = sum_k w[t,k] * y[dest[t,k]]
//   stb_moe_gather_bwd  : gy[dest[t,k]] = w[t,k] * g[t], gw[t,k] = <y[dest[t,k]], g[t]>, padding rows of gy = 0
//
// Rows are bf16 with H a multiple of 8 (16-byte words); accumulation is fp32.  All kernels are bandwidth bound:
// one warp per row / token, 16-byte accesses, the K source rows of a token loaded together.
#include <cuda_bf16.h>

#include "common.cuh"

namespace stb {

constexpr int kChunk = 512;          // slots per warp in the index kernels
constexpr int kIndexWarps = 4;       // warps per block in the index kernels
constexpr int kMaxTopK = 16;

__device__ __forceinline__ int slot_expert(const long long* ids, int i, int n_slots, int E) {
  if (i >= n_slots) return -2;
  const long long e = ids[i];
  return (e >= 0 && e < E) ? static_cast<int>(e) : -1;
}

// chunk_hist[c][e] = number of slots of chunk c routed to expert e; also fills slot_of_row with -1
__global__ void moe_hist_kernel(const long long* __restrict__ ids, int n_slots, int E, int n_chunks,
                                int* __restrict__ chunk_hist, int* __restrict__ slot_of_row, int rows) {
  extern __shared__ int smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) slot_of_row[r] = -1;
  int* hist = smem + warp * E;
  const int c = blockIdx.x * kIndexWarps + warp;
  if (c >= n_chunks) return;
  for (int e = lane; e < E; e += 32) hist[e] = 0;
  __syncwarp();
  const int begin = c * kChunk;
  for (int i = begin + lane; i < begin + kChunk; i += 32) {
    const int e = slot_expert(ids, i, n_slots, E);
    if (e >= 0) atomicAdd(&hist[e], 1);
  }
  __syncwarp();
  for (int e = lane; e < E; e += 32) chunk_hist[static_cast<long long>(c) * E + e] = hist[e];
}

// one block: exclusive scan of chunk_hist over chunks (per expert), counts, 128-aligned segment starts, tile groups
// Segment starts are clamped to `rows` (a multiple of 128): when the caller sized the buffers by a capacity bound
// instead of the exact count and more slots arrive, the overflowing slots are dropped (dest -1) and the status
// word records kErrMoeCapacity, so the step fails loudly instead of writing out of bounds.
__global__ void moe_scan_kernel(int* __restrict__ chunk_hist, int n_chunks, int E, int* __restrict__ counts,
                                int* __restrict__ offsets, int* __restrict__ tile_group, int n_tiles, int rows,
                                int* status) {
  extern __shared__ int smem[];  // E + 1 segment starts
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < n_chunks; ++c) {
      const long long at = static_cast<long long>(c) * E + e;
      const int v = chunk_hist[at];
      chunk_hist[at] = run;
      run += v;
    }
    counts[e] = run;
    smem[e + 1] = (run + 127) & ~127;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    smem[0] = 0;
    for (int e = 0; e < E; ++e) smem[e + 1] += smem[e];
    if (smem[E] > rows) report_error(status, kErrMoeCapacity);
    for (int e = 0; e <= E; ++e) smem[e] = min(smem[e], rows);
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = smem[e];
  for (int t = threadIdx.x; t < n_tiles; t += blockDim.x) {
    const int row = t * 128;
    int lo = 0, hi = E;  // first e with smem[e + 1] > row
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (smem[mid + 1] > row) hi = mid; else lo = mid + 1;
    }
    tile_group[t] = lo < E ? lo : -1;
  }
}

// dest[i] = offsets[e] + (slots of e in earlier chunks) + (slots of e earlier in this chunk); slot_of_row[dest] = i
__global__ void moe_rank_kernel(const long long* __restrict__ ids, int n_slots, int E, int n_chunks,
                                const int* __restrict__ chunk_hist, const int* __restrict__ offsets,
                                long long* __restrict__ dest, int* __restrict__ slot_of_row, int rows) {
  extern __shared__ int smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* next = smem + warp * E;
  const int c = blockIdx.x * kIndexWarps + warp;
  if (c >= n_chunks) return;
  // offsets[e + 1] bounds expert e's segment (clamped to the buffer); ranks past it are dropped
  int* limit = next + kIndexWarps * E;
  for (int e = lane; e < E; e += 32) {
    next[e] = offsets[e] + chunk_hist[static_cast<long long>(c) * E + e];
    limit[e] = offsets[e + 1];
  }
  __syncwarp();
  const int begin = c * kChunk;
  const unsigned lt = (1u << lane) - 1u;
  for (int i = begin + lane; i < begin + kChunk; i += 32) {
    const int e = slot_expert(ids, i, n_slots, E);
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int leader = __ffs(same) - 1;
    int base = 0;
    if (lane == leader && e >= 0) {
      base = next[e];
      next[e] = base + __popc(same);
    }
    base = __shfl_sync(0xffffffffu, base, leader);
    __syncwarp();
    if (e >= 0) {
      const int d = base + __popc(same & lt);
      if (d < limit[e] && d < rows) {
        dest[i] = d;
        slot_of_row[d] = i;
      } else {
        dest[i] = -1;
      }
    } else if (e == -1) {
      dest[i] = -1;
    }
  }
}

// ---------------------------------------------------------------------------------------------- row movers
struct Acc8 {
  float v[8];
};
__device__ __forceinline__ void zero8(Acc8& a) {
#pragma unroll
  for (int i = 0; i < 8; ++i) a.v[i] = 0.f;
}
__device__ __forceinline__ void fma8(Acc8& a, const uint4& q, float w) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    a.v[2 * i] = fmaf(w, f.x, a.v[2 * i]);
    a.v[2 * i + 1] = fmaf(w, f.y, a.v[2 * i + 1]);
  }
}
__device__ __forceinline__ uint4 pack8(const Acc8& a) {
  uint4 q;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(a.v[2 * i], a.v[2 * i + 1]);
  return q;
}
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b) {
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
    s = fmaf(fa.x, fb.x, s);
    s = fmaf(fa.y, fb.y, s);
  }
  return s;
}

__global__ void moe_scatter_kernel(const uint4* __restrict__ x, const int* __restrict__ slot_of_row,
                                   const int* __restrict__ offsets, int E, int K, int h16, int rows,
                                   uint4* __restrict__ out) {
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int used = min(offsets[E], rows);
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < used; r += gridDim.x * wpb) {
    const int s = slot_of_row[r];
    uint4* o = out + static_cast<long long>(r) * h16;
    if (s >= 0) {
      const uint4* src = x + static_cast<long long>(s / K) * h16;
      for (int j = lane; j < h16; j += 32) o[j] = src[j];
    } else {
      for (int j = lane; j < h16; j += 32) o[j] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// out[t] = sum_k w[t,k] * y[dest[t,k]]  (w == nullptr: plain sum, the backward of the scatter)
template <int KT>
__global__ void __launch_bounds__(256, KT <= 8 ? 2 : 1) moe_gather_kernel(const uint4* __restrict__ y, const long long* __restrict__ dest,
                                  const float* __restrict__ w, int T, int K, int h16, uint4* __restrict__ out) {
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    long long d[KT];
    float wt[KT];
#pragma unroll
    for (int k = 0; k < KT; ++k) {
      d[k] = k < K ? dest[static_cast<long long>(t) * K + k] : -1;
      wt[k] = (k < K && d[k] >= 0) ? (w ? w[static_cast<long long>(t) * K + k] : 1.f) : 0.f;
    }
    for (int j = lane; j < h16; j += 32) {
      uint4 q[KT];
#pragma unroll
      for (int k = 0; k < KT; ++k)
        if (d[k] >= 0) q[k] = y[d[k] * h16 + j];
      Acc8 a;
      zero8(a);
#pragma unroll
      for (int k = 0; k < KT; ++k)
        if (d[k] >= 0) fma8(a, q[k], wt[k]);
      out[static_cast<long long>(t) * h16 + j] = pack8(a);
    }
  }
}

// warps [0, T): token t -> gy rows of its slots and gw[t, :]; warps [T, T + rows): zero the padding rows of gy
template <int KT>
__global__ void __launch_bounds__(256, KT <= 8 ? 2 : 1) moe_gather_bwd_kernel(const uint4* __restrict__ g, const uint4* __restrict__ y,
                                      const long long* __restrict__ dest, const float* __restrict__ w,
                                      const int* __restrict__ slot_of_row, const int* __restrict__ offsets, int E,
                                      int T, int K, int h16, int rows, uint4* __restrict__ gy,
                                      float* __restrict__ gw) {
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int used = min(offsets[E], rows);
  for (int u = blockIdx.x * wpb + (threadIdx.x >> 5); u < T + used; u += gridDim.x * wpb) {
    if (u >= T) {
      const int r = u - T;
      if (slot_of_row[r] < 0) {
        uint4* o = gy + static_cast<long long>(r) * h16;
        for (int j = lane; j < h16; j += 32) o[j] = make_uint4(0u, 0u, 0u, 0u);
      }
      continue;
    }
    const int t = u;
    long long d[KT];
    float wt[KT], dot[KT];
#pragma unroll
    for (int k = 0; k < KT; ++k) {
      d[k] = k < K ? dest[static_cast<long long>(t) * K + k] : -1;
      wt[k] = (k < K && d[k] >= 0) ? w[static_cast<long long>(t) * K + k] : 0.f;
      dot[k] = 0.f;
    }
    for (int j = lane; j < h16; j += 32) {
      const uint4 gq = g[static_cast<long long>(t) * h16 + j];
      uint4 q[KT];
#pragma unroll
      for (int k = 0; k < KT; ++k)
        if (d[k] >= 0) q[k] = y[d[k] * h16 + j];
#pragma unroll
      for (int k = 0; k < KT; ++k) {
        if (d[k] < 0) continue;
        dot[k] += dot8(q[k], gq);
        Acc8 a;
        zero8(a);
        fma8(a, gq, wt[k]);
        gy[d[k] * h16 + j] = pack8(a);
      }
    }
#pragma unroll
    for (int k = 0; k < KT; ++k) {
      float s = dot[k];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0 && k < K) gw[static_cast<long long>(t) * K + k] = s;
    }
  }
}

static int row_grid(long long warps_needed, int threads) {
  const int wpb = threads / 32;
  long long grid = (warps_needed + wpb - 1) / wpb;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  return static_cast<int>(grid);
}

static int last_error() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

}  // namespace stb

using namespace stb;

extern "C" int stb_moe_index_chunks(int n_slots) { return (n_slots + kChunk - 1) / kChunk; }

// chunk_hist: int32 scratch of stb_moe_index_chunks(n_slots) * E words.
extern "C" int stb_moe_index(const void* ids, int n_slots, int E, int rows, void* dest, void* offsets, void* counts,
                             void* tile_group, int n_tiles, void* slot_of_row, void* chunk_hist, int* status,
                             cudaStream_t stream) {
  if (E < 1 || E > 1024 || n_slots < 0 || rows < 0 || (rows & 127)) return -kErrBadArgument;
  const int n_chunks = stb_moe_index_chunks(n_slots);
  const size_t smem = static_cast<size_t>(kIndexWarps) * E * sizeof(int);
  int blocks = (n_chunks + kIndexWarps - 1) / kIndexWarps;
  if (blocks < 1) blocks = 1;
  // the histogram launch also fills slot_of_row: give it enough threads for that when there are few chunks
  const int fill_blocks = (rows + kIndexWarps * 32 * 8 - 1) / (kIndexWarps * 32 * 8);
  moe_hist_kernel<<<blocks > fill_blocks ? blocks : fill_blocks, kIndexWarps * 32, smem, stream>>>(
      static_cast<const long long*>(ids), n_slots, E, n_chunks, static_cast<int*>(chunk_hist),
      static_cast<int*>(slot_of_row), rows);
  moe_scan_kernel<<<1, 1024, (E + 1) * sizeof(int), stream>>>(static_cast<int*>(chunk_hist), n_chunks, E,
                                                               static_cast<int*>(counts), static_cast<int*>(offsets),
                                                               static_cast<int*>(tile_group), n_tiles, rows, status);
  moe_rank_kernel<<<blocks, kIndexWarps * 32, 2 * smem, stream>>>(static_cast<const long long*>(ids), n_slots, E, n_chunks,
                                                               static_cast<const int*>(chunk_hist),
                                                               static_cast<const int*>(offsets),
                                                               static_cast<long long*>(dest),
                                                               static_cast<int*>(slot_of_row), rows);
  return last_error();
}

extern "C" int stb_moe_scatter(const void* x, const void* slot_of_row, const void* offsets, int E, int K, int H,
                               int rows, void* out, cudaStream_t stream) {
  if ((H & 7) || K < 1) return -kErrBadArgument;
  moe_scatter_kernel<<<row_grid(rows, 256), 256, 0, stream>>>(static_cast<const uint4*>(x),
                                                              static_cast<const int*>(slot_of_row),
                                                              static_cast<const int*>(offsets), E, K, H / 8, rows,
                                                              static_cast<uint4*>(out));
  return last_error();
}

template <int KT>
static void launch_gather(const void* y, const void* dest, const void* w, int T, int K, int H, void* out,
                          cudaStream_t stream) {
  moe_gather_kernel<KT><<<row_grid(T, 256), 256, 0, stream>>>(static_cast<const uint4*>(y),
                                                              static_cast<const long long*>(dest),
                                                              static_cast<const float*>(w), T, K, H / 8,
                                                              static_cast<uint4*>(out));
}

// w may be null (plain sum over the K slots: the backward of the scatter)
extern "C" int stb_moe_gather(const void* y, const void* dest, const void* w, int T, int K, int H, void* out,
                              cudaStream_t stream) {
  if ((H & 7) || K < 1 || K > kMaxTopK) return -kErrBadArgument;
  if (K <= 2) launch_gather<2>(y, dest, w, T, K, H, out, stream);
  else if (K <= 4) launch_gather<4>(y, dest, w, T, K, H, out, stream);
  else if (K <= 8) launch_gather<8>(y, dest, w, T, K, H, out, stream);
  else launch_gather<16>(y, dest, w, T, K, H, out, stream);
  return last_error();
}

template <int KT>
static void launch_gather_bwd(const void* g, const void* y, const void* dest, const void* w, const void* slot_of_row,
                              const void* offsets, int E, int T, int K, int H, int rows, void* gy, void* gw,
                              cudaStream_t stream) {
  moe_gather_bwd_kernel<KT><<<row_grid(static_cast<long long>(T) + rows, 256), 256, 0, stream>>>(
      static_cast<const uint4*>(g), static_cast<const uint4*>(y), static_cast<const long long*>(dest),
      static_cast<const float*>(w), static_cast<const int*>(slot_of_row), static_cast<const int*>(offsets), E, T, K,
      H / 8, rows, static_cast<uint4*>(gy), static_cast<float*>(gw));
}

extern "C" int stb_moe_gather_bwd(const void* g, const void* y, const void* dest, const void* w,
                                  const void* slot_of_row, const void* offsets, int E, int T, int K, int H, int rows,
                                  void* gy, void* gw, cudaStream_t stream) {
  if ((H & 7) || K < 1 || K > kMaxTopK) return -kErrBadArgument;
  if (K <= 2) launch_gather_bwd<2>(g, y, dest, w, slot_of_row, offsets, E, T, K, H, rows, gy, gw, stream);
  else if (K <= 4) launch_gather_bwd<4>(g, y, dest, w, slot_of_row, offsets, E, T, K, H, rows, gy, gw, stream);
  else if (K <= 8) launch_gather_bwd<8>(g, y, dest, w, slot_of_row, offsets, E, T, K, H, rows, gy, gw, stream);
  else launch_gather_bwd<16>(g, y, dest, w, slot_of_row, offsets, E, T, K, H, rows, gy, gw, stream);
  return last_error();
}

// ------------------------------------------------------------------------------------------------ router
// One warp per token: probabilities (softmax or sigmoid), top-k of (prob + selection bias) with the tie-break of
// a stable descending sort (lower expert index first), renormalised routing weights, and the per-expert sums the
// auxiliary loss needs.  Stands where the reference sorts every row of the [T, E] probability matrix
// (steptronoss/model/common/moe_block.py:224-337).  Per-expert sums are deterministic: every warp adds its tokens
// in order into its own shared-memory row, the block adds its warps in order and writes one partial row per
// block; the caller sums the partial rows.
namespace stb {

constexpr int kRouterWarps = 8;
constexpr int kRouterMaxE = 512;

struct RouterArgs {
  const float* logits;  // [T, E]
  const float* bias;    // [E] added for selection only, or null
  int T, E, K;
  int sigmoid;          // 1: sigmoid scores, weights and probabilities renormalised by their sums
  int norm_topk;        // softmax only: renormalise the k selected probabilities
  float eps;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// p[e] of one token into shared memory; returns sum_e p[e] (softmax: 1 by construction, returned as computed)
__device__ __forceinline__ float router_probs(const RouterArgs& a, const float* row, float* p, int lane,
                                              float* absmax) {
  float m = -INFINITY, am = 0.f;
  for (int e = lane; e < a.E; e += 32) {
    const float l = row[e];
    p[e] = l;
    m = fmaxf(m, l);
    am = fmaxf(am, fabsf(l));
  }
  *absmax = warp_max(am);
  float s = 0.f;
  if (a.sigmoid) {
    for (int e = lane; e < a.E; e += 32) {
      const float v = 1.f / (1.f + expf(-p[e]));
      p[e] = v;
      s += v;
    }
    return warp_sum(s);
  }
  m = warp_max(m);
  for (int e = lane; e < a.E; e += 32) {
    const float v = expf(p[e] - m);
    p[e] = v;
    s += v;
  }
  s = warp_sum(s);
  const float inv = 1.f / s;
  for (int e = lane; e < a.E; e += 32) p[e] *= inv;
  return 1.f;
}

__global__ void router_fwd_kernel(const RouterArgs a, long long* __restrict__ ids, float* __restrict__ weights,
                                  float* __restrict__ part_prob, int* __restrict__ part_hist,
                                  float* __restrict__ part_stats) {
  extern __shared__ float rsm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* p = rsm + warp * a.E;                              // probabilities of the current token
  float* sel = rsm + (kRouterWarps + warp) * a.E;           // selection scores, consumed by the top-k rounds
  float* acc = rsm + (2 * kRouterWarps + warp) * a.E;       // this warp's per-expert probability sums
  int* cnt = reinterpret_cast<int*>(rsm + (3 * kRouterWarps + warp) * a.E);
  for (int e = lane; e < a.E; e += 32) {
    acc[e] = 0.f;
    cnt[e] = 0;
  }
  float absmax_all = 0.f, pmax_sum = 0.f;
  for (int t = blockIdx.x * kRouterWarps + warp; t < a.T; t += gridDim.x * kRouterWarps) {
    __syncwarp();
    float am;
    const float S = router_probs(a, a.logits + static_cast<long long>(t) * a.E, p, lane, &am);
    absmax_all = fmaxf(absmax_all, am);
    __syncwarp();
    const float invS = a.sigmoid ? 1.f / (S + a.eps) : 1.f;
    float pm = 0.f;
    for (int e = lane; e < a.E; e += 32) {
      const float v = p[e];
      sel[e] = a.bias ? v + a.bias[e] : v;
      acc[e] += v * invS;
      pm = fmaxf(pm, v);
    }
    pmax_sum += warp_max(pm);
    __syncwarp();
    float top_p = 0.f;   // lane k keeps the k-th selected probability
    int top_e = -1;
    float top_sum = 0.f;
    for (int k = 0; k < a.K; ++k) {
      float best = -INFINITY;
      int arg = 0x7fffffff;
      for (int e = lane; e < a.E; e += 32) {
        const float v = sel[e];
        if (v > best) {  // strided scan visits indices in increasing order: first maximum kept
          best = v;
          arg = e;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) {
          best = ob;
          arg = oa;
        }
      }
      if (arg >= a.E) arg = k;  // all scores NaN: any fixed choice keeps indices in range
      const float pv = p[arg];
      top_sum += pv;
      if (lane == k) {
        top_p = pv;
        top_e = arg;
      }
      if (lane == 0) {
        sel[arg] = -INFINITY;
        cnt[arg] += 1;
      }
      __syncwarp();
    }
    if (lane < a.K) {
      const bool renorm = a.sigmoid || a.norm_topk;
      ids[static_cast<long long>(t) * a.K + lane] = top_e;
      weights[static_cast<long long>(t) * a.K + lane] = renorm ? top_p / (top_sum + a.eps) : top_p;
    }
  }
  __syncthreads();
  // block partials: warps added in order
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
    float s = 0.f;
    int c = 0;
    for (int w = 0; w < kRouterWarps; ++w) {
      s += rsm[(2 * kRouterWarps + w) * a.E + e];
      c += reinterpret_cast<int*>(rsm)[(3 * kRouterWarps + w) * a.E + e];
    }
    part_prob[static_cast<long long>(blockIdx.x) * a.E + e] = s;
    part_hist[static_cast<long long>(blockIdx.x) * a.E + e] = c;
  }
  __shared__ float red[2][kRouterWarps];
  if (lane == 0) {
    red[0][warp] = absmax_all;
    red[1][warp] = pmax_sum;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float am = 0.f, ps = 0.f;
    for (int w = 0; w < kRouterWarps; ++w) {
      am = fmaxf(am, red[0][w]);
      ps += red[1][w];
    }
    part_stats[2 * blockIdx.x] = am;
    part_stats[2 * blockIdx.x + 1] = ps;
  }
}

// dlogits from the gradients of the routing weights (g_w [T, K]) and of the per-expert probability sums (g_ps [E])
__global__ void router_bwd_kernel(const RouterArgs a, const long long* __restrict__ ids,
                                  const float* __restrict__ g_w, const float* __restrict__ g_ps,
                                  float* __restrict__ dlogits) {
  extern __shared__ float rsm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* p = rsm + warp * a.E;
  float* dp = rsm + (kRouterWarps + warp) * a.E;
  for (int t = blockIdx.x * kRouterWarps + warp; t < a.T; t += gridDim.x * kRouterWarps) {
    __syncwarp();
    float am;
    const float S = router_probs(a, a.logits + static_cast<long long>(t) * a.E, p, lane, &am);
    __syncwarp();
    // gradient reaching p through the per-expert sums
    if (a.sigmoid) {
      const float invS = 1.f / (S + a.eps);
      float dotv = 0.f;
      for (int e = lane; e < a.E; e += 32) dotv += (g_ps ? g_ps[e] : 0.f) * p[e];
      dotv = warp_sum(dotv) * invS;  // sum_j g_j * probn_j
      for (int e = lane; e < a.E; e += 32) dp[e] = ((g_ps ? g_ps[e] : 0.f) - dotv) * invS;
    } else {
      for (int e = lane; e < a.E; e += 32) dp[e] = g_ps ? g_ps[e] : 0.f;
    }
    __syncwarp();
    // gradient reaching p through the k routing weights
    int e_k = 0;
    float p_k = 0.f, g_k = 0.f;
    if (lane < a.K) {
      e_k = static_cast<int>(ids[static_cast<long long>(t) * a.K + lane]);
      p_k = p[e_k];
      g_k = g_w[static_cast<long long>(t) * a.K + lane];
    }
    if (a.sigmoid || a.norm_topk) {
      const float s_top = warp_sum(p_k) + a.eps;
      const float gdot = warp_sum(g_k * p_k) / s_top;  // sum_k g_k * w_k
      if (lane < a.K) dp[e_k] += (g_k - gdot) / s_top;
    } else if (lane < a.K) {
      dp[e_k] += g_k;
    }
    __syncwarp();
    float* out = dlogits + static_cast<long long>(t) * a.E;
    if (a.sigmoid) {
      for (int e = lane; e < a.E; e += 32) out[e] = dp[e] * p[e] * (1.f - p[e]);
    } else {
      float dotv = 0.f;
      for (int e = lane; e < a.E; e += 32) dotv += dp[e] * p[e];
      dotv = warp_sum(dotv);
      for (int e = lane; e < a.E; e += 32) out[e] = p[e] * (dp[e] - dotv);
    }
  }
}

static int router_grid(int T) {
  int grid = (T + kRouterWarps - 1) / kRouterWarps;
  const int cap = sm_count() * 2;
  if (grid > cap) grid = cap;
  return grid < 1 ? 1 : grid;
}

}  // namespace stb

// Sums of the per-CTA partials of router_fwd_kernel in one launch: prob_sum [E], hist [E] (int32 and a float copy for
// the auxiliary loss), stats = [max |logit|, mean over tokens of the largest probability] and the share of the
// busiest expert (max hist / sum hist).  One CTA; thread e owns expert e (E <= 512).
__global__ void __launch_bounds__(512)
router_finalize_kernel(const float* __restrict__ part_prob, const int* __restrict__ part_hist,
                       const float* __restrict__ part_stats, int grid, int E, int T, float* __restrict__ prob_sum,
                       int* __restrict__ hist, float* __restrict__ hist_f, float* __restrict__ stats3) {
  __shared__ int s_max[16], s_sum[16];
  __shared__ float s_lmax[16], s_psum[16];
  const int e = threadIdx.x;
  float ps = 0.f;
  int h = 0;
  if (e < E) {
    for (int g = 0; g < grid; ++g) {
      ps += part_prob[static_cast<long long>(g) * E + e];
      h += part_hist[static_cast<long long>(g) * E + e];
    }
    prob_sum[e] = ps;
    hist[e] = h;
    hist_f[e] = static_cast<float>(h);
  }
  float lmax = 0.f, psum = 0.f;
  for (int g = e; g < grid; g += blockDim.x) {
    lmax = fmaxf(lmax, part_stats[2 * g]);
    psum += part_stats[2 * g + 1];
  }
  int hm = h, hs = h;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    hm = max(hm, __shfl_xor_sync(0xffffffffu, hm, o));
    hs += __shfl_xor_sync(0xffffffffu, hs, o);
    lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
    psum += __shfl_xor_sync(0xffffffffu, psum, o);
  }
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) { s_max[w] = hm; s_sum[w] = hs; s_lmax[w] = lmax; s_psum[w] = psum; }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    for (int i = 1; i < nw; ++i) {
      hm = max(hm, s_max[i]); hs += s_sum[i]; lmax = fmaxf(lmax, s_lmax[i]); psum += s_psum[i];
    }
    stats3[0] = lmax;
    stats3[1] = psum / static_cast<float>(T > 0 ? T : 1);
    stats3[2] = static_cast<float>(hm) / static_cast<float>(hs > 0 ? hs : 1);
  }
}

extern "C" int stb_router_grid(int T) { return router_grid(T); }

// part_prob / part_hist: [stb_router_grid(T), E]; part_stats: [grid, 2] (max |logit|, sum over tokens of max prob)
extern "C" int stb_router_fwd(const void* logits, const void* bias, int T, int E, int K, int sigmoid, int norm_topk,
                              float eps, void* ids, void* weights, void* part_prob, void* part_hist, void* part_stats,
                              cudaStream_t stream) {
  if (E < 1 || E > kRouterMaxE || K < 1 || K > 32 || K > E) return -kErrBadArgument;
  RouterArgs a{static_cast<const float*>(logits), static_cast<const float*>(bias), T, E, K, sigmoid, norm_topk, eps};
  const size_t smem = static_cast<size_t>(4) * kRouterWarps * E * sizeof(float);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(router_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         4 * kRouterWarps * kRouterMaxE * static_cast<int>(sizeof(float)));
    attr_set = true;
  }
  router_fwd_kernel<<<router_grid(T), kRouterWarps * 32, smem, stream>>>(
      a, static_cast<long long*>(ids), static_cast<float*>(weights), static_cast<float*>(part_prob),
      static_cast<int*>(part_hist), static_cast<float*>(part_stats));
  return last_error();
}

extern "C" int stb_router_bwd(const void* logits, int T, int E, int K, int sigmoid, int norm_topk, float eps,
                              const void* ids, const void* g_w, const void* g_ps, void* dlogits,
                              cudaStream_t stream) {
  if (E < 1 || E > kRouterMaxE || K < 1 || K > 32 || K > E) return -kErrBadArgument;
  RouterArgs a{static_cast<const float*>(logits), nullptr, T, E, K, sigmoid, norm_topk, eps};
  const size_t smem = static_cast<size_t>(2) * kRouterWarps * E * sizeof(float);
  int grid = (T + kRouterWarps - 1) / kRouterWarps;
  const int cap = sm_count() * 8;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  router_bwd_kernel<<<grid, kRouterWarps * 32, smem, stream>>>(a, static_cast<const long long*>(ids),
                                                               static_cast<const float*>(g_w),
                                                               static_cast<const float*>(g_ps),
                                                               static_cast<float*>(dlogits));
  return last_error();
}

extern "C" int stb_router_finalize(const void* part_prob, const void* part_hist, const void* part_stats, int grid, int E,
                                   int T, void* prob_sum, void* hist, void* hist_f, void* stats3, cudaStream_t stream) {
  if (E <= 0 || E > 512 || grid <= 0) return -kErrBadArgument;
  const int threads = (E + 31) / 32 * 32;
  router_finalize_kernel<<<1, threads, 0, stream>>>(
      static_cast<const float*>(part_prob), static_cast<const int*>(part_hist), static_cast<const float*>(part_stats),
      grid, E, T, static_cast<float*>(prob_sum), static_cast<int*>(hist), static_cast<float*>(hist_f),
      static_cast<float*>(stats3));
  return -static_cast<int>(cudaGetLastError());
}
