// Row scatter into other GPUs' memory over NVLink, with epoch flags: the data-movement half of the
// expert-parallel dispatcher (tokens to the ranks that host their experts, expert outputs back to the
// tokens' ranks).  Stands where the reference runs variable-size NCCL all-to-alls preceded by a host-side
// exchange of the split sizes (steptronoss/model/ep_dispatcher/token_dispatcher.py:14-118): here every row
// has a fixed landing position in the destination's buffer, so nothing is read back to the host.
//
//   stb_peer_scatter_rows : row i of `src` (src_row[i]) is copied to row dst_row[i] of the buffer of rank
//                           dst_rank[i] (entries with dst_row < 0 are skipped); when the whole grid is done,
//                           the flag word [epoch slot][this rank] of every peer is set to `epoch`.
//   stb_peer_wait_flags   : waits (bounded) until every peer has raised this rank's flag word for `epoch`.
//
// Flags carry the call number, buffers alternate between two slots by epoch parity; a slot written in call
// e was consumed in call e-2, which every writer's call e-1 already depended on.
#include "common.cuh"

namespace stb {

constexpr int kPeerMaxRanks = 8;
struct PeerBases {
  void* p[kPeerMaxRanks];
};

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One warp per row. row_bytes is a multiple of 4; rows whose size and addresses allow it move in 16-byte words.
__global__ void peer_scatter_rows_kernel(const uint8_t* __restrict__ src, long long src_pitch, int row_bytes,
                                         const int* __restrict__ src_row, const int* __restrict__ dst_rank,
                                         const int* __restrict__ dst_row, int n,
                                         const __grid_constant__ PeerBases bases, long long dst_pitch,
                                         const __grid_constant__ PeerBases flags, int flag_index, int world, int rank,
                                         uint32_t epoch, uint32_t* done_counter) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = blockIdx.x * warps_per_block + (threadIdx.x >> 5); i < n; i += gridDim.x * warps_per_block) {
    const int dr = dst_row[i];
    if (dr < 0) continue;
    const int d = dst_rank[i];
    const uint8_t* s = src + static_cast<long long>(src_row[i]) * src_pitch;
    uint8_t* t = static_cast<uint8_t*>(bases.p[d]) + static_cast<long long>(dr) * dst_pitch;
    if ((row_bytes & 15) == 0 && ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(t)) & 15) == 0) {
      const int n16 = row_bytes >> 4;
      for (int j = lane; j < n16; j += 32)
        reinterpret_cast<uint4*>(t)[j] = reinterpret_cast<const uint4*>(s)[j];
    } else {
      const int n4 = row_bytes >> 2;
      for (int j = lane; j < n4; j += 32)
        reinterpret_cast<uint32_t*>(t)[j] = reinterpret_cast<const uint32_t*>(s)[j];
    }
  }
  // the last block to finish publishes the flags (all stores of all blocks are ordered before them)
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;  // ready for the next launch on this stream
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        st_release_sys_u32(static_cast<uint32_t*>(flags.p[r]) + flag_index * kPeerMaxRanks + rank, epoch);
    }
  }
}

__global__ void peer_wait_flags_kernel(const uint32_t* flags, int flag_index, int world, uint32_t epoch,
                                       unsigned long long budget_ns, int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  const uint32_t* f = flags + flag_index * kPeerMaxRanks + r;
  uint64_t t0 = 0;   // the wall clock is slow to read: not before the first miss
  for (uint32_t i = 0;; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys_u32(f) - epoch) >= 0) return;
    if (i == 0) t0 = global_timer_ns();
    if ((i & 15u) == 15u && global_timer_ns() - t0 > budget_ns) {
      report_error(status, kErrPeerFlagWait);
      return;
    }
    __nanosleep(200);
  }
}

}  // namespace stb

using namespace stb;

// bases[r] / flag_pages[r]: destination buffer (this call's slot) and flag page of rank r as mapped here.
// flag_index selects one of the flag rows of the page (e.g. 2 * kind + slot); done_counter: one zeroed word
// of local scratch, reset by the kernel.  Indices are int32 device arrays of length n.
extern "C" int stb_peer_scatter_rows(const void* src, long long src_pitch_bytes, int row_bytes, const int* src_row,
                                     const int* dst_rank, const int* dst_row, int n, void* const* bases,
                                     long long dst_pitch_bytes, void* const* flag_pages, int flag_index, int world,
                                     int rank, unsigned epoch, void* done_counter, cudaStream_t stream) {
  if (world < 1 || world > kPeerMaxRanks || (row_bytes & 3) || row_bytes <= 0) return -kErrBadArgument;
  PeerBases b{}, f{};
  for (int i = 0; i < world; ++i) {
    b.p[i] = bases[i];
    f.p[i] = flag_pages[i];
  }
  const int threads = 256, warps = threads / 32;
  int grid = (n + warps - 1) / warps;
  const int cap = sm_count() * 8;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  peer_scatter_rows_kernel<<<grid, threads, 0, stream>>>(static_cast<const uint8_t*>(src), src_pitch_bytes, row_bytes,
                                                         src_row, dst_rank, dst_row, n, b, dst_pitch_bytes, f,
                                                         flag_index, world, rank, epoch,
                                                         static_cast<uint32_t*>(done_counter));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

extern "C" int stb_peer_wait_flags(const void* flag_page_self, int flag_index, int world, unsigned epoch,
                                   unsigned long long wait_ns, int* status, cudaStream_t stream) {
  if (world < 1 || world > kPeerMaxRanks) return -kErrBadArgument;
  peer_wait_flags_kernel<<<1, 32, 0, stream>>>(static_cast<const uint32_t*>(flag_page_self), flag_index, world, epoch,
                                               wait_ns, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

// ------------------------------------------------------------------------------------------------------------
// Expert-parallel dispatch / return / sum with fixed landing rows: token t of source rank s lands in row
// s*T + t of every destination that hosts one of its experts, so no positions, counts or prefix sums are
// exchanged, and the receiver tells fresh rows from stale ones by the call number in front of each metadata row.
//
//   stb_ep_dispatch : per token, the set of destination ranks follows from its k expert ids; the row of x goes to
//                     each of them (x may be null), together with a metadata row [tag | k local ids (-1 = foreign)
//                     | k weights as bits (0 = foreign)] (weights may be null: rows only, the backward of combine).
//   stb_ep_return   : the way back: receive-buffer row r = s*T + t that is marked valid goes to row rank*T + t of
//                     source s, optionally with a second, small fp32 row (the gradient of the routing weights).
//   stb_ep_sum      : at the source: out[t] = sum over the destinations of token t, in rank order, of the rows that
//                     came back (fp32 accumulation), and gw[t, k] = the entry that the host of expert ids[t, k] sent.
namespace stb {

struct EpShape {
  int T, K, world, rank, per_rank;
};

__device__ __forceinline__ void publish_when_grid_done(uint32_t* done_counter, const PeerBases& flags, int flag_index,
                                                       int world, int rank, uint32_t epoch) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        st_release_sys_u32(static_cast<uint32_t*>(flags.p[r]) + flag_index * kPeerMaxRanks + rank, epoch);
    }
  }
}

// destination rank of the lane's slot (lane < K), -1 for ignored slots and idle lanes
__device__ __forceinline__ int slot_rank(const long long* ids, int t, int lane, const EpShape& s, long long* e_out) {
  long long e = -1;
  if (lane < s.K) e = ids[static_cast<long long>(t) * s.K + lane];
  *e_out = e;
  if (e < 0) return -1;
  const int d = static_cast<int>(e / s.per_rank);
  return d < s.world ? d : -1;
}

__global__ void ep_dispatch_kernel(const uint4* __restrict__ x, long long x_pitch16, int n16,
                                   const long long* __restrict__ ids, const float* __restrict__ weights,
                                   const __grid_constant__ PeerBases xb, long long meta_offset, int tag,
                                   const __grid_constant__ PeerBases flags, int flag_index, uint32_t epoch,
                                   uint32_t* done_counter, const EpShape s) {
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int meta_words = 1 + 2 * s.K;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < s.T; t += gridDim.x * wpb) {
    long long e;
    const int d_lane = slot_rank(ids, t, lane, s, &e);
    const float w_lane = (weights && lane < s.K) ? weights[static_cast<long long>(t) * s.K + lane] : 0.f;
    unsigned hit = 0;
    for (int d = 0; d < s.world; ++d)
      if (__any_sync(0xffffffffu, d_lane == d)) hit |= 1u << d;
    const long long row = static_cast<long long>(s.rank) * s.T + t;
    if (weights) {
      // lane 0: tag, lanes 1..K: local ids, lanes K+1..2K: weight bits
      const int k = lane == 0 ? 0 : (lane <= s.K ? lane - 1 : lane - 1 - s.K);
      const long long e_k = __shfl_sync(0xffffffffu, e, k);
      const int d_k = __shfl_sync(0xffffffffu, d_lane, k);
      const float w_k = __shfl_sync(0xffffffffu, w_lane, k);
      for (int d = 0; d < s.world; ++d) {
        if (!(hit >> d & 1u) || lane >= meta_words) continue;
        int v;
        if (lane == 0) v = tag;
        else if (lane <= s.K) v = d_k == d ? static_cast<int>(e_k - static_cast<long long>(d) * s.per_rank) : -1;
        else v = d_k == d ? __float_as_int(w_k) : 0;
        int* m = reinterpret_cast<int*>(static_cast<uint8_t*>(xb.p[d]) + meta_offset) + row * meta_words;
        m[lane] = v;
      }
    }
    if (x) {
      const uint4* src = x + static_cast<long long>(t) * x_pitch16;
      for (int base = 0; base < n16; base += 256) {
        uint4 q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int j = base + i * 32 + lane;
          if (j < n16) q[i] = src[j];
        }
        for (int d = 0; d < s.world; ++d) {
          if (!(hit >> d & 1u)) continue;
          uint4* dst = static_cast<uint4*>(xb.p[d]) + row * n16;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int j = base + i * 32 + lane;
            if (j < n16) dst[j] = q[i];
          }
        }
      }
    }
  }
  publish_when_grid_done(done_counter, flags, flag_index, s.world, s.rank, epoch);
}

__global__ void ep_return_kernel(const uint4* __restrict__ rows, int n16, const float* __restrict__ wrows,
                                 const uint8_t* __restrict__ valid, const __grid_constant__ PeerBases bb,
                                 long long w_offset, const __grid_constant__ PeerBases flags, int flag_index,
                                 uint32_t epoch, uint32_t* done_counter, const EpShape s) {
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int total = s.world * s.T;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < total; r += gridDim.x * wpb) {
    if (!valid[r]) continue;
    const int src_rank = r / s.T, t = r - src_rank * s.T;
    const long long row = static_cast<long long>(s.rank) * s.T + t;
    if (rows) {
      const uint4* a = rows + static_cast<long long>(r) * n16;
      uint4* dst = static_cast<uint4*>(bb.p[src_rank]) + row * n16;
      for (int base = 0; base < n16; base += 256) {
        uint4 q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int j = base + i * 32 + lane;
          if (j < n16) q[i] = a[j];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int j = base + i * 32 + lane;
          if (j < n16) dst[j] = q[i];
        }
      }
    }
    if (wrows && lane < s.K) {
      float* dw = reinterpret_cast<float*>(static_cast<uint8_t*>(bb.p[src_rank]) + w_offset) + row * s.K;
      dw[lane] = wrows[static_cast<long long>(r) * s.K + lane];
    }
  }
  publish_when_grid_done(done_counter, flags, flag_index, s.world, s.rank, epoch);
}

__global__ void ep_sum_kernel(const uint4* __restrict__ back, int n16, const float* __restrict__ back_w,
                              const long long* __restrict__ ids, uint4* __restrict__ out, float* __restrict__ gw,
                              const EpShape s) {
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < s.T; t += gridDim.x * wpb) {
    long long e;
    const int d_lane = slot_rank(ids, t, lane, s, &e);
    unsigned hit = 0;
    for (int d = 0; d < s.world; ++d)
      if (__any_sync(0xffffffffu, d_lane == d)) hit |= 1u << d;
    if (gw && lane < s.K)
      gw[static_cast<long long>(t) * s.K + lane] =
          d_lane >= 0 ? back_w[(static_cast<long long>(d_lane) * s.T + t) * s.K + lane] : 0.f;
    if (!out) continue;
    for (int j = lane; j < n16; j += 32) {
      uint4 q[kPeerMaxRanks];
#pragma unroll
      for (int d = 0; d < kPeerMaxRanks; ++d)
        if (hit >> d & 1u) q[d] = back[(static_cast<long long>(d) * s.T + t) * n16 + j];
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
      for (int d = 0; d < kPeerMaxRanks; ++d) {
        if (!(hit >> d & 1u)) continue;
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&q[d]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(p[i]);
          acc[2 * i] += f.x;
          acc[2 * i + 1] += f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      out[static_cast<long long>(t) * n16 + j] = o;
    }
  }
}

static int ep_grid(long long warps, int threads) {
  const int wpb = threads / 32;
  long long g = (warps + wpb - 1) / wpb;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (g > cap) g = cap;
  return g < 1 ? 1 : static_cast<int>(g);
}

static bool ep_shape_ok(const EpShape& s) {
  return s.world >= 1 && s.world <= kPeerMaxRanks && s.K >= 1 && s.K <= 15 && s.per_rank >= 1 && s.T >= 0;
}

}  // namespace stb

// x: [T, row_bytes] rows with pitch x_pitch_bytes (null: metadata only); weights: fp32 [T, K] (null: rows only).
// bases[r]: this call's slot of rank r's receive buffer: world*T rows of row_bytes, then at meta_offset world*T
// metadata rows of (1 + 2K) int32.  row_bytes, pitches and offsets are multiples of 16.
extern "C" int stb_ep_dispatch(const void* x, long long x_pitch_bytes, int row_bytes, const void* ids,
                               const void* weights, void* const* bases, long long meta_offset, int tag,
                               void* const* flag_pages, int flag_index, unsigned epoch, void* done_counter, int T,
                               int K, int world, int rank, int per_rank, cudaStream_t stream) {
  EpShape s{T, K, world, rank, per_rank};
  if (!ep_shape_ok(s) || (row_bytes & 15) || (x_pitch_bytes & 15) || (meta_offset & 15)) return -kErrBadArgument;
  PeerBases b{}, f{};
  for (int i = 0; i < world; ++i) {
    b.p[i] = bases[i];
    f.p[i] = flag_pages[i];
  }
  ep_dispatch_kernel<<<ep_grid(T, 256), 256, 0, stream>>>(
      static_cast<const uint4*>(x), x_pitch_bytes / 16, row_bytes / 16, static_cast<const long long*>(ids),
      static_cast<const float*>(weights), b, meta_offset, tag, f, flag_index, epoch,
      static_cast<uint32_t*>(done_counter), s);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

// rows: [world*T, row_bytes] contiguous (null: none); wrows: fp32 [world*T, K] (null: none); valid: uint8 [world*T].
// bases[r]: this call's slot of rank r's return buffer: world*T rows of row_bytes, then at w_offset world*T rows of
// K fp32.
extern "C" int stb_ep_return(const void* rows, int row_bytes, const void* wrows, const void* valid,
                             void* const* bases, long long w_offset, void* const* flag_pages, int flag_index,
                             unsigned epoch, void* done_counter, int T, int K, int world, int rank,
                             cudaStream_t stream) {
  EpShape s{T, K, world, rank, 1};
  if (!ep_shape_ok(s) || (row_bytes & 15) || (w_offset & 15)) return -kErrBadArgument;
  PeerBases b{}, f{};
  for (int i = 0; i < world; ++i) {
    b.p[i] = bases[i];
    f.p[i] = flag_pages[i];
  }
  ep_return_kernel<<<ep_grid(static_cast<long long>(world) * T, 256), 256, 0, stream>>>(
      static_cast<const uint4*>(rows), row_bytes / 16, static_cast<const float*>(wrows),
      static_cast<const uint8_t*>(valid), b, w_offset, f, flag_index, epoch, static_cast<uint32_t*>(done_counter), s);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

// back: bf16 rows [world*T, H] of this rank's return buffer (null: none); back_w: fp32 [world*T, K] (null: none).
extern "C" int stb_ep_sum(const void* back, int H, const void* back_w, const void* ids, void* out, void* gw, int T,
                          int K, int world, int rank, int per_rank, cudaStream_t stream) {
  EpShape s{T, K, world, rank, per_rank};
  if (!ep_shape_ok(s) || (H & 7)) return -kErrBadArgument;
  ep_sum_kernel<<<ep_grid(T, 256), 256, 0, stream>>>(static_cast<const uint4*>(back), H / 8,
                                                     static_cast<const float*>(back_w),
                                                     static_cast<const long long*>(ids), static_cast<uint4*>(out),
                                                     static_cast<float*>(gw), s);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
