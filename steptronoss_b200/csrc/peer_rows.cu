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
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 0;; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys_u32(f) - epoch) >= 0) return;
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
