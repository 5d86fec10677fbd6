// Copy kernels that measure what one GPU can move to or from a peer's memory over NVLink with the
// access patterns the fused kernels of this library use (benchmarks/benchmark_peer_bandwidth.py):
//
//   mode 0  push, plain stores : 16-byte loads from local memory, 16-byte stores into the peer's buffer
//   mode 1  push, bulk copies  : cp.async.bulk local -> shared memory ring -> cp.async.bulk into the peer
//   mode 2  pull, plain loads  : 16-byte loads from the peer, 16-byte stores to local memory
//   mode 3  pull, bulk copies  : cp.async.bulk peer -> shared memory ring -> cp.async.bulk to local memory
//
// The reference probes its NCCL all-reduce bandwidth at start-up (steptronoss/utils/utils.py:377-433);
// this is the same kind of probe for the peer-memory paths.  No load uses cluster broadcast.
#include "common.cuh"

namespace stb {

constexpr int kBwStages = 4;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}

// src -> dst, `bytes` a multiple of 16; grid-stride over 16-byte words with `U` loads in flight per thread.
__global__ void __launch_bounds__(256) peer_copy_plain_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                              long long n16) {
  constexpr int U = 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long base = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; base < n16; base += stride * U) {
    uint4 v[U];
#pragma unroll
    for (int q = 0; q < U; ++q) {
      const long long i = base + q * stride;
      if (i < n16) v[q] = src[i];
    }
#pragma unroll
    for (int q = 0; q < U; ++q) {
      const long long i = base + q * stride;
      if (i < n16) dst[i] = v[q];
    }
  }
}

// One thread per CTA drives a ring of kBwStages chunks: bulk load into shared memory, bulk store out of it.
__global__ void __launch_bounds__(32) peer_copy_bulk_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                            long long bytes, int chunk, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kBwStages) * chunk);
  if (threadIdx.x == 0) {
    for (int i = 0; i < kBwStages; ++i) mbar_init(&bars[i], 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const long long num_chunks = (bytes + chunk - 1) / chunk;
  // prologue: fill the ring
  long long next = blockIdx.x;
  uint32_t issued = 0;
  for (; issued < kBwStages && next < num_chunks; ++issued, next += gridDim.x) {
    const long long off = next * chunk;
    const uint32_t len = static_cast<uint32_t>(min(static_cast<long long>(chunk), bytes - off));
    mbar_arrive_expect_tx(&bars[issued], len);
    bulk_load(smem + static_cast<size_t>(issued) * chunk, src + off, len, &bars[issued]);
  }
  uint32_t done = 0;
  for (long long c = blockIdx.x; c < num_chunks; c += gridDim.x, ++done) {
    const int st = done % kBwStages;
    if (!mbar_wait(&bars[st], (done / kBwStages) & 1)) {
      report_error(status, kErrProducerWait);
      break;
    }
    const long long off = c * chunk;
    const uint32_t len = static_cast<uint32_t>(min(static_cast<long long>(chunk), bytes - off));
    fence_proxy_async_smem();
    bulk_store(dst + off, smem + static_cast<size_t>(st) * chunk, len);
    tma_store_commit();
    if (next < num_chunks) {
      // the stage is refilled once the store issued from it has read shared memory
      tma_store_wait_read<0>();
      const long long noff = next * chunk;
      const uint32_t nlen = static_cast<uint32_t>(min(static_cast<long long>(chunk), bytes - noff));
      mbar_arrive_expect_tx(&bars[st], nlen);
      bulk_load(smem + static_cast<size_t>(st) * chunk, src + noff, nlen, &bars[st]);
      next += gridDim.x;
    }
  }
  tma_store_wait<0>();
}


// The same ring with the extras of the fused GEMM+collective kernels switched on one by one (`feat` bits):
//   1  every chunk is also stored to a second, local destination (the own copy of gathered rows)
//   2  every 8th chunk: wait until all but the newest 6 store groups have completed, fence, write a flag word
//      at `flag` (peer memory) - the per-part completion signal
//   4  five more warps of the CTA spin on an mbarrier that is only released at the end (the idle MMA and
//      epilogue warps of a comm CTA)
//   8  the ring is driven by the non-blocking state machine of the fused kernels (try_wait + nanosleep)
template <int STAGES>
__global__ void __launch_bounds__(192) peer_copy_ring_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                             uint8_t* __restrict__ dst2, uint32_t* flag, long long bytes,
                                                             int chunk, int feat, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(STAGES) * chunk);
  uint64_t* park = bars + STAGES;
  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) mbar_init(&bars[i], 1);
    mbar_init(park, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x >= 32) {
    if ((feat & 4) && (threadIdx.x & 31) == 0) mbar_wait(park, 0);   // bounded: 2 s
    return;
  }
  if (threadIdx.x != 0) return;
  const long long num_chunks = (bytes + chunk - 1) / chunk;
  auto issue = [&](long long c, int st) {
    const long long off = c * chunk;
    const uint32_t len = static_cast<uint32_t>(min(static_cast<long long>(chunk), bytes - off));
    mbar_arrive_expect_tx(&bars[st], len);
    bulk_load(smem + static_cast<size_t>(st) * chunk, src + off, len, &bars[st]);
  };
  auto store = [&](long long c, int st, uint32_t n) {
    const long long off = c * chunk;
    const uint32_t len = static_cast<uint32_t>(min(static_cast<long long>(chunk), bytes - off));
    fence_proxy_async_smem();
    bulk_store(dst + off, smem + static_cast<size_t>(st) * chunk, len);
    if (feat & 1) bulk_store(dst2 + off, smem + static_cast<size_t>(st) * chunk, len);
    tma_store_commit();
    if ((feat & 2) && (n & 7u) == 7u) {
      tma_store_wait<6>();
      asm volatile("fence.proxy.async.global;" ::: "memory");
      __threadfence_system();
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(flag + blockIdx.x), "r"(n) : "memory");
    }
    tma_store_wait_read<0>();
  };
  long long next = blockIdx.x;
  uint32_t filled = 0, stored = 0;
  if (!(feat & 8)) {
    for (; filled < STAGES && next < num_chunks; ++filled, next += gridDim.x) issue(next, filled);
    for (long long c = blockIdx.x; c < num_chunks; c += gridDim.x, ++stored) {
      const int st = stored % STAGES;
      if (!mbar_wait(&bars[st], (stored / STAGES) & 1)) {
        report_error(status, kErrProducerWait);
        break;
      }
      store(c, st, stored);
      if (next < num_chunks) {
        issue(next, st);
        next += gridDim.x;
      }
    }
  } else {
    long long c_store = blockIdx.x;
    uint32_t idle = 0;
    for (;;) {
      bool progress = false;
      if (next < num_chunks && filled - stored < static_cast<uint32_t>(STAGES)) {
        issue(next, filled % STAGES);
        next += gridDim.x;
        ++filled;
        progress = true;
      }
      if (stored < filled && mbar_try_wait(&bars[stored % STAGES], (stored / STAGES) & 1)) {
        store(c_store, stored % STAGES, stored);
        c_store += gridDim.x;
        ++stored;
        progress = true;
      }
      if (next >= num_chunks && stored == filled) break;
      if (progress) idle = 0;
      else {
        if (++idle > (1u << 24)) {
          report_error(status, kErrProducerWait);
          break;
        }
        __nanosleep(32);
      }
    }
  }
  tma_store_wait<0>();
  mbar_arrive(park);
}

}  // namespace stb

using namespace stb;

// Copies `bytes` (multiple of 16) from src to dst with `grid` CTAs; either pointer may be peer memory.
//   bulk = 0: 256 threads per CTA, 16-byte loads and stores;  bulk = 1: shared-memory ring of `chunk`-byte bulk copies
//   (chunk a multiple of 128, at most 48 KB).
extern "C" int stb_peer_copy(const void* src, void* dst, long long bytes, int grid, int bulk, int chunk, int* status,
                             cudaStream_t stream) {
  if (bytes <= 0 || (bytes & 15) || grid <= 0) return -kErrBadArgument;
  if (!bulk) {
    peer_copy_plain_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), bytes / 16);
  } else {
    if (chunk < 128 || (chunk & 127) || chunk > 48 * 1024) return -kErrBadArgument;
    const int smem = kBwStages * chunk + 256;
    cudaError_t e = cudaFuncSetAttribute(peer_copy_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return -static_cast<int>(e);
    peer_copy_bulk_kernel<<<grid, 32, smem, stream>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), bytes,
                                                      chunk, status);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

// Ring variants (see peer_copy_ring_kernel): dst2 = local scratch of `bytes`, flag = grid words of peer memory.
extern "C" int stb_peer_copy_ring(const void* src, void* dst, void* dst2, void* flag, long long bytes, int grid,
                                  int chunk, int stages, int feat, int* status, cudaStream_t stream) {
  if (bytes <= 0 || (bytes & 15) || grid <= 0 || chunk < 128 || (chunk & 127)) return -kErrBadArgument;
  if (stages != 4 && stages != 6) return -kErrBadArgument;
  const int smem = stages * chunk + 256 + 1024;
  auto kern = stages == 4 ? peer_copy_ring_kernel<4> : peer_copy_ring_kernel<6>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return -static_cast<int>(e);
  kern<<<grid, 192, smem, stream>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst),
                                    static_cast<uint8_t*>(dst2), static_cast<uint32_t*>(flag), bytes, chunk, feat, status);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
