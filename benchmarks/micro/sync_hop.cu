// Micro-benchmark: latency of one synchronisation "hop" between a single issuing thread and 128 worker threads.
#include "common.cuh"
#include <cstdio>
using namespace stb;

// mode 0: A signalled by tcgen05.commit (no MMA outstanding), B by 128 software arrives
// mode 1: A signalled by software arrive of the issuing thread
// extra_pollers: additional warps that spin on a third barrier that never completes (until the end)
__global__ void __launch_bounds__(320, 1) hop_kernel(int iters, int mode, int extra, long long* out) {
  __shared__ __align__(8) uint64_t bars[4];
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);     // A: issuer -> workers
    mbar_init(&bars[1], 128);   // B: workers -> issuer
    mbar_init(&bars[2], 1);     // never completes until the end
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, 32); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  long long t0 = clock64();
  long long fails = 0, done = 0;
  if (warp == 1) {
    if (lane == 0) {
      for (int j = 0; j < iters; ++j) {
        if (mode == 0) umma_commit(&bars[0]); else mbar_arrive(&bars[0]);
        if (!mbar_wait(&bars[1], j & 1)) fails++;
        tc_fence_after();
        done++;
      }
      mbar_arrive(&bars[2]);
      if (blockIdx.x == 0) { out[1] = fails; out[2] = done; out[3] = clock64() - t0; }
    }
  } else if (warp >= 2 && warp < 6) {
    for (int j = 0; j < iters; ++j) {
      mbar_wait(&bars[0], j & 1);
      tc_fence_after();
      tc_fence_before();
      mbar_arrive(&bars[1]);
    }
  } else if (warp >= 6 && warp < 6 + extra) {
    mbar_wait(&bars[2], 0);
  }
  __syncthreads();
  long long t1 = clock64();
  if (threadIdx.x == 0 && blockIdx.x == 0) out[0] = t1 - t0;
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_slot, 32); }
}

int main() {
  long long* d; cudaMalloc(&d, 32);
  const int iters = 2000;
  for (int mode = 0; mode < 2; ++mode)
    for (int extra = 0; extra <= 4; extra += 4) {
      cudaMemset(d, 0, 32);
      for (int rep = 0; rep < 2; ++rep) hop_kernel<<<148, 320>>>(iters, mode, extra, d);
      cudaError_t le = cudaGetLastError();
      if (le != cudaSuccess) printf("launch error: %s\n", cudaGetErrorString(le));
      cudaError_t e = cudaDeviceSynchronize();
      long long hh[4] = {0, 0, 0, 0}; cudaMemcpy(hh, d, 32, cudaMemcpyDeviceToHost);
      printf("mode %d extra_pollers %d: total %lld clks, issuer loop %lld clks = %.1f per round trip; fails %lld done %lld err=%d\n", mode, extra, hh[0], hh[3], double(hh[3]) / iters, hh[1], hh[2], int(e));
    }
  return 0;
}
