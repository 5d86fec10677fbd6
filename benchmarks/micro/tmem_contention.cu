// Does tcgen05.ld / tcgen05.st traffic from other warps slow down a chain of tcgen05.mma?
#include "attention_common.cuh"
#include <cstdio>
using namespace stb;
constexpr int kSmem = 200 * 1024;

// load_mode 0: no concurrent TMEM traffic; 1: four warps load 128 columns per round; 2: load 128 + store 64 columns
template <int load_mode>
__global__ void __launch_bounds__(192, 1) k(int groups, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int done;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (kSmem - 2048) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_barrier_init(); done = 0; }
  if (warp == 4) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (warp == 4) {
    if (lane == 0) {
      const uint32_t sA = smem_u32(smem), sB = smem_u32(smem + 65536);
      const long long t0 = clock64();
      for (int g = 0; g < groups; ++g) {
        mma_128x128x128<false, false>(tmem, sA, sB + (g & 1) * 32768, false);            // S = Q K^T
        mma_128x128x128_ta<true>(tmem + 256, tmem + 128, sB + (g & 1) * 32768, g > 0);   // O += P V
      }
      umma_commit(&bar);
      mbar_wait(&bar, 0);
      const long long t1 = clock64();
      if (blockIdx.x == 0) out[0] = t1 - t0;
      done = 1;
    }
  } else if (warp < 4 && load_mode > 0) {
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    long long rounds = 0;
    uint32_t sink = 0;
    while (!done) {
      uint32_t v[32];
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld_32x32(tmem + lane_addr + 384 + c * 32, v);
        tmem_wait_ld();
        sink ^= v[lane & 31];
      }
      if (load_mode > 1) {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) tmem_st_32x32(tmem + lane_addr + 384 + c * 32, v);
        tmem_wait_st();
      }
      ++rounds;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) { out[1] = rounds; out[2] = sink; }
  }
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

template <int load_mode>
void run(long long* d) {
  cudaFuncSetAttribute(k<load_mode>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  const int groups = 512;
  long long h[3] = {0, 0, 0};
  for (int rep = 0; rep < 2; ++rep) {
    cudaMemset(d, 0, 24);
    k<load_mode><<<148, 192, kSmem>>>(groups, d);
    cudaError_t le = cudaGetLastError();
    cudaError_t e = cudaDeviceSynchronize();
    if (le != cudaSuccess || e != cudaSuccess) printf("error %s / %s\n", cudaGetErrorString(le), cudaGetErrorString(e));
    cudaMemcpy(h, d, 24, cudaMemcpyDeviceToHost);
  }
  printf("load_mode %d: %.1f clks per MMA step (16 steps per tile); loader rounds per tile %.2f\n", load_mode,
         double(h[0]) / (groups * 16), double(h[1]) / groups);
}

int main() {
  long long* d; cudaMalloc(&d, 24);
  run<0>(d); run<1>(d); run<2>(d);
  return 0;
}
