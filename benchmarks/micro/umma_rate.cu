// Micro-benchmark: sustained rate of tcgen05.mma variants issued back to back by one thread (operands = whatever
// is in shared memory / TMEM; results are not checked).
#include "attention_common.cuh"
#include <cstdio>
using namespace stb;

constexpr int kSmem = 200 * 1024;

// mode 0: 128x128x16, A smem K-major, B smem K-major (Q K^T)
// mode 1: 128x128x16, A TMEM, B smem MN-major (P V)
// mode 2: alternate mode 0 and mode 1 instructions
// mode 3: 128x256x16, A smem, B smem (GEMM tile)
// mode 4: 128x64x16, A TMEM, B smem K-major
// mode 5: 128x128x16, A TMEM, B smem K-major (Q from TMEM)
template <int mode, int issuers>
__global__ void __launch_bounds__(128, 1) mma_kernel(int groups, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t bar;
  __shared__ __align__(8) uint64_t bar2;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (kSmem - 2048) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(&bar, issuers); mbar_init(&bar2, 1 << 20); fence_barrier_init(); }
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (warp >= 1 && warp < 1 + issuers && lane == 0) {
    const uint32_t sA = smem_u32(smem), sB = smem_u32(smem + 65536);
    const uint32_t tm = tmem_slot + (warp - 1) * 128;
    constexpr uint32_t id_kk = umma_idesc_bf16(128, 128, 0, 0), id_kmn = umma_idesc_bf16(128, 128, 0, 1);
    constexpr uint32_t id_256 = umma_idesc_bf16(128, 256, 0, 0), id_64 = umma_idesc_bf16(128, 64, 0, 0);
    const long long t0 = clock64();
    if (mode == 6) {
      volatile int* stage_src = reinterpret_cast<volatile int*>(smem + 190 * 1024);
      for (int g = 0; g < groups; ++g) {
        const int st = (g + *stage_src) & 1;    // runtime stage, like the ring of the attention kernels
        mma_128x128x128<false, false>(tm, sA, sB + st * 32768, false);
        umma_commit(&bar2);
      }
    } else if (mode == 7) {
      volatile int* stage_src = reinterpret_cast<volatile int*>(smem + 190 * 1024);
      for (int g = 0; g < groups; ++g) {
        const int st = (g + *stage_src) & 1;
        mma_128x128x128<false, true>(tm, sA, sB + st * 32768, g > 0);
        umma_commit(&bar2);
      }
    } else
    for (int g = 0; g < groups; ++g) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint64_t da = umma_smem_desc(sA + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
        const uint64_t dbk = umma_smem_desc(sB + (g & 1) * 32768 + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
        const uint64_t dbmn = umma_smem_desc(sB + (g & 1) * 32768 + k * 2048, 16384, 1024);
        if (mode == 0) umma_bf16(tm, da, dbk, id_kk, k > 0);
        else if (mode == 1) umma_bf16_a_tmem(tm + 256, tmem + k * 8, dbmn, id_kmn, 1);
        else if (mode == 2) { umma_bf16(tmem, da, dbk, id_kk, k > 0); umma_bf16_a_tmem(tmem + 256, tmem + 128 + k * 8, dbmn, id_kmn, 1); }
        else if (mode == 3) umma_bf16(tmem, da, dbk, id_256, k > 0);
        else if (mode == 4) umma_bf16_a_tmem(tmem, tmem + 384 + k * 8, dbk, id_64, k > 0);
        else if (mode == 8) umma_bf16(tm, da, dbk, id_64, k > 0);
        else umma_bf16_a_tmem(tmem, tmem + 384 + k * 8, dbk, id_kk, k > 0);
      }
    }
    const long long t_issue = clock64();
    umma_commit(&bar);
    mbar_wait(&bar, 0);
    const long long t1 = clock64();
    if (blockIdx.x == 0 && warp == 1) { out[0] = t1 - t0; out[1] = t_issue - t0; }
  }
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

template <int mode, int issuers>
void run(const char* name, double flop, long long* d) {
  cudaFuncSetAttribute(mma_kernel<mode, issuers>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  const int groups = 512;
  long long h[2] = {0, 0};
  for (int rep = 0; rep < 2; ++rep) {
    cudaMemset(d, 0, 16);
    mma_kernel<mode, issuers><<<148, 128, kSmem>>>(groups, d);
    cudaError_t le = cudaGetLastError();
    cudaError_t e = cudaDeviceSynchronize();
    if (le != cudaSuccess || e != cudaSuccess) printf("error %s / %s\n", cudaGetErrorString(le), cudaGetErrorString(e));
    cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
  }
  const double per = double(h[0]) / (groups * 8);
  printf("mode %d issuers %d (%s): %.1f clks per step per issuer (issue loop alone %.1f), %.0f FLOP/clk/SM of 8192\n", mode, issuers, name, per,
         double(h[1]) / (groups * 8), issuers * flop / per);
}

int main() {
  long long* d; cudaMalloc(&d, 16);
  run<0, 1>("128x128x16 A smem B smem", 128. * 128 * 16 * 2, d);
  run<0, 2>("128x128x16 A smem B smem", 128. * 128 * 16 * 2, d);
  run<1, 1>("128x128x16 A tmem B smem(MN)", 128. * 128 * 16 * 2, d);
  run<1, 2>("128x128x16 A tmem B smem(MN)", 128. * 128 * 16 * 2, d);
  run<2, 1>("alternate", 2 * 128. * 128 * 16 * 2, d);
  run<3, 1>("128x256x16 A smem B smem", 128. * 256 * 16 * 2, d);
  run<5, 1>("128x128x16 A tmem B smem(K)", 128. * 128 * 16 * 2, d);
  run<8, 1>("128x64x16 A smem B smem", 128. * 64 * 16 * 2, d);
  run<4, 1>("128x64x16 A tmem B smem", 128. * 64 * 16 * 2, d);
  run<6, 1>("attention helper QK, runtime stage, commit per tile", 128. * 128 * 16 * 2, d);
  run<7, 1>("attention helper PV (B MN-major), runtime stage", 128. * 128 * 16 * 2, d);
  return 0;
}
