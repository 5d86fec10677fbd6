// Block-scaled fp8 (e4m3) GEMM for sm_100a, dense and grouped by row tiles (expert-major MoE activations):
//
//     Y[r, n] = sum over 128-wide k blocks kb of  sx[r, kb] * sw[g, n / 128, kb] * (Xq[r, kb] . Wq[g, n, kb])
//
// Xq [M, K] e4m3 with one fp32 scale per row and 128 columns ("1 x 128"), Wq [G, N, K] e4m3 with one fp32 scale per
// 128 x 128 block, Y bf16.  The reference has this recipe only as an unused Triton path (its grouped GEMM back-ends
// are bf16: steptronoss/model/utils/moe_utils.py:423-453); the shapes are those of DeepSeek-style block scaling.
//
// The tensor pipe cannot apply fp32 scales that change every 128 k, so the sum is split the classic way: per k block
// four tcgen05.mma.kind::f8f6f4 steps (K = 32 each) produce an unscaled 128 x 128 partial product in one of four
// TMEM buffers; eight promotion warps read the partial, multiply it by the two scales and add it to fp32
// accumulators that they keep in registers (64 columns of one row per thread), while the tensor pipe fills the
// other buffers (TMEM loads are slow while the tensor pipe is busy, so the ring is four deep).  After the last k block the same warps convert to bf16 and store their rows.
//
//   warp 0      TMA producer: A and B tiles of 128 rows x 128 bytes (one swizzle span = one k block), 6-stage ring
//   warp 1      MMA issuer
//   warps 2..9  promotion + epilogue: warp w owns TMEM lanes 32 * (w % 4) and columns 64 * ((w - 2) / 4)
#include "common.cuh"

#include <cuda_fp8.h>

namespace stb {

constexpr int kF8BlockM = 128, kF8BlockN = 128, kF8BlockK = 128;
constexpr int kF8Stages = 6;
constexpr int kF8Parts = 4;                              // partial-product buffers in TMEM (4 x 128 columns)
constexpr int kF8TileBytes = 128 * 128;                 // one operand tile: 128 rows of 128 bytes
constexpr int kF8StageBytes = 2 * kF8TileBytes;
constexpr int kF8Threads = 320;
constexpr int kF8Smem = kF8Stages * kF8StageBytes + 256 + 1024;

struct Fp8GemmParams {
  int M, N, K;
  long long ldc;
  const int* tile_group;     // [ceil(M/128)] group of each row tile, -1 = skip; nullptr = dense (group 0)
  const float* sx;           // [M][K/128]
  const float* sw;           // [G][N/128][K/128]
  __nv_bfloat16* C;
  int* status;
};

// Instruction descriptor of kind::f8f6f4 with e4m3 inputs (format 0), fp32 accumulation, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// 4 steps of K = 32 over one 128-byte swizzle span; the first step overwrites the accumulator.
__device__ __forceinline__ void umma4_e4m3(uint32_t d, uint64_t a0, uint64_t b0, uint32_t idesc) {
  const uint64_t a1 = umma_desc_advance(a0, 32), a2 = umma_desc_advance(a0, 64), a3 = umma_desc_advance(a0, 96);
  const uint64_t b1 = umma_desc_advance(b0, 32), b2 = umma_desc_advance(b0, 64), b3 = umma_desc_advance(b0, 96);
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, 0, 0;\n\t"
      "setp.eq.b32 q, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %5, %9, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %2, %6, %9, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %3, %7, %9, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %4, %8, %9, q;\n\t}"
      ::"r"(d), "l"(a0), "l"(a1), "l"(a2), "l"(a3), "l"(b0), "l"(b1), "l"(b2), "l"(b3), "r"(idesc)
      : "memory");
}

__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const Fp8GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kF8Stages * kF8StageBytes);
  uint64_t* empty_bar = full_bar + kF8Stages;
  uint64_t* part_full = empty_bar + kF8Stages;     // [kF8Parts] partial product of a k block is in TMEM
  uint64_t* part_empty = part_full + kF8Parts;     // the promotion warps have read it (8 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part_empty + kF8Parts);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + kF8BlockM - 1) / kF8BlockM;
  const int num_n = p.N / kF8BlockN;
  const int num_tiles = num_m * num_n;
  const int k_blocks = p.K / kF8BlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kF8Stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < kF8Parts; ++a) {
      mbar_init(&part_full[a], 1);
      mbar_init(&part_empty[a], 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kF8Parts * kF8BlockN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile order: all n tiles of a row tile one after the other, so that the A rows stay in L2
  auto tile_coord = [&](int tile, int& m_tile, int& n_tile, int& group) {
    m_tile = tile / num_n;
    n_tile = tile - m_tile * num_n;
    group = p.tile_group != nullptr ? p.tile_group[m_tile] : 0;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
        int m_tile, n_tile, group;
        tile_coord(tile, m_tile, n_tile, group);
        if (group < 0) continue;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kF8Stages;
          if (!mbar_wait(&empty_bar[s], ((it / kF8Stages) & 1) ^ 1)) {
            report_error(p.status, kErrProducerWait);
            *abort_flag = 1;
            break;
          }
          uint8_t* sa = smem + s * kF8StageBytes;
          mbar_arrive_expect_tx(&full_bar[s], kF8StageBytes);
          tma_load_2d(sa, &tmap_a, &full_bar[s], kb * kF8BlockK, m_tile * kF8BlockM);
          tma_load_2d(sa + kF8TileBytes, &tmap_b, &full_bar[s], kb * kF8BlockK, group * p.N + n_tile * kF8BlockN);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_e4m3(kF8BlockM, kF8BlockN);
      uint32_t it = 0;      // k blocks issued so far = ring position = partial-buffer sequence number
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok && !*abort_flag; tile += gridDim.x) {
        int m_tile, n_tile, group;
        tile_coord(tile, m_tile, n_tile, group);
        if (group < 0) continue;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kF8Stages, buf = it % kF8Parts;
          ok = mbar_wait(&part_empty[buf], ((it / kF8Parts) & 1) ^ 1);
          if (ok) ok = mbar_wait(&full_bar[s], (it / kF8Stages) & 1);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kF8StageBytes);
          umma4_e4m3(tmem_base + buf * kF8BlockN, umma_smem_desc(sa, 16, 1024),
                     umma_smem_desc(sa + kF8TileBytes, 16, 1024), idesc);
          umma_commit(&empty_bar[s]);
          umma_commit(&part_full[buf]);
        }
      }
      if (!ok) { report_error(p.status, kErrMmaWaitFull); *abort_flag = 1; }
    }
  } else {
    const int quarter = warp & 3;                 // TMEM lanes [32 * quarter, +32)
    const int half = (warp - 2) >> 2;             // columns [64 * half, +64) of the tile
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int kbs = k_blocks;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_tile, n_tile, group;
      tile_coord(tile, m_tile, n_tile, group);
      if (group < 0) continue;
      const int row = m_tile * kF8BlockM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const float* sx_row = p.sx + static_cast<long long>(row_ok ? row : 0) * kbs;
      const float* sw_blk = p.sw + (static_cast<long long>(group) * num_n + n_tile) * kbs;
      float acc[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = 0.f;
      for (int kb = 0; kb < kbs; ++kb, ++it) {
        const int buf = it % kF8Parts;
        const float scale = __ldg(sx_row + kb) * __ldg(sw_blk + kb);   // issued before the wait
        if (*abort_flag) ok = false;
        if (ok) ok = mbar_wait(&part_full[buf], (it / kF8Parts) & 1);
        ok = __all_sync(0xffffffffu, ok);         // the TMEM loads below are warp-wide
        if (!ok) break;
        tc_fence_after();
        uint32_t v[64];
        {
          uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&v[0]);
          uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&v[32]);
          tmem_ld_32x32(tmem_base + lane_addr + buf * kF8BlockN + half * 64, lo);
          tmem_ld_32x32(tmem_base + lane_addr + buf * kF8BlockN + half * 64 + 32, hi);
        }
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&part_empty[buf]);   // the tensor pipe may overwrite the buffer
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] = fmaf(__uint_as_float(v[i]), scale, acc[i]);
      }
      if (!ok) break;
      if (row_ok) {
        __nv_bfloat16* crow = p.C + static_cast<long long>(row) * p.ldc + n_tile * kF8BlockN + half * 64;
#pragma unroll
        for (int j = 0; j < 64; j += 8) {
          uint4 o;
          o.x = pack_bf16(acc[j], acc[j + 1]); o.y = pack_bf16(acc[j + 2], acc[j + 3]);
          o.z = pack_bf16(acc[j + 4], acc[j + 5]); o.w = pack_bf16(acc[j + 6], acc[j + 7]);
          *reinterpret_cast<uint4*>(crow + j) = o;
        }
      }
    }
    if (!ok) { report_error(p.status, kErrEpilogueWait); *abort_flag = 1; }
  }

  __syncthreads();
  if (*abort_flag) drain_delay();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kF8Parts * kF8BlockN);
  }
}

// ------------------------------------------------------------------------------------------------ quantisation
__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

// One warp per (row, 128-column block): scale = amax / 448, q = x / scale.
__global__ void __launch_bounds__(256)
quant_rows_1x128_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                        float* __restrict__ sx, long long rows, int kbs) {
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= rows * kbs) return;
  const long long r = wid / kbs;
  const int kb = static_cast<int>(wid % kbs);
  const uint2 raw = *reinterpret_cast<const uint2*>(x + r * ldx + kb * 128 + lane * 4);
  float f[4] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y)};
  float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = amax > 0.f ? amax * (1.f / 448.f) : 1.f;
  const float inv = 1.f / scale;
  const uint32_t packed = to_e4m3(f[0] * inv) | (to_e4m3(f[1] * inv) << 8) | (to_e4m3(f[2] * inv) << 16) |
                          (static_cast<uint32_t>(to_e4m3(f[3] * inv)) << 24);
  *reinterpret_cast<uint32_t*>(q + r * ldq + kb * 128 + lane * 4) = packed;
  if (lane == 0) sx[r * kbs + kb] = scale;
}

// One CTA of 256 threads per 128 x 128 block of a row-major matrix [R][K]: a thread handles half a row.
__global__ void __launch_bounds__(256)
quant_blocks_128x128_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, uint8_t* __restrict__ q, long long ldq,
                            float* __restrict__ sw, int kbs) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const int rb = blockIdx.y, kb = blockIdx.x;
  const int row = threadIdx.x >> 1, part = threadIdx.x & 1;
  const __nv_bfloat16* src = w + (static_cast<long long>(rb) * 128 + row) * ldw + kb * 128 + part * 64;
  uint4 raw[8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    raw[i] = *reinterpret_cast<const uint4*>(src + i * 8);
    const uint32_t u[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(u[j])), fabsf(bf16_hi(u[j]))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    const float scale = m > 0.f ? m * (1.f / 448.f) : 1.f;
    s_scale = scale;
    sw[static_cast<long long>(rb) * kbs + kb] = scale;
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
  uint8_t* dst = q + (static_cast<long long>(rb) * 128 + row) * ldq + kb * 128 + part * 64;
#pragma unroll
  for (int i = 0; i < 8; i += 2) {   // 16 values -> 16 bytes
    uint32_t out[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t u[4] = {raw[i + h].x, raw[i + h].y, raw[i + h].z, raw[i + h].w};
      out[h * 2] = to_e4m3(bf16_lo(u[0]) * inv) | (to_e4m3(bf16_hi(u[0]) * inv) << 8) |
                   (to_e4m3(bf16_lo(u[1]) * inv) << 16) | (static_cast<uint32_t>(to_e4m3(bf16_hi(u[1]) * inv)) << 24);
      out[h * 2 + 1] = to_e4m3(bf16_lo(u[2]) * inv) | (to_e4m3(bf16_hi(u[2]) * inv) << 8) |
                       (to_e4m3(bf16_lo(u[3]) * inv) << 16) | (static_cast<uint32_t>(to_e4m3(bf16_hi(u[3]) * inv)) << 24);
    }
    *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

}  // namespace stb

using namespace stb;

// xq [M][K] e4m3 (row stride lda bytes), sx [M][K/128]; wq [G*N][K] e4m3 (row stride ldb bytes), sw [G][N/128][K/128];
// C [M][N] bf16 (row stride ldc elements).  tile_group: group of every 128-row tile (-1 = skip) or null for G = 1.
extern "C" int stb_gemm_fp8_block_scaled(const void* xq, const float* sx, const void* wq, const float* sw, void* C,
                                         const int* tile_group, int M, int N, int K, int num_groups, long long lda,
                                         long long ldb, long long ldc, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % kF8BlockK) || (N % kF8BlockN) || (lda & 15) || (ldb & 15) || (ldc & 7) || num_groups < 1)
    return -kErrBadArgument;
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, xq, 1, K, M, static_cast<uint64_t>(lda), kF8BlockK, kF8BlockM, 1);
  if (r) return r;
  r = make_tmap_2d(&tb, wq, 1, K, static_cast<uint64_t>(N) * num_groups, static_cast<uint64_t>(ldb), kF8BlockK,
                   kF8BlockN, 1);
  if (r) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kF8Smem);
    if (e != cudaSuccess) return -static_cast<int>(e);
    configured = true;
  }
  Fp8GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.tile_group = tile_group; p.sx = sx; p.sw = sw;
  p.C = static_cast<__nv_bfloat16*>(C); p.status = status;
  const int tiles = ((M + kF8BlockM - 1) / kF8BlockM) * (N / kF8BlockN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_fp8_kernel<<<grid, kF8Threads, kF8Smem, stream>>>(ta, tb, p);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_quant_rows_1x128(const void* x, long long ldx, void* q, long long ldq, float* sx, long long rows,
                                    int K, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K <= 0 || (K % 128) || (ldx & 3) || (ldq & 3)) return -kErrBadArgument;
  const long long warps = rows * (K / 128);
  const long long blocks = (warps * 32 + 255) / 256;
  quant_rows_1x128_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq, sx, rows, K / 128);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_quant_blocks_128x128(const void* w, long long ldw, void* q, long long ldq, float* sw, long long rows,
                                        int K, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K <= 0 || (K % 128) || (rows % 128) || (ldw & 7) || (ldq & 15)) return -kErrBadArgument;
  quant_blocks_128x128_kernel<<<dim3(K / 128, static_cast<unsigned>(rows / 128)), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(w), ldw, static_cast<uint8_t*>(q), ldq, sw, K / 128);
  return -static_cast<int>(cudaGetLastError());
}
