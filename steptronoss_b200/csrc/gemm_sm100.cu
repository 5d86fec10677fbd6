// bf16 GEMM for sm_100a: persistent, warp-specialised, TMA-fed, tcgen05.mma with fp32
// accumulators double-buffered in TMEM.
//
//   C[M,N] (=|+=) A[M,K] * B[N,K]^T          operands may each be K-major or MN-major in memory
//
// which covers the three products of a linear layer without any transposed copy:
//   forward  y  = x  * W^T : A = x  (K-major),            B = W (K-major)
//   dgrad    dx = dy * W   : A = dy (K-major),            B = W  stored [K_red][N_out] -> MN-major
//   wgrad    dW = dy^T * x : A = dy stored [K_red][M_out] -> MN-major, B = x stored [K_red][N_out] -> MN-major
// The wgrad form accumulates straight into an fp32 gradient buffer (beta = 1), the role that
// apex's wgrad_gemm_accum_fp32 plays for the reference (steptronoss/core/tensor_parallel/layers.py:244-249).
//
// Grouped (mixture-of-experts) variants share the kernel:
//   mode 1 "grouped rows": A/C rows are expert-major segments aligned to 128 rows; tile_group[m_tile]
//          selects which expert's B matrix a row tile multiplies (fwd and dgrad of expert FFNs);
//   mode 2 "grouped reduction": per expert g, C[g] (+)= A[rows_g]^T B[rows_g] with the reduction
//          running over that expert's row segment (expert wgrad).
// These replace the reference's Triton grouped GEMM and its python-loop backward
// (steptronoss/model/optimizations/grouped_gemm/triton.py:45-316).
//
// CTA layout (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (+TMEM owner),
// warps 2..5 = epilogue (each owns the 32 TMEM lanes of its warp-id mod 4).
#include "common.cuh"

#include <cstdlib>

namespace stb {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;   // 64 bf16 = 128 B = one swizzle span
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;

struct GemmParams {
  int M, N, K;
  int ldc;
  int mode;              // 0 dense, 1 grouped rows, 2 grouped reduction
  int num_groups;        // modes 1,2
  int group_n_stride;    // mode 1: B row (K-major) or k (MN-major) offset per group
  const int* tile_group; // mode 1: [ceil(M/128)] group id per row tile, -1 = skip tile
  const int* group_offsets;  // mode 2: [num_groups+1] row offsets (multiples of 64)
  long long group_c_stride;  // mode 2: elements between consecutive groups' C
  int* status;
  float alpha;
  // dense mode, bf16 output written by TMA: C = alpha * A B^T + beta * addend (addend may be C itself)
  const __nv_bfloat16* addend;
  long long ld_add;
  float beta;
  // dense mode with a symmetric result (X X^T, A^2 of a symmetric A): tiles that lie entirely below the diagonal
  // are not computed; the caller mirrors the upper triangle afterwards
  int upper_only;
  // dense mode with fp32 reduce-add output (weight gradients): the reduction extent is cut into k_splits parts that
  // different CTAs add into C, so that a product with few output tiles still fills whole waves of the grid
  int k_splits;
};

template <int BLOCK_N>
struct GemmSmem {
  static constexpr int kStages = (BLOCK_N == 256) ? 4 : 5;
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BLOCK_N * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kStoreBytes = 4 * 2 * 4096;  // per epilogue warp: two 32-row x 128-byte staging tiles
  static constexpr int kTotal = kStages * kStageBytes + kStoreBytes + kBarrierBytes + 1024;  // + alignment slack
};

struct TileCoord {
  int m_tile, n_tile, group, k_begin, k_blocks;
  bool valid;
};

// Tile order: row tiles are walked in bands of kBand so that the CTAs running at the same time
// share A and B tiles in L2.
__device__ __forceinline__ void decode_tile(const GemmParams& p, int tile, int num_m, int num_n, TileCoord& t,
                                            int block_n = 0) {
  constexpr int kBand = 8;
  if (p.upper_only && block_n > 0) {
    // compact enumeration of the tiles that reach the diagonal, row tile after row tile, so that the CTAs of the
    // persistent grid get equal shares of real work
    int rem = tile;
    t.m_tile = 0; t.n_tile = 0;
    for (int i = 0; i < num_m; ++i) {
      const int n_min = (i * kBlockM) / block_n;
      const int cnt = num_n - n_min;
      if (rem < cnt) { t.m_tile = i; t.n_tile = n_min + rem; break; }
      rem -= cnt;
    }
    t.k_begin = 0;
    t.k_blocks = (p.K + kBlockK - 1) / kBlockK;
    t.group = 0;
    t.valid = true;
    return;
  }
  if (p.mode == 2) {
    const int per_group = num_m * num_n;
    t.group = tile / per_group;
    const int r = tile - t.group * per_group;
    t.m_tile = r % num_m;
    t.n_tile = r / num_m;
    const int b = p.group_offsets[t.group], e = p.group_offsets[t.group + 1];
    t.k_begin = b;
    t.k_blocks = (e - b + kBlockK - 1) / kBlockK;
    t.valid = true;
    return;
  }
  int split = 0;
  if (p.k_splits > 1) {   // splits of one output tile are a whole pass over the tiles apart
    split = tile / (num_m * num_n);
    tile -= split * num_m * num_n;
  }
  const int in_band = kBand * num_n;
  const int band = tile / in_band;
  const int first_m = band * kBand;
  const int band_rows = min(num_m - first_m, kBand);
  const int r = tile - band * in_band;
  t.m_tile = first_m + r % band_rows;
  t.n_tile = r / band_rows;
  t.k_begin = 0;
  t.k_blocks = (p.K + kBlockK - 1) / kBlockK;
  if (p.k_splits > 1) {
    const int per = (t.k_blocks + p.k_splits - 1) / p.k_splits;
    t.k_begin = split * per * kBlockK;
    t.k_blocks = max(0, min(per, t.k_blocks - split * per));
  }
  t.group = 0;
  t.valid = true;
  if (p.mode == 1) {
    t.group = p.tile_group[t.m_tile];
    t.valid = t.group >= 0;
  }
}

// Number of 128 x block_n tiles of a square result that reach the diagonal or lie above it.
__host__ __device__ inline int upper_tile_count(int num_m, int num_n, int block_n) {
  int total = 0;
  for (int i = 0; i < num_m; ++i) total += num_n - (i * kBlockM) / block_n;
  return total;
}

template <int BLOCK_N, bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, void* __restrict__ Cptr, const GemmParams p) {
  using S = GemmSmem<BLOCK_N>;
  constexpr int kStages = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* store_stage = smem + kStages * S::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(store_stage + S::kStoreBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (p.M + kBlockM - 1) / kBlockM;
  const int num_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int num_tiles = p.upper_only ? upper_tile_count(num_m, num_n, BLOCK_N)
                                     : num_m * num_n * (p.mode == 2 ? p.num_groups : (p.k_splits > 1 ? p.k_splits : 1));

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BLOCK_N);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
        TileCoord t;
        decode_tile(p, tile, num_m, num_n, t, BLOCK_N);
        if (!t.valid) continue;
        const int m0 = t.m_tile * kBlockM;
        const int n0 = t.n_tile * BLOCK_N;
        for (int kb = 0; kb < t.k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
            report_error(p.status, kErrProducerWait);
            *abort_flag = 1;
            break;
          }
          uint8_t* sa = smem + s * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          mbar_arrive_expect_tx(&full_bar[s], S::kStageBytes);
          const int k0 = t.k_begin + kb * kBlockK;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmap_a, &full_bar[s], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j)
              tma_load_2d(sa + j * (kBlockK * 128), &tmap_a, &full_bar[s], m0 + j * 64, k0);
          }
          if constexpr (!B_MN) {
            const int brow = n0 + (p.mode == 1 ? t.group * p.group_n_stride : 0);
            tma_load_2d(sb, &tmap_b, &full_bar[s], k0, brow);
          } else {
            const int bk = k0 + (p.mode == 1 ? t.group * p.group_n_stride : 0);
#pragma unroll
            for (int j = 0; j < BLOCK_N / 64; ++j)
              tma_load_2d(sb + j * (kBlockK * 128), &tmap_b, &full_bar[s], n0 + j * 64, bk);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(kBlockM, BLOCK_N, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0, local_tile = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
        TileCoord t;
        decode_tile(p, tile, num_m, num_n, t, BLOCK_N);
        if (!t.valid) continue;
        const int acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1)) {
          report_error(p.status, kErrMmaWaitTmem);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        bool ok = true;
        for (int kb = 0; kb < t.k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&full_bar[s], ph)) {
            report_error(p.status, kErrMmaWaitFull);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            // K-major: step 32 B inside the 128 B swizzle span. MN-major: step 16 k-rows of 128 B.
            const uint64_t da = A_MN ? umma_smem_desc(sa + k * (kUmmaK * 128), kBlockK * 128, 1024)
                                     : umma_smem_desc(sa + k * (kUmmaK * 2), 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc(sb + k * (kUmmaK * 128), kBlockK * 128, 1024)
                                     : umma_smem_desc(sb + k * (kUmmaK * 2), 16, 1024);
            umma_bf16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
        }
        if (!ok) break;
        if (t.k_blocks == 0) {
          // empty reduction (an expert without rows): nothing was issued; the epilogue writes zeros
        }
        umma_commit(&tmem_full[acc]);
        ++local_tile;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    uint32_t local_tile = 0;
    uint32_t store_count = 0;
    for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
      TileCoord t;
      decode_tile(p, tile, num_m, num_n, t, BLOCK_N);
      if (!t.valid) continue;
      const int acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_ph)) {
        report_error(p.status, kErrEpilogueWait);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int n0 = t.n_tile * BLOCK_N;
      const bool zero_acc = (t.k_blocks == 0);
      // rows of this warp inside C (grouped reduction: every group owns M consecutive rows of the map)
      const int row0 = t.m_tile * kBlockM + quarter * 32 + (p.mode == 2 ? t.group * p.M : 0);
      constexpr bool kTmaStore = OUT_F32 || !ACCUM;  // bf16 read-modify-write keeps the direct path
      if constexpr (kTmaStore) {
        // Stage 32 rows x 128 bytes (32 fp32 or 64 bf16 columns) in shared memory with the 128-byte
        // swizzle, then one TMA store (or TMA fp32 reduce-add for beta = 1) per staged tile.  The TMA
        // unit clips rows and columns outside C, so there are no edge guards here.
        constexpr int kColsPerStore = OUT_F32 ? 32 : 64;
        uint8_t* my_stage = store_stage + (warp - 2) * 8192;
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / kColsPerStore; ++c) {
          uint32_t v[OUT_F32 ? 32 : 64];
          {
            uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&v[0]);
            tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BLOCK_N + c * kColsPerStore, lo);
            if constexpr (!OUT_F32) {
              uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&v[32]);
              tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BLOCK_N + c * 64 + 32, hi);
            }
            tmem_wait_ld();
          }
          const int col0 = n0 + c * kColsPerStore;
          if (col0 >= p.N) continue;  // warp-uniform
          uint8_t* buf = my_stage + (store_count & 1) * 4096;
          if (store_count >= 2) {
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
          }
          uint4 chunks[8];
          if constexpr (OUT_F32) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              chunks[j].x = __float_as_uint(zero_acc ? 0.f : __uint_as_float(v[4 * j]) * p.alpha);
              chunks[j].y = __float_as_uint(zero_acc ? 0.f : __uint_as_float(v[4 * j + 1]) * p.alpha);
              chunks[j].z = __float_as_uint(zero_acc ? 0.f : __uint_as_float(v[4 * j + 2]) * p.alpha);
              chunks[j].w = __float_as_uint(zero_acc ? 0.f : __uint_as_float(v[4 * j + 3]) * p.alpha);
            }
          } else {
            // optional scaled addend: this lane's row, the 64 columns of the chunk (rows and columns past the matrix
            // are clipped by the TMA store, so they only have to be kept from being read)
            const int arow = row0 + lane;
            const bool add_ok = p.addend != nullptr && arow < p.M;
            const __nv_bfloat16* arow_ptr = p.addend + static_cast<long long>(add_ok ? arow : 0) * p.ld_add + col0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float f[8];
#pragma unroll
              for (int q = 0; q < 8; ++q) f[q] = zero_acc ? 0.f : __uint_as_float(v[8 * j + q]) * p.alpha;
              if (add_ok && col0 + 8 * j < p.N) {
                const uint4 d = *reinterpret_cast<const uint4*>(arow_ptr + 8 * j);
                f[0] = fmaf(p.beta, bf16_lo(d.x), f[0]); f[1] = fmaf(p.beta, bf16_hi(d.x), f[1]);
                f[2] = fmaf(p.beta, bf16_lo(d.y), f[2]); f[3] = fmaf(p.beta, bf16_hi(d.y), f[3]);
                f[4] = fmaf(p.beta, bf16_lo(d.z), f[4]); f[5] = fmaf(p.beta, bf16_hi(d.z), f[5]);
                f[6] = fmaf(p.beta, bf16_lo(d.w), f[6]); f[7] = fmaf(p.beta, bf16_hi(d.w), f[7]);
              }
              chunks[j].x = pack_bf16(f[0], f[1]); chunks[j].y = pack_bf16(f[2], f[3]);
              chunks[j].z = pack_bf16(f[4], f[5]); chunks[j].w = pack_bf16(f[6], f[7]);
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = chunks[j];
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if constexpr (ACCUM) tma_reduce_add_2d(&tmap_c, buf, col0, row0);
            else tma_store_2d(&tmap_c, buf, col0, row0);
            tma_store_commit();
          }
          ++store_count;
        }
      } else {
      const int row = t.m_tile * kBlockM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const long long cbase =
          (p.mode == 2 ? static_cast<long long>(t.group) * p.group_c_stride : 0) + static_cast<long long>(row) * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BLOCK_N + c * 32, v);
        tmem_wait_ld();
        const int col0 = n0 + c * 32;
        if (!row_ok || col0 >= p.N) continue;
        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cptr) + cbase + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (col0 + j < p.N) {
            float f[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) f[q] = zero_acc ? 0.f : __uint_as_float(v[j + q]) * p.alpha;
            const uint4 old = *reinterpret_cast<const uint4*>(crow + j);
            f[0] += bf16_lo(old.x); f[1] += bf16_hi(old.x); f[2] += bf16_lo(old.y); f[3] += bf16_hi(old.y);
            f[4] += bf16_lo(old.z); f[5] += bf16_hi(old.z); f[6] += bf16_lo(old.w); f[7] += bf16_hi(old.w);
            uint4 o;
            o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
            o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
            *reinterpret_cast<uint4*>(crow + j) = o;
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      ++local_tile;
    }
    if (lane == 0) tma_store_wait<0>();  // this warp's bulk stores have completed before the CTA retires
  }

  __syncthreads();
  if (*abort_flag) drain_delay();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BLOCK_N);
  }
}

template <int BLOCK_N, bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, void* C,
                       const GemmParams& p, cudaStream_t st) {
  using S = GemmSmem<BLOCK_N>;
  auto kern = gemm_bf16_kernel<BLOCK_N, A_MN, B_MN, OUT_F32, ACCUM>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return -static_cast<int>(e);
    configured = true;
  }
  const int num_m = (p.M + kBlockM - 1) / kBlockM;
  const int num_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const long long tiles = p.upper_only ? upper_tile_count(num_m, num_n, BLOCK_N)
                                       : static_cast<long long>(num_m) * num_n *
                                             (p.mode == 2 ? p.num_groups : (p.k_splits > 1 ? p.k_splits : 1));
  if (tiles == 0) return 0;
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  kern<<<grid, kGemmThreads, S::kTotal, st>>>(ta, tb, tc, C, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

template <int BLOCK_N, bool A_MN, bool B_MN>
static int dispatch_out(const CUtensorMap& ta, const CUtensorMap& tb, void* C, const GemmParams& p, int out_f32,
                        int accumulate, cudaStream_t st) {
  // C as a 2-D map of 32-row x 128-byte boxes for the epilogue's TMA stores / reduce-adds
  CUtensorMap tc;
  const uint64_t rows = static_cast<uint64_t>(p.M) * (p.mode == 2 ? p.num_groups : 1);
  int r = out_f32 ? make_tmap_2d(&tc, C, 4, p.N, rows, static_cast<uint64_t>(p.ldc) * 4, 32, 32, 1)
                  : make_tmap_2d(&tc, C, 2, p.N, rows, static_cast<uint64_t>(p.ldc) * 2, 64, 32, 1);
  if (r) return r;
  if (out_f32) {
    return accumulate ? launch_gemm<BLOCK_N, A_MN, B_MN, true, true>(ta, tb, tc, C, p, st)
                      : launch_gemm<BLOCK_N, A_MN, B_MN, true, false>(ta, tb, tc, C, p, st);
  }
  return accumulate ? launch_gemm<BLOCK_N, A_MN, B_MN, false, true>(ta, tb, tc, C, p, st)
                    : launch_gemm<BLOCK_N, A_MN, B_MN, false, false>(ta, tb, tc, C, p, st);
}

template <int BLOCK_N>
static int dispatch_major(const CUtensorMap& ta, const CUtensorMap& tb, void* C, const GemmParams& p, int a_mn,
                          int b_mn, int out_f32, int accumulate, cudaStream_t st) {
  if (!a_mn && !b_mn) return dispatch_out<BLOCK_N, false, false>(ta, tb, C, p, out_f32, accumulate, st);
  if (!a_mn && b_mn) return dispatch_out<BLOCK_N, false, true>(ta, tb, C, p, out_f32, accumulate, st);
  if (a_mn && b_mn) return dispatch_out<BLOCK_N, true, true>(ta, tb, C, p, out_f32, accumulate, st);
  return dispatch_out<BLOCK_N, true, false>(ta, tb, C, p, out_f32, accumulate, st);
}

// N tile: 256 wide whenever the problem has more than 128 columns. A 128x128 tile streams 32 KB of
// operands per 64-deep k-block, which is the shared-memory bandwidth of an SM at tensor-core rate, so
// the narrow tile only pays off when N itself is narrow.
static int choose_block_n(long long /*num_m*/, int N, int /*groups*/) { return N > 128 ? 256 : 128; }

// Split of the reduction extent for products that add into an fp32 C (TMA reduce-add makes the partial sums of
// several CTAs safe): the smallest split that brings the last wave of the persistent grid to 92 % or more of a full
// one, with at least 16 k blocks per part.  STB200_WGRAD_SPLITK=0 switches it off (then the sums of a tile always
// come from one CTA, in one order).
static int choose_k_splits(int M, int N, int K, int bn) {
  static const bool off = [] { const char* e = getenv("STB200_WGRAD_SPLITK"); return e != nullptr && e[0] == '0'; }();
  if (off) return 1;
  const long long tiles = static_cast<long long>((M + kBlockM - 1) / kBlockM) * ((N + bn - 1) / bn);
  const int kb = (K + kBlockK - 1) / kBlockK, sms = sm_count();
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= 4; ++s) {   // every part adds the whole tile into C once more: keep the extra traffic small
    if (s > 1 && kb / s < 16) break;
    const long long units = tiles * s;
    const double eff = static_cast<double>(units) / (static_cast<double>((units + sms - 1) / sms) * sms);
    if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
    if (best_eff >= 0.92) break;
  }
  return best;
}

// C[r][c] = C[c][r] for c < r: completes a symmetric matrix whose upper triangle (by tiles) was computed.
// One CTA of 32 x 8 threads per 32 x 32 block on or below the diagonal.
__global__ void __launch_bounds__(256)
mirror_upper_kernel(__nv_bfloat16* __restrict__ C, int n, long long ld) {
  __shared__ __nv_bfloat16 tile[32][33];
  const int bi = blockIdx.y, bj = blockIdx.x;     // destination block (rows bi, columns bj)
  if (bj > bi) return;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  // source block (rows bj, columns bi), read row-wise
  for (int r = ty; r < 32; r += 8) {
    const int sr = bj * 32 + r, sc = bi * 32 + tx;
    tile[r][tx] = (sr < n && sc < n) ? C[static_cast<long long>(sr) * ld + sc] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int dr = bi * 32 + r, dc = bj * 32 + tx;
    if (dr < n && dc < n && dc < dr) C[static_cast<long long>(dr) * ld + dc] = tile[tx][r];
  }
}

}  // namespace stb

using namespace stb;

extern "C" int stb_mirror_upper_bf16(void* C, int n, long long ld, cudaStream_t stream) {
  if (n <= 0) return 0;
  const unsigned blocks = static_cast<unsigned>((n + 31) / 32);
  mirror_upper_kernel<<<dim3(blocks, blocks), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(C), n, ld);
  return -static_cast<int>(cudaGetLastError());
}

// A: K-major -> stored [M][lda]; MN-major -> stored [K][lda].   (lda/ldb/ldc in elements)
// B: K-major -> stored [N][ldb]; MN-major -> stored [K][ldb].
// Requirements: 16-byte aligned bases, lda/ldb multiples of 8, N and ldc multiples of 8.
// The same with C = alpha * A B^T + beta * addend (bf16 [M][ld_add], may be C; bf16 output only) and, for a square
// symmetric result, only the tiles that reach the diagonal or lie above it (upper_only; mirror afterwards).
extern "C" int stb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                             int a_mn_major, int b_mn_major, int out_f32, int accumulate, float alpha, int* status,
                             cudaStream_t stream);
static int gemm_bf16_impl(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                          int a_mn_major, int b_mn_major, int out_f32, int accumulate, float alpha, const void* addend,
                          long long ld_add, float beta, int upper_only, int* status, cudaStream_t stream);

extern "C" int stb_gemm_bf16_ex(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                int a_mn_major, int b_mn_major, float alpha, const void* addend, long long ld_add,
                                float beta, int upper_only, int* status, cudaStream_t stream) {
  if (addend != nullptr && ((ld_add & 7) || (reinterpret_cast<uintptr_t>(addend) & 15))) return -kErrBadArgument;
  if (upper_only && M != N) return -kErrBadArgument;
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, 0, 0, alpha, addend, ld_add, beta,
                        upper_only, status, stream);
}

extern "C" int stb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                             int a_mn_major, int b_mn_major, int out_f32, int accumulate, float alpha, int* status,
                             cudaStream_t stream) {
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, out_f32, accumulate, alpha, nullptr, 0,
                        0.f, 0, status, stream);
}

static int gemm_bf16_impl(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                          int a_mn_major, int b_mn_major, int out_f32, int accumulate, float alpha, const void* addend,
                          long long ld_add, float beta, int upper_only, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (N & 7) || (lda & 7) || (ldb & 7) || (ldc & 3)) return -kErrBadArgument;
  const int bn = choose_block_n((M + kBlockM - 1) / kBlockM, N, 1);
  CUtensorMap ta, tb;
  int r;
  if (!a_mn_major) r = make_tmap_2d_bf16(&ta, A, K, M, static_cast<uint64_t>(lda) * 2, kBlockK, kBlockM, 1);
  else r = make_tmap_2d_bf16(&ta, A, M, K, static_cast<uint64_t>(lda) * 2, 64, kBlockK, 1);
  if (r) return r;
  if (!b_mn_major) r = make_tmap_2d_bf16(&tb, B, K, N, static_cast<uint64_t>(ldb) * 2, kBlockK, bn, 1);
  else r = make_tmap_2d_bf16(&tb, B, N, K, static_cast<uint64_t>(ldb) * 2, 64, kBlockK, 1);
  if (r) return r;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.mode = 0; p.status = status; p.alpha = alpha;
  p.addend = static_cast<const __nv_bfloat16*>(addend); p.ld_add = ld_add; p.beta = beta; p.upper_only = upper_only;
  p.k_splits = (out_f32 && accumulate) ? choose_k_splits(M, N, K, bn) : 1;
  return bn == 256 ? dispatch_major<256>(ta, tb, C, p, a_mn_major, b_mn_major, out_f32, accumulate, stream)
                   : dispatch_major<128>(ta, tb, C, p, a_mn_major, b_mn_major, out_f32, accumulate, stream);
}

// Grouped rows (expert FFN forward / dgrad). A: [M][lda] K-major, rows grouped into expert
// segments aligned to 128 rows; tile_group[m_tile] gives the expert (or -1 to skip the tile).
//   b_mn_major = 0: B stored [G][N][ldb] (K contiguous)   -> y_g = x_g * W_g^T
//   b_mn_major = 1: B stored [G][K][ldb] (N contiguous)   -> y_g = x_g * W_g
extern "C" int stb_gemm_bf16_grouped_rows(const void* A, const void* B, void* C, const int* tile_group, int M, int N,
                                          int K, int num_groups, int lda, int ldb, int ldc, int b_mn_major,
                                          int out_f32, int accumulate, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (N & 7) || (lda & 7) || (ldb & 7) || (ldc & 3)) return -kErrBadArgument;
  const int bn = (N % 256 == 0) ? 256 : 128;
  if (!b_mn_major && (N % bn) != 0) return -kErrBadArgument;  // a B tile must not run into the next expert
  if (b_mn_major && (K % kBlockK) != 0) return -kErrBadArgument;
  CUtensorMap ta, tb;
  int r = make_tmap_2d_bf16(&ta, A, K, M, static_cast<uint64_t>(lda) * 2, kBlockK, kBlockM, 1);
  if (r) return r;
  if (!b_mn_major)
    r = make_tmap_2d_bf16(&tb, B, K, static_cast<uint64_t>(N) * num_groups, static_cast<uint64_t>(ldb) * 2, kBlockK, bn, 1);
  else
    r = make_tmap_2d_bf16(&tb, B, N, static_cast<uint64_t>(K) * num_groups, static_cast<uint64_t>(ldb) * 2, 64, kBlockK, 1);
  if (r) return r;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.mode = 1; p.num_groups = num_groups;
  p.group_n_stride = b_mn_major ? K : N;
  p.tile_group = tile_group; p.status = status; p.alpha = 1.f;
  return bn == 256 ? dispatch_major<256>(ta, tb, C, p, 0, b_mn_major, out_f32, accumulate, stream)
                   : dispatch_major<128>(ta, tb, C, p, 0, b_mn_major, out_f32, accumulate, stream);
}

// Grouped reduction (expert wgrad): for each g, C[g][M][N] (+)= A[rows_g][M]^T * B[rows_g][N], both operands
// stored row-major by token (MN-major); group_offsets[g] are multiples of 64 and padding rows are zero.
extern "C" int stb_gemm_bf16_grouped_reduce(const void* A, const void* B, void* C, const int* group_offsets,
                                            int total_rows, int M, int N, int num_groups, int lda, int ldb, int ldc,
                                            int out_f32, int accumulate, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || num_groups <= 0) return 0;
  if ((N & 7) || (M & 127) || (lda & 7) || (ldb & 7) || (ldc & 3)) return -kErrBadArgument;
  const int bn = (N % 256 == 0) ? 256 : 128;
  CUtensorMap ta, tb;
  int r = make_tmap_2d_bf16(&ta, A, M, total_rows, static_cast<uint64_t>(lda) * 2, 64, kBlockK, 1);
  if (r) return r;
  r = make_tmap_2d_bf16(&tb, B, N, total_rows, static_cast<uint64_t>(ldb) * 2, 64, kBlockK, 1);
  if (r) return r;
  GemmParams p{};
  p.M = M; p.N = N; p.K = total_rows; p.ldc = ldc; p.mode = 2; p.num_groups = num_groups;
  p.group_offsets = group_offsets; p.group_c_stride = static_cast<long long>(M) * ldc;
  p.status = status; p.alpha = 1.f;
  return bn == 256 ? dispatch_major<256>(ta, tb, C, p, 1, 1, out_f32, accumulate, stream)
                   : dispatch_major<128>(ta, tb, C, p, 1, 1, out_f32, accumulate, stream);
}
