// Flash-attention backward for sm_100a: one pipelined kernel template for both gradient passes.
//
// A CTA keeps two 128-row tiles resident ("fixed": K,V for the dK/dV pass, Q,dO for the dQ pass) and
// streams 64-row tiles of the other side ("stream": Q,dO resp. K,V) through a 3-stage TMA ring.
// Per streamed tile:
//     S'  = F1 * G1^T          [128 x 64]   (dkv: K Q^T = S^T ; dq: Q K^T = S)
//     dP' = F2 * G2^T          [128 x 64]   (dkv: V dO^T     ; dq: dO V^T)
//   softmax threads (one per fixed row): P' = exp2(S' * c - lse), dS' = P' o (dP' - delta) * scale -> smem
//     dkv: dV += P' * G2 (dO)  ,  dK += dS' * G1 (Q)        dq: dQ += dS' * G1 (K)
// S' / dP' are double buffered in TMEM so that the products of tile i+1 run while the softmax threads
// work on tile i; the output accumulators stay in TMEM for the whole CTA.  Both passes recompute S, so
// no atomics are needed and the gradients are bitwise reproducible.
//
// The kernels are bound by shared-memory bandwidth rather than by the tensor pipe (a 128x64x16 product with both
// operands in shared memory reads 6 KB in the 32 cycles it computes).  In the dQ pass the fixed tiles Q and dO are
// therefore copied once per CTA into TMEM (64 columns each, two bf16 per column) and serve as the A operand of
// S and dP from there; only the streamed K / V tiles are read from shared memory.
//
// The dK/dV pass loops over q heads of the GQA group inside the CTA, so dK and dV come out summed over them.
// With few kv heads and key blocks (4 kv heads x 33 blocks is less than one wave of 148 SMs) the group is
// split over `splits` CTAs; each writes fp32 partials and `attn_dkv_reduce_kernel` adds them in split order,
// which keeps the gradients bitwise reproducible.
#include "attention_common.cuh"

namespace stb {

constexpr int kSB = 64;                       // streamed rows per iteration
constexpr int kStreamTile = kSB * kD * 2;     // 16 KB: [64][128] bf16 as two [64][64] slabs of 8 KB
constexpr int kStreamSlab = kSB * 128;        // 8 KB
constexpr int kPTile = 128 * kSB * 2;         // 16 KB: [128][64] bf16, one swizzled slab
constexpr int kBwdStages = 3;
constexpr int kBwdThreads = 320;                // producer warp, MMA warp, 8 softmax warps (2 per TMEM lane quarter)
constexpr int kBwdSmem = 2 * kTileBytes + kBwdStages * 2 * kStreamTile + 2 * 2 * kPTile + 1024 + 1024 + 512;

// A [128][K] K-major (two 64-col slabs of 16 KB) x B [64][K] K-major (two slabs of 8 KB) -> D [128 x 64]
__device__ __forceinline__ void mma_fixed_stream_t(uint32_t d_tmem, uint32_t sa, uint32_t sb) {
  constexpr uint32_t idesc = umma_idesc_bf16(128, kSB, 0, 0);
  const uint64_t da = umma_smem_desc(sa, 16, 1024), db = umma_smem_desc(sb, 16, 1024);
  umma4_ss(d_tmem, da, umma_desc_advance(da, 32), umma_desc_advance(da, 64), umma_desc_advance(da, 96), db,
           umma_desc_advance(db, 32), umma_desc_advance(db, 64), umma_desc_advance(db, 96), idesc, 0u);
  umma4_ss(d_tmem, umma_desc_advance(da, kSlabBytes), umma_desc_advance(da, kSlabBytes + 32),
           umma_desc_advance(da, kSlabBytes + 64), umma_desc_advance(da, kSlabBytes + 96),
           umma_desc_advance(db, kStreamSlab), umma_desc_advance(db, kStreamSlab + 32),
           umma_desc_advance(db, kStreamSlab + 64), umma_desc_advance(db, kStreamSlab + 96), idesc, 1u);
}

// A [128][128] bf16 in TMEM (64 columns) x B [64][K] K-major (two slabs of 8 KB) -> D [128 x 64]
__device__ __forceinline__ void mma_tmem_stream_t(uint32_t d_tmem, uint32_t a_tmem, uint32_t sb) {
  constexpr uint32_t idesc = umma_idesc_bf16(128, kSB, 0, 0);
  const uint64_t db = umma_smem_desc(sb, 16, 1024);
  umma4_ts(d_tmem, a_tmem, a_tmem + 8, a_tmem + 16, a_tmem + 24, db, umma_desc_advance(db, 32),
           umma_desc_advance(db, 64), umma_desc_advance(db, 96), idesc, 0u);
  umma4_ts(d_tmem, a_tmem + 32, a_tmem + 40, a_tmem + 48, a_tmem + 56, umma_desc_advance(db, kStreamSlab),
           umma_desc_advance(db, kStreamSlab + 32), umma_desc_advance(db, kStreamSlab + 64),
           umma_desc_advance(db, kStreamSlab + 96), idesc, 1u);
}

// A [128][64] K-major (one slab) x B stored [64 rows = K][128 = N] (MN-major, two slabs of 8 KB) -> D [128 x 128]
__device__ __forceinline__ void mma_p_stream(uint32_t d_tmem, uint32_t sa, uint32_t sb, bool accumulate) {
  constexpr uint32_t idesc = umma_idesc_bf16(128, 128, 0, 1);
  const uint64_t da = umma_smem_desc(sa, 16, 1024), db = umma_smem_desc(sb, kStreamSlab, 1024);
  umma4_ss(d_tmem, da, umma_desc_advance(da, 32), umma_desc_advance(da, 64), umma_desc_advance(da, 96), db,
           umma_desc_advance(db, 2048), umma_desc_advance(db, 4096), umma_desc_advance(db, 6144), idesc,
           accumulate ? 1u : 0u);
}

__device__ __forceinline__ void load_stream_tile(void* dst, const CUtensorMap* m, uint64_t* bar, int head, int row) {
  tma_load_3d(dst, m, bar, 0, head, row);
  tma_load_3d(static_cast<uint8_t*>(dst) + kStreamSlab, m, bar, 64, head, row);
}

// Softmax-gradient math of one thread for its 32 columns of a streamed tile:
//   P' = exp2(S' * c - lse),  dS' = P' o (dP' - delta)      (the softmax scale is applied to dK / dQ in the epilogue)
// `cl` holds the per-column constants of the dK/dV pass ([64] lse * log2e, then [64] delta); the dQ pass has them
// per row.  MASK is decided per tile by the caller, so interior tiles run without a predicate per element.
template <bool DKV, bool MASK>
__device__ __forceinline__ void bwd_tile_math(const AttnParams& p, const SegInfo& s, const uint32_t (&sv)[32],
                                              const uint32_t (&dv)[32], const float* cl, int half, int r, int fi, int g0,
                                              float sl2, float row_lse2, float row_delta, uint8_t* pP, uint8_t* pdS) {
#pragma unroll
  for (int c8l = 0; c8l < 4; ++c8l) {
    const int c8 = half * 4 + c8l;
    float lse8[8], dl8[8];
    if (DKV) {
      const float4 l0 = *reinterpret_cast<const float4*>(cl + c8 * 8), l1 = *reinterpret_cast<const float4*>(cl + c8 * 8 + 4);
      const float4 d0 = *reinterpret_cast<const float4*>(cl + 64 + c8 * 8), d1 = *reinterpret_cast<const float4*>(cl + 64 + c8 * 8 + 4);
      lse8[0] = l0.x; lse8[1] = l0.y; lse8[2] = l0.z; lse8[3] = l0.w; lse8[4] = l1.x; lse8[5] = l1.y; lse8[6] = l1.z; lse8[7] = l1.w;
      dl8[0] = d0.x; dl8[1] = d0.y; dl8[2] = d0.z; dl8[3] = d0.w; dl8[4] = d1.x; dl8[5] = d1.y; dl8[6] = d1.z; dl8[7] = d1.w;
    }
    float pv[8], dd[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int lc = c8l * 8 + i;          // index into this thread's 32 columns
      const float lse2 = DKV ? lse8[i] : row_lse2;
      const float dl = DKV ? dl8[i] : row_delta;
      float pr = exp2f(fmaf(__uint_as_float(sv[lc]), sl2, -lse2));
      if (MASK) {
        const int col = half * 32 + lc;    // column of the streamed tile
        const bool vis = DKV ? visible(p, s, g0 + col, fi) : visible(p, s, fi, g0 + col);
        if (!vis) pr = 0.f;
      }
      pv[i] = pr;
      dd[i] = pr * (__uint_as_float(dv[lc]) - dl);
    }
    const uint32_t a = swz(r, c8);
    if (DKV)
      *reinterpret_cast<uint4*>(pP + a) =
          make_uint4(pack_bf16(pv[0], pv[1]), pack_bf16(pv[2], pv[3]), pack_bf16(pv[4], pv[5]), pack_bf16(pv[6], pv[7]));
    *reinterpret_cast<uint4*>(pdS + a) =
        make_uint4(pack_bf16(dd[0], dd[1]), pack_bf16(dd[2], dd[3]), pack_bf16(dd[4], dd[5]), pack_bf16(dd[6], dd[7]));
  }
}

template <bool DKV>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_f1, const __grid_constant__ CUtensorMap tmap_f2,
                const __grid_constant__ CUtensorMap tmap_g1, const __grid_constant__ CUtensorMap tmap_g2,
                const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sF1 = smem;
  uint8_t* sF2 = sF1 + kTileBytes;
  uint8_t* sG = sF2 + kTileBytes;                       // stages x (G1 | G2)
  uint8_t* sP = sG + kBwdStages * 2 * kStreamTile;      // 2 buffers x (P' | dS')
  float* s_lse = reinterpret_cast<float*>(sP + 4 * kPTile);   // [2][64] lse*log2e, then [2][64] delta
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s_lse) + 1024);
  uint64_t* f_full = bars;                      // fixed tiles landed
  uint64_t* g_full = bars + 1;                  // [3]
  uint64_t* g_empty = bars + 4;                 // [3]
  uint64_t* sdp_full = bars + 7;                // [2] S', dP' in TMEM
  uint64_t* pds_full = bars + 9;                // [2] P', dS' in smem (128 arrivals)
  uint64_t* acc_full = bars + 11;
  uint64_t* f_tmem = bars + 12;                 // dQ pass: Q and dO copied into TMEM (256 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.hq / p.hkv;
  const int blk = DKV ? static_cast<int>(blockIdx.y) : static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);
  const int seg = p.blk_seg[blk];
  if (seg < 0) return;
  const SegInfo s = seg_info(p, seg);
  const int row_abs0 = p.blk_row0[blk];
  // fixed rows: keys (dkv) or queries (dq), relative to the segment
  const int f0 = row_abs0 - (DKV ? s.k_begin : s.q_begin);
  const int splits = DKV ? p.splits : 1;
  const int head_f = DKV ? static_cast<int>(blockIdx.x) / splits : static_cast<int>(blockIdx.x);  // kv head ; q head
  const int split = DKV ? static_cast<int>(blockIdx.x) % splits : 0;
  const int gps = group / splits;  // q heads per CTA in the dK/dV pass
  const int kvh = DKV ? head_f : head_f / group;

  // streamed range [g_lo, g_hi) in rows of the other side
  int g_lo, g_hi;
  if (DKV) {
    g_lo = p.causal ? max(0, f0 - s.off) : 0;
    g_hi = s.q_len;
    if (p.window > 0) g_hi = min(g_hi, f0 + kBN - 1 - s.off + p.window);
  } else {
    g_hi = s.k_len;
    if (p.causal) g_hi = min(g_hi, f0 + kBM + s.off);
    g_lo = (p.window > 0) ? max(0, f0 + s.off - p.window + 1) : 0;
  }
  const int sb0 = g_lo / kSB;
  const int nsb = (g_hi > g_lo) ? (g_hi + kSB - 1) / kSB - sb0 : 0;
  const int iters = nsb * (DKV ? gps : 1);

  if (threadIdx.x == 0) {
    mbar_init(f_full, 1);
    for (int i = 0; i < kBwdStages; ++i) {
      mbar_init(&g_full[i], 1);
      mbar_init(&g_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sdp_full[i], 1);
      mbar_init(&pds_full[i], 256);
    }
    mbar_init(acc_full, 1);
    mbar_init(f_tmem, 256);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;  // S'[2] 0,64 ; dP'[2] 128,192 ; acc1 256 ; acc2 384 (dQ pass: Q 384, dO 448)

  if (warp == 0) {
    if (lane == 0 && iters > 0) {
      mbar_arrive_expect_tx(f_full, 2 * kTileBytes);
      const int f_row = DKV ? key_row(p, row_abs0) : row_abs0;   // fixed rows are keys in the dK/dV pass
      load_tile(sF1, &tmap_f1, f_full, head_f, f_row);
      load_tile(sF2, &tmap_f2, f_full, head_f, f_row);
      for (int it = 0; it < iters && !*abort_flag; ++it) {
        const int st = it % kBwdStages;
        if (!mbar_wait(&g_empty[st], ((it / kBwdStages) & 1) ^ 1)) {
          report_error(p.status, kErrProducerWait);
          *abort_flag = 1;
          break;
        }
        const int hg = DKV ? kvh * group + split * gps + it / nsb : kvh;
        const int grow = DKV ? s.q_begin + (sb0 + it % nsb) * kSB : key_row(p, s.k_begin + (sb0 + it % nsb) * kSB);
        uint8_t* g1 = sG + st * 2 * kStreamTile;
        mbar_arrive_expect_tx(&g_full[st], 2 * kStreamTile);
        load_stream_tile(g1, &tmap_g1, &g_full[st], hg, grow);
        load_stream_tile(g1 + kStreamTile, &tmap_g2, &g_full[st], hg, grow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && iters > 0) {
      bool ok = mbar_wait(f_full, 0);
      if (!DKV && ok) ok = mbar_wait(f_tmem, 0);
      const uint32_t aF1 = smem_u32(sF1), aF2 = smem_u32(sF2);
      auto issue_sdp = [&](int it) -> bool {
        const int st = it % kBwdStages;
        if (!mbar_wait(&g_full[st], (it / kBwdStages) & 1)) return false;
        tc_fence_after();
        const uint32_t g1 = smem_u32(sG + st * 2 * kStreamTile);
        if (DKV) {
          mma_fixed_stream_t(tmem + (it & 1) * kSB, aF1, g1);
          mma_fixed_stream_t(tmem + 128 + (it & 1) * kSB, aF2, g1 + kStreamTile);
        } else {
          mma_tmem_stream_t(tmem + (it & 1) * kSB, tmem + 384, g1);
          mma_tmem_stream_t(tmem + 128 + (it & 1) * kSB, tmem + 448, g1 + kStreamTile);
        }
        umma_commit(&sdp_full[it & 1]);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int it = 0; it < iters && ok && !*abort_flag; ++it) {
        if (it + 1 < iters) {
          ok = issue_sdp(it + 1);
          if (!ok) break;
        }
        ok = mbar_wait(&pds_full[it & 1], (it >> 1) & 1);
        if (!ok) break;
        tc_fence_after();
        const int st = it % kBwdStages;
        const uint32_t g1 = smem_u32(sG + st * 2 * kStreamTile);
        const uint32_t pbuf = smem_u32(sP + (it & 1) * 2 * kPTile);
        if (DKV) {
          mma_p_stream(tmem + 256, pbuf, g1 + kStreamTile, it > 0);   // dV += P'  * dO
          mma_p_stream(tmem + 384, pbuf + kPTile, g1, it > 0);       // dK += dS' * Q
        } else {
          mma_p_stream(tmem + 256, pbuf + kPTile, g1, it > 0);       // dQ += dS' * K
        }
        umma_commit(&g_empty[st]);
      }
      if (ok) umma_commit(acc_full);
      if (!ok) { report_error(p.status, kErrMmaWaitFull); *abort_flag = 1; }
    }
  } else {
    // Two warps share each TMEM lane quarter: warps 2..5 take columns [0,32) of every streamed tile,
    // warps 6..9 columns [32,64).  A scheduler then always has two softmax warps to alternate between.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;               // 0 or 1
    const int r = quarter * 32 + lane;              // fixed row owned by this thread
    const int t128 = threadIdx.x - 64;              // 0..255 among the softmax threads
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    const int fi = f0 + r;                          // row inside the segment (key for dkv, query for dq)
    float row_lse2 = 0.f, row_delta = 0.f;
    bool frow_ok;
    if (DKV) {
      // keys in front of the document (context parallelism: the range starts at a tile boundary) belong to another
      // segment, whose CTA writes their gradients
      frow_ok = fi < s.k_len && fi >= s.k_skip;
    } else {
      const long long q_abs = static_cast<long long>(row_abs0) + r;
      frow_ok = (fi < s.q_len) && (q_abs < p.total_q);
      if (frow_ok) {
        row_lse2 = p.LSE[static_cast<long long>(head_f) * p.total_q + q_abs] * kLog2e;
        row_delta = p.delta[static_cast<long long>(head_f) * p.total_q + q_abs];
      }
    }
    bool ok = true;
    if (!DKV && iters > 0) {
      // group 0 copies its row of Q, group 1 its row of dO: 16 chunks of 16 bytes from the swizzled tile
      ok = mbar_wait(f_full, 0);
      const uint8_t* src = half == 0 ? sF1 : sF2;
      const uint32_t dst = tmem + lane_addr + 384 + half * 64;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {          // 64 columns of the row = one 128-byte slab row = 32 TMEM columns
        uint32_t w[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 x = *reinterpret_cast<const uint4*>(src + hh * kSlabBytes + swz(r, c));
          w[c * 4] = x.x; w[c * 4 + 1] = x.y; w[c * 4 + 2] = x.z; w[c * 4 + 3] = x.w;
        }
        tmem_st_32x32(dst + hh * 32, w);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(f_tmem);
    }
    // All softmax threads run every iteration (the dK/dV pass meets at a named barrier in each one); after
    // a timed-out wait the remaining waits are skipped, so a failure cannot strand the other threads.
    for (int it = 0; it < iters; ++it) {
      const int g0 = (sb0 + it % nsb) * kSB;        // first streamed row of this tile (segment relative)
      const int buf = it & 1;
      if (*abort_flag) ok = false;
      if (DKV) {
        // per-column constants of the 64 streamed queries: threads 0..63 fetch lse, 64..127 fetch delta
        const int hq_i = kvh * group + split * gps + it / nsb;
        const int c = t128 & 63;
        const long long q_abs = static_cast<long long>(s.q_begin) + g0 + c;
        const bool qok = (g0 + c < s.q_len) && (q_abs < p.total_q);
        if (t128 < 128) {
          float val = 0.f;
          if (qok) {
            val = (t128 < 64) ? p.LSE[static_cast<long long>(hq_i) * p.total_q + q_abs] * kLog2e
                              : p.delta[static_cast<long long>(hq_i) * p.total_q + q_abs];
          } else if (t128 < 64) {
            val = INFINITY;  // exp2(x - inf) = 0 for rows past the segment
          }
          s_lse[buf * 128 + t128] = val;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
      if (ok) ok = mbar_wait(&sdp_full[buf], (it >> 1) & 1);
      if (!ok) continue;
      tc_fence_after();
      uint32_t sv[32], dv[32];
      tmem_ld_32x32(tmem + lane_addr + buf * kSB + half * 32, sv);
      tmem_ld_32x32(tmem + lane_addr + 128 + buf * kSB + half * 32, dv);
      tmem_wait_ld();
      // does any (fixed row, streamed row) pair of this tile fall outside the mask?
      bool need_mask;
      if (DKV) {
        need_mask = (f0 + kBN > s.k_len) || (f0 < s.k_skip) || (g0 + kSB > s.q_len) ||
                    (p.causal && f0 + kBN - 1 > g0 + s.off) || (p.window > 0 && f0 <= g0 + kSB - 1 + s.off - p.window);
      } else {
        need_mask = (f0 + kBM > s.q_len) || (g0 + kSB > s.k_len) || (g0 < s.k_skip) ||
                    (p.causal && g0 + kSB - 1 > f0 + s.off) || (p.window > 0 && g0 <= f0 + kBM - 1 + s.off - p.window);
      }
      uint8_t* pP = sP + buf * 2 * kPTile;
      uint8_t* pdS = pP + kPTile;
      const float* cl = s_lse + buf * 128;
      if (!frow_ok) {
        // a fixed row past the end of its segment: its P' and dS' rows are zero
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int c8l = 0; c8l < 4; ++c8l) {
          const uint32_t a = swz(r, half * 4 + c8l);
          if (DKV) *reinterpret_cast<uint4*>(pP + a) = z;
          *reinterpret_cast<uint4*>(pdS + a) = z;
        }
      } else if (need_mask) {
        bwd_tile_math<DKV, true>(p, s, sv, dv, cl, half, r, fi, g0, sl2, row_lse2, row_delta, pP, pdS);
      } else {
        bwd_tile_math<DKV, false>(p, s, sv, dv, cl, half, r, fi, g0, sl2, row_lse2, row_delta, pP, pdS);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&pds_full[buf]);
    }
    if (ok && iters > 0 && !*abort_flag) ok = mbar_wait(acc_full, 0);
    if (!ok) { report_error(p.status, kErrSoftmaxWait); *abort_flag = 1; }
    if (iters > 0) tc_fence_after();
    const long long f_abs = static_cast<long long>(DKV ? key_row(p, row_abs0) : row_abs0) + r;
    const bool store_ok = DKV ? (frow_ok && f_abs < p.total_k) : frow_ok;
#pragma unroll 1
    for (int which = 0; which < (DKV ? 2 : 1); ++which) {
      __nv_bfloat16* base;
      if (DKV) base = which == 0 ? p.dV + f_abs * p.dv_stride + static_cast<long long>(kvh) * kD
                                 : p.dK + (f_abs * p.hkv + kvh) * kD;
      else base = p.dQ + (f_abs * p.hq + head_f) * kD;
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t v[32];
        if (iters > 0 && ok) {
          tmem_ld_32x32(tmem + lane_addr + 256 + which * 128 + c * 32, v);
          tmem_wait_ld();
          if (!DKV || which == 1) {   // dK and dQ were accumulated from unscaled dS'
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * p.scale);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (DKV && splits > 1) {
          if (store_ok) {
            float4* part = reinterpret_cast<float4*>(
                p.dkv_part + (((static_cast<long long>(split) * 2 + which) * p.total_k + f_abs) * p.hkv + kvh) * kD +
                c * 32);
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              part[i >> 2] = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]),
                                         __uint_as_float(v[i + 3]));
          }
        } else if (store_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
            o.y = pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
            o.z = pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
            o.w = pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
            *reinterpret_cast<uint4*>(base + c * 32 + i) = o;
          }
        }
      }
    }
    tc_fence_before();
  }

  __syncthreads();
  if (*abort_flag) drain_delay();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// dV / dK = sum over splits (in order) of the fp32 partials; one thread per 4 elements
__global__ void __launch_bounds__(256)
attn_dkv_reduce_kernel(const float* __restrict__ part, int splits, long long total_k, int hkv,
                       __nv_bfloat16* __restrict__ dK, __nv_bfloat16* __restrict__ dV, long long dv_stride) {
  const long long per = total_k * hkv * (kD / 4);  // float4 words of one [Tk][hkv][D] array
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < 2 * per;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int which = i >= per;
    const long long w = i - which * per;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float4 v = reinterpret_cast<const float4*>(part)[(static_cast<long long>(s) * 2 + which) * per + w];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const long long d4 = w % (kD / 4), th = w / (kD / 4);
    const long long t = th / hkv, h = th % hkv;
    __nv_bfloat16* dst = which == 0 ? dV + t * dv_stride + h * kD + d4 * 4 : dK + (t * hkv + h) * kD + d4 * 4;
    *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
  }
}

// delta[h][t] = sum_d dO[t][h][d] * O[t][h][d]; one warp per (t, h)
__global__ void __launch_bounds__(256)
attn_delta2_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO, float* __restrict__ delta,
                   int T, int hq) {
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(T) * hq) return;
  const long long t = wid / hq;
  const int h = static_cast<int>(wid % hq);
  const uint2 a = *reinterpret_cast<const uint2*>(O + wid * kD + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dO + wid * kD + lane * 4);
  float sum = bf16_lo(a.x) * bf16_lo(b.x) + bf16_hi(a.x) * bf16_hi(b.x) + bf16_lo(a.y) * bf16_lo(b.y) +
              bf16_hi(a.y) * bf16_hi(b.y);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = sum;
}

}  // namespace stb

using namespace stb;

// How many CTAs share the q heads of one kv head in the dK/dV pass: 1 when (kv heads x key blocks) already fills
// two waves, otherwise the smallest divisor of the group size that does (at most the group size).
extern "C" int stb_attn_bwd_splits(int hq, int hkv, int num_k_blocks) {
  if (hkv <= 0 || hq % hkv) return 1;
  const int group = hq / hkv;
  const long long want = 2LL * sm_count();
  for (int s = 1; s <= group; ++s) {
    if (group % s) continue;
    if (static_cast<long long>(hkv) * s * num_k_blocks >= want) return s;
  }
  return group;
}

// Backward. dq [Tq][hq][D], dk [Tk][hkv][D] contiguous; dv rows with stride dv_stride (elements).
// dkv_part: fp32 scratch of splits * 2 * total_k * hkv * head_dim floats when splits > 1 (else unused).
// q_blk_*: schedule over 128-row q blocks; k_blk_*: schedule over 128-row key blocks.
// delta: scratch [hq][Tq] floats.
extern "C" int stb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, float* delta, void* dq, void* dk, void* dv, const int* cu_q,
                            const int* cu_k, const int* q_blk_seg, const int* q_blk_row0, int num_q_blocks,
                            const int* k_blk_seg, const int* k_blk_row0, int num_k_blocks, int total_q, int total_k,
                            int hq, int hkv, int head_dim, long long q_stride, long long k_stride, long long v_stride,
                            long long dv_stride, int causal, int window, float scale, float* dkv_part, int splits,
                            const int* seg_k_begin, const int* seg_k_len, const int* seg_k_skip, int cp, int chunk_len,
                            int* status, cudaStream_t st) {
  if (total_q <= 0 || total_k <= 0) return 0;
  if (head_dim != kD || hq % hkv) return -kErrBadArgument;
  if (splits < 1 || (hq / hkv) % splits || (splits > 1 && dkv_part == nullptr)) return -kErrBadArgument;
  const long long do_stride = static_cast<long long>(hq) * kD;
  CUtensorMap q128, k128, v128, do128, q64, k64, v64, do64;
  int r;
  if ((r = make_head_map(&q128, q, hq, total_q, q_stride, 128))) return r;
  if ((r = make_head_map(&k128, k, hkv, total_k, k_stride, 128))) return r;
  if ((r = make_head_map(&v128, v, hkv, total_k, v_stride, 128))) return r;
  if ((r = make_head_map(&do128, d_o, hq, total_q, do_stride, 128))) return r;
  if ((r = make_head_map(&q64, q, hq, total_q, q_stride, 64))) return r;
  if ((r = make_head_map(&k64, k, hkv, total_k, k_stride, 64))) return r;
  if ((r = make_head_map(&v64, v, hkv, total_k, v_stride, 64))) return r;
  if ((r = make_head_map(&do64, d_o, hq, total_q, do_stride, 64))) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
    if (e != cudaSuccess) return -static_cast<int>(e);
    e = cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
    if (e != cudaSuccess) return -static_cast<int>(e);
    configured = true;
  }
  const long long warps = static_cast<long long>(total_q) * hq;
  attn_delta2_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, total_q, hq);
  AttnParams p{};
  p.cu_q = cu_q; p.cu_k = cu_k;
  p.hq = hq; p.hkv = hkv; p.causal = causal; p.window = window; p.scale = scale;
  p.total_q = total_q; p.total_k = total_k;
  p.LSE = const_cast<float*>(lse); p.delta = delta;
  p.dQ = static_cast<__nv_bfloat16*>(dq); p.dK = static_cast<__nv_bfloat16*>(dk);
  p.dV = static_cast<__nv_bfloat16*>(dv); p.dv_stride = dv_stride; p.status = status;
  p.dkv_part = dkv_part; p.splits = splits;
  if (seg_k_begin != nullptr) {
    if (cp < 1 || chunk_len <= 0 || (chunk_len % kBN) || seg_k_len == nullptr || seg_k_skip == nullptr)
      return -kErrBadArgument;
    p.seg_k_begin = seg_k_begin; p.seg_k_len = seg_k_len; p.seg_k_skip = seg_k_skip; p.cp = cp; p.chunk_len = chunk_len;
  }
  // dK / dV: fixed = (K, V) of a kv head, streamed = (Q, dO) of the group's q heads
  p.blk_seg = k_blk_seg; p.blk_row0 = k_blk_row0;
  if (num_k_blocks > 0) {
    attn_bwd_kernel<true><<<dim3(hkv * splits, num_k_blocks), kBwdThreads, kBwdSmem, st>>>(k128, v128, q64, do64, p);
    if (splits > 1) {
      const long long words = 2LL * total_k * hkv * (kD / 4);
      long long blocks = (words + 255) / 256;
      const long long cap = static_cast<long long>(sm_count()) * 16;
      if (blocks > cap) blocks = cap;
      attn_dkv_reduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
          dkv_part, splits, total_k, hkv, static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dv), dv_stride);
    }
  }
  // dQ: fixed = (Q, dO) of a q head, streamed = (K, V)
  p.blk_seg = q_blk_seg; p.blk_row0 = q_blk_row0;
  if (num_q_blocks > 0)
    attn_bwd_kernel<false><<<dim3(hq, num_q_blocks), kBwdThreads, kBwdSmem, st>>>(q128, do128, k64, v64, p);
  return -static_cast<int>(cudaGetLastError());
}
