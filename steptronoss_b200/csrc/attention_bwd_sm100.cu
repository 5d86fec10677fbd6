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

#include <cstdlib>

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
  uint64_t* pds_full = bars + 9;                // [2] P', dS' in smem (one arrival per softmax warp)
  uint64_t* acc_full = bars + 11;
  uint64_t* f_tmem = bars + 12;                 // dQ pass: Q and dO copied into TMEM (one arrival per softmax warp)
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
      mbar_init(&pds_full[i], 8);    // one arrival per softmax warp
    }
    mbar_init(acc_full, 1);
    mbar_init(f_tmem, 8);
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
      mbar_arrive_warp(f_tmem);
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
      ok = __all_sync(0xffffffffu, ok);             // warp-wide TMEM loads and the warp's single arrival follow
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
      mbar_arrive_warp(&pds_full[buf]);
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

// ---------------------------------------------------------------------------------------------------------------
// dQ pass with 128-key tiles.
//
// A 128x64x16 step reads its A operand for 64 columns of output only and runs at 54 % (A in shared memory) or 72 %
// (A in TMEM) of the tensor rate, a 128x128x16 step at 100 % (`benchmarks/micro/umma_rate.cu`).  This kernel
// therefore streams K / V in tiles of 128 keys: S = Q K^T and dP = dO V^T are 128x128x128 products with Q and dO in
// TMEM, dQ += dS K takes dS [128 q][128 keys] from shared memory.  S and dP have one TMEM buffer each; the softmax
// threads free it as soon as their 64 columns are in registers, so the products of the next tile run while they
// compute, and dS has one shared-memory tile whose previous consumer (dQ of the tile before) has long finished when
// it is written again.
//
//   warp 0      TMA producer: Q, dO once; K_j, V_j (32 KB each) through a 3-stage ring whose third stage reuses the
//               Q / dO landing zone once those are in TMEM
//   warp 1      MMA issuer
//   warps 2..17 warp w: TMEM lanes 32 * (w % 4) (its q rows), key columns 32 * ((w - 2) / 4) of every tile.  Sixteen
//               softmax warps (four per scheduler) because the per-element chain scale -> exp2 -> subtract -> multiply
//               is latency-bound: with eight warps the 64 columns of a thread took 2200 cycles per tile, twice
//               what the exp2 pipe needs.
// TMEM columns: S 0, dP 128, dQ 256, Q 384, dO 448.
// dS of one thread's 32 columns of a tile: P = exp2(S c - lse), dS = P (dP - delta), packed in place into sv[0..15].
template <bool MASK>
__device__ __forceinline__ void dq_tile_math(const AttnParams& p, const SegInfo& s, uint32_t (&sv)[32],
                                             const uint32_t (&dv)[32], int fi, int col0, float sl2, float row_lse2,
                                             float row_delta) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float pa = exp2f(fmaf(__uint_as_float(sv[2 * i]), sl2, -row_lse2));
    float pb = exp2f(fmaf(__uint_as_float(sv[2 * i + 1]), sl2, -row_lse2));
    if (MASK) {
      if (!visible(p, s, fi, col0 + 2 * i)) pa = 0.f;
      if (!visible(p, s, fi, col0 + 2 * i + 1)) pb = 0.f;
    }
    sv[i] = pack_bf16(pa * (__uint_as_float(dv[2 * i]) - row_delta), pb * (__uint_as_float(dv[2 * i + 1]) - row_delta));
  }
}

constexpr int kDqThreads = 576;
constexpr int kDqSoftmaxThreads = 512;
constexpr int kDqStages = 3;
constexpr int kDqSmem = 3 * 2 * kTileBytes + kTileBytes + 1024 + 256;   // ring (stage 2 = Q | dO zone) + dS

__global__ void __launch_bounds__(kDqThreads, 1)
attn_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
               const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
               const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sRing = smem;                                   // stage s: K at +0, V at +kTileBytes
  uint8_t* sF = sRing + 2 * 2 * kTileBytes;                // Q | dO, later ring stage 2
  uint8_t* sDS = sRing + 3 * 2 * kTileBytes;               // dS [128 q][128 keys] bf16, two 64-key slabs
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + kTileBytes);
  uint64_t* f_full = bars;                 // Q, dO landed
  uint64_t* f_tmem = bars + 1;             // Q, dO copied into TMEM (one arrival per softmax warp)
  uint64_t* kv_full = bars + 2;            // [3]
  uint64_t* kv_empty = bars + 5;           // [3]
  uint64_t* sdp_full = bars + 8;           // S, dP of a tile are in TMEM
  uint64_t* s_free = bars + 9;             // the softmax threads hold them in registers (one arrival per warp)
  uint64_t* ds_full = bars + 10;           // dS of a tile is in shared memory (one arrival per warp)
  uint64_t* ds_empty = bars + 11;          // dQ += dS K of a tile has finished
  uint64_t* acc_full = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blk = static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);   // heavy causal blocks first
  const int seg = p.blk_seg[blk];
  if (seg < 0) return;
  const SegInfo s = seg_info(p, seg);
  const int row_abs0 = p.blk_row0[blk];
  const int f0 = row_abs0 - s.q_begin;           // first q row of the block inside the segment
  const int head = static_cast<int>(blockIdx.x);
  const int kvh = head / (p.hq / p.hkv);
  int g_hi = s.k_len;
  if (p.causal) g_hi = min(g_hi, f0 + kBM + s.off);
  const int g_lo = (p.window > 0) ? max(0, f0 + s.off - p.window + 1) : 0;
  const int tb0 = g_lo / kBN;
  const int iters = (g_hi > g_lo) ? (g_hi + kBN - 1) / kBN - tb0 : 0;

  if (threadIdx.x == 0) {
    mbar_init(f_full, 1);
    mbar_init(f_tmem, kDqSoftmaxThreads / 32);      // barriers count warps: see mbar_arrive_warp
    for (int i = 0; i < kDqStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(s_free, kDqSoftmaxThreads / 32);
    mbar_init(ds_full, kDqSoftmaxThreads / 32);
    mbar_init(ds_empty, 1);
    mbar_init(acc_full, 1);
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
  const uint32_t tmem = *tmem_slot;
  auto stage_ptr = [&](int st) -> uint8_t* { return st == 2 ? sF : sRing + st * 2 * kTileBytes; };

  if (warp == 0) {
    if (lane == 0 && iters > 0) {
      mbar_arrive_expect_tx(f_full, 2 * kTileBytes);
      load_tile(sF, &tmap_q, f_full, head, row_abs0);
      load_tile(sF + kTileBytes, &tmap_do, f_full, head, row_abs0);
      for (int it = 0; it < iters && !*abort_flag; ++it) {
        const int st = it % kDqStages;
        bool ok = mbar_wait(&kv_empty[st], ((it / kDqStages) & 1) ^ 1);
        if (ok && it == 2) ok = mbar_wait(f_tmem, 0);     // stage 2 is the Q | dO zone: free once they are in TMEM
        if (!ok) {
          report_error(p.status, kErrProducerWait);
          *abort_flag = 1;
          break;
        }
        uint8_t* dst = stage_ptr(st);
        const int krow = key_row(p, s.k_begin + (tb0 + it) * kBN);
        mbar_arrive_expect_tx(&kv_full[st], 2 * kTileBytes);
        load_tile(dst, &tmap_k, &kv_full[st], kvh, krow);
        load_tile(dst + kTileBytes, &tmap_v, &kv_full[st], kvh, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && iters > 0) {
      bool ok = mbar_wait(f_tmem, 0);
      auto issue_sdp = [&](int it) -> bool {
        const int st = it % kDqStages;
        if (!mbar_wait(&kv_full[st], (it / kDqStages) & 1)) return false;
        tc_fence_after();
        const uint32_t kv = smem_u32(stage_ptr(st));
        mma_128x128x128_ta<false>(tmem + 0, tmem + 384, kv, false);                  // S  = Q  K^T
        mma_128x128x128_ta<false>(tmem + 128, tmem + 448, kv + kTileBytes, false);   // dP = dO V^T
        umma_commit(sdp_full);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int it = 0; it < iters && ok && !*abort_flag; ++it) {
        if (it + 1 < iters) {
          ok = mbar_wait(s_free, it & 1);          // S, dP of tile `it` are in registers
          if (ok) { tc_fence_after(); ok = issue_sdp(it + 1); }
          if (!ok) break;
        }
        ok = mbar_wait(ds_full, it & 1);
        if (!ok) break;
        tc_fence_after();
        const int st = it % kDqStages;
        // dQ += dS K : A = dS (K-major over keys), B = K tile ([keys][D] -> MN-major)
        mma_128x128x128<false, true>(tmem + 256, smem_u32(sDS), smem_u32(stage_ptr(st)), it > 0);
        umma_commit(ds_empty);
        umma_commit(&kv_empty[st]);
      }
      if (ok) umma_commit(acc_full);
      if (!ok) { report_error(p.status, kErrMmaWaitFull); *abort_flag = 1; }
    }
  } else {
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;               // key columns [32 * part, +32) of every tile
    const int r = quarter * 32 + lane;              // q row of the block owned by this thread
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    const int fi = f0 + r;
    const long long q_abs = static_cast<long long>(row_abs0) + r;
    const bool frow_ok = (fi < s.q_len) && (q_abs < p.total_q);
    float row_lse2 = 0.f, row_delta = 0.f;
    if (frow_ok) {
      row_lse2 = p.LSE[static_cast<long long>(head) * p.total_q + q_abs] * kLog2e;
      row_delta = p.delta[static_cast<long long>(head) * p.total_q + q_abs];
    }
    bool ok = true;
    if (iters > 0) {
      // parts 0, 1 copy the two halves of their row of Q, parts 2, 3 of dO into TMEM (A operands of S and dP):
      // 64 columns of the row = one 128-byte slab row = 32 TMEM columns
      ok = mbar_wait(f_full, 0);
      {
        const uint8_t* src = sF + (part >> 1) * kTileBytes + (part & 1) * kSlabBytes;
        uint32_t w[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 x = *reinterpret_cast<const uint4*>(src + swz(r, c));
          w[c * 4] = x.x; w[c * 4 + 1] = x.y; w[c * 4 + 2] = x.z; w[c * 4 + 3] = x.w;
        }
        tmem_st_32x32(tmem + lane_addr + 384 + part * 32, w);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(f_tmem);
    }
    for (int it = 0; it < iters && ok; ++it) {
      const int g0 = (tb0 + it) * kBN;              // first key of the tile (segment relative)
      if (*abort_flag) { ok = false; break; }
      ok = __all_sync(0xffffffffu, mbar_wait(sdp_full, it & 1));
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[32], dv[32];
      tmem_ld_32x32(tmem + lane_addr + part * 32, sv);
      tmem_ld_32x32(tmem + lane_addr + 128 + part * 32, dv);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive_warp(s_free);                        // the products of the next tile may overwrite S and dP
      const bool need_mask = (f0 + kBM > s.q_len) || (g0 + kBN > s.k_len) || (g0 < s.k_skip) ||
                             (p.causal && g0 + kBN - 1 > f0 + s.off) ||
                             (p.window > 0 && g0 <= f0 + kBM - 1 + s.off - p.window);
      // in place: sv[i] becomes the packed pair of dS values of columns (2i, 2i+1); the masked variant only runs on
      // tiles that touch the diagonal, the window edge or the end of the segment
      if (!frow_ok) {
#pragma unroll
        for (int i = 0; i < 16; ++i) sv[i] = 0u;
      } else if (need_mask) {
        dq_tile_math<true>(p, s, sv, dv, fi, g0 + part * 32, sl2, row_lse2, row_delta);
      } else {
        dq_tile_math<false>(p, s, sv, dv, fi, g0 + part * 32, sl2, row_lse2, row_delta);
      }
      // the dS tile of the previous iteration must have been consumed (asked this late, it almost always has)
      if (it > 0) ok = __all_sync(0xffffffffu, mbar_wait(ds_empty, (it - 1) & 1));
      uint8_t* slab = sDS + (part >> 1) * kSlabBytes;      // 64 keys per slab, this thread's 32 keys = 4 chunks of 16 bytes
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4*>(slab + swz(r, (part & 1) * 4 + c)) = make_uint4(sv[c * 4], sv[c * 4 + 1], sv[c * 4 + 2], sv[c * 4 + 3]);
      fence_proxy_async_smem();
      mbar_arrive_warp(ds_full);
    }
    if (ok && iters > 0 && !*abort_flag) ok = mbar_wait(acc_full, 0);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) { report_error(p.status, kErrSoftmaxWait); *abort_flag = 1; }
    if (iters > 0) tc_fence_after();
    __nv_bfloat16* base = p.dQ + (q_abs * p.hq + head) * kD;
    {
      const int c = part;                           // each part stores 32 of the 128 columns of dQ
      uint32_t v[32];
      if (iters > 0 && ok) {
        tmem_ld_32x32(tmem + lane_addr + 256 + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * p.scale);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (frow_ok) {
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
    e = cudaFuncSetAttribute(attn_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDqSmem);
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
  // (a dK/dV pass with 128-row streamed tiles, P' and dS' kept in TMEM over S' and dP', was built and measured: its
  // products run at the full tensor rate, but with one S' / dP' buffer the softmax of a tile and the products
  // around it cannot overlap; 1 x 8192 backward 2.72 ms against 2.35 ms with this pass)
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
  // STB200_ATTN_DQ=1 selects the earlier dQ pass with 64-key tiles
  static const bool dq64 = [] { const char* e = getenv("STB200_ATTN_DQ"); return e != nullptr && e[0] == '1'; }();
  if (num_q_blocks > 0) {
    if (dq64) attn_bwd_kernel<false><<<dim3(hq, num_q_blocks), kBwdThreads, kBwdSmem, st>>>(q128, do128, k64, v64, p);
    else attn_dq_kernel<<<dim3(hq, num_q_blocks), kDqThreads, kDqSmem, st>>>(q128, do128, k128, v128, p);
  }
  return -static_cast<int>(cudaGetLastError());
}
