// Flash attention for sm_100a: packed variable-length sequences, causal and sliding-window masks,
// grouped-query heads, head_dim 128.  QK^T, PV and all five backward products run on tcgen05.mma
// with accumulators in TMEM; operands arrive by TMA (128-byte swizzle); softmax rows live one per
// thread (thread r of the four softmax warps owns TMEM lane r).
//
// Replaces the FlashAttention-2 / SDPA paths of the reference AttentionCore
// (steptronoss/model/common/attention_core.py:119-400) including its separate q / k segment
// tables (q rows of a segment are the last Lq of its Lk keys, as under context parallelism).
//
// Kernels
//   attn_fwd_kernel   : CTA = (q block of 128 rows, q head). Loop over key blocks: S = Q K^T (TMEM,
//                       double buffered) -> softmax threads -> P (bf16, smem) -> O += P V (TMEM), with
//                       the accumulator rescaled only when a row maximum moves by more than 2^8.
//                       Writes O and LSE.
//   attn_bwd_dq_kernel: same decomposition; per key block S and dP = dO V^T, dS = P o (dP - delta),
//                       dQ += dS K accumulated in TMEM.
//   attn_bwd_dkv_kernel: CTA = (key block of 128, kv head); loops over the q heads of the group and
//                       the q blocks that see this key block; dV += P^T dO, dK += dS^T Q in TMEM.
//   attn_delta_kernel : delta[h][t] = sum_d dO o O.
// S is recomputed in both backward kernels, which removes every atomic and makes the gradients
// deterministic.
#include "attention_common.cuh"

namespace stb {

// =============================================================================== forward / dQ
// MODE 0: forward.  MODE 1: dQ.
template <int MODE>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_rowblock_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                     const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // fwd : Q | K0 V0 | K1 V1 | P0 | P1              = 32 + 128 + 64 = 224 KB
  // dq  : Q | K0 V0 | K1 V1 | dO | dS              = 32 + 128 + 64 = 224 KB
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + kTileBytes;
  uint8_t* sX0 = sKV + 4 * kTileBytes;  // fwd: P0, dq: dO
  uint8_t* sX1 = sX0 + kTileBytes;      // fwd: P1, dq: dS
  uint64_t* bars = reinterpret_cast<uint64_t*>(sX1 + kTileBytes);
  uint64_t* q_full = bars;            // 1
  uint64_t* kv_full = bars + 1;       // 2
  uint64_t* kv_empty = bars + 3;      // 2
  uint64_t* s_full = bars + 5;        // 2
  uint64_t* p_full = bars + 7;        // 2
  uint64_t* pv_full = bars + 9;       // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x;
  // later q blocks of a causal document see more keys: launch them first so the tail of the grid is light
  const int blk = static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);
  const int seg = p.blk_seg[blk];
  if (seg < 0) return;  // uniform for the CTA, before any barrier or TMEM use
  const SegInfo s = seg_info(p, seg);
  const int q_abs0 = p.blk_row0[blk];
  const int q0 = q_abs0 - s.q_begin;
  const int kvh = head / (p.hq / p.hkv);
  int jb0, jb1;
  kv_range(p, s, q0, jb0, jb1);
  const int nkb = jb1 - jb0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&pv_full[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns. fwd: S0 0, S1 128, O 256.   dq: S 0, dP 128, dQ 256.

  if (warp == 0) {
    if (lane == 0 && nkb > 0) {
      const uint32_t qbytes = (MODE == 1) ? 2 * kTileBytes : kTileBytes;
      mbar_arrive_expect_tx(q_full, qbytes);
      load_tile(sQ, &tmap_q, q_full, head, q_abs0);
      if (MODE == 1) load_tile(sX0, &tmap_do, q_full, head, q_abs0);
      for (int j = 0; j < nkb && !*abort_flag; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1)) {
          report_error(p.status, kErrProducerWait);
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&kv_full[st], 2 * kTileBytes);
        const int krow = s.k_begin + (jb0 + j) * kBN;
        load_tile(sKV + st * 2 * kTileBytes, &tmap_k, &kv_full[st], kvh, krow);
        load_tile(sKV + st * 2 * kTileBytes + kTileBytes, &tmap_v, &kv_full[st], kvh, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nkb > 0) {
      bool ok = mbar_wait(q_full, 0);
      if (!ok) { report_error(p.status, kErrMmaWaitFull); *abort_flag = 1; }
      const uint32_t aQ = smem_u32(sQ);
      if (MODE == 0) {
        if (ok) {
          ok = mbar_wait(&kv_full[0], 0);
          if (ok) {
            tc_fence_after();
            mma_128x128x128<false, false>(tmem + 0, aQ, smem_u32(sKV), false);
            umma_commit(&s_full[0]);
          }
        }
        for (int j = 0; j < nkb && ok && !*abort_flag; ++j) {
          const int st = j & 1;
          if (j + 1 < nkb) {
            const int sn = (j + 1) & 1;
            ok = mbar_wait(&kv_full[sn], ((j + 1) >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            mma_128x128x128<false, false>(tmem + sn * 128, aQ, smem_u32(sKV + sn * 2 * kTileBytes), false);
            umma_commit(&s_full[sn]);
          }
          ok = mbar_wait(&p_full[st], (j >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          // O += P_j V_j : A = P (K-major over keys), B = V ([keys][D] -> MN-major)
          mma_128x128x128<false, true>(tmem + 256, smem_u32(st ? sX1 : sX0),
                                       smem_u32(sKV + st * 2 * kTileBytes + kTileBytes), j > 0);
          umma_commit(&pv_full[0]);
          umma_commit(&kv_empty[st]);
        }
      } else {
        for (int j = 0; j < nkb && ok && !*abort_flag; ++j) {
          const int st = j & 1;
          ok = mbar_wait(&kv_full[st], (j >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          const uint32_t aK = smem_u32(sKV + st * 2 * kTileBytes), aV = aK + kTileBytes;
          mma_128x128x128<false, false>(tmem + 0, aQ, aK, false);                // S  = Q K^T
          mma_128x128x128<false, false>(tmem + 128, smem_u32(sX0), aV, false);   // dP = dO V^T
          umma_commit(&s_full[0]);
          ok = mbar_wait(&p_full[0], j & 1);
          if (!ok) break;
          tc_fence_after();
          // dQ += dS K : A = dS (K-major over keys), B = K ([keys][D] -> MN-major)
          mma_128x128x128<false, true>(tmem + 256, smem_u32(sX1), aK, j > 0);
          umma_commit(&kv_empty[st]);
          if (j == nkb - 1) umma_commit(&pv_full[0]);
        }
      }
      if (!ok) { report_error(p.status, kErrMmaWaitFull); *abort_flag = 1; }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue threads
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;           // row of the block owned by this thread
    const int qi = q0 + r;                       // row inside the segment
    const long long q_abs = static_cast<long long>(q_abs0) + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    if (MODE == 0) {
      // The output accumulates in TMEM (PV issued with accumulate = 1). The exponent reference m_ref of a
      // row only moves when the row maximum outgrows it by more than kRescaleGap (in log2 units): until
      // then probabilities are at most 2^kRescaleGap, which fp32 accumulation and bf16 P hold without loss,
      // and the accumulator is left untouched.  When a row does move its reference, its warp reads the
      // accumulator rows back, scales them and stores them again before releasing P for the next PV.
      constexpr float kRescaleGap = 8.f;
      float m_ref = -INFINITY, l = 0.f;
      bool ok = true;
      for (int j = 0; j < nkb && ok && !*abort_flag; ++j) {
        const int st = j & 1;
        ok = mbar_wait(&s_full[st], (j >> 1) & 1);
        if (!ok) break;
        tc_fence_after();
        const int kb = (jb0 + j) * kBN;
        // a block needs element masks when it touches the diagonal, the window edge or the segment end
        const bool need_mask = (kb + kBN > s.k_len) || (p.causal && kb + kBN - 1 > q0 + s.off) ||
                               (p.window > 0 && kb <= q0 + kBM - 1 + s.off - p.window) || (q0 + kBM > s.q_len);
        uint32_t v[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t (&part)[32] = *reinterpret_cast<uint32_t (*)[32]>(&v[c * 32]);
          tmem_ld_32x32(tmem + lane_addr + st * 128 + c * 32, part);
        }
        tmem_wait_ld();
        float mx = -INFINITY;
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 128; ++i) {
            if (!visible(p, s, qi, kb + i)) v[i] = 0xff800000u;  // -inf
            mx = fmaxf(mx, __uint_as_float(v[i]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 128; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
        const float m_cand = mx * sl2;
        const bool moves = m_cand > m_ref + kRescaleGap || (m_ref == -INFINITY && m_cand > -INFINITY);
        if (__any_sync(0xffffffffu, moves)) {
          const float m_new = moves ? m_cand : m_ref;
          const float factor = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
          if (j > 0) {
            // every PV issued so far must have landed before the accumulator is rewritten
            ok = mbar_wait(&pv_full[0], (j - 1) & 1);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
              tmem_ld_32x32(tmem + lane_addr + 256 + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
              tmem_st_32x32(tmem + lane_addr + 256 + c * 32, o);
            }
            tmem_wait_st();
          }
          l *= factor;
          m_ref = m_new;
        }
        const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
        float rowsum = 0.f;
        uint8_t* sP = st ? sX1 : sX0;
#pragma unroll
        for (int c8 = 0; c8 < 16; ++c8) {  // 16 chunks of 8 keys = 16 bytes of bf16
          float pr[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            pr[i] = exp2f(__uint_as_float(v[c8 * 8 + i]) * sl2 - m_use);
            rowsum += pr[i];
          }
          uint8_t* slab = sP + (c8 >> 3) * kSlabBytes;
          *reinterpret_cast<uint4*>(slab + swz(r, c8 & 7)) =
              make_uint4(pack_bf16(pr[0], pr[1]), pack_bf16(pr[2], pr[3]), pack_bf16(pr[4], pr[5]), pack_bf16(pr[6], pr[7]));
        }
        l += rowsum;
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&p_full[st]);
      }
      float inv = 0.f;
      if (ok && nkb > 0 && !*abort_flag) {
        ok = mbar_wait(&pv_full[0], (nkb - 1) & 1);
        if (ok) tc_fence_after();
        inv = (l > 0.f) ? 1.f / l : 0.f;
      }
      if (!ok) { report_error(p.status, kErrSoftmaxWait); *abort_flag = 1; }
      const bool store_row = qi < s.q_len && q_abs < p.total_q;
      __nv_bfloat16* orow = p.O + (q_abs * p.hq + head) * kD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        if (nkb > 0 && ok) {
          tmem_ld_32x32(tmem + lane_addr + 256 + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (store_row) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + i) = w;
          }
        }
      }
      if (store_row)
        p.LSE[static_cast<long long>(head) * p.total_q + q_abs] = (l > 0.f) ? (m_ref * kLn2 + logf(l)) : -INFINITY;
    } else {
      // dQ mode
      const bool row_ok = (qi < s.q_len) && (q_abs < p.total_q);
      const float lse2 = row_ok ? p.LSE[static_cast<long long>(head) * p.total_q + q_abs] * kLog2e : 0.f;
      const float dl = row_ok ? p.delta[static_cast<long long>(head) * p.total_q + q_abs] : 0.f;
      bool ok = true;
      for (int j = 0; j < nkb && ok && !*abort_flag; ++j) {
        ok = mbar_wait(&s_full[0], j & 1);
        if (!ok) break;
        tc_fence_after();
        const int kb = (jb0 + j) * kBN;
#pragma unroll 1
        for (int hblk = 0; hblk < 2; ++hblk) {  // 64 keys per TMEM round trip
          uint32_t sv[64], dv[64];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t (&a)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sv[c * 32]);
            uint32_t (&b)[32] = *reinterpret_cast<uint32_t (*)[32]>(&dv[c * 32]);
            tmem_ld_32x32(tmem + lane_addr + hblk * 64 + c * 32, a);
            tmem_ld_32x32(tmem + lane_addr + 128 + hblk * 64 + c * 32, b);
          }
          tmem_wait_ld();
          uint8_t* slab = sX1 + hblk * kSlabBytes;
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            float d[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int col = c8 * 8 + i;
              d[i] = 0.f;
              if (row_ok && visible(p, s, qi, kb + hblk * 64 + col)) {
                const float pr = exp2f(__uint_as_float(sv[col]) * sl2 - lse2);
                d[i] = pr * (__uint_as_float(dv[col]) - dl) * p.scale;
              }
            }
            *reinterpret_cast<uint4*>(slab + swz(r, c8)) =
                make_uint4(pack_bf16(d[0], d[1]), pack_bf16(d[2], d[3]), pack_bf16(d[4], d[5]), pack_bf16(d[6], d[7]));
          }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&p_full[0]);
      }
      if (ok && nkb > 0 && !*abort_flag) ok = mbar_wait(&pv_full[0], 0);
      if (!ok) { report_error(p.status, kErrSoftmaxWait); *abort_flag = 1; }
      if (nkb > 0) tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        if (nkb > 0 && ok) {
          tmem_ld_32x32(tmem + lane_addr + 256 + c * 32, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (row_ok) {
          __nv_bfloat16* drow = p.dQ + (q_abs * p.hq + head) * kD + c * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
            o.y = pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
            o.z = pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
            o.w = pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
            *reinterpret_cast<uint4*>(drow + i) = o;
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

// =============================================================================== dK / dV
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                    const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTileBytes;
  uint8_t* sQ = sV + kTileBytes;
  uint8_t* sdO = sQ + kTileBytes;
  uint8_t* sP = sdO + kTileBytes;
  uint8_t* sdS = sP + kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + kTileBytes);
  uint64_t* kv_full = bars;       // K,V tile landed
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;  // S and dP in TMEM
  uint64_t* pds_full = bars + 4;  // P and dS in smem (128 arrivals)
  uint64_t* acc_full = bars + 5;  // all MMAs done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x;
  const int blk = blockIdx.y;
  const int seg = p.blk_seg[blk];
  if (seg < 0) return;
  const SegInfo s = seg_info(p, seg);
  const int k_abs0 = p.blk_row0[blk];
  const int k0 = k_abs0 - s.k_begin;
  const int group = p.hq / p.hkv;
  // q blocks that can see keys [k0, k0+128): causal -> q >= k0 - off ; window -> q <= k0+127 - off + window - 1
  int qlo = 0, qhi = s.q_len;
  if (p.causal) qlo = max(0, k0 - s.off);
  if (p.window > 0) qhi = min(s.q_len, k0 + kBN - 1 - s.off + p.window);
  const int ib0 = qlo / kBM;
  const int ib1 = (qhi > qlo) ? (qhi + kBM - 1) / kBM : ib0;
  const int nqb = ib1 - ib0;
  const int iters = nqb * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 128);
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
  const uint32_t tmem = *tmem_slot;  // S 0, dP 128, dV 256, dK 384

  if (warp == 0) {
    if (lane == 0 && iters > 0) {
      mbar_arrive_expect_tx(kv_full, 2 * kTileBytes);
      load_tile(sK, &tmap_k, kv_full, kvh, k_abs0);
      load_tile(sV, &tmap_v, kv_full, kvh, k_abs0);
      for (int it = 0; it < iters && !*abort_flag; ++it) {
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1)) {
          report_error(p.status, kErrProducerWait);
          *abort_flag = 1;
          break;
        }
        const int h = kvh * group + it / nqb;
        const int qrow = s.q_begin + (ib0 + it % nqb) * kBM;
        mbar_arrive_expect_tx(qdo_full, 2 * kTileBytes);
        load_tile(sQ, &tmap_q, qdo_full, h, qrow);
        load_tile(sdO, &tmap_do, qdo_full, h, qrow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && iters > 0) {
      bool ok = mbar_wait(kv_full, 0);
      for (int it = 0; it < iters && ok && !*abort_flag; ++it) {
        ok = mbar_wait(qdo_full, it & 1);
        if (!ok) break;
        tc_fence_after();
        mma_128x128x128<false, false>(tmem + 0, smem_u32(sQ), smem_u32(sK), false);     // S  = Q K^T
        mma_128x128x128<false, false>(tmem + 128, smem_u32(sdO), smem_u32(sV), false);  // dP = dO V^T
        umma_commit(sdp_full);
        ok = mbar_wait(pds_full, it & 1);
        if (!ok) break;
        tc_fence_after();
        // dV += P^T dO : A = P stored [q][keys] read as [K = q][M = keys]; B = dO stored [q][D]
        mma_128x128x128<true, true>(tmem + 256, smem_u32(sP), smem_u32(sdO), it > 0);
        // dK += dS^T Q
        mma_128x128x128<true, true>(tmem + 384, smem_u32(sdS), smem_u32(sQ), it > 0);
        umma_commit(qdo_empty);
      }
      if (ok) umma_commit(acc_full);
      if (!ok) { report_error(p.status, kErrMmaWaitFull); *abort_flag = 1; }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    bool ok = true;
    for (int it = 0; it < iters && ok && !*abort_flag; ++it) {
      const int h = kvh * group + it / nqb;
      const int q0 = (ib0 + it % nqb) * kBM;
      const int qi = q0 + r;
      const long long q_abs = static_cast<long long>(s.q_begin) + qi;
      const bool row_ok = (qi < s.q_len) && (q_abs < p.total_q);
      const float lse2 = row_ok ? p.LSE[static_cast<long long>(h) * p.total_q + q_abs] * kLog2e : 0.f;
      const float dl = row_ok ? p.delta[static_cast<long long>(h) * p.total_q + q_abs] : 0.f;
      ok = mbar_wait(sdp_full, it & 1);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int hblk = 0; hblk < 2; ++hblk) {  // 64 keys per TMEM round trip
        uint32_t sv[64], dv[64];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t (&a)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sv[c * 32]);
          uint32_t (&b)[32] = *reinterpret_cast<uint32_t (*)[32]>(&dv[c * 32]);
          tmem_ld_32x32(tmem + lane_addr + hblk * 64 + c * 32, a);
          tmem_ld_32x32(tmem + lane_addr + 128 + hblk * 64 + c * 32, b);
        }
        tmem_wait_ld();
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
          float pv[8], dd[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int col = c8 * 8 + i;
            pv[i] = 0.f;
            dd[i] = 0.f;
            if (row_ok && visible(p, s, qi, k0 + hblk * 64 + col)) {
              pv[i] = exp2f(__uint_as_float(sv[col]) * sl2 - lse2);
              dd[i] = pv[i] * (__uint_as_float(dv[col]) - dl) * p.scale;
            }
          }
          const uint32_t a = hblk * kSlabBytes + swz(r, c8);
          *reinterpret_cast<uint4*>(sP + a) =
              make_uint4(pack_bf16(pv[0], pv[1]), pack_bf16(pv[2], pv[3]), pack_bf16(pv[4], pv[5]), pack_bf16(pv[6], pv[7]));
          *reinterpret_cast<uint4*>(sdS + a) =
              make_uint4(pack_bf16(dd[0], dd[1]), pack_bf16(dd[2], dd[3]), pack_bf16(dd[4], dd[5]), pack_bf16(dd[6], dd[7]));
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_full);
    }
    if (ok && iters > 0 && !*abort_flag) ok = mbar_wait(acc_full, 0);
    if (!ok) { report_error(p.status, kErrSoftmaxWait); *abort_flag = 1; }
    if (iters > 0) tc_fence_after();
    // thread r owns key row r of this block
    const int kk = k0 + r;
    const long long k_abs = static_cast<long long>(k_abs0) + r;
    const bool key_ok = (kk < s.k_len) && (k_abs < p.total_k);
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* base = which == 0 ? p.dV + k_abs * p.dv_stride + static_cast<long long>(kvh) * kD
                                       : p.dK + (k_abs * p.hkv + kvh) * kD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        if (iters > 0 && ok) {
          tmem_ld_32x32(tmem + lane_addr + 256 + which * 128 + c * 32, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (key_ok) {
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

// delta[h][t] = sum_d dO[t][h][d] * O[t][h][d]; one warp per (t, h)
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO, float* __restrict__ delta,
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

constexpr int kAttnSmem = 7 * kTileBytes + 1024 + 256;      // fwd / dq
constexpr int kAttnSmemDkv = 6 * kTileBytes + 1024 + 256;   // dkv

int make_head_map(CUtensorMap* m, const void* base, int heads, long long rows, long long row_stride_elems, int box_rows) {
  // dims: D (inner), heads, rows; a box is 64 columns of one head for 128 rows
  return make_tmap_3d_bf16(m, base, kD, heads, rows, static_cast<uint64_t>(kD) * 2,
                           static_cast<uint64_t>(row_stride_elems) * 2, 64, 1, box_rows, 1);
}

}  // namespace stb

using namespace stb;

// q [Tq][hq][D] with row stride q_stride (elements); k, v [Tk][hkv][D] with row strides k_stride, v_stride.
// blk_seg / blk_row0: schedule of q blocks (num_blocks entries, seg < 0 = unused).
extern "C" int stb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_q,
                            const int* cu_k, const int* blk_seg, const int* blk_row0, int num_blocks, int total_q,
                            int total_k, int hq, int hkv, int head_dim, long long q_stride, long long k_stride,
                            long long v_stride, int causal, int window, float scale, int* status, cudaStream_t st) {
  if (num_blocks <= 0 || total_q <= 0) return 0;
  if (head_dim != kD || hq % hkv) return -kErrBadArgument;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_head_map(&tq, q, hq, total_q, q_stride, 128))) return r;
  if ((r = make_head_map(&tk, k, hkv, total_k, k_stride, 128))) return r;
  if ((r = make_head_map(&tv, v, hkv, total_k, v_stride, 128))) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_rowblock_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
    if (e != cudaSuccess) return -static_cast<int>(e);
    configured = true;
  }
  AttnParams p{};
  p.cu_q = cu_q; p.cu_k = cu_k; p.blk_seg = blk_seg; p.blk_row0 = blk_row0;
  p.hq = hq; p.hkv = hkv; p.causal = causal; p.window = window; p.scale = scale;
  p.total_q = total_q; p.total_k = total_k;
  p.O = static_cast<__nv_bfloat16*>(o); p.LSE = lse; p.status = status;
  attn_rowblock_kernel<0><<<dim3(hq, num_blocks), kAttnThreads, kAttnSmem, st>>>(tq, tk, tv, tq, p);
  return -static_cast<int>(cudaGetLastError());
}

// Backward. dq [Tq][hq][D], dk [Tk][hkv][D] contiguous; dv rows with stride dv_stride.
// q_blk_*: schedule over q blocks; k_blk_*: schedule over key blocks. delta: scratch [hq][Tq] floats.
extern "C" int stb_attn_bwd_legacy(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, float* delta, void* dq, void* dk, void* dv, const int* cu_q,
                            const int* cu_k, const int* q_blk_seg, const int* q_blk_row0, int num_q_blocks,
                            const int* k_blk_seg, const int* k_blk_row0, int num_k_blocks, int total_q, int total_k,
                            int hq, int hkv, int head_dim, long long q_stride, long long k_stride, long long v_stride,
                            long long dv_stride, int causal, int window, float scale, int* status, cudaStream_t st) {
  if (total_q <= 0 || total_k <= 0) return 0;
  if (head_dim != kD || hq % hkv) return -kErrBadArgument;
  CUtensorMap tq, tk, tv, tdo;
  int r;
  if ((r = make_head_map(&tq, q, hq, total_q, q_stride, 128))) return r;
  if ((r = make_head_map(&tk, k, hkv, total_k, k_stride, 128))) return r;
  if ((r = make_head_map(&tv, v, hkv, total_k, v_stride, 128))) return r;
  if ((r = make_head_map(&tdo, d_o, hq, total_q, static_cast<long long>(hq) * kD, 128))) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_rowblock_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
    if (e != cudaSuccess) return -static_cast<int>(e);
    e = cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmemDkv);
    if (e != cudaSuccess) return -static_cast<int>(e);
    configured = true;
  }
  const long long warps = static_cast<long long>(total_q) * hq;
  attn_delta_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, total_q, hq);
  AttnParams p{};
  p.cu_q = cu_q; p.cu_k = cu_k;
  p.hq = hq; p.hkv = hkv; p.causal = causal; p.window = window; p.scale = scale;
  p.total_q = total_q; p.total_k = total_k;
  p.LSE = const_cast<float*>(lse); p.delta = delta;
  p.dQ = static_cast<__nv_bfloat16*>(dq); p.dK = static_cast<__nv_bfloat16*>(dk);
  p.dV = static_cast<__nv_bfloat16*>(dv); p.dv_stride = dv_stride; p.status = status;
  p.blk_seg = q_blk_seg; p.blk_row0 = q_blk_row0;
  if (num_q_blocks > 0)
    attn_rowblock_kernel<1><<<dim3(hq, num_q_blocks), kAttnThreads, kAttnSmem, st>>>(tq, tk, tv, tdo, p);
  p.blk_seg = k_blk_seg; p.blk_row0 = k_blk_row0;
  if (num_k_blocks > 0)
    attn_bwd_dkv_kernel<<<dim3(hkv, num_k_blocks), kAttnThreads, kAttnSmemDkv, st>>>(tq, tk, tv, tdo, p);
  return -static_cast<int>(cudaGetLastError());
}
