// Flash attention forward for sm_100a: packed variable-length sequences, causal and sliding-window
// masks, grouped-query heads, head_dim 128.  QK^T and PV run on tcgen05.mma with accumulators in TMEM;
// operands arrive by TMA (128-byte swizzle).
//
// Replaces the FlashAttention-2 / SDPA paths of the reference AttentionCore
// (steptronoss/model/common/attention_core.py:119-400) including its separate q / k segment tables
// (q rows of a segment are the last Lq of its Lk keys, as under context parallelism).
//
// CTA = (q block of 128 rows, q head), 320 threads:
//   warp 0      TMA producer: Q once, then K/V tiles of 128 keys through a 2-stage ring
//   warp 1      MMA issuer: S_j = Q K_j^T into one of two TMEM buffers, O += P_j V_j
//   warps 2..9  softmax: two warps per TMEM lane quarter, each thread owns one row and one half
//               (64 keys) of every S tile, so every scheduler always has two softmax warps to
//               alternate between.  The two halves of a row exchange their partial maximum through
//               shared memory once per tile.
// The output accumulates in TMEM.  A row's exponent reference only moves when its maximum outgrows
// it by more than 2^8; only then are the accumulator rows read back, scaled and stored again.
// The backward kernels live in attention_bwd_sm100.cu.
#include "attention_common.cuh"

#include <cstdlib>

namespace stb {

constexpr int kFwdThreads = 320;
constexpr int kFwdXchgBytes = 2 * 2 * 128 * 2;   // [parity][half][row] bf16 partial maxima (reused for the final sums)
constexpr int kFwdSmem = 7 * kTileBytes + 1024 + kFwdXchgBytes + 128;

__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // Q | K0 V0 | K1 V1 | P0 | P1 = 32 + 128 + 64 = 224 KB
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + kTileBytes;
  uint8_t* sP0 = sKV + 4 * kTileBytes;
  uint8_t* sP1 = sP0 + kTileBytes;
  __nv_bfloat16* xchg = reinterpret_cast<__nv_bfloat16*>(sP1 + kTileBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xchg) + kFwdXchgBytes);
  uint64_t* q_full = bars;            // 1
  uint64_t* kv_full = bars + 1;       // 2
  uint64_t* kv_empty = bars + 3;      // 2
  uint64_t* s_full = bars + 5;        // 2
  uint64_t* p_full = bars + 7;        // 2
  uint64_t* pv_done = bars + 9;       // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
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
      mbar_init(&p_full[i], 8);      // one arrival per softmax warp
    }
    mbar_init(pv_done, 1);
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
  const uint32_t tmem = *tmem_slot;  // columns: S0 0, S1 128, O 256

  if (warp == 0) {
    if (lane == 0 && nkb > 0) {
      mbar_arrive_expect_tx(q_full, kTileBytes);
      load_tile(sQ, &tmap_q, q_full, head, q_abs0);
      for (int j = 0; j < nkb && !*abort_flag; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1)) {
          report_error(p.status, kErrProducerWait);
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&kv_full[st], 2 * kTileBytes);
        const int krow = key_row(p, s.k_begin + (jb0 + j) * kBN);
        load_tile(sKV + st * 2 * kTileBytes, &tmap_k, &kv_full[st], kvh, krow);
        load_tile(sKV + st * 2 * kTileBytes + kTileBytes, &tmap_v, &kv_full[st], kvh, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nkb > 0) {
      bool ok = mbar_wait(q_full, 0);
      const uint32_t aQ = smem_u32(sQ);
      if (ok) ok = mbar_wait(&kv_full[0], 0);
      if (ok) {
        tc_fence_after();
        mma_128x128x128<false, false>(tmem + 0, aQ, smem_u32(sKV), false);
        umma_commit(&s_full[0]);
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
        mma_128x128x128<false, true>(tmem + 256, smem_u32(st ? sP1 : sP0),
                                     smem_u32(sKV + st * 2 * kTileBytes + kTileBytes), j > 0);
        umma_commit(pv_done);
        umma_commit(&kv_empty[st]);
      }
      if (!ok) { report_error(p.status, kErrMmaWaitFull); *abort_flag = 1; }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue threads
    const int quarter = warp & 3;                // TMEM lanes [32*quarter, +32)
    const int half = (warp - 2) >> 2;            // keys [64*half, +64) of every tile, O columns likewise
    const int r = quarter * 32 + lane;           // row of the block owned by this thread
    const int qi = q0 + r;                       // row inside the segment
    const long long q_abs = static_cast<long long>(q_abs0) + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    constexpr float kRescaleGap = 8.f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    // Every softmax thread runs all nkb iterations and meets its row partner at one named barrier per
    // iteration, whatever happens: after a timed-out wait (ok == false) the remaining waits are skipped
    // and the iterations only keep the barrier counts aligned, so a failure can never strand a partner.
    for (int j = 0; j < nkb; ++j) {
      const int st = j & 1;
      if (*abort_flag) ok = false;
      if (ok) ok = mbar_wait(&s_full[st], (j >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);             // warp-wide TMEM loads and the warp's single arrival follow
      if (!ok) {
        asm volatile("bar.sync 1, 256;" ::: "memory");
        continue;
      }
      tc_fence_after();
      const int kb = (jb0 + j) * kBN + half * 64;  // first key of this thread's 64 columns
      // a tile needs element masks when it touches the diagonal, the window edge or the segment end
      const int kt = (jb0 + j) * kBN;
      const bool need_mask = (kt + kBN > s.k_len) || (kt < s.k_skip) || (p.causal && kt + kBN - 1 > q0 + s.off) ||
                             (p.window > 0 && kt <= q0 + kBM - 1 + s.off - p.window) || (q0 + kBM > s.q_len);
      uint32_t v[64];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t (&part)[32] = *reinterpret_cast<uint32_t (*)[32]>(&v[c * 32]);
        tmem_ld_32x32(tmem + lane_addr + st * 128 + half * 64 + c * 32, part);
      }
      tmem_wait_ld();
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (!visible(p, s, qi, kb + i)) v[i] = 0xff800000u;  // -inf
      }
      // eight independent chains instead of one of 64 dependent maxima
      float mx8[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx8[i] = __uint_as_float(v[i]);
#pragma unroll
      for (int i = 8; i < 64; ++i) mx8[i & 7] = fmaxf(mx8[i & 7], __uint_as_float(v[i]));
      float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
      // exchange the partial maximum with the thread that owns the other half of this row; both use the
      // bf16-rounded values so that they arrive at the same reference
      __nv_bfloat16* slot = xchg + (j & 1) * 256;
      const __nv_bfloat16 mine = __float2bfloat16_rn(mx);
      slot[half * 128 + r] = mine;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mx = fmaxf(__bfloat162float(mine), __bfloat162float(slot[(half ^ 1) * 128 + r]));
      const float m_cand = mx * sl2;
      const bool moves = m_cand > m_ref + kRescaleGap || (m_ref == -INFINITY && m_cand > -INFINITY);
      if (__any_sync(0xffffffffu, moves)) {
        const float m_new = moves ? m_cand : m_ref;
        const float factor = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
        if (j > 0) {
          // every PV issued so far must have landed before the accumulator is rewritten
          ok = mbar_wait(pv_done, (j - 1) & 1);
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < (ok ? 2 : 0); ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem + lane_addr + 256 + half * 64 + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tmem_st_32x32(tmem + lane_addr + 256 + half * 64 + c * 32, o);
          }
          tmem_wait_st();
        }
        l *= factor;
        m_ref = m_new;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      float rs8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};   // independent partial sums (no 64-long add chain)
      uint8_t* slab = (st ? sP1 : sP0) + half * kSlabBytes;  // 64 keys = one 128-byte-wide slab
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {  // 8 chunks of 8 keys = 16 bytes of bf16
        float pr[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          pr[i] = exp2f(fmaf(__uint_as_float(v[c8 * 8 + i]), sl2, -m_use));
          rs8[i] += pr[i];
        }
        *reinterpret_cast<uint4*>(slab + swz(r, c8)) =
            make_uint4(pack_bf16(pr[0], pr[1]), pack_bf16(pr[2], pr[3]), pack_bf16(pr[4], pr[5]), pack_bf16(pr[6], pr[7]));
      }
      l += ((rs8[0] + rs8[1]) + (rs8[2] + rs8[3])) + ((rs8[4] + rs8[5]) + (rs8[6] + rs8[7]));
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive_warp(&p_full[st]);
    }
    // total row sum = sum of the two halves (fp32 exchange through the same scratch, viewed as floats)
    float* fx = reinterpret_cast<float*>(xchg);
    asm volatile("bar.sync 1, 256;" ::: "memory");  // nobody still reads the last maxima
    fx[half * 128 + r] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const float l_tot = l + fx[(half ^ 1) * 128 + r];
    float inv = 0.f;
    if (ok && nkb > 0 && !*abort_flag) {
      ok = mbar_wait(pv_done, (nkb - 1) & 1);
      if (ok) tc_fence_after();
      inv = (l_tot > 0.f) ? 1.f / l_tot : 0.f;
    }
    if (!ok) { report_error(p.status, kErrSoftmaxWait); *abort_flag = 1; }
    const bool store_row = qi < s.q_len && q_abs < p.total_q;
    __nv_bfloat16* orow = p.O + (q_abs * p.hq + head) * kD + half * 64;
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      uint32_t o[32];
      if (nkb > 0 && ok) {
        tmem_ld_32x32(tmem + lane_addr + 256 + half * 64 + c * 32, o);
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
    if (store_row && half == 0)
      p.LSE[static_cast<long long>(head) * p.total_q + q_abs] =
          (l_tot > 0.f) ? (m_ref * kLn2 + logf(l_tot)) : -INFINITY;
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


// ---------------------------------------------------------------------------------------------------------------
// Forward, two q heads per CTA.
//
// The two heads belong to the same kv head (grouped-query attention) and cover the same 128 q rows, so they share
// every K / V tile, the key range and the masks.  While the softmax warps of one head work on S_j, the tensor pipe
// runs P V and the next Q K^T of the other head:
//
//   warp 0      TMA producer: both Q tiles once, then K_j, V_j through a 4-stage ring of 32 KB tiles
//   warp 1      MMA issuer, per key tile and head t:  O_t += P_t V_j ;  S_t = Q_t K_{j+1}^T
//   warps 2..5  softmax of head 0, warps 6..9 softmax of head 1: one thread per row, the whole row of 128 keys
//               in registers, so a row's maximum and sum need no exchange between threads
//
// P never touches shared memory: a softmax thread stores its bf16 row over the first 64 columns of its own S row
// in TMEM, and P V takes its A operand from there.  tcgen05.mma of one thread run in issue order, so the Q K^T
// that overwrites S_t is issued right behind the P V that reads P_t; the commit behind that Q K^T therefore also
// tells the softmax warps that every earlier P V of the head has landed, which is what the (rare) rescale of the
// output accumulator needs.  TMEM columns: S0 0, S1 128, O0 256, O1 384.
constexpr int kFwd2Threads = 320;
constexpr int kFwd2Stages = 4;
constexpr int kFwd2Smem = (2 + kFwd2Stages) * kTileBytes + 1024 + 256;

__global__ void __launch_bounds__(kFwd2Threads, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                            // Q of head 0 | Q of head 1
  uint8_t* sKV = smem + 2 * kTileBytes;          // ring: K_0 V_0 K_1 V_1 ...
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + kFwd2Stages * kTileBytes);
  uint64_t* q_full = bars;                       // 1
  uint64_t* kv_full = bars + 1;                  // kFwd2Stages
  uint64_t* kv_empty = kv_full + kFwd2Stages;    // kFwd2Stages
  uint64_t* s_full = kv_empty + kFwd2Stages;     // 2
  uint64_t* p_full = s_full + 2;                 // 2
  uint64_t* o_done = p_full + 2;                 // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head0 = blockIdx.x * 2;
  const int blk = static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);   // heavy causal blocks first
  const int seg = p.blk_seg[blk];
  if (seg < 0) return;  // uniform for the CTA, before any barrier or TMEM use
  const SegInfo s = seg_info(p, seg);
  const int q_abs0 = p.blk_row0[blk];
  const int q0 = q_abs0 - s.q_begin;
  const int kvh = head0 / (p.hq / p.hkv);
  int jb0, jb1;
  kv_range(p, s, q0, jb0, jb1);
  const int nkb = jb1 - jb0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kFwd2Stages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);      // one arrival per softmax warp of the head
      mbar_init(&o_done[i], 1);
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

  if (warp == 0) {
    if (lane == 0 && nkb > 0) {
      mbar_arrive_expect_tx(q_full, 2 * kTileBytes);
      load_tile(sQ, &tmap_q, q_full, head0, q_abs0);
      load_tile(sQ + kTileBytes, &tmap_q, q_full, head0 + 1, q_abs0);
      for (int i = 0; i < 2 * nkb && !*abort_flag; ++i) {   // item 2j = K_j, item 2j+1 = V_j
        const int st = i % kFwd2Stages;
        if (!mbar_wait(&kv_empty[st], ((i / kFwd2Stages) & 1) ^ 1)) {
          report_error(p.status, kErrProducerWait);
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&kv_full[st], kTileBytes);
        const int krow = key_row(p, s.k_begin + (jb0 + (i >> 1)) * kBN);
        load_tile(sKV + st * kTileBytes, (i & 1) ? &tmap_v : &tmap_k, &kv_full[st], kvh, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nkb > 0) {
      const uint32_t aQ = smem_u32(sQ);
      bool ok = mbar_wait(q_full, 0);
      if (ok) ok = mbar_wait(&kv_full[0], 0);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t) {
          mma_128x128x128<false, false>(tmem + t * 128, aQ + t * kTileBytes, smem_u32(sKV), false);
          umma_commit(&s_full[t]);
        }
        umma_commit(&kv_empty[0]);
      }
      for (int j = 0; j < nkb && ok && !*abort_flag; ++j) {
        const int iv = 2 * j + 1, ik = 2 * j + 2;               // ring items of V_j and K_{j+1}
        const int sv = iv % kFwd2Stages, sk = ik % kFwd2Stages;
        const bool more = j + 1 < nkb;
        ok = mbar_wait(&kv_full[sv], (iv / kFwd2Stages) & 1);
        if (ok && more) ok = mbar_wait(&kv_full[sk], (ik / kFwd2Stages) & 1);
        const uint32_t aV = smem_u32(sKV + sv * kTileBytes), aK = smem_u32(sKV + sk * kTileBytes);
        for (int t = 0; t < 2 && ok; ++t) {
          ok = mbar_wait(&p_full[t], j & 1);
          if (!ok) break;
          tc_fence_after();
          // O_t += P_t V_j : A = P_t in TMEM (16 keys = 8 columns per step), B = V ([keys][D], MN-major)
          mma_128x128x128_ta<true>(tmem + 256 + t * 128, tmem + t * 128, aV, j > 0);
          if (more) {
            mma_128x128x128<false, false>(tmem + t * 128, aQ + t * kTileBytes, aK, false);
            umma_commit(&s_full[t]);
          } else {
            umma_commit(&o_done[t]);
          }
        }
        if (ok) {
          umma_commit(&kv_empty[sv]);
          if (more) umma_commit(&kv_empty[sk]);
        }
      }
      if (!ok) { report_error(p.status, kErrMmaWaitFull); *abort_flag = 1; }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue threads
    const int t = (warp - 2) >> 2;               // which of the two heads
    const int quarter = warp & 3;                // TMEM lanes [32*quarter, +32)
    const int r = quarter * 32 + lane;           // row of the block owned by this thread
    const int qi = q0 + r;                       // row inside the segment
    const int head = head0 + t;
    const long long q_abs = static_cast<long long>(q_abs0) + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_addr + t * 128, tO = tmem + lane_addr + 256 + t * 128;
    const float sl2 = p.scale * kLog2e;
    constexpr float kRescaleGap = 8.f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nkb && ok; ++j) {
      if (*abort_flag) { ok = false; break; }
      ok = mbar_wait(&s_full[t], j & 1);
      if (!ok) break;
      tc_fence_after();
      const int kt = (jb0 + j) * kBN;            // first key of the tile
      // a tile needs element masks when it touches the diagonal, the window edge or the segment end
      const bool need_mask = (kt + kBN > s.k_len) || (kt < s.k_skip) || (p.causal && kt + kBN - 1 > q0 + s.off) ||
                             (p.window > 0 && kt <= q0 + kBM - 1 + s.off - p.window) || (q0 + kBM > s.q_len);
      uint32_t v[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t (&part)[32] = *reinterpret_cast<uint32_t (*)[32]>(&v[c * 32]);
        tmem_ld_32x32(tS + c * 32, part);
      }
      tmem_wait_ld();
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (!visible(p, s, qi, kt + i)) v[i] = 0xff800000u;  // -inf
      }
      float mx8[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx8[i] = __uint_as_float(v[i]);
#pragma unroll
      for (int i = 8; i < 128; ++i) mx8[i & 7] = fmaxf(mx8[i & 7], __uint_as_float(v[i]));
      const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                             fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
      const float m_cand = mx * sl2;
      const bool moves = m_cand > m_ref + kRescaleGap || (m_ref == -INFINITY && m_cand > -INFINITY);
      if (__any_sync(0xffffffffu, moves)) {
        const float m_new = moves ? m_cand : m_ref;
        const float factor = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
        if (j > 0) {   // every P V of this head issued so far has landed (see the note above the kernel)
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tO + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tmem_st_32x32(tO + c * 32, o);
          }
        }
        l *= factor;
        m_ref = m_new;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      float rs8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int h = 0; h < 2; ++h) {              // 64 keys -> 32 columns of packed bf16
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float a = exp2f(fmaf(__uint_as_float(v[h * 64 + 2 * i]), sl2, -m_use));
          const float b = exp2f(fmaf(__uint_as_float(v[h * 64 + 2 * i + 1]), sl2, -m_use));
          rs8[i & 7] += a + b;
          pk[i] = pack_bf16(a, b);
        }
        tmem_st_32x32(tS + h * 32, pk);
      }
      l += ((rs8[0] + rs8[1]) + (rs8[2] + rs8[3])) + ((rs8[4] + rs8[5]) + (rs8[6] + rs8[7]));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(&p_full[t]);
    }
    float inv = 0.f;
    if (ok && nkb > 0 && !*abort_flag) {
      ok = mbar_wait(&o_done[t], 0);
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
        tmem_ld_32x32(tO + c * 32, o);
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


int make_head_map(CUtensorMap* m, const void* base, int heads, long long rows, long long row_stride_elems, int box_rows) {
  // dims: D (inner), heads, rows; a box is 64 columns of one head for box_rows rows
  return make_tmap_3d_bf16(m, base, kD, heads, rows, static_cast<uint64_t>(kD) * 2,
                           static_cast<uint64_t>(row_stride_elems) * 2, 64, 1, box_rows, 1);
}

}  // namespace stb

using namespace stb;

// q [Tq][hq][D] with row stride q_stride (elements); k, v [Tk][hkv][D] with row strides k_stride, v_stride.
// blk_seg / blk_row0: schedule of q blocks (num_blocks entries, seg < 0 = unused).
// seg_k_begin / seg_k_len / seg_k_skip (optional, with cp and chunk_len): keys addressed by global position in a
// rank-major [cp][2*chunk_len] buffer, see AttnParams; cu_k is then unused.
extern "C" int stb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_q,
                            const int* cu_k, const int* blk_seg, const int* blk_row0, int num_blocks, int total_q,
                            int total_k, int hq, int hkv, int head_dim, long long q_stride, long long k_stride,
                            long long v_stride, int causal, int window, float scale, const int* seg_k_begin,
                            const int* seg_k_len, const int* seg_k_skip, int cp, int chunk_len, int* status,
                            cudaStream_t st) {
  if (num_blocks <= 0 || total_q <= 0) return 0;
  if (head_dim != kD || hq % hkv) return -kErrBadArgument;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_head_map(&tq, q, hq, total_q, q_stride, 128))) return r;
  if ((r = make_head_map(&tk, k, hkv, total_k, k_stride, 128))) return r;
  if ((r = make_head_map(&tv, v, hkv, total_k, v_stride, 128))) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem);
    if (e != cudaSuccess) return -static_cast<int>(e);
    configured = true;
  }
  AttnParams p{};
  p.cu_q = cu_q; p.cu_k = cu_k; p.blk_seg = blk_seg; p.blk_row0 = blk_row0;
  p.hq = hq; p.hkv = hkv; p.causal = causal; p.window = window; p.scale = scale;
  p.total_q = total_q; p.total_k = total_k;
  p.O = static_cast<__nv_bfloat16*>(o); p.LSE = lse; p.status = status;
  if (seg_k_begin != nullptr) {
    if (cp < 1 || chunk_len <= 0 || (chunk_len % kBN) || seg_k_len == nullptr || seg_k_skip == nullptr)
      return -kErrBadArgument;
    p.seg_k_begin = seg_k_begin; p.seg_k_len = seg_k_len; p.seg_k_skip = seg_k_skip; p.cp = cp; p.chunk_len = chunk_len;
  }
  // two q heads of one kv head per CTA whenever the group size allows it; STB200_ATTN_FWD=1 keeps one head per CTA
  static const bool one_head = [] { const char* e = getenv("STB200_ATTN_FWD"); return e != nullptr && e[0] == '1'; }();
  if (!one_head && (hq / hkv) % 2 == 0) {
    static bool configured2 = false;
    if (!configured2) {
      cudaError_t e = cudaFuncSetAttribute(attn_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwd2Smem);
      if (e != cudaSuccess) return -static_cast<int>(e);
      configured2 = true;
    }
    attn_fwd2_kernel<<<dim3(hq / 2, num_blocks), kFwd2Threads, kFwd2Smem, st>>>(tq, tk, tv, p);
  } else {
    attn_fwd_kernel<<<dim3(hq, num_blocks), kFwdThreads, kFwdSmem, st>>>(tq, tk, tv, p);
  }
  return -static_cast<int>(cudaGetLastError());
}
