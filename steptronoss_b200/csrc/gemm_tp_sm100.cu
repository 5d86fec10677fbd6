// Sequence-parallel projections as single kernels over NVLink peer memory (sm_100a).
//
//   gemm_ag_kernel : C = all_gather_rows(x) * B^T.   The gathered matrix lives in symmetric memory.  Four
//                    "comm" warps in every CTA push this rank's rows, 16-row slices at a time, straight into
//                    every peer's gathered buffer (plain 16-byte peer stores: posted writes keep NVLink busy, a
//                    few thousand threads saturate the links, and a slice is complete after one fence) and raise
//                    a per-row-tile flag on the peer when a tile is complete.  The TMA producer of the tcgen05
//                    GEMM waits for the flag of the row tile it is about to load, so products of rows that have
//                    arrived overlap the transfer of the rest.  Own rows are multiplied first (read where the
//                    caller left them); the peers' row tiles follow in the order they arrive (every peer pushes
//                    its tiles in ascending order to all ranks at once: tile i of every peer, then tile i+1).
//   gemm_rs_kernel : out = reduce_scatter_rows(A * B^T).  The epilogue TMA-stores every bf16 partial tile into a
//                    local staging matrix, at full speed: no store of the tensor pipeline's critical path ever
//                    crosses NVLink.  The four extra warps of every CTA forward finished row tiles that another
//                    rank owns into that rank's receive slot (plain peer stores, a flag per tile) and add the tp
//                    partial copies of the row tiles this rank owns in fixed rank order (fp32), the own partial
//                    straight out of the staging matrix.  Row blocks are computed next-rank first, own block
//                    last, and the forwarding / reduction units are handed out in that same order.
//
// They replace the NCCL collective + cuBLAS pairs of the reference's sequence-parallel linears
// (steptronoss/core/tensor_parallel/layers.py:151-346, mappings.py:103-300).
//
// Cross-rank protocol.  Flags are uint32 words in each rank's symmetric flag page, written into the peer's
// page with st.release.sys and polled in the own page (relaxed loads, one acquire fence after the poll that
// succeeds); they carry the call number ("epoch", compared wrap-safe), so nothing is ever reset.  Gathered and
// receive buffers have two slots used alternately by epoch parity.  A slot written in call e was last read in
// call e-2 (and by what the caller ran right after it), and no rank can leave call e-1 before every peer has
// entered call e-1 (each call consumes data that every peer produces inside the same call), so two slots need no
// further hand-shake.  GEMM tiles and the work of the extra warps are claimed from device counters, not assigned
// by CTA index, so progress never depends on a CTA that is not resident (for instance while a collective of
// another stream holds some SMs and is itself waiting for the peer).  Every wait is bounded by the caller's
// budget; on time-out the kernel records a code in the status word, drains and returns.
#include "common.cuh"
#include <string.h>

namespace stb {

constexpr int kTpBlockM = 128;
constexpr int kTpBlockN = 256;
constexpr int kTpBlockK = 64;
constexpr int kTpStages = 4;
constexpr int kTpThreads = 384;      // producer, MMA, 4 epilogue warps, 6 comm/reduce warps
constexpr int kTpAuxThreads = 192;
constexpr int kTpParts = 8;          // a 128-row tile is moved as 8 slices of 16 rows
constexpr int kTpPartRows = kTpBlockM / kTpParts;
constexpr int kTpMaxRanks = 8;

// Layout of the symmetric flag page (uint32 words).
constexpr int kTpMaxRowTiles = 1024;              // row tiles of 128 per rank
constexpr int kFlagRsBase = 64;                   // [slot 2][row tile][src 8]   partial tile of `src` has landed
constexpr int kFlagAgBase = kFlagRsBase + 2 * kTpMaxRowTiles * kTpMaxRanks;  // [slot 2][src 8][row tile] staged
constexpr int kFlagWords = kFlagAgBase + 2 * kTpMaxRanks * kTpMaxRowTiles;
constexpr int kAuxLoads = 8;                      // 16-byte loads each aux thread keeps in flight
constexpr int kRsParts = 16;                      // the reduction works on 8-row slices: a short tail after the
constexpr int kRsPartRows = kTpBlockM / kRsParts; // last partial tile has landed

// Layout of the local counter scratch (uint32 words), zeroed by the host function before each launch.
constexpr int kCtrClaim = 0;      // next comm (forward) unit; [1] next reduce unit
constexpr int kCtrTileClaim = 2;  // next GEMM tile
constexpr int kSchedDepth = 4;    // claimed tiles the producer may run ahead of the slowest consumer
constexpr int kCtrTiles = 8;      // AG: [row tile] slices pushed;  RS: [row tile] epilogue warps finished,
                                  //                                     [row tiles + row tile] slices forwarded

constexpr int kTpABytes = kTpBlockM * kTpBlockK * 2;
constexpr int kTpBBytes = kTpBlockN * kTpBlockK * 2;
constexpr int kTpStageBytes = kTpABytes + kTpBBytes;
constexpr int kTpStoreBytes = 4 * 2 * 4096;
constexpr int kTpSmem = kTpStages * kTpStageBytes + kTpStoreBytes + 256 + 1024;

struct PeerPtrs {
  void* p[kTpMaxRanks];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded spin until *p >= target (wrap-safe). Returns false on time-out or when the CTA has aborted.  The polls
// are relaxed loads; one acquire fence follows the poll that succeeds.
template <bool SYS>
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t target, uint64_t budget_ns,
                                             const volatile int* abort_flag) {
  uint64_t t0 = 0;
  for (uint32_t i = 0;; ++i) {
    const uint32_t v = SYS ? ld_relaxed_sys(p) : ld_relaxed_gpu(p);
    if (static_cast<int32_t>(v - target) >= 0) {
      if (SYS) asm volatile("fence.acq_rel.sys;" ::: "memory");
      else asm volatile("fence.acq_rel.gpu;" ::: "memory");
      return true;
    }
    if ((i & 63u) == 63u) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();   // slow to read: once per 64 polls
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) return false;
    }
    if (i >= 4) __nanosleep(i < 64 ? 40 : 200);
  }
}

__device__ __forceinline__ void aux_barrier() { asm volatile("bar.sync 2, 192;" ::: "memory"); }

// All-gather: own rows first, then the peers' row tiles in arrival order (tile i of every peer lands at about the
// same time, before tile i+1 of any peer).
__device__ __forceinline__ int ag_m_tile(int logical, int tiles_per_rank, int rank, int tp) {
  if (logical < tiles_per_rank) return rank * tiles_per_rank + logical;
  const int j = logical - tiles_per_rank;
  return ((rank + 1 + j % (tp - 1)) % tp) * tiles_per_rank + j / (tp - 1);
}
// Round-robin over the rank blocks (next rank first): the tiles bound for each peer are spread over the whole
// kernel, so the NVLink write rate is 1/tp-th of the epilogue's output rate instead of all of it for a while.
__device__ __forceinline__ int interleaved_m_tile(int logical, int tiles_per_rank, int rank, int tp) {
  return ((rank + 1 + logical % tp) % tp) * tiles_per_rank + logical / tp;
}

// Tile order: bands of 8 row tiles x all column tiles, so concurrently running CTAs share operands in L2
// and row tiles complete (or are needed) progressively.
__device__ __forceinline__ void decode_tp_tile(int tile, int num_m, int num_n, int& m_logical, int& n_tile) {
  constexpr int kBand = 8;
  const int in_band = kBand * num_n;
  const int band = tile / in_band;
  const int first_m = band * kBand;
  const int band_rows = min(num_m - first_m, kBand);
  const int r = tile - band * in_band;
  m_logical = first_m + r % band_rows;
  n_tile = r / band_rows;
}

struct TpCommon {
  int M, N, K;          // M = tp * rows_local
  int rank, tp, rows_local;
  uint32_t epoch;
  uint32_t* ctrs;       // local counter scratch
  unsigned long long wait_ns;
  int* status;
  unsigned long long* trace;  // optional [gridDim.x][8] device-timer stamps (ns) of the phases of every CTA
};

// Phase stamps for performance analysis (no effect when the caller passes no trace buffer).
enum TraceSlot { kTrEntry = 0, kTrFirstLoad = 1, kTrProducerDone = 2, kTrMmaDone = 3, kTrEpilogueDone = 4,
                 kTrAuxFirst = 5, kTrAuxDone = 6, kTrExit = 7 };
__device__ __forceinline__ void tp_trace(const TpCommon& c, int slot) {
  if (c.trace != nullptr) c.trace[blockIdx.x * 8 + slot] = global_timer_ns();
}

struct TpShared {
  uint8_t* smem;
  uint8_t* store_stage;
  uint64_t *full_bar, *empty_bar, *tmem_full, *tmem_empty;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
  volatile int* claim_slot;
  uint64_t *sched_full, *sched_empty;
  volatile int* tile_ring;
};

__device__ __forceinline__ TpShared tp_carve(uint8_t* smem_raw) {
  TpShared s;
  s.smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  s.store_stage = s.smem + kTpStages * kTpStageBytes;
  s.full_bar = reinterpret_cast<uint64_t*>(s.store_stage + kTpStoreBytes);
  s.empty_bar = s.full_bar + kTpStages;
  s.tmem_full = s.empty_bar + kTpStages;
  s.tmem_empty = s.tmem_full + 2;
  s.tmem_slot = reinterpret_cast<uint32_t*>(s.tmem_empty + 2);
  s.abort_flag = reinterpret_cast<volatile int*>(s.tmem_slot + 1);
  s.claim_slot = s.abort_flag + 1;
  s.sched_full = s.tmem_empty + 4;   // 8-byte aligned, past the three words above
  s.sched_empty = s.sched_full + kSchedDepth;
  s.tile_ring = reinterpret_cast<volatile int*>(s.sched_empty + kSchedDepth);
  return s;
}

__device__ __forceinline__ void tp_prologue(const TpShared& s, int warp) {
  if (threadIdx.x == 0) {
    for (int i = 0; i < kTpStages; ++i) {
      mbar_init(&s.full_bar[i], 1);
      mbar_init(&s.empty_bar[i], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&s.tmem_full[a], 1);
      mbar_init(&s.tmem_empty[a], 4);
    }
    for (int i = 0; i < kSchedDepth; ++i) {
      mbar_init(&s.sched_full[i], 1);
      mbar_init(&s.sched_empty[i], 5);  // MMA thread + 4 epilogue warps
    }
    *s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(s.tmem_slot, 2 * kTpBlockN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

__device__ __forceinline__ void tp_epilogue_sync(const TpShared& s, int warp, uint32_t tmem_base) {
  __syncthreads();
  if (*s.abort_flag) drain_delay();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * kTpBlockN);
  }
}

// Tile scheduler: the producer thread claims tile numbers from a device counter and hands them to the MMA
// thread and the epilogue warps through a small ring in shared memory.  -1 ends the stream, -2 = failed wait.
// `claimed` holds a tile number claimed ahead of time, so the latency of the atomic is off the critical path.
__device__ __forceinline__ int sched_produce(const TpShared& s, const TpCommon& c, uint32_t q, int num_tiles,
                                             uint32_t& claimed) {
  const int slot = q % kSchedDepth;
  if (!mbar_wait_budget(&s.sched_empty[slot], ((q / kSchedDepth) & 1) ^ 1, c.wait_ns, s.abort_flag)) return -2;
  int tile = static_cast<int>(claimed);
  if (tile >= num_tiles) tile = -1;
  else claimed = atomicAdd(&c.ctrs[kCtrTileClaim], 1u);
  s.tile_ring[slot] = tile;
  mbar_arrive(&s.sched_full[slot]);
  return tile;
}
__device__ __forceinline__ int sched_consume(const TpShared& s, const TpCommon& c, uint32_t q) {
  const int slot = q % kSchedDepth;
  if (!mbar_wait_budget(&s.sched_full[slot], (q / kSchedDepth) & 1, c.wait_ns, s.abort_flag)) return -2;
  const int tile = s.tile_ring[slot];
  mbar_arrive(&s.sched_empty[slot]);
  return tile;
}
// Producer side of a failed wait / end of stream: wake the consumers with the end marker where possible.
__device__ __forceinline__ void sched_fail(const TpShared& s, const TpCommon& c, int code) {
  if (!*s.abort_flag) report_error(c.status, code);
  *s.abort_flag = 1;
}

// One k-block of operand loads for the 128 x 256 tile at (m0, n0).
template <bool B_MN>
__device__ __forceinline__ void tp_load_stage(const TpShared& s, int stage, const CUtensorMap* ta, const CUtensorMap* tb,
                                              int k0, int m0, int n0) {
  uint8_t* sa = s.smem + stage * kTpStageBytes;
  uint8_t* sb = sa + kTpABytes;
  mbar_arrive_expect_tx(&s.full_bar[stage], kTpStageBytes);
  tma_load_2d(sa, ta, &s.full_bar[stage], k0, m0);
  if constexpr (!B_MN) {
    tma_load_2d(sb, tb, &s.full_bar[stage], k0, n0);
  } else {
#pragma unroll
    for (int j = 0; j < kTpBlockN / 64; ++j) tma_load_2d(sb + j * (kTpBlockK * 128), tb, &s.full_bar[stage], n0 + j * 64, k0);
  }
}

// MMA issue loop shared by both kernels (A is always K-major here).
template <bool B_MN>
__device__ __forceinline__ void tp_mma_loop(const TpShared& s, const TpCommon& c, uint32_t tmem_base, int k_blocks) {
  constexpr uint32_t idesc = umma_idesc_bf16(kTpBlockM, kTpBlockN, 0, B_MN ? 1 : 0);
  uint32_t it = 0, local_tile = 0;
  for (;; ++local_tile) {
    const int tile = sched_consume(s, c, local_tile);
    if (tile < 0) {
      if (tile == -2) sched_fail(s, c, kErrMmaWaitFull);
      return;
    }
    const int acc = local_tile & 1;
    if (!mbar_wait_budget(&s.tmem_empty[acc], ((local_tile >> 1) & 1) ^ 1, c.wait_ns, s.abort_flag)) {
      sched_fail(s, c, kErrMmaWaitTmem);
      return;
    }
    tc_fence_after();
    const uint32_t d_tmem = tmem_base + acc * kTpBlockN;
    for (int kb = 0; kb < k_blocks; ++kb, ++it) {
      const int st = it % kTpStages;
      if (!mbar_wait_budget(&s.full_bar[st], (it / kTpStages) & 1, c.wait_ns, s.abort_flag)) {
        sched_fail(s, c, kErrMmaWaitFull);
        return;
      }
      tc_fence_after();
      const uint32_t sa = smem_u32(s.smem + st * kTpStageBytes);
      const uint32_t sb = sa + kTpABytes;
#pragma unroll
      for (int k = 0; k < kTpBlockK / 16; ++k) {
        const uint64_t da = umma_smem_desc(sa + k * 32, 16, 1024);
        const uint64_t db = B_MN ? umma_smem_desc(sb + k * (16 * 128), kTpBlockK * 128, 1024)
                                 : umma_smem_desc(sb + k * 32, 16, 1024);
        umma_bf16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit(&s.empty_bar[st]);
    }
    umma_commit(&s.tmem_full[acc]);
  }
}

// Epilogue of one warp for one accumulator: TMEM -> bf16 -> swizzled smem -> TMA stores through `tc` at
// (n0 + .., row0).  Returns with the stores committed (not waited).
__device__ __forceinline__ void tp_store_tile(const TpShared& s, uint32_t tmem_base, int acc, int quarter, int ep_warp,
                                              int lane, const CUtensorMap* tc, int n0, int row0, int N,
                                              uint32_t& store_count) {
  uint8_t* my_stage = s.store_stage + ep_warp * 8192;
#pragma unroll 1
  for (int c = 0; c < kTpBlockN / 64; ++c) {
    uint32_t v[64];
    {
      uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&v[0]);
      uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&v[32]);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kTpBlockN + c * 64;
      tmem_ld_32x32(taddr, lo);
      tmem_ld_32x32(taddr + 32, hi);
      tmem_wait_ld();
    }
    const int col0 = n0 + c * 64;
    if (col0 >= N) continue;  // warp-uniform
    uint8_t* buf = my_stage + (store_count & 1) * 4096;
    if (store_count >= 2) {
      if (lane == 0) tma_store_wait_read<1>();
      __syncwarp();
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint4 ch;
      ch.x = pack_bf16(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
      ch.y = pack_bf16(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
      ch.z = pack_bf16(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
      ch.w = pack_bf16(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
      *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = ch;
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tc, buf, col0, row0);
      tma_store_commit();
    }
    ++store_count;
  }
}

// Claim the next unit of comm / reduce work for the 128 aux threads of this CTA.
__device__ __forceinline__ int aux_claim(const TpShared& s, uint32_t* ctrs, int tid) {
  if (tid == 0) *s.claim_slot = static_cast<int>(atomicAdd(&ctrs[kCtrClaim], 1u));
  aux_barrier();
  const int u = *s.claim_slot;
  aux_barrier();
  return u;
}

// Thread 0 of the aux group waits, every aux thread learns the outcome.
template <bool SYS>
__device__ __forceinline__ bool aux_wait_flag(const TpShared& s, const TpCommon& c, const uint32_t* flag,
                                              uint32_t target, int tid) {
  if (tid == 0) *s.claim_slot = wait_flag_ge<SYS>(flag, target, c.wait_ns, s.abort_flag) ? 1 : 0;
  aux_barrier();
  const bool ok = *s.claim_slot != 0;
  aux_barrier();
  return ok;
}

// ===================================================================================== all-gather -> GEMM
struct AgArgs {
  TpCommon c;
  const __nv_bfloat16* x_local;   // [rows_local][ldx]
  long long ldx;
  PeerPtrs gathered;              // this call's gathered buffer [M][K] of every rank (own entry: local memory)
  int gather_own;                 // also copy this rank's own rows into the own gathered buffer
  PeerPtrs flags;                 // flag page of every rank
  int ldc;
};

template <bool B_MN>
__global__ void __launch_bounds__(kTpThreads, 1)
gemm_ag_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_x,
               const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_c, const AgArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const TpShared s = tp_carve(smem_raw);
  const TpCommon& c = a.c;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = c.M / kTpBlockM;
  const int num_n = (c.N + kTpBlockN - 1) / kTpBlockN;
  const int num_tiles = num_m * num_n;
  const int tiles_per_rank = c.rows_local / kTpBlockM;
  const int k_blocks = (c.K + kTpBlockK - 1) / kTpBlockK;
  const int slot = c.epoch & 1;

  tp_prologue(s, warp);
  const uint32_t tmem_base = *s.tmem_slot;
  if (threadIdx.x == 0) tp_trace(c, kTrEntry);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      unsigned long long ready_mask = 0;  // row tiles < 64 already seen complete (and proxy-fenced) by this thread
      uint32_t claimed = atomicAdd(&c.ctrs[kCtrTileClaim], 1u);
      for (uint32_t q = 0;; ++q) {
        const int tile = sched_produce(s, c, q, num_tiles, claimed);
        if (tile < 0) {
          if (tile == -2) sched_fail(s, c, kErrProducerWait);
          tp_trace(c, kTrProducerDone);
          break;
        }
        int m_log, n_tile;
        decode_tp_tile(tile, num_m, num_n, m_log, n_tile);
        const int m_tile = ag_m_tile(m_log, tiles_per_rank, c.rank, c.tp);
        // Own rows are read where the caller left them; a peer's rows must have landed in the gathered buffer
        // (the peer raises the tile's flag after its stores).
        const bool own = (m_tile / tiles_per_rank) == c.rank;
        if (!own && !(m_tile < 64 && ((ready_mask >> m_tile) & 1ull))) {
          const uint32_t* flag = reinterpret_cast<const uint32_t*>(a.flags.p[c.rank]) + kFlagAgBase +
                                 (slot * kTpMaxRanks + m_tile / tiles_per_rank) * kTpMaxRowTiles +
                                 m_tile % tiles_per_rank;
          if (!wait_flag_ge<true>(flag, c.epoch, c.wait_ns, s.abort_flag)) {
            sched_fail(s, c, kErrPeerFlagWait);
            break;
          }
          fence_proxy_async_global();  // the peer's stores, acquired above -> visible to the TMA reads
          if (m_tile < 64) ready_mask |= 1ull << m_tile;
        }
        const CUtensorMap* ta = own ? &tmap_x : &tmap_a;
        const int a_row = own ? (m_tile % tiles_per_rank) * kTpBlockM : m_tile * kTpBlockM;
        bool ok = true;
        if (q == 0) tp_trace(c, kTrFirstLoad);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int st = it % kTpStages;
          if (!mbar_wait_budget(&s.empty_bar[st], ((it / kTpStages) & 1) ^ 1, c.wait_ns, s.abort_flag)) {
            sched_fail(s, c, kErrProducerWait);
            ok = false;
            break;
          }
          tp_load_stage<B_MN>(s, st, ta, &tmap_b, kb * kTpBlockK, a_row, n_tile * kTpBlockN);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      tp_mma_loop<B_MN>(s, c, tmem_base, k_blocks);
      tp_trace(c, kTrMmaDone);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    uint32_t local_tile = 0, store_count = 0;
    for (;;) {
      int tile = 0;
      if (lane == 0) tile = sched_consume(s, c, local_tile);
      tile = __shfl_sync(0xffffffffu, tile, 0);
      if (tile < 0) {
        if (tile == -2 && lane == 0) sched_fail(s, c, kErrEpilogueWait);
        break;
      }
      int m_log, n_tile;
      decode_tp_tile(tile, num_m, num_n, m_log, n_tile);
      const int m_tile = ag_m_tile(m_log, tiles_per_rank, c.rank, c.tp);
      const int acc = local_tile & 1;
      if (!mbar_wait_budget(&s.tmem_full[acc], (local_tile >> 1) & 1, c.wait_ns, s.abort_flag)) {
        sched_fail(s, c, kErrEpilogueWait);
        break;
      }
      tc_fence_after();
      tp_store_tile(s, tmem_base, acc, quarter, warp - 2, lane, &tmap_c, n_tile * kTpBlockN,
                    m_tile * kTpBlockM + quarter * 32, c.N, store_count);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.tmem_empty[acc]);
      ++local_tile;
    }
    if (lane == 0) tma_store_wait<0>();
    if (warp == 2 && lane == 0) tp_trace(c, kTrEpilogueDone);
  } else {
    // ------------------------------------------------------------------ comm warps
    // Unit = 16 rows of one of this rank's row tiles: read once, stored into every peer's gathered buffer
    // (and the own one when asked to); the unit that completes a tile raises its flag on every peer.
    const int tid = threadIdx.x - 192;
    const int total_units = tiles_per_rank * kTpParts;
    const int vec_per_row = c.K / 8;
    const int total_vec = kTpPartRows * vec_per_row;
    if (tid == 0) tp_trace(c, kTrAuxFirst);
    for (;;) {
      const int u = aux_claim(s, c.ctrs, tid);
      if (u >= total_units || *s.abort_flag) {
        if (tid == 0) tp_trace(c, kTrAuxDone);
        break;
      }
      const int m_local = u / kTpParts, part = u % kTpParts;
      const long long src_row = static_cast<long long>(m_local) * kTpBlockM + part * kTpPartRows;
      const __nv_bfloat16* from = a.x_local + src_row * a.ldx;
      const long long dst_off = (static_cast<long long>(c.rank) * c.rows_local + src_row) * c.K;
      for (int base = tid; base < total_vec; base += kTpAuxThreads * kAuxLoads) {
        uint4 v[kAuxLoads];
#pragma unroll
        for (int q = 0; q < kAuxLoads; ++q) {
          const int idx = base + q * kTpAuxThreads;
          if (idx < total_vec) {
            const int r = idx / vec_per_row, col = idx - r * vec_per_row;
            v[q] = ld_cg_v4(from + r * a.ldx + col * 8);
          }
        }
        for (int pr = 1; pr <= c.tp; ++pr) {
          const int dst_rank = (c.rank + pr) % c.tp;  // peers in ring order, own buffer last
          if (dst_rank == c.rank && !a.gather_own) continue;
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.gathered.p[dst_rank]) + dst_off;
#pragma unroll
          for (int q = 0; q < kAuxLoads; ++q) {
            const int idx = base + q * kTpAuxThreads;
            if (idx < total_vec) *reinterpret_cast<uint4*>(dst + static_cast<long long>(idx) * 8) = v[q];
          }
        }
      }
      __threadfence_system();
      aux_barrier();
      if (tid == 0) {
        const uint32_t done = atomicAdd(&c.ctrs[kCtrTiles + m_local], 1u);
        if (done == static_cast<uint32_t>(kTpParts - 1)) {
          __threadfence_system();
          for (int r = 0; r < c.tp; ++r)
            if (r != c.rank)
              st_release_sys(reinterpret_cast<uint32_t*>(a.flags.p[r]) + kFlagAgBase +
                                 (slot * kTpMaxRanks + c.rank) * kTpMaxRowTiles + m_local,
                             c.epoch);
        }
      }
    }
    if (num_tiles == 0) {
      // Gather only: no product consumes the tiles, so wait here until every peer's rows have landed
      // (the row tiles are spread over the CTAs).
      bool ok = true;
      for (int t = blockIdx.x; t < num_m && ok; t += gridDim.x) {
        if (t / tiles_per_rank == c.rank) continue;
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(a.flags.p[c.rank]) + kFlagAgBase +
                               (slot * kTpMaxRanks + t / tiles_per_rank) * kTpMaxRowTiles + t % tiles_per_rank;
        ok = aux_wait_flag<true>(s, c, flag, c.epoch, tid);
        if (!ok && tid == 0) sched_fail(s, c, kErrPeerFlagWait);
      }
    }
  }
  tp_epilogue_sync(s, warp, tmem_base);
  if (threadIdx.x == 0) tp_trace(c, kTrExit);
}

// Sum the TP partial copies of a few rows (fixed rank order, fp32) and write bf16.  in[src] points at the first
// row of the unit inside the partial copy of rank `src`.
template <int TP>
__device__ __forceinline__ void reduce_unit(const __nv_bfloat16* const (&in)[kTpMaxRanks], __nv_bfloat16* __restrict__ out0,
                                            long long ldo, int vec_per_row, int total_vec, int tid) {
  constexpr int U = (8 / TP) > 0 ? (8 / TP) : 1;  // 8 loads in flight per thread
  for (int base = tid; base < total_vec; base += kTpAuxThreads * U) {
    uint4 v[U][TP];
#pragma unroll
    for (int q = 0; q < U; ++q) {
      const int idx = base + q * kTpAuxThreads;
      if (idx < total_vec) {
#pragma unroll
        for (int src = 0; src < TP; ++src) v[q][src] = ld_cg_v4(in[src] + static_cast<long long>(idx) * 8);
      }
    }
#pragma unroll
    for (int q = 0; q < U; ++q) {
      const int idx = base + q * kTpAuxThreads;
      if (idx < total_vec) {
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int src = 0; src < TP; ++src) {
          f[0] += bf16_lo(v[q][src].x); f[1] += bf16_hi(v[q][src].x); f[2] += bf16_lo(v[q][src].y);
          f[3] += bf16_hi(v[q][src].y); f[4] += bf16_lo(v[q][src].z); f[5] += bf16_hi(v[q][src].z);
          f[6] += bf16_lo(v[q][src].w); f[7] += bf16_hi(v[q][src].w);
        }
        uint4 o;
        o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
        o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
        const int r = idx / vec_per_row, col = idx - r * vec_per_row;
        *reinterpret_cast<uint4*>(out0 + r * ldo + col * 8) = o;
      }
    }
  }
}

// ===================================================================================== GEMM -> reduce-scatter
struct RsArgs {
  TpCommon c;
  __nv_bfloat16* out;             // [rows_local][ldo]
  long long ldo;
  const __nv_bfloat16* staging;   // local [M][N]: every partial tile this rank computes
  const __nv_bfloat16* recv_self; // this call's receive slot of this rank: [tp src][rows_local][N]
  PeerPtrs recv;                  // receive slot of every rank
  PeerPtrs flags;                 // flag page of every rank
};

template <bool B_MN>
__global__ void __launch_bounds__(kTpThreads, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_stage, const RsArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const TpShared s = tp_carve(smem_raw);
  const TpCommon& c = a.c;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = c.M / kTpBlockM;
  const int num_n = (c.N + kTpBlockN - 1) / kTpBlockN;
  const int num_tiles = num_m * num_n;
  const int tiles_per_rank = c.rows_local / kTpBlockM;
  const int k_blocks = (c.K + kTpBlockK - 1) / kTpBlockK;
  const int slot = c.epoch & 1;
  const uint32_t tile_done = static_cast<uint32_t>(num_n * 4);   // epilogue warps that store a share of a row tile

  tp_prologue(s, warp);
  const uint32_t tmem_base = *s.tmem_slot;
  if (threadIdx.x == 0) tp_trace(c, kTrEntry);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t claimed = atomicAdd(&c.ctrs[kCtrTileClaim], 1u);
      for (uint32_t q = 0;; ++q) {
        const int tile = sched_produce(s, c, q, num_tiles, claimed);
        if (tile < 0) {
          if (tile == -2) sched_fail(s, c, kErrProducerWait);
          tp_trace(c, kTrProducerDone);
          break;
        }
        int m_log, n_tile;
        decode_tp_tile(tile, num_m, num_n, m_log, n_tile);
        const int m_tile = interleaved_m_tile(m_log, tiles_per_rank, c.rank, c.tp);
        bool ok = true;
        if (q == 0) tp_trace(c, kTrFirstLoad);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int st = it % kTpStages;
          if (!mbar_wait_budget(&s.empty_bar[st], ((it / kTpStages) & 1) ^ 1, c.wait_ns, s.abort_flag)) {
            sched_fail(s, c, kErrProducerWait);
            ok = false;
            break;
          }
          tp_load_stage<B_MN>(s, st, &tmap_a, &tmap_b, kb * kTpBlockK, m_tile * kTpBlockM, n_tile * kTpBlockN);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      tp_mma_loop<B_MN>(s, c, tmem_base, k_blocks);
      tp_trace(c, kTrMmaDone);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue: partial tiles to the staging matrix
    const int quarter = warp & 3;
    uint32_t local_tile = 0, store_count = 0;
    int pending_m = -1;  // row tile whose stores are issued but not yet known complete
    // lane 0: the bulk stores of `m_tile` by this warp have been performed -> count it
    auto signal_tile = [&](int m_tile) {
      fence_proxy_async_global();
      __threadfence();
      atomicAdd(&c.ctrs[kCtrTiles + m_tile], 1u);
    };
    for (;;) {
      int tile = 0;
      if (lane == 0) tile = sched_consume(s, c, local_tile);
      tile = __shfl_sync(0xffffffffu, tile, 0);
      if (tile < 0) {
        if (tile == -2 && lane == 0) sched_fail(s, c, kErrEpilogueWait);
        break;
      }
      int m_log, n_tile;
      decode_tp_tile(tile, num_m, num_n, m_log, n_tile);
      const int m_tile = interleaved_m_tile(m_log, tiles_per_rank, c.rank, c.tp);
      const int acc = local_tile & 1;
      if (lane == 0 && pending_m >= 0) {
        // The stores of the previous tile were issued a tile's MMA time ago at most: let them complete and count
        // the tile now, while this warp would only be waiting for the next accumulator anyway.  Forwarding and
        // reduction of a row tile then start one GEMM wave earlier than with a count deferred past the next tile.
        tma_store_wait<0>();
        signal_tile(pending_m);
        pending_m = -1;
      }
      if (!mbar_wait_budget(&s.tmem_full[acc], (local_tile >> 1) & 1, c.wait_ns, s.abort_flag)) {
        sched_fail(s, c, kErrEpilogueWait);
        break;
      }
      tc_fence_after();
      tp_store_tile(s, tmem_base, acc, quarter, warp - 2, lane, &tmap_stage, n_tile * kTpBlockN,
                    m_tile * kTpBlockM + quarter * 32, c.N, store_count);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s.tmem_empty[acc]);
        pending_m = m_tile;
      }
      __syncwarp();
      ++local_tile;
    }
    if (lane == 0) {
      tma_store_wait<0>();
      if (pending_m >= 0) signal_tile(pending_m);
      if (warp == 2) tp_trace(c, kTrEpilogueDone);
    }
  } else {
    // ------------------------------------------------------------------ forward / reduce warps
    // Two streams of units, each handed out in the order the row tiles are computed:
    //   forward  16-row slices of finished row tiles that another rank owns: staging -> owner's receive slot
    //   reduce   8-row slices of the row tiles this rank owns: sum of the tp partial copies
    // The aux group of a CTA holds at most one claimed unit of each stream and never blocks on either: it polls
    // whether the held unit of its preferred stream can run, else whether the other one can, else sleeps briefly.
    // Groups of even CTAs prefer forwarding, groups of odd CTAs prefer reducing: half the groups already saturate
    // NVLink, and the reduction (HBM traffic) then proceeds beside the forwarding instead of after it.  Every
    // claimed forward unit is sent as soon as this rank's own GEMM has produced its tile and the group is free,
    // whatever the peers do, so the waits between ranks cannot form a cycle.
    const int tid = threadIdx.x - 192;
    constexpr int kFwdParts = kTpParts, kFwdRows = kTpPartRows;
    const int total_fwd = (num_m - tiles_per_rank) * kFwdParts;
    const int total_red = tiles_per_rank * kRsParts;
    const int vec_per_row = c.N / 8;
    const long long slot_stride = static_cast<long long>(c.rows_local) * c.N;
    const uint32_t* my_flags = reinterpret_cast<const uint32_t*>(a.flags.p[c.rank]) + kFlagRsBase +
                               slot * kTpMaxRowTiles * kTpMaxRanks;
    // decision of thread 0 for this round, published to the group: 0 nothing ready, 1 forward, 2 reduce, 3 stop
    auto publish = [&](int v) {
      if (tid == 0) *s.claim_slot = v;
      aux_barrier();
      const int r = *s.claim_slot;
      aux_barrier();
      return r;
    };
    auto fwd_tile = [&](int u) {
      const int jt = u / kFwdParts;
      const int logical = (jt / (c.tp - 1)) * c.tp + jt % (c.tp - 1);   // own tiles (logical % tp == tp - 1) skipped
      return interleaved_m_tile(logical, tiles_per_rank, c.rank, c.tp);
    };
    if (tid == 0) tp_trace(c, kTrAuxFirst);
    // thread 0 owns the claims and the readiness checks; the unit numbers travel through shared memory
    int fwd_u = -1, red_u = -1;            // held units (-1: none held, -2: stream exhausted)
    int fwd_ready_tile = -1, red_ready_tile = -1;
    uint64_t t_idle = 0;
    uint32_t idle_polls = 0;
    for (;;) {
      int decision = 0;
      if (tid == 0) {
        if (*s.abort_flag) decision = 3;
        if (decision == 0 && fwd_u == -1) {
          const int u = static_cast<int>(atomicAdd(&c.ctrs[kCtrClaim], 1u));
          fwd_u = u < total_fwd ? u : -2;
        }
        if (decision == 0 && red_u == -1) {
          const int u = static_cast<int>(atomicAdd(&c.ctrs[kCtrClaim + 1], 1u));
          red_u = u < total_red ? u : -2;
        }
        auto try_forward = [&]() {
          if (decision != 0 || fwd_u < 0) return;
          const int m_tile = fwd_tile(fwd_u);
          if (m_tile == fwd_ready_tile || ld_relaxed_gpu(&c.ctrs[kCtrTiles + m_tile]) >= tile_done) {
            if (m_tile != fwd_ready_tile) {
              asm volatile("fence.acq_rel.gpu;" ::: "memory");
              fence_proxy_async_global();   // the epilogue's bulk stores -> visible to plain loads
              fwd_ready_tile = m_tile;
            }
            decision = 1;
          }
        };
        auto try_reduce = [&]() {
          if (decision != 0 || red_u < 0) return;
          const int m_local = red_u / kRsParts;
          bool ready = m_local == red_ready_tile;
          if (!ready) {
            ready = ld_relaxed_gpu(&c.ctrs[kCtrTiles + c.rank * tiles_per_rank + m_local]) >= tile_done;
            for (int src = 0; src < c.tp && ready; ++src)
              if (src != c.rank)
                ready = static_cast<int32_t>(ld_relaxed_sys(my_flags + m_local * kTpMaxRanks + src) - c.epoch) >= 0;
            if (ready) {
              asm volatile("fence.acq_rel.sys;" ::: "memory");
              fence_proxy_async_global();   // the own partial was written through the async proxy (bulk stores)
              red_ready_tile = m_local;
            }
          }
          if (ready) decision = 2;
        };
        if (blockIdx.x & 1) {
          try_reduce();
          try_forward();
        } else {
          try_forward();
          try_reduce();
        }
        if (decision == 0 && fwd_u == -2 && red_u == -2) decision = 3;
        if (decision == 0) {
          if ((++idle_polls & 63u) == 0) {         // the timer is slow to read
            const uint64_t now = global_timer_ns();
            if (t_idle == 0) t_idle = now;
            else if (now - t_idle > c.wait_ns) {
              sched_fail(s, c, fwd_u >= 0 ? kErrEpilogueWait : kErrPeerFlagWait);
              decision = 3;
            }
          }
        } else {
          t_idle = 0;
          idle_polls = 0;
        }
        s.tile_ring[kSchedDepth] = decision == 1 ? fwd_u : red_u;   // spare word after the tile ring
      }
      decision = publish(decision);
      if (decision == 3) break;
      if (decision == 0) {
        __nanosleep(100);
        continue;
      }
      const int u = s.tile_ring[kSchedDepth];
      if (decision == 1) {
        // ---- forward 16 rows of a finished remote tile to its owner
        const int part = u % kFwdParts;
        const int m_tile = fwd_tile(u);
        const int dest = m_tile / tiles_per_rank, m_local = m_tile % tiles_per_rank;
        const long long row_in_tile = static_cast<long long>(part) * kFwdRows;
        const __nv_bfloat16* from = a.staging + (static_cast<long long>(m_tile) * kTpBlockM + row_in_tile) * c.N;
        __nv_bfloat16* to = reinterpret_cast<__nv_bfloat16*>(a.recv.p[dest]) +
                            (static_cast<long long>(c.rank) * c.rows_local + m_local * kTpBlockM + row_in_tile) * c.N;
        const int total_vec = kFwdRows * vec_per_row;     // rows are contiguous on both sides
        constexpr int kFwdLoads = 8;                      // 16-byte loads each thread keeps in flight
        for (int base = tid; base < total_vec; base += kTpAuxThreads * kFwdLoads) {
          uint4 v[kFwdLoads];
#pragma unroll
          for (int q = 0; q < kFwdLoads; ++q) {
            const int idx = base + q * kTpAuxThreads;
            if (idx < total_vec) v[q] = ld_cg_v4(from + static_cast<long long>(idx) * 8);
          }
#pragma unroll
          for (int q = 0; q < kFwdLoads; ++q) {
            const int idx = base + q * kTpAuxThreads;
            if (idx < total_vec) *reinterpret_cast<uint4*>(to + static_cast<long long>(idx) * 8) = v[q];
          }
        }
        __threadfence_system();
        aux_barrier();
        if (tid == 0) {
          const uint32_t done = atomicAdd(&c.ctrs[kCtrTiles + num_m + m_tile], 1u);
          if (done == static_cast<uint32_t>(kFwdParts - 1)) {
            __threadfence_system();
            st_release_sys(reinterpret_cast<uint32_t*>(a.flags.p[dest]) + kFlagRsBase +
                               (slot * kTpMaxRowTiles + m_local) * kTpMaxRanks + c.rank,
                           c.epoch);
          }
          fwd_u = -1;
        }
      } else {
        // ---- reduce 8 rows of an own tile
        const int m_local = u / kRsParts, part = u % kRsParts;
        const long long row0 = static_cast<long long>(m_local) * kTpBlockM + part * kRsPartRows;
        const __nv_bfloat16* in[kTpMaxRanks];
#pragma unroll
        for (int src = 0; src < kTpMaxRanks; ++src)
          in[src] = (src == c.rank) ? a.staging + (static_cast<long long>(c.rank) * c.rows_local + row0) * c.N
                                    : a.recv_self + src * slot_stride + row0 * c.N;
        __nv_bfloat16* out0 = a.out + row0 * a.ldo;
        const int total_vec = kRsPartRows * vec_per_row;
        switch (c.tp) {
          case 2: reduce_unit<2>(in, out0, a.ldo, vec_per_row, total_vec, tid); break;
          case 4: reduce_unit<4>(in, out0, a.ldo, vec_per_row, total_vec, tid); break;
          case 8: reduce_unit<8>(in, out0, a.ldo, vec_per_row, total_vec, tid); break;
          default: reduce_unit<1>(in, out0, a.ldo, vec_per_row, total_vec, tid); break;
        }
        if (tid == 0) red_u = -1;
      }
    }
    if (tid == 0) tp_trace(c, kTrAuxDone);
  }
  tp_epilogue_sync(s, warp, tmem_base);
  if (threadIdx.x == 0) tp_trace(c, kTrExit);
}

template <typename Kern>
static int tp_configure(Kern kern) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kTpSmem);
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

static int tp_check(int rows_local, int N, int K, int tp, int rank) {
  if ((tp != 2 && tp != 4 && tp != 8) || rank < 0 || rank >= tp) return -kErrBadArgument;
  if (rows_local <= 0 || (rows_local % kTpBlockM) || rows_local / kTpBlockM > kTpMaxRowTiles) return -kErrBadArgument;
  if (K <= 0 || (K & 7) || N < 0 || (N & 7)) return -kErrBadArgument;
  return 0;
}

}  // namespace stb

using namespace stb;

// Words of symmetric flag memory a rank must provide (zero-initialised once, before the first call).
extern "C" int stb_tp_flag_words() { return kFlagWords; }
// Words of local counter scratch needed for `row_tiles` = tp * rows_local / 128 row tiles.
extern "C" int stb_tp_ctr_words(int row_tiles) { return kCtrTiles + 2 * row_tiles; }

// C[tp*rows_local, N] = all_gather_rows(x_local) * B^T (b_mn_major = 0, B stored [N][ldb]) or * B
// (b_mn_major = 1, B stored [K][ldb]); `gathered` [tp*rows_local][K] receives the gathered rows.
// N = 0 gathers only; gather_own = 0 leaves this rank's own rows of the gathered matrix unwritten (the product
// reads them from x_local).  gathered_ptrs[r] / flag_ptrs[r]: rank r's gathered buffer for this call (slot =
// epoch & 1, tp*rows_local*K bf16, symmetric memory) and flag page, as mapped into this process; the result is
// in gathered_ptrs[rank] and stays valid until the second-next call on the group.  epoch: 1, 2, 3, ... per group,
// the same on every rank.  ctrs: local scratch of stb_tp_ctr_words(row tiles) words.
extern "C" int stb_gemm_ag_bf16(const void* x_local, long long ldx, void* const* gathered_ptrs,
                                void* const* flag_ptrs, const void* B, void* C, int rows_local, int N, int K, int ldb,
                                int ldc, int b_mn_major, int gather_own, int rank, int tp, unsigned epoch, void* ctrs,
                                unsigned long long wait_ns, int* status, void* trace, cudaStream_t stream) {
  int r = tp_check(rows_local, N, K, tp, rank);
  if (r) return r;
  if ((ldx & 7) || (N > 0 && ((ldb & 7) || (ldc & 7)))) return -kErrBadArgument;
  const int M = tp * rows_local;
  CUtensorMap ta, tx, tb, tc;
  r = make_tmap_2d_bf16(&ta, gathered_ptrs[rank], K, M, static_cast<uint64_t>(K) * 2, kTpBlockK, kTpBlockM, 1);
  if (r) return r;
  r = make_tmap_2d_bf16(&tx, x_local, K, rows_local, static_cast<uint64_t>(ldx) * 2, kTpBlockK, kTpBlockM, 1);
  if (r) return r;
  if (N > 0) {
    if (!b_mn_major) r = make_tmap_2d_bf16(&tb, B, K, N, static_cast<uint64_t>(ldb) * 2, kTpBlockK, kTpBlockN, 1);
    else r = make_tmap_2d_bf16(&tb, B, N, K, static_cast<uint64_t>(ldb) * 2, 64, kTpBlockK, 1);
    if (r) return r;
    r = make_tmap_2d(&tc, C, 2, N, M, static_cast<uint64_t>(ldc) * 2, 64, 32, 1);
    if (r) return r;
  } else {
    tb = ta;
    tc = ta;
  }
  AgArgs a{};
  a.c.M = M; a.c.N = N; a.c.K = K; a.c.rank = rank; a.c.tp = tp; a.c.rows_local = rows_local;
  a.c.epoch = epoch; a.c.ctrs = static_cast<uint32_t*>(ctrs); a.c.wait_ns = wait_ns; a.c.status = status;
  a.c.trace = static_cast<unsigned long long*>(trace);
  a.x_local = static_cast<const __nv_bfloat16*>(x_local);
  a.ldx = ldx;
  a.gather_own = gather_own;
  a.ldc = ldc;
  for (int i = 0; i < tp; ++i) {
    a.gathered.p[i] = gathered_ptrs[i];
    a.flags.p[i] = flag_ptrs[i];
  }
  cudaError_t e = cudaMemsetAsync(ctrs, 0, sizeof(uint32_t) * (kCtrTiles + 2 * (M / kTpBlockM)), stream);
  if (e != cudaSuccess) return -static_cast<int>(e);
  static bool configured[2] = {false, false};
  if (!configured[b_mn_major ? 1 : 0]) {
    r = b_mn_major ? tp_configure(gemm_ag_kernel<true>) : tp_configure(gemm_ag_kernel<false>);
    if (r) return r;
    configured[b_mn_major ? 1 : 0] = true;
  }
  const int grid = sm_count();
  if (b_mn_major) gemm_ag_kernel<true><<<grid, kTpThreads, kTpSmem, stream>>>(ta, tx, tb, tc, a);
  else gemm_ag_kernel<false><<<grid, kTpThreads, kTpSmem, stream>>>(ta, tx, tb, tc, a);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

// out[rows_local, N] = reduce_scatter_rows(A[tp*rows_local, K] * B^T or * B).  recv_ptrs[r]: rank r's receive
// slot for this call (slot = epoch & 1; tp*rows_local*N bf16), flag_ptrs[r]: rank r's flag page.  staging: local
// scratch of tp*rows_local*N bf16 (this rank's partial products; free again when the call has finished).
extern "C" int stb_gemm_rs_bf16(const void* A, int lda, const void* B, int ldb, int b_mn_major, void* out,
                                long long ldo, void* staging, void* const* recv_ptrs, void* const* flag_ptrs,
                                int rows_local, int N, int K, int rank, int tp, unsigned epoch, void* ctrs,
                                unsigned long long wait_ns, int* status, void* trace, cudaStream_t stream) {
  int r = tp_check(rows_local, N, K, tp, rank);
  if (r) return r;
  if (N <= 0 || (lda & 7) || (ldb & 7) || (ldo & 7) || staging == nullptr) return -kErrBadArgument;
  const int M = tp * rows_local;
  CUtensorMap ta, tb, ts;
  r = make_tmap_2d_bf16(&ta, A, K, M, static_cast<uint64_t>(lda) * 2, kTpBlockK, kTpBlockM, 1);
  if (r) return r;
  if (!b_mn_major) r = make_tmap_2d_bf16(&tb, B, K, N, static_cast<uint64_t>(ldb) * 2, kTpBlockK, kTpBlockN, 1);
  else r = make_tmap_2d_bf16(&tb, B, N, K, static_cast<uint64_t>(ldb) * 2, 64, kTpBlockK, 1);
  if (r) return r;
  r = make_tmap_2d(&ts, staging, 2, N, M, static_cast<uint64_t>(N) * 2, 64, 32, 1);
  if (r) return r;
  RsArgs a{};
  a.c.M = M; a.c.N = N; a.c.K = K; a.c.rank = rank; a.c.tp = tp; a.c.rows_local = rows_local;
  a.c.epoch = epoch; a.c.ctrs = static_cast<uint32_t*>(ctrs); a.c.wait_ns = wait_ns; a.c.status = status;
  a.c.trace = static_cast<unsigned long long*>(trace);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.ldo = ldo;
  a.staging = static_cast<const __nv_bfloat16*>(staging);
  a.recv_self = static_cast<const __nv_bfloat16*>(recv_ptrs[rank]);
  for (int i = 0; i < tp; ++i) {
    a.recv.p[i] = recv_ptrs[i];
    a.flags.p[i] = flag_ptrs[i];
  }
  cudaError_t e = cudaMemsetAsync(ctrs, 0, sizeof(uint32_t) * (kCtrTiles + 2 * (M / kTpBlockM)), stream);
  if (e != cudaSuccess) return -static_cast<int>(e);
  static bool configured[2] = {false, false};
  if (!configured[b_mn_major ? 1 : 0]) {
    r = b_mn_major ? tp_configure(gemm_rs_kernel<true>) : tp_configure(gemm_rs_kernel<false>);
    if (r) return r;
    configured[b_mn_major ? 1 : 0] = true;
  }
  const int grid = sm_count();
  if (b_mn_major) gemm_rs_kernel<true><<<grid, kTpThreads, kTpSmem, stream>>>(ta, tb, ts, a);
  else gemm_rs_kernel<false><<<grid, kTpThreads, kTpSmem, stream>>>(ta, tb, ts, a);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

// ------------------------------------------------------------------------------------ peer memory plumbing
// Device memory that other processes of the node can map (cudaMalloc + CUDA IPC handles).
extern "C" int stb_symm_alloc(void** ptr, unsigned long long bytes, void* handle64) {
  cudaFree(nullptr);  // binds the primary context to this thread
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return -static_cast<int>(e);
  e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return -static_cast<int>(e);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), *ptr);
  if (e != cudaSuccess) return -static_cast<int>(e);
  e = cudaDeviceSynchronize();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
extern "C" int stb_symm_open(void** ptr, const void* handle64) {
  cudaFree(nullptr);  // binds the primary context to this thread
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
extern "C" int stb_symm_close(void* ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
extern "C" int stb_symm_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
