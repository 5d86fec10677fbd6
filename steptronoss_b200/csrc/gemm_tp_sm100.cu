// Sequence-parallel projections as single kernels over NVLink peer memory (sm_100a).
//
//   gemm_ag_kernel : C = all_gather_rows(x) * B^T.   The gathered matrix lives in symmetric memory.
//   gemm_rs_kernel : out = reduce_scatter_rows(A * B^T).
//
// Both are the persistent tcgen05 GEMM of gemm_sm100.cu (TMA producer warp, MMA warp, four epilogue warps,
// tiles claimed from a device counter) plus a communication role that a few CTAs take.  Measured on this
// hardware, sixteen CTAs that each drive a ring of 32 KB cp.async.bulk copies (global -> shared -> peer global)
// saturate a GPU's NVLink ports (about 675 GB/s per direction), while 16-byte stores issued by a few warps of
// every CTA or 128-byte TMA tensor stores from the GEMM epilogue reach 440-550 GB/s and stall the tensor pipe.
// So the first `n_comm` CTAs to start (a ticket from a device counter: roles never depend on a CTA that is not
// resident) become "comm CTAs": one thread of theirs moves rows with bulk copies through the shared memory that
// the GEMM stages would otherwise use.
//
//   all-gather -> GEMM   comm CTAs push this rank's rows, 32 KB at a time, into every peer's gathered matrix (one
//                        load, tp-1 stores).  A comm CTA owns whole 32-row parts of a row tile, so it alone knows
//                        when a part has landed and raises that part's flag on the peers (no counting across
//                        CTAs, no atomics on the path); when the rows are out the comm CTAs turn into GEMM CTAs.  The TMA producer of a GEMM CTA waits
//                        for the flag of the row tile it is about to load.  Own rows are multiplied first (read
//                        where the caller left them), the peers' row tiles then in the order they arrive.
//   GEMM -> reduce-scatter  the epilogue TMA-stores bf16 partial tiles into a local staging matrix at full speed;
//                        comm CTAs copy every finished row tile that another rank owns into that rank's receive
//                        slot and raise its flag; four "reduce" warps per CTA add the tp partial copies of the
//                        row tiles this rank owns in fixed rank order (fp32) as they complete (the own partial
//                        straight out of the staging matrix).  Row blocks are computed next-rank first, own last.
//
// They replace the NCCL collective + cuBLAS pairs of the reference's sequence-parallel linears
// (steptronoss/core/tensor_parallel/layers.py:151-346, mappings.py:103-300).
//
// Cross-rank protocol.  Flags are uint32 words in each rank's symmetric flag page, written into the peer's
// page with st.release.sys and read from the own page with ld.acquire.sys; they carry the call number
// ("epoch", compared wrap-safe), so nothing is ever reset.  Gathered and receive buffers have two slots
// used alternately by epoch parity.  A slot written in call e was last read in call e-2 (and by what the
// caller ran right after it), and no rank can leave call e-1 before every peer has entered call e-1 (each
// call consumes data that every peer produces inside the same call), so two slots need no further hand-shake.
// GEMM tiles and reduce units are claimed from device counters and the communication work is striped over the
// CTAs that hold a comm ticket (tickets go to CTAs that are running), so progress never depends on a CTA that is
// not resident.  Every wait is bounded by the caller's budget; on time-out the kernel records a
// code in the status word, drains and returns.  No load uses cluster broadcast; peers are only written to.
#include "common.cuh"
#include <string.h>

namespace stb {

constexpr int kTpBlockM = 128;
constexpr int kTpBlockN = 256;
constexpr int kTpBlockK = 64;
constexpr int kTpStages = 4;
constexpr int kTpThreads = 320;      // producer / comm, MMA, 4 epilogue warps, 4 reduce warps (reduce-scatter only)
constexpr int kTpAuxThreads = 128;
constexpr int kTpMaxRanks = 8;

// Layout of the symmetric flag page (uint32 words).
constexpr int kTpMaxRowTiles = 1024;              // row tiles of 128 per rank
constexpr int kTpParts = 4;                       // a row tile travels as 4 parts of 32 rows, each with its own flag
constexpr int kTpPartRows = kTpBlockM / kTpParts;
constexpr int kFlagRsBase = 64;                   // [slot 2][row tile][src 8][part 4]   part of the partial tile of `src` has landed
constexpr int kFlagAgBase = kFlagRsBase + 2 * kTpMaxRowTiles * kTpMaxRanks * kTpParts;  // [slot 2][src 8][row tile][part 4]
constexpr int kFlagWords = kFlagAgBase + 2 * kTpMaxRanks * kTpMaxRowTiles * kTpParts;
constexpr int kRsParts = 16;                      // the reduction works on 8-row slices: a short tail after the
constexpr int kRsPartRows = kTpBlockM / kRsParts; // last partial tile has landed

// Layout of the local counter scratch (uint32 words), zeroed by the host function before each launch.
constexpr int kCtrClaim = 0;      // next reduce unit
constexpr int kCtrTicket = 1;     // CTAs that have started (the first n_comm become comm CTAs)
constexpr int kCtrTileClaim = 2;  // next GEMM tile
constexpr int kSchedDepth = 4;    // claimed tiles the producer may run ahead of the slowest consumer
constexpr int kCtrTiles = 8;      // [row tile]  reduce-scatter: epilogue warps that have stored their share of the tile

constexpr int kTpABytes = kTpBlockM * kTpBlockK * 2;
constexpr int kTpBBytes = kTpBlockN * kTpBlockK * 2;
constexpr int kTpStageBytes = kTpABytes + kTpBBytes;
constexpr int kTpStoreBytes = 4 * 2 * 4096;
constexpr int kTpBarrierBytes = 512;
constexpr int kTpSmem = kTpStages * kTpStageBytes + kTpStoreBytes + kTpBarrierBytes + 1024;

// Communication ring of a comm CTA: it reuses the GEMM operand stages.
constexpr int kCommStageBytes = 32 * 1024;
constexpr int kCommStages = (kTpStages * kTpStageBytes) / kCommStageBytes;   // 6
constexpr int kCommLag = 3;       // a unit's completion is signalled once three younger store groups were issued
constexpr int kCommPend = 8;      // ring of store groups issued but not yet known complete (> kCommLag)
static_assert(kCommStages * kCommStageBytes <= kTpStages * kTpStageBytes, "ring must fit in the operand stages");

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
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// Untiled bulk copies: global -> shared (completion counted on an mbarrier) and shared -> global (bulk group).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}

// Bounded spin until *p >= target (wrap-safe). Returns false on time-out or when the CTA has aborted.
template <bool SYS>
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t target, uint64_t budget_ns,
                                             const volatile int* abort_flag) {
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 0;; ++i) {
    const uint32_t v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if (static_cast<int32_t>(v - target) >= 0) return true;
    if ((i & 15u) == 15u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > budget_ns) return false;
    }
    if (i >= 4) __nanosleep(i < 64 ? 40 : 200);
  }
}

__device__ __forceinline__ void aux_barrier() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// All-gather: own rows first, then the peers' row tiles in arrival order (every peer pushes its tiles in
// ascending order to all ranks at once, so tile i of every peer lands at about the same time).
__device__ __forceinline__ int ag_m_tile(int logical, int tiles_per_rank, int rank, int tp) {
  if (logical < tiles_per_rank) return rank * tiles_per_rank + logical;
  const int j = logical - tiles_per_rank;
  return ((rank + 1 + j % (tp - 1)) % tp) * tiles_per_rank + j / (tp - 1);
}
// Reduce-scatter: round-robin over the rank blocks (next rank first, own block last): the tiles bound for each
// peer are spread over the whole kernel.
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
  int n_comm;           // CTAs that take the communication role
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
  uint64_t *sched_full, *sched_empty, *comm_bar;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
  volatile int* claim_slot;
  volatile int* role_slot;
  volatile int* tile_ring;
  volatile int* pend_tile;   // [kCommPend] completion ring of the comm thread
};

__device__ __forceinline__ TpShared tp_carve(uint8_t* smem_raw) {
  TpShared s;
  s.smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  s.store_stage = s.smem + kTpStages * kTpStageBytes;
  s.full_bar = reinterpret_cast<uint64_t*>(s.store_stage + kTpStoreBytes);
  s.empty_bar = s.full_bar + kTpStages;
  s.tmem_full = s.empty_bar + kTpStages;
  s.tmem_empty = s.tmem_full + 2;
  s.sched_full = s.tmem_empty + 2;
  s.sched_empty = s.sched_full + kSchedDepth;
  s.comm_bar = s.sched_empty + kSchedDepth;
  s.tmem_slot = reinterpret_cast<uint32_t*>(s.comm_bar + kCommStages);
  s.abort_flag = reinterpret_cast<volatile int*>(s.tmem_slot + 1);
  s.claim_slot = s.abort_flag + 1;
  s.role_slot = s.abort_flag + 2;
  s.tile_ring = s.abort_flag + 3;
  s.pend_tile = s.tile_ring + kSchedDepth;
  return s;
}
static_assert((2 * kTpStages + 4 + 2 * kSchedDepth + kCommStages) * 8 + (5 + kSchedDepth + kCommPend) * 4 <= kTpBarrierBytes,
              "barrier region too small");

// Returns this CTA's communication ticket (0 .. n_comm-1), or -1 when it only computes.
__device__ __forceinline__ int tp_prologue(const TpShared& s, const TpCommon& c, int warp) {
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
    for (int i = 0; i < kCommStages; ++i) mbar_init(&s.comm_bar[i], 1);
    *s.abort_flag = 0;
    const uint32_t ticket = atomicAdd(&c.ctrs[kCtrTicket], 1u);
    *s.role_slot = ticket < static_cast<uint32_t>(c.n_comm) ? static_cast<int>(ticket) : -1;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(s.tmem_slot, 2 * kTpBlockN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  return *s.role_slot;
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
// A CTA that computes no tiles at all: send the end marker as the first (and only) entry of the stream.
__device__ __forceinline__ void sched_end_now(const TpShared& s) {
  s.tile_ring[0] = -1;
  mbar_arrive(&s.sched_full[0]);
}
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

// Claim the next unit of reduce work for the 128 aux threads of this CTA.
__device__ __forceinline__ int aux_claim(const TpShared& s, uint32_t* ctrs, int tid) {
  if (tid == 0) *s.claim_slot = static_cast<int>(atomicAdd(&ctrs[kCtrClaim], 1u));
  aux_barrier();
  const int u = *s.claim_slot;
  aux_barrier();
  return u;
}

// ------------------------------------------------------------------------------------- communication ring
// How a part ([32 rows x cols] bf16) is cut into units of at most kCommStageBytes: `rows` whole rows per unit
// when a row fits (rows a power of two), else one row piece of `chunk_cols` columns per unit.
struct CopyGeom {
  int rows;          // rows per unit
  int chunk_cols;    // columns per unit
  int col_chunks;    // units per row (1 when whole rows are moved)
  int units_per_part;
};
__host__ __device__ inline CopyGeom copy_geom(int cols) {
  CopyGeom g;
  const int row_bytes = cols * 2;
  if (row_bytes <= kCommStageBytes) {
    int r = 1;
    while (r * 2 * row_bytes <= kCommStageBytes && r * 2 <= kTpPartRows) r *= 2;
    g.rows = r;
    g.chunk_cols = cols;
    g.col_chunks = 1;
  } else {
    g.rows = 1;
    g.chunk_cols = kCommStageBytes / 2;
    g.col_chunks = (cols + g.chunk_cols - 1) / g.chunk_cols;
  }
  g.units_per_part = (kTpPartRows / g.rows) * g.col_chunks;
  return g;
}
// (row inside the part, first column, columns) of unit `sub` of a part
__device__ __forceinline__ void unit_window(const CopyGeom& g, int sub, int total_cols, int& row, int& col0, int& cols) {
  row = g.col_chunks == 1 ? sub * g.rows : sub / g.col_chunks;
  col0 = g.col_chunks == 1 ? 0 : (sub % g.col_chunks) * g.chunk_cols;
  cols = min(g.chunk_cols, total_cols - col0);
}

struct CommJob {
  const uint8_t* src;     // first byte of the unit in local memory
  long long src_pitch;    // bytes between rows at the source
  long long dst_off;      // byte offset of the unit in every destination buffer (rows are contiguous there)
  int rows, row_bytes;
  int item;               // the part this unit belongs to
  int last;               // 1: the last unit of its part
};

// One thread of a comm CTA moves its share of the parts through the ring: item = ticket, ticket + n_comm, ...;
// per unit: (wait until the part's source is ready) -> bulk load into a stage -> bulk store to every destination.
// A part's completion callback runs once the store group of its last unit has completed; that is checked
// kCommLag store groups later, so the ring never waits for a round trip over NVLink.
// Policy: num_items(), units_per_item(), describe(item, sub, job), ready(item), num_dests(job), dest(job, i), complete(item).
template <class Policy>
__device__ bool comm_ring_run(const TpShared& s, const TpCommon& c, int ticket, const Policy& pol) {
  const int num_items = pol.num_items();
  const int upi = pol.units_per_item();
  int item = ticket, sub = 0;            // next unit to load
  int ready_item = -1;                   // last item whose source was seen ready
  uint32_t filled = 0, stored = 0, signalled = 0;
  CommJob inflight[kCommStages];
  uint64_t t_idle = 0;
  bool ok = true;
  for (;;) {
    bool progress = false;
    if (item < num_items && filled - stored < static_cast<uint32_t>(kCommStages)) {
      if (ready_item != item && pol.ready(item)) ready_item = item;
      if (ready_item == item) {
        CommJob j;
        pol.describe(item, sub, j);
        j.item = item;
        j.last = (sub == upi - 1) ? 1 : 0;
        const int st = filled % kCommStages;
        uint8_t* dst = s.smem + st * kCommStageBytes;
        const uint32_t bytes = static_cast<uint32_t>(j.rows) * j.row_bytes;
        mbar_arrive_expect_tx(&s.comm_bar[st], bytes);
        if (j.src_pitch == j.row_bytes) {
          bulk_load(dst, j.src, bytes, &s.comm_bar[st]);
        } else {
          for (int r = 0; r < j.rows; ++r)
            bulk_load(dst + r * j.row_bytes, j.src + r * j.src_pitch, j.row_bytes, &s.comm_bar[st]);
        }
#pragma unroll
        for (int i = 0; i < kCommStages; ++i)
          if (i == st) inflight[i] = j;
        ++filled;
        if (++sub == upi) {
          sub = 0;
          item += c.n_comm;
        }
        progress = true;
      }
    }
    if (stored < filled) {
      const int st = stored % kCommStages;
      if (mbar_try_wait(&s.comm_bar[st], (stored / kCommStages) & 1)) {
        CommJob j{};
#pragma unroll
        for (int i = 0; i < kCommStages; ++i)
          if (i == st) j = inflight[i];
        const uint8_t* src = s.smem + st * kCommStageBytes;
        const uint32_t bytes = static_cast<uint32_t>(j.rows) * j.row_bytes;
        fence_proxy_async_smem();
        const int nd = pol.num_dests(j);
        for (int d = 0; d < nd; ++d) bulk_store(pol.dest(j, d) + j.dst_off, src, bytes);
        tma_store_commit();
        s.pend_tile[stored % kCommPend] = j.last ? j.item : -1;
        ++stored;
        if (stored - signalled > static_cast<uint32_t>(kCommLag)) {
          const int done_item = s.pend_tile[signalled % kCommPend];
          if (done_item >= 0) {
            tma_store_wait<kCommLag>();            // every group but the newest kCommLag has completed
            pol.complete(done_item);
          }
          ++signalled;
        }
        tma_store_wait_read<0>();                  // the stage may be refilled
        progress = true;
      }
    }
    if (item >= num_items && stored == filled) break;
    if (progress) {
      t_idle = 0;
    } else {
      if (t_idle == 0) t_idle = global_timer_ns();
      else if (*s.abort_flag || global_timer_ns() - t_idle > c.wait_ns) {
        ok = false;
        break;
      }
      __nanosleep(64);
    }
  }
  tma_store_wait<0>();
  if (ok)
    for (; signalled < stored; ++signalled) {
      const int done_item = s.pend_tile[signalled % kCommPend];
      if (done_item >= 0) pol.complete(done_item);
    }
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

struct AgCommPolicy {
  const AgArgs& a;
  CopyGeom g;
  int tiles_per_rank, slot;
  __device__ int num_items() const { return tiles_per_rank * kTpParts; }
  __device__ int units_per_item() const { return g.units_per_part; }
  __device__ void describe(int item, int sub, CommJob& j) const {
    int row, col0, cols;
    unit_window(g, sub, a.c.K, row, col0, cols);
    row += item * kTpPartRows;                       // row inside this rank's block
    j.src = reinterpret_cast<const uint8_t*>(a.x_local + static_cast<long long>(row) * a.ldx + col0);
    j.rows = g.rows;
    j.row_bytes = cols * 2;
    j.src_pitch = g.col_chunks == 1 ? a.ldx * 2 : j.row_bytes;   // a single row piece is one contiguous load
    j.dst_off = ((static_cast<long long>(a.c.rank) * a.c.rows_local + row) * a.c.K + col0) * 2;
  }
  __device__ bool ready(int) const { return true; }
  __device__ int num_dests(const CommJob&) const { return a.c.tp - 1 + (a.gather_own ? 1 : 0); }
  __device__ uint8_t* dest(const CommJob&, int i) const {   // peers in ring order, the own buffer last
    return static_cast<uint8_t*>(a.gathered.p[(a.c.rank + 1 + i) % a.c.tp]);
  }
  // the part's rows have landed on every peer: tell them
  __device__ void complete(int item) const {
    fence_proxy_async_global();
    __threadfence_system();        // one release fence, then plain system-scope stores of the flag to every peer
    for (int r = 0; r < a.c.tp; ++r)
      if (r != a.c.rank)
        st_relaxed_sys(reinterpret_cast<uint32_t*>(a.flags.p[r]) + kFlagAgBase +
                           ((slot * kTpMaxRanks + a.c.rank) * kTpMaxRowTiles) * kTpParts + item,
                       a.c.epoch);
  }
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

  const int ticket = tp_prologue(s, c, warp);
  const uint32_t tmem_base = *s.tmem_slot;
  if (threadIdx.x == 0) tp_trace(c, kTrEntry);

  if (warp == 0) {
    if (lane == 0) {
      bool alive = true;
      if (ticket >= 0) {
        // ---------------------------------------------------------------- push this rank's rows to every peer
        tp_trace(c, kTrAuxFirst);
        const AgCommPolicy pol{a, copy_geom(c.K), tiles_per_rank, slot};
        if (!comm_ring_run(s, c, ticket, pol)) {
          sched_fail(s, c, kErrProducerWait);
          alive = false;
        }
        tp_trace(c, kTrAuxDone);
      }
      // ------------------------------------------------------------------ TMA producer
      uint32_t it = 0;
      unsigned long long ready_mask = 0;  // row tiles < 64 already seen complete (and proxy-fenced) by this thread
      uint32_t claimed = alive ? atomicAdd(&c.ctrs[kCtrTileClaim], 1u) : 0u;
      for (uint32_t q = 0; alive; ++q) {
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
                                 ((slot * kTpMaxRanks + m_tile / tiles_per_rank) * kTpMaxRowTiles +
                                  m_tile % tiles_per_rank) * kTpParts;
          bool landed = true;
          for (int part = 0; part < kTpParts && landed; ++part)
            landed = wait_flag_ge<true>(flag + part, c.epoch, c.wait_ns, s.abort_flag);
          if (!landed) {
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
      if (num_tiles == 0 && alive) {
        // Gather only: no product consumes the tiles, so wait here until every peer's rows have landed
        // (the row tiles are spread over the CTAs).
        for (int t = blockIdx.x; t < num_m; t += gridDim.x) {
          if (t / tiles_per_rank == c.rank) continue;
          const uint32_t* flag = reinterpret_cast<const uint32_t*>(a.flags.p[c.rank]) + kFlagAgBase +
                                 ((slot * kTpMaxRanks + t / tiles_per_rank) * kTpMaxRowTiles + t % tiles_per_rank) * kTpParts;
          bool landed = true;
          for (int part = 0; part < kTpParts && landed; ++part)
            landed = wait_flag_ge<true>(flag + part, c.epoch, c.wait_ns, s.abort_flag);
          if (!landed) {
            sched_fail(s, c, kErrPeerFlagWait);
            break;
          }
        }
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

struct RsCommPolicy {
  const RsArgs& a;
  CopyGeom g;
  int tiles_per_rank, num_m, slot;
  uint32_t tile_done;             // epilogue warps per finished row tile
  // item = (remote row tile in the order the tiles are computed, part)
  __device__ int num_items() const { return (num_m - tiles_per_rank) * kTpParts; }
  __device__ int units_per_item() const { return g.units_per_part; }
  __device__ int tile_of(int item) const {
    const int tp = a.c.tp, jt = item / kTpParts;
    const int logical = (jt / (tp - 1)) * tp + jt % (tp - 1);      // own tiles (logical % tp == tp - 1) skipped
    return interleaved_m_tile(logical, tiles_per_rank, a.c.rank, tp);
  }
  __device__ void describe(int item, int sub, CommJob& j) const {
    const int m_tile = tile_of(item), m_local = m_tile % tiles_per_rank;
    int row, col0, cols;
    unit_window(g, sub, a.c.N, row, col0, cols);
    row += (item % kTpParts) * kTpPartRows;          // row inside the tile
    j.src = reinterpret_cast<const uint8_t*>(a.staging + (static_cast<long long>(m_tile) * kTpBlockM + row) * a.c.N + col0);
    j.rows = g.rows;
    j.row_bytes = cols * 2;
    j.src_pitch = g.col_chunks == 1 ? static_cast<long long>(a.c.N) * 2 : j.row_bytes;
    j.dst_off = ((static_cast<long long>(a.c.rank) * a.c.rows_local + m_local * kTpBlockM + row) * a.c.N + col0) * 2;
  }
  __device__ bool ready(int item) const {
    if (ld_acquire_gpu(&a.c.ctrs[kCtrTiles + tile_of(item)]) < tile_done) return false;
    fence_proxy_async_global();   // the epilogue's bulk stores, acquired above -> visible to the bulk loads
    return true;
  }
  __device__ int num_dests(const CommJob&) const { return 1; }
  __device__ uint8_t* dest(const CommJob& j, int) const {
    return static_cast<uint8_t*>(a.recv.p[tile_of(j.item) / tiles_per_rank]);
  }
  __device__ void complete(int item) const {
    const int m_tile = tile_of(item);
    const int dest = m_tile / tiles_per_rank, m_local = m_tile % tiles_per_rank;
    fence_proxy_async_global();
    st_release_sys(reinterpret_cast<uint32_t*>(a.flags.p[dest]) + kFlagRsBase +
                       (((slot * kTpMaxRowTiles + m_local) * kTpMaxRanks + a.c.rank) * kTpParts) + item % kTpParts,
                   a.c.epoch);
  }
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
  const uint32_t tile_done = static_cast<uint32_t>(num_n * 4);

  const int ticket = tp_prologue(s, c, warp);
  const uint32_t tmem_base = *s.tmem_slot;
  if (threadIdx.x == 0) tp_trace(c, kTrEntry);

  if (warp == 0) {
    if (lane == 0) {
      if (ticket >= 0) {
        // ---------------------------------------------------------------- finished row tiles to their owners
        sched_end_now(s);   // this CTA computes no tiles: its MMA and epilogue warps leave at once
        const RsCommPolicy pol{a, copy_geom(c.N), tiles_per_rank, num_m, slot, tile_done};
        if (!comm_ring_run(s, c, ticket, pol)) sched_fail(s, c, kErrProducerWait);
        tp_trace(c, kTrProducerDone);
      } else {
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
      if (!mbar_wait_budget(&s.tmem_full[acc], (local_tile >> 1) & 1, c.wait_ns, s.abort_flag)) {
        sched_fail(s, c, kErrEpilogueWait);
        break;
      }
      tc_fence_after();
      const uint32_t before = store_count;
      tp_store_tile(s, tmem_base, acc, quarter, warp - 2, lane, &tmap_stage, n_tile * kTpBlockN,
                    m_tile * kTpBlockM + quarter * 32, c.N, store_count);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s.tmem_empty[acc]);
        if (pending_m >= 0) {
          // bulk groups retire in order: with at most this tile's groups outstanding, the previous tile is done
          if (store_count - before == 4) tma_store_wait<4>();
          else tma_store_wait<0>();
          signal_tile(pending_m);
          if (store_count - before != 4) {
            signal_tile(m_tile);
            pending_m = -1;
          } else {
            pending_m = m_tile;
          }
        } else {
          pending_m = m_tile;
        }
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
    // ------------------------------------------------------------------ reduce warps: rows this rank owns
    const int tid = threadIdx.x - 192;
    const int total_units = tiles_per_rank * kRsParts;
    const int vec_per_row = c.N / 8;
    const int total_vec = kRsPartRows * vec_per_row;
    const long long slot_stride = static_cast<long long>(c.rows_local) * c.N;
    const uint32_t* my_flags = reinterpret_cast<const uint32_t*>(a.flags.p[c.rank]) + kFlagRsBase +
                               slot * kTpMaxRowTiles * kTpMaxRanks * kTpParts;
    int ready_part = -1;            // (row tile, part) whose partial copies were last seen complete
    bool failed = false;
    if (tid == 0) tp_trace(c, kTrAuxFirst);
    for (;;) {
      const int u = aux_claim(s, c.ctrs, tid);
      if (u >= total_units || failed || *s.abort_flag) {
        if (tid == 0) tp_trace(c, kTrAuxDone);
        break;
      }
      const int m_local = u / kRsParts, part = u % kRsParts;
      const int tpart = part / (kRsParts / kTpParts);      // the 32-row part this 8-row slice lies in
      if (m_local * kTpParts + tpart != ready_part) {
        // one thread waits for that part of the partial tile of every rank (the own one in the staging matrix),
        // then everybody learns the outcome
        if (tid == 0) {
          int good = 1;
          for (int src = 0; src < c.tp && good; ++src) {
            if (src == c.rank)
              good = wait_flag_ge<false>(&c.ctrs[kCtrTiles + c.rank * tiles_per_rank + m_local], tile_done, c.wait_ns,
                                         s.abort_flag) ? 1 : 0;
            else
              good = wait_flag_ge<true>(my_flags + (m_local * kTpMaxRanks + src) * kTpParts + tpart, c.epoch, c.wait_ns,
                                        s.abort_flag) ? 1 : 0;
          }
          // partial tiles were written through the async proxy (bulk stores): order them before the plain loads
          fence_proxy_async_global();
          *s.claim_slot = good;
        }
        aux_barrier();
        const bool ok = *s.claim_slot != 0;
        aux_barrier();
        if (!ok) {
          if (tid == 0) {
            report_error(c.status, kErrPeerFlagWait);
            *s.abort_flag = 1;
          }
          failed = true;
          continue;
        }
        ready_part = m_local * kTpParts + tpart;
      }
      const long long row0 = static_cast<long long>(m_local) * kTpBlockM + part * kRsPartRows;
      const __nv_bfloat16* in[kTpMaxRanks];
#pragma unroll
      for (int src = 0; src < kTpMaxRanks; ++src)
        in[src] = (src == c.rank) ? a.staging + (static_cast<long long>(c.rank) * c.rows_local + row0) * c.N
                                  : a.recv_self + src * slot_stride + row0 * c.N;
      __nv_bfloat16* out0 = a.out + row0 * a.ldo;
      switch (c.tp) {
        case 2: reduce_unit<2>(in, out0, a.ldo, vec_per_row, total_vec, tid); break;
        case 4: reduce_unit<4>(in, out0, a.ldo, vec_per_row, total_vec, tid); break;
        case 8: reduce_unit<8>(in, out0, a.ldo, vec_per_row, total_vec, tid); break;
        default: reduce_unit<1>(in, out0, a.ldo, vec_per_row, total_vec, tid); break;
      }
    }
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

// Comm CTAs for a transfer of `bytes` over NVLink that should not outlast a GEMM of `flops`: one CTA moves about
// 35 GB/s through its ring and sixteen saturate the links; a few more than the rate asks for keep the tail short.
static int choose_comm_ctas(double bytes, double flops, int grid) {
  const double t_gemm = flops / 1.3e15 + 5e-6;
  int n = static_cast<int>(bytes / t_gemm / 35e9) + 3;
  if (n < 4) n = 4;
  if (n > 20) n = 20;
  if (n > grid / 2) n = grid / 2 > 0 ? grid / 2 : 1;
  return n;
}

}  // namespace stb

using namespace stb;

// Words of symmetric flag memory a rank must provide (zero-initialised once, before the first call).
extern "C" int stb_tp_flag_words() { return kFlagWords; }
// Words of local counter scratch needed for `row_tiles` = tp * rows_local / 128 row tiles.
extern "C" int stb_tp_ctr_words(int row_tiles) { return kCtrTiles + row_tiles; }

// C[tp*rows_local, N] = all_gather_rows(x_local) * B^T (b_mn_major = 0, B stored [N][ldb]) or * B
// (b_mn_major = 1, B stored [K][ldb]); `gathered` [tp*rows_local][K] receives the gathered rows.
// N = 0 gathers only; gather_own = 0 leaves this rank's own rows of the gathered matrix unwritten (the product
// reads them from x_local).  gathered_ptrs[r] / flag_ptrs[r]: rank r's gathered buffer for this call (slot =
// epoch & 1, tp*rows_local*K bf16, symmetric memory) and flag page, as mapped into this process; the result is
// in gathered_ptrs[rank] and stays valid until the second-next call on the group.  epoch: 1, 2, 3, ... per group,
// the same on every rank.  ctrs: local scratch of stb_tp_ctr_words(row tiles) words.  comm_ctas: CTAs that push
// the rows before they join the product (0 = chosen from the sizes).
extern "C" int stb_gemm_ag_bf16(const void* x_local, long long ldx, void* const* gathered_ptrs,
                                void* const* flag_ptrs, const void* B, void* C, int rows_local, int N, int K, int ldb,
                                int ldc, int b_mn_major, int gather_own, int rank, int tp, unsigned epoch, void* ctrs,
                                unsigned long long wait_ns, int comm_ctas, int* status, void* trace,
                                cudaStream_t stream) {
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
  int grid = sm_count();
  const double out_bytes = static_cast<double>(tp - 1) * rows_local * K * 2;
  if (comm_ctas <= 0) {
    // these CTAs join the product once the rows are out, so a few more than the rate asks for cost nothing
    comm_ctas = choose_comm_ctas(out_bytes, 2.0 * M * static_cast<double>(N) * K, grid);
    if (comm_ctas < 12) comm_ctas = 12;
  }
  if (N == 0) {
    comm_ctas = comm_ctas < 16 ? 16 : comm_ctas;   // nothing to multiply: only the comm CTAs are launched
    grid = comm_ctas;
  }
  if (comm_ctas > grid) comm_ctas = grid;
  AgArgs a{};
  a.c.M = M; a.c.N = N; a.c.K = K; a.c.rank = rank; a.c.tp = tp; a.c.rows_local = rows_local;
  a.c.n_comm = comm_ctas;
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
  cudaError_t e = cudaMemsetAsync(ctrs, 0, sizeof(uint32_t) * (kCtrTiles + M / kTpBlockM), stream);
  if (e != cudaSuccess) return -static_cast<int>(e);
  static bool configured[2] = {false, false};
  if (!configured[b_mn_major ? 1 : 0]) {
    r = b_mn_major ? tp_configure(gemm_ag_kernel<true>) : tp_configure(gemm_ag_kernel<false>);
    if (r) return r;
    configured[b_mn_major ? 1 : 0] = true;
  }
  if (b_mn_major) gemm_ag_kernel<true><<<grid, kTpThreads, kTpSmem, stream>>>(ta, tx, tb, tc, a);
  else gemm_ag_kernel<false><<<grid, kTpThreads, kTpSmem, stream>>>(ta, tx, tb, tc, a);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

// out[rows_local, N] = reduce_scatter_rows(A[tp*rows_local, K] * B^T or * B).  recv_ptrs[r]: rank r's receive
// slot for this call (slot = epoch & 1; tp*rows_local*N bf16), flag_ptrs[r]: rank r's flag page.  staging: local
// scratch of tp*rows_local*N bf16 (the rank's partial products; free again when the call has finished).
// comm_ctas: CTAs that copy finished row tiles to their owners instead of computing (0 = chosen from the sizes).
extern "C" int stb_gemm_rs_bf16(const void* A, int lda, const void* B, int ldb, int b_mn_major, void* out,
                                long long ldo, void* staging, void* const* recv_ptrs, void* const* flag_ptrs,
                                int rows_local, int N, int K, int rank, int tp, unsigned epoch, void* ctrs,
                                unsigned long long wait_ns, int comm_ctas, int* status, void* trace,
                                cudaStream_t stream) {
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
  const int grid = sm_count();
  const double out_bytes = static_cast<double>(tp - 1) * rows_local * N * 2;
  if (comm_ctas <= 0) comm_ctas = choose_comm_ctas(out_bytes, 2.0 * M * static_cast<double>(N) * K, grid);
  if (comm_ctas >= grid) comm_ctas = grid - 1;
  if (comm_ctas < 1) return -kErrBadArgument;    // one CTA cannot both compute and send
  RsArgs a{};
  a.c.M = M; a.c.N = N; a.c.K = K; a.c.rank = rank; a.c.tp = tp; a.c.rows_local = rows_local;
  a.c.n_comm = comm_ctas;
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
  cudaError_t e = cudaMemsetAsync(ctrs, 0, sizeof(uint32_t) * (kCtrTiles + M / kTpBlockM), stream);
  if (e != cudaSuccess) return -static_cast<int>(e);
  static bool configured[2] = {false, false};
  if (!configured[b_mn_major ? 1 : 0]) {
    r = b_mn_major ? tp_configure(gemm_rs_kernel<true>) : tp_configure(gemm_rs_kernel<false>);
    if (r) return r;
    configured[b_mn_major ? 1 : 0] = true;
  }
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
