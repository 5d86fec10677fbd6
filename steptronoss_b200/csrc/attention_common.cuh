// Shared pieces of the sm_100a attention kernels: tile geometry, launch parameters, the 128-byte
// swizzle address function, packed-segment bookkeeping and the visibility (mask) predicate.
#pragma once
#include "common.cuh"

namespace stb {

constexpr int kD = 128;        // head dim
constexpr int kBM = 128;       // q rows per block
constexpr int kBN = 128;       // keys per block
constexpr int kTileBytes = 128 * kD * 2;   // 32 KB: one [128][128] bf16 tile as two 64-column slabs
constexpr int kSlabBytes = 128 * 128;      // 16 KB: [128 rows][64 cols]
constexpr int kAttnThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct AttnParams {
  const int* cu_q;
  const int* cu_k;
  const int* blk_seg;   // per block: segment id or -1
  const int* blk_row0;  // per block: first absolute row (q rows for fwd/dq, key rows for dkv)
  int hq, hkv;
  int causal, window;
  float scale;          // softmax scale (1/sqrt(D))
  int total_q, total_k;
  // forward
  __nv_bfloat16* O;     // [Tq][hq][D]
  float* LSE;           // [hq][Tq]  (natural log)
  // backward
  const float* delta;   // [hq][Tq]
  __nv_bfloat16* dQ;    // [Tq][hq][D]
  __nv_bfloat16* dK;    // [Tk][hkv][D]
  __nv_bfloat16* dV;    // rows with stride dv_stride
  long long dv_stride;
  int* status;
  // dK/dV pass with the q heads of a GQA group split over several CTAs (few kv heads, short sequences):
  // fp32 partials [split][dV, dK][Tk][hkv][D], summed in split order by a second kernel
  float* dkv_part;
  int splits;
  // Keys addressed by their global position (context parallelism): the K / V (and dK / dV) rows live in a
  // rank-major buffer [cp][2 * chunk_len] that holds every rank's two load-balanced chunks, and per-segment tables
  // replace cu_k.  A segment's key range starts at a multiple of 128 at or before its document, so that no
  // 128-key tile straddles two chunks; the keys in front of the document are masked (seg_k_skip of them).
  const int* seg_k_begin;  // global position of the first key row of the range (multiple of 128)
  const int* seg_k_len;    // rows from seg_k_begin to the segment's last key
  const int* seg_k_skip;   // leading rows of the range that belong to an earlier document
  int cp, chunk_len;       // chunk_len == 0: keys are addressed by plain row numbers
};

// 128-byte-swizzled address of (row, 16-byte chunk) inside a [128][64 bf16] slab.
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

// One 128x128x128 product out of 8 UMMA (K = 16 each).
//   A_KMAJOR: A tile is [M rows][K] (slabs split K); otherwise [K rows][M] (slabs split M).
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void mma_128x128x128(uint32_t d_tmem, uint32_t sa, uint32_t sb, bool accumulate) {
  constexpr uint32_t idesc = umma_idesc_bf16(128, 128, A_MN ? 1 : 0, B_MN ? 1 : 0);
  // step k of an MN-major operand starts 16 rows = 2048 bytes further; of a K-major operand 32 bytes further inside
  // a 64-column slab, and in the second slab from k = 4 on
  const uint64_t da = A_MN ? umma_smem_desc(sa, kSlabBytes, 1024) : umma_smem_desc(sa, 16, 1024);
  const uint64_t db = B_MN ? umma_smem_desc(sb, kSlabBytes, 1024) : umma_smem_desc(sb, 16, 1024);
  constexpr uint32_t sa1 = A_MN ? 2048 : 32, sa4 = A_MN ? 4 * 2048 : kSlabBytes;
  constexpr uint32_t sb1 = B_MN ? 2048 : 32, sb4 = B_MN ? 4 * 2048 : kSlabBytes;
  umma4_ss(d_tmem, da, umma_desc_advance(da, sa1), umma_desc_advance(da, 2 * sa1), umma_desc_advance(da, 3 * sa1), db,
           umma_desc_advance(db, sb1), umma_desc_advance(db, 2 * sb1), umma_desc_advance(db, 3 * sb1), idesc,
           accumulate ? 1u : 0u);
  umma4_ss(d_tmem, umma_desc_advance(da, sa4), umma_desc_advance(da, sa4 + sa1), umma_desc_advance(da, sa4 + 2 * sa1),
           umma_desc_advance(da, sa4 + 3 * sa1), umma_desc_advance(db, sb4), umma_desc_advance(db, sb4 + sb1),
           umma_desc_advance(db, sb4 + 2 * sb1), umma_desc_advance(db, sb4 + 3 * sb1), idesc, 1u);
}

// The same with A = [128 lanes][128 K] bf16 in TMEM (64 columns).
template <bool B_MN>
__device__ __forceinline__ void mma_128x128x128_ta(uint32_t d_tmem, uint32_t ta, uint32_t sb, bool accumulate) {
  constexpr uint32_t idesc = umma_idesc_bf16(128, 128, 0, B_MN ? 1 : 0);
  const uint64_t db = B_MN ? umma_smem_desc(sb, kSlabBytes, 1024) : umma_smem_desc(sb, 16, 1024);
  constexpr uint32_t sb1 = B_MN ? 2048 : 32, sb4 = B_MN ? 4 * 2048 : kSlabBytes;
  umma4_ts(d_tmem, ta, ta + 8, ta + 16, ta + 24, db, umma_desc_advance(db, sb1), umma_desc_advance(db, 2 * sb1),
           umma_desc_advance(db, 3 * sb1), idesc, accumulate ? 1u : 0u);
  umma4_ts(d_tmem, ta + 32, ta + 40, ta + 48, ta + 56, umma_desc_advance(db, sb4), umma_desc_advance(db, sb4 + sb1),
           umma_desc_advance(db, sb4 + 2 * sb1), umma_desc_advance(db, sb4 + 3 * sb1), idesc, 1u);
}

__device__ __forceinline__ void load_tile(void* dst, const CUtensorMap* m, uint64_t* bar, int head, int row) {
  tma_load_3d(dst, m, bar, 0, head, row);
  tma_load_3d(static_cast<uint8_t*>(dst) + kSlabBytes, m, bar, 64, head, row);
}

struct SegInfo {
  int q_begin, q_len, k_begin, k_len, off, k_skip;
};

__device__ __forceinline__ SegInfo seg_info(const AttnParams& p, int seg) {
  SegInfo s;
  s.q_begin = p.cu_q[seg];
  s.q_len = p.cu_q[seg + 1] - s.q_begin;
  if (p.seg_k_begin != nullptr) {
    s.k_begin = p.seg_k_begin[seg];
    s.k_len = p.seg_k_len[seg];
    s.k_skip = p.seg_k_skip[seg];
  } else {
    s.k_begin = p.cu_k[seg];
    s.k_len = p.cu_k[seg + 1] - s.k_begin;
    s.k_skip = 0;
  }
  s.off = s.k_len - s.q_len;
  return s;
}

// Row of the K / V buffer that holds global key position g.  Load-balanced context parallelism cuts the sequence
// into 2*cp chunks and gives rank r the chunks r and 2*cp-1-r; the buffer stores rank after rank.  g is a multiple
// of 64 and chunk_len a multiple of 128, so a 64- or 128-row tile starting at g stays inside one chunk.
__device__ __forceinline__ int key_row(const AttnParams& p, int g) {
  if (p.chunk_len == 0) return g;
  const int c = g / p.chunk_len, in_chunk = g - c * p.chunk_len;
  const int rank = c < p.cp ? c : 2 * p.cp - 1 - c;
  return rank * 2 * p.chunk_len + (c < p.cp ? 0 : p.chunk_len) + in_chunk;
}

// key-block range [jb0, jb1) visible to q rows [q0, q0+128) of a segment (relative indices)
__device__ __forceinline__ void kv_range(const AttnParams& p, const SegInfo& s, int q0, int& jb0, int& jb1) {
  int kend = s.k_len;
  if (p.causal) kend = min(kend, q0 + kBM + s.off);
  int kbeg = 0;
  if (p.window > 0) kbeg = max(0, q0 + s.off - p.window + 1);
  if (kend <= kbeg) { jb0 = 0; jb1 = 0; return; }
  jb0 = kbeg / kBN;
  jb1 = (kend + kBN - 1) / kBN;
}

__device__ __forceinline__ bool visible(const AttnParams& p, const SegInfo& s, int qi, int kk) {
  bool ok = (kk < s.k_len) && (kk >= s.k_skip) && (qi < s.q_len);
  if (p.causal) ok = ok && (kk <= qi + s.off);
  if (p.window > 0) ok = ok && (kk > qi + s.off - p.window);
  return ok;
}


int make_head_map(CUtensorMap* m, const void* base, int heads, long long rows, long long row_stride_elems, int box_rows);

}  // namespace stb
