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
};

// 128-byte-swizzled address of (row, 16-byte chunk) inside a [128][64 bf16] slab.
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

// One 128x128x128 product out of 8 UMMA (K = 16 each).
//   A_KMAJOR: A tile is [M rows][K] (slabs split K); otherwise [K rows][M] (slabs split M).
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void mma_128x128x128(uint32_t d_tmem, uint32_t sa, uint32_t sb, bool accumulate) {
  constexpr uint32_t idesc = umma_idesc_bf16(128, 128, A_MN ? 1 : 0, B_MN ? 1 : 0);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint64_t da = A_MN ? umma_smem_desc(sa + k * 2048, kSlabBytes, 1024)
                             : umma_smem_desc(sa + (k >> 2) * kSlabBytes + (k & 3) * 32, 16, 1024);
    const uint64_t db = B_MN ? umma_smem_desc(sb + k * 2048, kSlabBytes, 1024)
                             : umma_smem_desc(sb + (k >> 2) * kSlabBytes + (k & 3) * 32, 16, 1024);
    umma_bf16(d_tmem, da, db, idesc, (accumulate || k > 0) ? 1u : 0u);
  }
}

__device__ __forceinline__ void load_tile(void* dst, const CUtensorMap* m, uint64_t* bar, int head, int row) {
  tma_load_3d(dst, m, bar, 0, head, row);
  tma_load_3d(static_cast<uint8_t*>(dst) + kSlabBytes, m, bar, 64, head, row);
}

struct SegInfo {
  int q_begin, q_len, k_begin, k_len, off;
};

__device__ __forceinline__ SegInfo seg_info(const AttnParams& p, int seg) {
  SegInfo s;
  s.q_begin = p.cu_q[seg];
  s.q_len = p.cu_q[seg + 1] - s.q_begin;
  s.k_begin = p.cu_k[seg];
  s.k_len = p.cu_k[seg + 1] - s.k_begin;
  s.off = s.k_len - s.q_len;
  return s;
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
  bool ok = (kk < s.k_len) && (qi < s.q_len);
  if (p.causal) ok = ok && (kk <= qi + s.off);
  if (p.window > 0) ok = ok && (kk > qi + s.off - p.window);
  return ok;
}


int make_head_map(CUtensorMap* m, const void* base, int heads, long long rows, long long row_stride_elems, int box_rows);

}  // namespace stb
