// Host utilities shared by the launchers: the driver entry point for tensor-map encoding
// (looked up at run time so the library links without libcuda) and device properties.
#include "common.cuh"

#include <cstring>
#include <mutex>

namespace stb {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

// The tensor-map encoder is a driver call and needs a current context on the calling thread; autograd
// runs backward on worker threads that have only selected a device through the runtime API, which binds
// the primary context lazily.  One cheap runtime call per thread makes the binding happen.
static void ensure_context_on_this_thread() {
  static thread_local bool ready = false;
  if (!ready) {
    cudaFree(nullptr);
    ready = true;
  }
}

// A tensor map is a pure function of (type, rank, base, extents, pitches, box, swizzle).  The caching allocator of
// the framework hands the same addresses back step after step, so the launchers ask for the same few hundred maps
// again and again; a direct-mapped per-thread table turns the driver call into a 64-byte compare.
namespace {

struct TmapKey {
  const void* base;
  uint64_t dims[3];
  uint64_t pitch[2];
  uint32_t box[3];
  uint32_t meta;   // rank | element bytes << 4 | swizzle << 8
};

struct alignas(64) TmapSlot {
  CUtensorMap map;
  TmapKey key;
  bool valid;
};

constexpr int kTmapSlots = 2048;

inline uint64_t tmap_hash(const TmapKey& k) {
  const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
  uint64_t h = 0x9E3779B97F4A7C15ull;
  for (size_t i = 0; i < sizeof(TmapKey) / 8; ++i) {
    h ^= w[i] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  }
  return h ^ (h >> 29);
}

int encode_cached(CUtensorMap* out, const TmapKey& key) {
  static_assert(sizeof(TmapKey) % 8 == 0, "key is hashed by 64-bit words");
  static thread_local TmapSlot* table = nullptr;
  if (table == nullptr) table = new TmapSlot[kTmapSlots]();   // lives as long as the thread's process
  TmapSlot& slot = table[tmap_hash(key) & (kTmapSlots - 1)];
  if (slot.valid && std::memcmp(&slot.key, &key, sizeof(TmapKey)) == 0) {
    *out = slot.map;
    return 0;
  }
  ensure_context_on_this_thread();
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  const int rank = key.meta & 15, elem = (key.meta >> 4) & 15, swz = (key.meta >> 8) & 1;
  cuuint64_t dims[3] = {key.dims[0], key.dims[1], key.dims[2]};
  cuuint64_t strides[2] = {key.pitch[0], key.pitch[1]};
  cuuint32_t box[3] = {key.box[0], key.box[1], key.box[2]};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dtype = elem == 4   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                    : elem == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                                : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = enc(out, dtype, rank,
                   const_cast<void*>(key.base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swz ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -static_cast<int>(r) - 1000;
  slot.map = *out;
  slot.key = key;
  slot.valid = true;
  return 0;
}

}  // namespace

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t pitch_bytes,
                 uint32_t box0, uint32_t box1, int swizzle128) {
  TmapKey k{};
  k.base = base;
  k.dims[0] = d0; k.dims[1] = d1;
  k.pitch[0] = pitch_bytes;
  k.box[0] = box0; k.box[1] = box1;
  k.meta = 2u | (static_cast<uint32_t>(elem_bytes == 4 ? 4 : elem_bytes == 1 ? 1 : 2) << 4) | (swizzle128 ? 1u << 8 : 0u);
  return encode_cached(out, k);
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t pitch_bytes,
                      uint32_t box0, uint32_t box1, int swizzle128) {
  return make_tmap_2d(out, base, 2, d0, d1, pitch_bytes, box0, box1, swizzle128);
}

int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1,
                      uint64_t pitch2, uint32_t box0, uint32_t box1, uint32_t box2, int swizzle128) {
  TmapKey k{};
  k.base = base;
  k.dims[0] = d0; k.dims[1] = d1; k.dims[2] = d2;
  k.pitch[0] = pitch1; k.pitch[1] = pitch2;
  k.box[0] = box0; k.box[1] = box1; k.box[2] = box2;
  k.meta = 3u | (2u << 4) | (swizzle128 ? 1u << 8 : 0u);
  return encode_cached(out, k);
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace stb

extern "C" int stb_sm_count() { return stb::sm_count(); }
extern "C" const char* stb_build_arch() { return "sm_100a"; }
