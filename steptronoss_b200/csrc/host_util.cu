// Host utilities shared by the launchers: the driver entry point for tensor-map encoding
// (looked up at run time so the library links without libcuda) and device properties.
#include "common.cuh"

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

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t pitch_bytes,
                      uint32_t box0, uint32_t box1, int swizzle128) {
  ensure_context_on_this_thread();
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {d0, d1};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
}

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t pitch_bytes,
                 uint32_t box0, uint32_t box1, int swizzle128) {
  ensure_context_on_this_thread();
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {d0, d1};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
}

int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1,
                      uint64_t pitch2, uint32_t box0, uint32_t box1, uint32_t box2, int swizzle128) {
  ensure_context_on_this_thread();
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {pitch1, pitch2};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
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
