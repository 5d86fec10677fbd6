// ZeRO-1 step over peer memory (NVLink), for data-parallel groups inside one node.
//
// The reference reduces gradients with `buf /= N; reduce_scatter_tensor`, takes the gradient norm in a separate
// pass, runs torch Adam on the owned shard and all-gathers the bf16 parameters
// (steptronoss/optimizer/zero1_gradient_manager.py:164-228).  Here the flat fp32 gradient buffer and the bf16
// parameter buffer of every rank live in memory that the other ranks of the group have mapped, and the step is
//
//   stb_zero_publish : "my gradients are complete" (flag = step number in every peer's flag page)
//   stb_zero_reduce  : waits (bounded) for every peer's flag, then for the owned shard only:
//                      g[i] = scale * sum over ranks r, in rank order, of grad_r[lo + i]   (peer loads, fp32)
//                      written into the own buffer in place, with the shard's squared norm as a by-product
//                      (per-block partials, added in block order: deterministic)
//   stb_adam_push    : the Adam update of the shard (same rule as stb_adam) whose bf16 result is stored into the
//                      parameter buffer of every rank of the group, so no all-gather follows
//   stb_zero_publish : "my parameter shard has landed everywhere"; the next forward waits for all peers' flags
//                      (stb_peer_wait_flags), which also tells it that every peer has finished reading its gradients.
//
// Ranks only write what they own (their shard of their own gradient buffer, their shard of every parameter
// buffer), so no two ranks ever write the same address.
#include "common.cuh"

namespace stb {

constexpr int kZeroMaxRanks = 8;
struct ZeroPtrs {
  void* p[kZeroMaxRanks];
};

__device__ __forceinline__ void zst_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t zld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void zero_publish_kernel(const __grid_constant__ ZeroPtrs flags, int flag_index, int world, int rank,
                                    uint32_t epoch) {
  __threadfence_system();
  if (threadIdx.x < world)
    zst_release_sys_u32(static_cast<uint32_t*>(flags.p[threadIdx.x]) + flag_index * kZeroMaxRanks + rank, epoch);
}

// n4: float4 words of the shard.  partials[blockIdx.x] = sum of squares of this block's results.
__global__ void __launch_bounds__(256)
zero_reduce_kernel(const __grid_constant__ ZeroPtrs grads, long long n4, int world, int rank, float scale,
                   float* __restrict__ partials, const uint32_t* __restrict__ flags_self, int flag_index,
                   uint32_t epoch, unsigned long long budget_ns, int* status) {
  __shared__ int ok;
  __shared__ float red[8];
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const uint32_t* f = flags_self + flag_index * kZeroMaxRanks + threadIdx.x;
    uint64_t t0 = 0;   // the wall clock is slow to read: not before the first miss
    for (uint32_t i = 0;; ++i) {
      if (static_cast<int32_t>(zld_acquire_sys_u32(f) - epoch) >= 0) break;
      if (i == 0) t0 = global_timer_ns();
      if ((i & 15u) == 15u && global_timer_ns() - t0 > budget_ns) {
        report_error(status, kErrPeerFlagWait);
        ok = 0;
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  float sq = 0.f;
  if (ok) {
    float4* own = static_cast<float4*>(grads.p[rank]);
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float4 v[kZeroMaxRanks];
#pragma unroll
      for (int r = 0; r < kZeroMaxRanks; ++r)
        if (r < world) v[r] = static_cast<const float4*>(grads.p[r])[i];
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < kZeroMaxRanks; ++r) {
        if (r >= world) continue;
        s.x += v[r].x;
        s.y += v[r].y;
        s.z += v[r].z;
        s.w += v[r].w;
      }
      s.x *= scale;
      s.y *= scale;
      s.z *= scale;
      s.w *= scale;
      own[i] = s;
      sq += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    // A shard whose wait ran out stays unreduced: poison its squared norm, so that the clip kernel sees a
    // non-finite norm on every rank (the norm is all-reduced) and the Adam kernels skip this step everywhere.
    partials[blockIdx.x] = ok ? t : __int_as_float(0x7fc00000);
  }
}

__global__ void zero_finish_kernel(const float* __restrict__ partials, int n, float* out, int accumulate) {
  // one warp, fixed order: lane l adds partials l, l+32, ...; then a shuffle tree
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += 32) s += partials[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

struct AdamChunkZ {
  long long offset;
  int len;
  float lr_mult;
  float weight_decay;
};

__global__ void __launch_bounds__(256)
adam_push_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                 const __grid_constant__ ZeroPtrs params, int world, const AdamChunkZ* __restrict__ chunks,
                 const float* __restrict__ scalars, float lr, float beta1, float beta2, float eps, float bc1, float bc2,
                 float grad_scale, int mode) {
  const AdamChunkZ c = chunks[blockIdx.x];
  const float clip = scalars ? scalars[2] : 1.f;
  if (scalars && scalars[3] == 0.f) return;
  const float gs = grad_scale * clip;
  const float lr_eff = lr * c.lr_mult;
  const float step_size = lr_eff / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  for (int i = threadIdx.x; i < c.len; i += blockDim.x) {
    const long long k = c.offset + i;
    float pv = p[k];
    float gv = g[k] * gs;
    if (mode == 0) gv += c.weight_decay * pv;
    else pv *= (1.f - lr_eff * c.weight_decay);
    const float mv = beta1 * m[k] + (1.f - beta1) * gv;
    const float vv = beta2 * v[k] + (1.f - beta2) * gv * gv;
    m[k] = mv;
    v[k] = vv;
    const float denom = sqrtf(vv) * inv_sqrt_bc2 + eps;
    pv -= step_size * mv / denom;
    p[k] = pv;
    const __nv_bfloat16 lp = __float2bfloat16_rn(pv);
#pragma unroll
    for (int r = 0; r < kZeroMaxRanks; ++r)
      if (r < world) static_cast<__nv_bfloat16*>(params.p[r])[k] = lp;
  }
}

}  // namespace stb

using namespace stb;

extern "C" int stb_zero_reduce_blocks() { return sm_count() * 8; }

extern "C" int stb_zero_publish(void* const* flag_pages, int flag_index, int world, int rank, unsigned epoch,
                                cudaStream_t stream) {
  if (world < 1 || world > kZeroMaxRanks) return -kErrBadArgument;
  ZeroPtrs f{};
  for (int i = 0; i < world; ++i) f.p[i] = flag_pages[i];
  zero_publish_kernel<<<1, 32, 0, stream>>>(f, flag_index, world, rank, epoch);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

// grads[r]: rank r's gradient buffer at the start of THIS rank's shard (fp32, 16-byte aligned); n: elements of the
// shard (multiple of 4); partials: stb_zero_reduce_blocks() floats; sq_out[0] (+)= squared norm of the result.
extern "C" int stb_zero_reduce(void* const* grads, long long n, int world, int rank, float scale, void* partials,
                               float* sq_out, int accumulate, const void* flag_page_self, int flag_index,
                               unsigned epoch, unsigned long long wait_ns, int* status, cudaStream_t stream) {
  if (world < 1 || world > kZeroMaxRanks || (n & 3)) return -kErrBadArgument;
  ZeroPtrs g{};
  for (int i = 0; i < world; ++i) {
    if (reinterpret_cast<uintptr_t>(grads[i]) & 15) return -kErrBadArgument;
    g.p[i] = grads[i];
  }
  const long long n4 = n / 4;
  long long blocks = (n4 + 255) / 256;
  const int cap = stb_zero_reduce_blocks();
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  zero_reduce_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      g, n4, world, rank, scale, static_cast<float*>(partials), static_cast<const uint32_t*>(flag_page_self),
      flag_index, epoch, wait_ns, status);
  zero_finish_kernel<<<1, 32, 0, stream>>>(static_cast<const float*>(partials), static_cast<int>(blocks), sq_out,
                                           accumulate);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

// params[r]: rank r's bf16 parameter buffer at the start of THIS rank's shard.  Other arguments as stb_adam.
extern "C" int stb_adam_push(float* p, const float* g, float* m, float* v, void* const* params, int world,
                             const void* chunks, int num_chunks, const float* scalars, float lr, float beta1,
                             float beta2, float eps, float bc1, float bc2, float grad_scale, int mode,
                             cudaStream_t stream) {
  if (world < 1 || world > kZeroMaxRanks) return -kErrBadArgument;
  if (num_chunks <= 0) return 0;
  ZeroPtrs q{};
  for (int i = 0; i < world; ++i) q.p[i] = params[i];
  adam_push_kernel<<<num_chunks, 256, 0, stream>>>(p, g, m, v, q, world, static_cast<const AdamChunkZ*>(chunks),
                                                   scalars, lr, beta1, beta2, eps, bc1, bc2, grad_scale, mode);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
