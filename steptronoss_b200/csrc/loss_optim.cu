// Vocab-parallel cross-entropy (two-phase, fused forward+backward) and the optimizer-side
// kernels: squared-norm reduction, fused Adam on flat fp32 shards with bf16 write-back, casts.
//
// Cross-entropy semantics follow steptronoss/core/tensor_parallel/cross_entropy.py:28-150
// (max, target logit and sum-exp reduced over the TP group; token accuracy; label smoothing is
// handled by the caller), restructured so that the fp32 logits tensor never exists: logits stay
// bf16 and are turned into their own gradient in place.
//
// Optimizer semantics follow steptronoss/exp/optimizer.py:44-62 (torch Adam with coupled L2
// decay on fp32 masters) and steptronoss/optimizer/clip_grads.py:20-147 (global L2 clip), with the
// clip coefficient kept on the device so the step never synchronises with the host.
#include "common.cuh"

namespace stb {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum2(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int kCeThreads = 512;

// Phase 1: per row of a [rows][V_local] bf16 logits shard: local max, sum exp(x - max), the target
// logit (if the label falls in this shard, else 0) and the local arg-max.
// stats[row] = {max, sumexp, target_logit, argmax_value};  argmax_idx[row] = global vocab index.
__global__ void __launch_bounds__(kCeThreads)
ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                float4* __restrict__ stats, long long* __restrict__ argmax_idx, int V, long long ld,
                long long vocab_start) {
  __shared__ float s_max[kCeThreads / 32];
  __shared__ float s_sum[kCeThreads / 32];
  __shared__ int s_arg[kCeThreads / 32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  const int nvec = V / 8;
  float m = -INFINITY, s = 0.f;
  int arg = 0;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    const uint4 u = *reinterpret_cast<const uint4*>(lr + v * 8);
    float f[8] = {bf16_lo(u.x), bf16_hi(u.x), bf16_lo(u.y), bf16_hi(u.y),
                  bf16_lo(u.z), bf16_hi(u.z), bf16_lo(u.w), bf16_hi(u.w)};
    float lm = f[0];
    int la = 0;
#pragma unroll
    for (int j = 1; j < 8; ++j)
      if (f[j] > lm) { lm = f[j]; la = j; }
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
      arg = v * 8 + la;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  // warp combine
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
    const float nm = fmaxf(m, om);
    const float a = (m == -INFINITY) ? 0.f : s * __expf(m - nm);
    const float b = (om == -INFINITY) ? 0.f : os * __expf(om - nm);
    if (om > m || (om == m && oa < arg)) arg = oa;
    s = a + b;
    m = nm;
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { s_max[w] = m; s_sum[w] = s; s_arg[w] = arg; }
  __syncthreads();
  if (w == 0) {
    m = (l < kCeThreads / 32) ? s_max[l] : -INFINITY;
    s = (l < kCeThreads / 32) ? s_sum[l] : 0.f;
    arg = (l < kCeThreads / 32) ? s_arg[l] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      const float nm = fmaxf(m, om);
      const float a = (m == -INFINITY) ? 0.f : s * __expf(m - nm);
      const float b = (om == -INFINITY) ? 0.f : os * __expf(om - nm);
      if (om > m || (om == m && oa < arg)) arg = oa;
      s = a + b;
      m = nm;
    }
    if (l == 0) {
      const long long lab = labels[row] - vocab_start;
      float tgt = 0.f;
      if (lab >= 0 && lab < V) tgt = __bfloat162float(lr[lab]);
      stats[row] = make_float4(m, s, tgt, m);
      argmax_idx[row] = vocab_start + arg;
    }
  }
}

// Phase 2: with the globally-reduced (gmax, gsum) per row: logits <- (softmax - onehot) * w[row]
// in place (bf16).  Rows with w == 0 get zeros.
__global__ void __launch_bounds__(kCeThreads)
ce_grad_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
               const float* __restrict__ gmax, const float* __restrict__ gsum, const float* __restrict__ weight,
               int V, long long ld, long long vocab_start) {
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const float w = weight[row];
  const float m = gmax[row];
  const float inv = w / gsum[row];
  const long long lab = labels[row] - vocab_start;
  const int nvec = V / 8;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    uint4 u = *reinterpret_cast<const uint4*>(lr + v * 8);
    float f[8] = {bf16_lo(u.x), bf16_hi(u.x), bf16_lo(u.y), bf16_hi(u.y),
                  bf16_lo(u.z), bf16_hi(u.z), bf16_lo(u.w), bf16_hi(u.w)};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float g = (w == 0.f) ? 0.f : __expf(f[j] - m) * inv;
      if (v * 8 + j == lab) g -= w;
      f[j] = g;
    }
    u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]);
    u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
    *reinterpret_cast<uint4*>(lr + v * 8) = u;
  }
}

// ============================================================================ norms / Adam
constexpr int kOptThreads = 512;

// partial[b] = sum of squares of the b-th slice; deterministic two-pass reduction.
__global__ void __launch_bounds__(kOptThreads)
sqnorm_partial_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[kOptThreads / 32];
  float s = 0.f;
  const long long n4 = n / 4;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) s += x[i] * x[i];
  s = warp_sum2(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = (threadIdx.x < kOptThreads / 32) ? red[threadIdx.x] : 0.f;
    t = warp_sum2(t);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
  }
}

// out[0] (+)= sum(partial[0..n))
__global__ void sum_partials_kernel(const float* __restrict__ partial, int n, float* __restrict__ out,
                                    int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = warp_sum2(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
    t = warp_sum2(t);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + t : t;
  }
}

// scalars[0] = total squared norm (already reduced across ranks) -> scalars[1] = norm,
// scalars[2] = clip coefficient min(1, max_norm / (norm + 1e-6)); scalars[3] = 1 when norm is finite.
__global__ void clip_coef_kernel(float* scalars, float max_norm) {
  const float nrm = sqrtf(scalars[0]);
  scalars[1] = nrm;
  float c = 1.f;
  if (max_norm > 0.f) c = fminf(1.f, max_norm / (nrm + 1e-6f));
  const bool finite = isfinite(nrm);
  scalars[2] = finite ? c : 0.f;
  scalars[3] = finite ? 1.f : 0.f;
}

struct AdamChunk {
  long long offset;  // element offset into the flat shard
  int len;
  float lr_mult;
  float weight_decay;
};

// Fused Adam on a flat fp32 shard. g is the (already reduced) fp32 gradient; `scalars[2]` is the clip
// coefficient, `grad_scale` the accumulation/averaging factor. mode 0: coupled L2 (torch.optim.Adam),
// mode 1: decoupled (AdamW). Writes the new bf16 parameter copy. A non-finite global norm
// (scalars[3] == 0) skips the update, matching a skipped iteration.
__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
            __nv_bfloat16* __restrict__ p_bf16, const AdamChunk* __restrict__ chunks, const float* __restrict__ scalars,
            float lr, float beta1, float beta2, float eps, float bc1, float bc2, float grad_scale, int mode) {
  const AdamChunk c = chunks[blockIdx.x];
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
    if (p_bf16) p_bf16[k] = __float2bfloat16_rn(pv);
  }
}

__global__ void __launch_bounds__(256)
cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16_rn(in[i]);
}

// acc[i] += g[i] (bf16 gradient folded into the fp32 accumulation buffer)
__global__ void __launch_bounds__(256)
accumulate_bf16_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ g, long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    acc[i] += __bfloat162float(g[i]);
}

__global__ void __launch_bounds__(256) scale_f32_kernel(float* __restrict__ x, long long n, float a) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    x[i] *= a;
}

// Device-side NaN/Inf probe: flag[0] |= 1 when any element is not finite (no host sync).
__global__ void __launch_bounds__(256)
nonfinite_flag_kernel(const __nv_bfloat16* __restrict__ x, long long n, int* __restrict__ flag) {
  bool bad = false;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    bad |= !isfinite(__bfloat162float(x[i]));
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(flag, 1);
}

static inline int grid_cap(long long items, int threads, int per_sm) {
  long long g = (items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * per_sm;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace stb

using namespace stb;

extern "C" int stb_ce_stats(const void* logits, const long long* labels, float* stats, long long* argmax_idx,
                            long long rows, int V, long long ld, long long vocab_start, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (V % 8 || ld % 8) return -kErrBadArgument;
  ce_stats_kernel<<<static_cast<unsigned>(rows), kCeThreads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(logits), labels, reinterpret_cast<float4*>(stats), argmax_idx, V, ld,
      vocab_start);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_ce_grad(void* logits, const long long* labels, const float* gmax, const float* gsum,
                           const float* weight, long long rows, int V, long long ld, long long vocab_start,
                           cudaStream_t st) {
  if (rows <= 0) return 0;
  if (V % 8 || ld % 8) return -kErrBadArgument;
  ce_grad_kernel<<<static_cast<unsigned>(rows), kCeThreads, 0, st>>>(static_cast<__nv_bfloat16*>(logits), labels, gmax,
                                                                    gsum, weight, V, ld, vocab_start);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_sqnorm_grid() { return sm_count() * 4; }

// partial: scratch of stb_sqnorm_grid() floats. out[0] (+)= ||x||^2.
extern "C" int stb_sqnorm(const float* x, long long n, float* partial, float* out, int accumulate, cudaStream_t st) {
  const int grid = stb_sqnorm_grid();
  sqnorm_partial_kernel<<<grid, kOptThreads, 0, st>>>(x, n, partial);
  sum_partials_kernel<<<1, 256, 0, st>>>(partial, grid, out, accumulate);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_clip_coef(float* scalars, float max_norm, cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>(scalars, max_norm);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_adam(float* p, const float* g, float* m, float* v, void* p_bf16, const void* chunks, int num_chunks,
                        const float* scalars, float lr, float beta1, float beta2, float eps, float bc1, float bc2,
                        float grad_scale, int mode, cudaStream_t st) {
  if (num_chunks <= 0) return 0;
  adam_kernel<<<num_chunks, 256, 0, st>>>(p, g, m, v, static_cast<__nv_bfloat16*>(p_bf16),
                                          static_cast<const AdamChunk*>(chunks), scalars, lr, beta1, beta2, eps, bc1,
                                          bc2, grad_scale, mode);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_cast_f32_bf16(const float* in, void* out, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_cap(n, 256, 8), 256, 0, st>>>(in, static_cast<__nv_bfloat16*>(out), n);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_accumulate_bf16(float* acc, const void* g, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  accumulate_bf16_kernel<<<grid_cap(n, 256, 8), 256, 0, st>>>(acc, static_cast<const __nv_bfloat16*>(g), n);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_scale_f32(float* x, long long n, float a, cudaStream_t st) {
  if (n <= 0) return 0;
  scale_f32_kernel<<<grid_cap(n, 256, 8), 256, 0, st>>>(x, n, a);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_nonfinite_flag(const void* x, long long n, int* flag, cudaStream_t st) {
  if (n <= 0) return 0;
  nonfinite_flag_kernel<<<grid_cap(n, 256, 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, flag);
  return -static_cast<int>(cudaGetLastError());
}

// ----------------------------------------------------------------------------- generalised advantage estimation
// adv_t = delta_t + gamma*lambda*adv_{t+1},  delta_t = r_t + gamma*v_{t+1} - v_t, restarted at every segment end
// (v_{T} = 0).  One thread walks one packed segment backwards; segments run in parallel.  Stands where the
// reference loops over time steps on the host (steptronoss/utils/rl_utils.py:180-210).
namespace stb {
__global__ void gae_kernel(const float* __restrict__ values, const float* __restrict__ rewards,
                           const int* __restrict__ cu, int n_seg, float gamma, float lambd,
                           float* __restrict__ adv, float* __restrict__ ret) {
  const int seg = blockIdx.x * blockDim.x + threadIdx.x;
  if (seg >= n_seg) return;
  const int b = cu[seg], e = cu[seg + 1];
  float next_v = 0.f, run = 0.f;
  for (int t = e - 1; t >= b; --t) {
    const float v = values[t];
    const float delta = rewards[t] + gamma * next_v - v;
    run = delta + gamma * lambd * run;
    adv[t] = run;
    ret[t] = run + v;
    next_v = v;
  }
}
}  // namespace stb

extern "C" int stb_gae(const float* values, const float* rewards, const int* cu_seqlens, int n_seg, float gamma,
                       float lambd, float* adv, float* ret, cudaStream_t st) {
  if (n_seg <= 0) return 0;
  stb::gae_kernel<<<(n_seg + 63) / 64, 64, 0, st>>>(values, rewards, cu_seqlens, n_seg, gamma, lambd, adv, ret);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
