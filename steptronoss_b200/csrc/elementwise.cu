// Memory-bound transformer ops for sm_100a: RMSNorm, fused per-head QK-norm + RoPE, SwiGLU,
// embedding gather / scatter-add.  All math is fp32 internally with bf16 (or fp32) storage and
// 16-byte vector accesses; each kernel touches every input byte once.
//
// Reference semantics: steptronoss/model/common/rms_norm.py:5-62 (fp32 compute, optional
// zero-centred gamma), steptronoss/model/common/rope.py:220-250 (half-split rotation with a
// position-id gather), steptronoss/model/common/feed_forward.py:20-26 (SwiGLU with optional clamps),
// steptronoss/core/tensor_parallel/layers.py:120-139 (vocab-sharded embedding).
#include "common.cuh"

namespace stb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  f[0] = bf16_lo(u.x); f[1] = bf16_hi(u.x); f[2] = bf16_lo(u.y); f[3] = bf16_hi(u.y);
  f[4] = bf16_lo(u.z); f[5] = bf16_hi(u.z); f[6] = bf16_lo(u.w); f[7] = bf16_hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]);
  u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
  return u;
}

// ============================================================================ RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * (w [+ 1]);  one CTA per row, the row stays in registers.
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // up to 256*8*4 = 8192 columns held in registers

// With `delta` the row that is normalised is s = bf16(x + delta), which is also written to `sum_out` (the residual
// stream of a pre-norm block: one pass instead of an add kernel followed by a norm kernel).
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd_out, int H, long long x_stride,
                   long long delta_stride, long long y_stride, long long sum_stride, float eps, int zero_centered) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * x_stride);
  const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + row * delta_stride) : nullptr;
  uint4* sr = sum_out ? reinterpret_cast<uint4*>(sum_out + row * sum_stride) : nullptr;
  const int nvec = H / 8;
  uint4 cache[kNormMaxVec];
  float ss = 0.f;
  // s = bf16(x + delta): what an elementwise bf16 add would have produced, so the statistics see the rounded sum
  auto load_row = [&](int v) -> uint4 {
    uint4 u = xr[v];
    if (dr != nullptr) {
      float a[8], b[8];
      unpack8(u, a);
      unpack8(dr[v], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
      u = pack8(a);
      if (sr != nullptr) sr[v] = u;
    }
    return u;
  };
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      cache[i] = load_row(v);
      float f[8];
      unpack8(cache[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  for (int v = threadIdx.x + kNormMaxVec * kNormThreads; v < nvec; v += kNormThreads) {
    float f[8];
    unpack8(load_row(v), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum<kNormThreads>(ss, red);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * y_stride);
  const float woff = zero_centered ? 1.f : 0.f;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      float f[8], g[8];
      unpack8(cache[i], f);
      unpack8(wr[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * (g[j] + woff);
      yr[v] = pack8(f);
    }
  }
  for (int v = threadIdx.x + kNormMaxVec * kNormThreads; v < nvec; v += kNormThreads) {
    float f[8], g[8];
    if (dr != nullptr) {       // very wide rows: the sum is recomputed (it was written to sum_out by this thread)
      float b[8];
      unpack8(xr[v], f);
      unpack8(dr[v], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += b[j];
      unpack8(pack8(f), f);
    } else {
      unpack8(xr[v], f);
    }
    unpack8(wr[v], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * (g[j] + woff);
    yr[v] = pack8(f);
  }
}

// dx = rstd * (g*w' - xhat * mean(g*w'*xhat));  dw partial[cta] = sum over the CTA's rows of g*xhat.
// Persistent over rows so that the weight-gradient partials stay in registers; the partials go to
// a [grid, H] fp32 scratch that rmsnorm_dw_reduce_kernel folds (in fixed order) into dw.
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const __nv_bfloat16* __restrict__ g, const float* __restrict__ rstd_in,
                   __nv_bfloat16* dx, float* __restrict__ dw_partial, int rows, int H, long long x_stride,
                   long long g_stride, long long dx_stride, int zero_centered, const __nv_bfloat16* dres,
                   long long dres_stride) {
  __shared__ float red[32];
  const int nvec = H / 8;
  float dw_acc[kNormMaxVec][8];
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const float woff = zero_centered ? 1.f : 0.f;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * x_stride);
    const uint4* gr = reinterpret_cast<const uint4*>(g + row * g_stride);
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * dx_stride);
    // gradient that reached the normalised tensor by another path (the residual stream); may alias dx
    const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + row * dres_stride) : nullptr;
    const float rstd = rstd_in[row];
    float xh[kNormMaxVec][8], gw[kNormMaxVec][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float xf[8], gf[8], wf[8];
        unpack8(xr[v], xf);
        unpack8(gr[v], gf);
        unpack8(wr[v], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = xf[j] * rstd;
          gw[i][j] = gf[j] * (wf[j] + woff);
          dw_acc[i][j] += gf[j] * xh[i][j];
          dot += gw[i][j] * xh[i][j];
        }
      }
    }
    dot = block_sum<kNormThreads>(dot, red) / H;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (gw[i][j] - xh[i][j] * dot) * rstd;
        if (rr != nullptr) {
          float old[8];
          unpack8(rr[v], old);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += old[j];
        }
        dxr[v] = pack8(o);
      }
    }
  }
  float* part = dw_partial + static_cast<long long>(blockIdx.x) * H;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      float4* dst = reinterpret_cast<float4*>(part + v * 8);
      dst[0] = make_float4(dw_acc[i][0], dw_acc[i][1], dw_acc[i][2], dw_acc[i][3]);
      dst[1] = make_float4(dw_acc[i][4], dw_acc[i][5], dw_acc[i][6], dw_acc[i][7]);
    }
  }
}

// dw[c] (+)= sum_p partial[p][c] in a fixed order (deterministic): a block owns 32 columns, its eight warps each
// add every eighth partial row (coalesced 128-byte reads), and warp 0 adds the eight sub-sums in order.
constexpr int kDwReduceWarps = 8;
__global__ void __launch_bounds__(32 * kDwReduceWarps)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int parts, int H, int accumulate,
                         long long part_stride) {
  __shared__ float sub[kDwReduceWarps][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < H)
    for (int p = ty; p < parts; p += kDwReduceWarps) s += partial[static_cast<long long>(p) * part_stride + c];
  sub[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kDwReduceWarps; ++i) t += sub[i][tx];
    dw[c] = accumulate ? dw[c] + t : t;
  }
}

// ============================================================================ QK-norm + RoPE
// qkv row layout per token: [q heads (hq*D) | k heads (hkv*D) | v heads (hkv*D)], D = 128.
// One warp per (token, head) for the hq + hkv normalised heads; lane l holds elements 4l..4l+3,
// the RoPE partner (i +- D/2) lives in lane l ^ 16.  cos/sin tables are fp32 [max_pos][rot/2];
// rot <= D is the rotary width (partial rotary leaves the tail untouched).  Output q [T][hq][D]
// and k [T][hkv][D]; v is consumed in place by the attention kernel.
constexpr int kHeadDim = 128;

__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ qw,
                       const __nv_bfloat16* __restrict__ kw, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, const int* __restrict__ pos, __nv_bfloat16* __restrict__ q_out,
                       __nv_bfloat16* __restrict__ k_out, float* __restrict__ rstd_out, int T, int hq, int hkv,
                       long long qkv_stride, int rot, float eps, int use_norm, int zero_centered) {
  const int heads = hq + hkv;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(T) * heads) return;
  const int t = static_cast<int>(wid / heads);
  const int h = static_cast<int>(wid % heads);
  const bool is_q = h < hq;
  const __nv_bfloat16* src = qkv + t * qkv_stride + static_cast<long long>(h) * kHeadDim + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  float f[4] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y)};
  if (use_norm) {
    float ss = f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3];
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / kHeadDim + eps);
    if (lane == 0 && rstd_out) rstd_out[wid] = rstd;
    const uint2 wraw = *reinterpret_cast<const uint2*>((is_q ? qw : kw) + lane * 4);
    const float woff = zero_centered ? 1.f : 0.f;
    f[0] *= rstd * (bf16_lo(wraw.x) + woff);
    f[1] *= rstd * (bf16_hi(wraw.x) + woff);
    f[2] *= rstd * (bf16_lo(wraw.y) + woff);
    f[3] *= rstd * (bf16_hi(wraw.y) + woff);
  }
  // rotation over the first `rot` elements, half-split: (i, i + rot/2)
  const int half = rot >> 1;
  float o[4];
  const int p = pos[t];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // partner exchange must be executed by all lanes
    const int i = lane * 4 + j;
    float partner;
    if (rot == kHeadDim) {
      partner = __shfl_xor_sync(0xffffffffu, f[j], 16);
    } else {
      // generic partial rotary: partner index i +- half may sit in any lane
      const int pi = (i < half) ? i + half : i - half;
      const int src_lane = (pi >> 2) & 31;
      const float c0 = __shfl_sync(0xffffffffu, f[0], src_lane);
      const float c1 = __shfl_sync(0xffffffffu, f[1], src_lane);
      const float c2 = __shfl_sync(0xffffffffu, f[2], src_lane);
      const float c3 = __shfl_sync(0xffffffffu, f[3], src_lane);
      const int pj = pi & 3;
      partner = pj == 0 ? c0 : pj == 1 ? c1 : pj == 2 ? c2 : c3;
    }
    if (i < rot) {
      const int fi = (i < half) ? i : i - half;
      const float c = cos_t[static_cast<long long>(p) * half + fi];
      const float s = sin_t[static_cast<long long>(p) * half + fi];
      o[j] = (i < half) ? f[j] * c - partner * s : f[j] * c + partner * s;
    } else {
      o[j] = f[j];
    }
  }
  uint2 outv;
  outv.x = pack_bf16(o[0], o[1]);
  outv.y = pack_bf16(o[2], o[3]);
  __nv_bfloat16* dst = is_q ? q_out + (static_cast<long long>(t) * hq + h) * kHeadDim
                            : k_out + (static_cast<long long>(t) * hkv + (h - hq)) * kHeadDim;
  *reinterpret_cast<uint2*>(dst + lane * 4) = outv;
}

// Backward: un-rotate the incoming gradient, then RMSNorm backward over the head; writes the q and
// k slices of dqkv and accumulates per-CTA weight-gradient partials [grid][2][D].
__global__ void __launch_bounds__(256)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ qw,
                       const __nv_bfloat16* __restrict__ kw, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, const int* __restrict__ pos,
                       const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                       const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dqkv,
                       float* __restrict__ dw_partial, int T, int hq, int hkv, long long qkv_stride,
                       long long dqkv_stride, int rot, int use_norm, int zero_centered) {
  __shared__ float sdw[2][kHeadDim];
  for (int i = threadIdx.x; i < 2 * kHeadDim; i += blockDim.x) (&sdw[0][0])[i] = 0.f;
  __syncthreads();
  const int heads = hq + hkv;
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const long long total = static_cast<long long>(T) * heads;
  const int half = rot >> 1;
  float dwq[4] = {0, 0, 0, 0}, dwk[4] = {0, 0, 0, 0};
  for (long long wid = static_cast<long long>(blockIdx.x) * warps_per_cta + (threadIdx.x >> 5); wid < total;
       wid += static_cast<long long>(gridDim.x) * warps_per_cta) {
    const int t = static_cast<int>(wid / heads);
    const int h = static_cast<int>(wid % heads);
    const bool is_q = h < hq;
    const __nv_bfloat16* gsrc = is_q ? dq + (static_cast<long long>(t) * hq + h) * kHeadDim
                                     : dk + (static_cast<long long>(t) * hkv + (h - hq)) * kHeadDim;
    const uint2 graw = *reinterpret_cast<const uint2*>(gsrc + lane * 4);
    float g[4] = {bf16_lo(graw.x), bf16_hi(graw.x), bf16_lo(graw.y), bf16_hi(graw.y)};
    const int p = pos[t];
    float gu[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = lane * 4 + j;
      float partner;
      if (rot == kHeadDim) {
        partner = __shfl_xor_sync(0xffffffffu, g[j], 16);
      } else {
        const int pi = (i < half) ? i + half : i - half;
        const int src_lane = (pi >> 2) & 31;
        const float c0 = __shfl_sync(0xffffffffu, g[0], src_lane);
        const float c1 = __shfl_sync(0xffffffffu, g[1], src_lane);
        const float c2 = __shfl_sync(0xffffffffu, g[2], src_lane);
        const float c3 = __shfl_sync(0xffffffffu, g[3], src_lane);
        const int pj = pi & 3;
        partner = pj == 0 ? c0 : pj == 1 ? c1 : pj == 2 ? c2 : c3;
      }
      if (i < rot) {
        const int fi = (i < half) ? i : i - half;
        const float c = cos_t[static_cast<long long>(p) * half + fi];
        const float s = sin_t[static_cast<long long>(p) * half + fi];
        // y1 = x1 c - x2 s ; y2 = x2 c + x1 s  =>  dx1 = g1 c + g2 s ; dx2 = g2 c - g1 s
        gu[j] = (i < half) ? g[j] * c + partner * s : g[j] * c - partner * s;
      } else {
        gu[j] = g[j];
      }
    }
    float o[4];
    if (use_norm) {
      const uint2 xraw =
          *reinterpret_cast<const uint2*>(qkv + t * qkv_stride + static_cast<long long>(h) * kHeadDim + lane * 4);
      const float x[4] = {bf16_lo(xraw.x), bf16_hi(xraw.x), bf16_lo(xraw.y), bf16_hi(xraw.y)};
      const uint2 wraw = *reinterpret_cast<const uint2*>((is_q ? qw : kw) + lane * 4);
      const float woff = zero_centered ? 1.f : 0.f;
      const float wv[4] = {bf16_lo(wraw.x) + woff, bf16_hi(wraw.x) + woff, bf16_lo(wraw.y) + woff,
                           bf16_hi(wraw.y) + woff};
      const float rstd = rstd_in[wid];
      float dot = 0.f, xh[4], gw[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xh[j] = x[j] * rstd;
        gw[j] = gu[j] * wv[j];
        dot += gw[j] * xh[j];
        if (is_q) dwq[j] += gu[j] * xh[j]; else dwk[j] += gu[j] * xh[j];
      }
      dot = warp_sum(dot) / kHeadDim;
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = (gw[j] - xh[j] * dot) * rstd;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = gu[j];
    }
    uint2 outv;
    outv.x = pack_bf16(o[0], o[1]);
    outv.y = pack_bf16(o[2], o[3]);
    *reinterpret_cast<uint2*>(dqkv + t * dqkv_stride + static_cast<long long>(h) * kHeadDim + lane * 4) = outv;
  }
  if (use_norm) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      atomicAdd(&sdw[0][lane * 4 + j], dwq[j]);
      atomicAdd(&sdw[1][lane * 4 + j], dwk[j]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * kHeadDim; i += blockDim.x)
      dw_partial[static_cast<long long>(blockIdx.x) * 2 * kHeadDim + i] = (&sdw[0][0])[i];
  }
}

// ============================================================================ SwiGLU
// in [rows][2F] = (gate | up) -> out [rows][F] = min(silu(gate), limit) * clamp(up, -limit, limit) when limit > 0
// (the activated gate is clamped from above, after the SiLU), silu(gate) * up otherwise.
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long rows, int F,
                  long long in_stride, long long out_stride, float limit) {
  const int vec_per_row = F / 8;
  const long long total = rows * vec_per_row;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / vec_per_row;
    const int v = static_cast<int>(idx % vec_per_row);
    const uint4 graw = *reinterpret_cast<const uint4*>(in + r * in_stride + v * 8);
    const uint4 uraw = *reinterpret_cast<const uint4*>(in + r * in_stride + F + v * 8);
    float g[8], u[8], o[8];
    unpack8(graw, g);
    unpack8(uraw, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gg = g[j];
      float uu = u[j];
      float act = gg / (1.f + __expf(-gg));
      if (limit > 0.f) {
        act = fminf(act, limit);
        uu = fminf(fmaxf(uu, -limit), limit);
      }
      o[j] = act * uu;
    }
    *reinterpret_cast<uint4*>(out + r * out_stride + v * 8) = pack8(o);
  }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ dout,
                  __nv_bfloat16* __restrict__ din, long long rows, int F, long long in_stride, long long dout_stride,
                  long long din_stride, float limit) {
  const int vec_per_row = F / 8;
  const long long total = rows * vec_per_row;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / vec_per_row;
    const int v = static_cast<int>(idx % vec_per_row);
    const uint4 graw = *reinterpret_cast<const uint4*>(in + r * in_stride + v * 8);
    const uint4 uraw = *reinterpret_cast<const uint4*>(in + r * in_stride + F + v * 8);
    const uint4 draw = *reinterpret_cast<const uint4*>(dout + r * dout_stride + v * 8);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(graw, g);
    unpack8(uraw, u);
    unpack8(draw, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gg = g[j];
      float uu = u[j];
      const float sig = 1.f / (1.f + __expf(-gg));
      const float silu = gg * sig;
      float act = silu;
      bool g_live = true, u_live = true;
      if (limit > 0.f) {                       // a clamp passes the gradient where its input lies inside the bounds
        g_live = silu <= limit;
        u_live = (uu >= -limit) && (uu <= limit);
        act = fminf(silu, limit);
        uu = fminf(fmaxf(uu, -limit), limit);
      }
      dg[j] = g_live ? d[j] * uu * (sig + silu * (1.f - sig)) : 0.f;
      du[j] = u_live ? d[j] * act : 0.f;
    }
    *reinterpret_cast<uint4*>(din + r * din_stride + v * 8) = pack8(dg);
    *reinterpret_cast<uint4*>(din + r * din_stride + F + v * 8) = pack8(du);
  }
}

// ============================================================================ Embedding
// out[t] = (vocab_start <= id < vocab_end) ? table[id - vocab_start] : 0
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                     __nv_bfloat16* __restrict__ out, long long T, int H, long long vocab_start, long long vocab_end) {
  const int vec_per_row = H / 8;
  const long long total = T * vec_per_row;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / vec_per_row;
    const int v = static_cast<int>(idx % vec_per_row);
    const long long id = ids[t];
    uint4 val = make_uint4(0, 0, 0, 0);
    if (id >= vocab_start && id < vocab_end)
      val = *reinterpret_cast<const uint4*>(table + (id - vocab_start) * H + v * 8);
    *reinterpret_cast<uint4*>(out + t * H + v * 8) = val;
  }
}

// grad_table[id - vocab_start] += g[t]  (fp32 accumulation buffer, atomic adds)
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ g,
                     float* __restrict__ grad_table, long long T, int H, long long vocab_start,
                     long long vocab_end) {
  const int vec_per_row = H / 8;
  const long long total = T * vec_per_row;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / vec_per_row;
    const int v = static_cast<int>(idx % vec_per_row);
    const long long id = ids[t];
    if (id < vocab_start || id >= vocab_end) continue;
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(g + t * H + v * 8), f);
    float* dst = grad_table + (id - vocab_start) * H + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, f[j]);
  }
}

// ============================================================================ residual add / casts
__global__ void __launch_bounds__(256)
add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ out, long long n8) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float x[8], y[8];
    unpack8(reinterpret_cast<const uint4*>(a)[i], x);
    unpack8(reinterpret_cast<const uint4*>(b)[i], y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    reinterpret_cast<uint4*>(out)[i] = pack8(x);
  }
}

static inline int grid_for(long long work_items, int threads, int per_sm = 8) {
  long long g = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * per_sm;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace stb

using namespace stb;

extern "C" int stb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int H,
                               long long x_stride, long long y_stride, float eps, int zero_centered,
                               cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H % 8) return -kErrBadArgument;
  rmsnorm_fwd_kernel<<<static_cast<unsigned>(rows), kNormThreads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), nullptr, static_cast<const __nv_bfloat16*>(w),
      static_cast<__nv_bfloat16*>(y), nullptr, rstd, H, x_stride, 0, y_stride, 0, eps, zero_centered);
  return -static_cast<int>(cudaGetLastError());
}

// s = x + delta (bf16, written to `sum`) and y = rmsnorm(s) in one pass; rstd is that of s.
extern "C" int stb_add_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* y, void* sum, float* rstd,
                                   long long rows, int H, long long x_stride, long long delta_stride,
                                   long long y_stride, long long sum_stride, float eps, int zero_centered,
                                   cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H % 8 || delta == nullptr || sum == nullptr) return -kErrBadArgument;
  rmsnorm_fwd_kernel<<<static_cast<unsigned>(rows), kNormThreads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(sum), rstd, H,
      x_stride, delta_stride, y_stride, sum_stride, eps, zero_centered);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_rmsnorm_bwd_grid(long long rows) {
  long long g = static_cast<long long>(sm_count()) * 4;
  return static_cast<int>(rows < g ? rows : g);
}

// dw_partial: caller-provided scratch of stb_rmsnorm_bwd_grid(rows) * H floats.
extern "C" int stb_rmsnorm_bwd(const void* x, const void* w, const void* g, const float* rstd, void* dx, float* dw,
                               float* dw_partial, long long rows, int H, long long x_stride, long long g_stride,
                               long long dx_stride, int zero_centered, int add_to_dx, int accumulate_dw,
                               cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H % 8 || H > kNormThreads * 8 * kNormMaxVec) return -kErrBadArgument;
  const int grid = stb_rmsnorm_bwd_grid(rows);
  rmsnorm_bwd_kernel<<<grid, kNormThreads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(g),
      rstd, static_cast<__nv_bfloat16*>(dx), dw_partial, static_cast<int>(rows), H, x_stride, g_stride, dx_stride,
      zero_centered, add_to_dx ? static_cast<const __nv_bfloat16*>(dx) : nullptr, dx_stride);
  if (dw != nullptr)
    rmsnorm_dw_reduce_kernel<<<(H + 31) / 32, 32 * kDwReduceWarps, 0, st>>>(dw_partial, dw, grid, H, accumulate_dw, H);
  return -static_cast<int>(cudaGetLastError());
}

// Backward of stb_add_rmsnorm_fwd: ds = dsum + rmsnorm_bwd(s, dy) is the gradient of both x and delta.
// s is the saved sum; dsum the gradient that reached it along the residual stream.
extern "C" int stb_add_rmsnorm_bwd(const void* s_in, const void* w, const void* g, const void* dsum, const float* rstd,
                                   void* ds, float* dw, float* dw_partial, long long rows, int H, long long s_stride,
                                   long long g_stride, long long dsum_stride, long long ds_stride, int zero_centered,
                                   int accumulate_dw, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H % 8 || H > kNormThreads * 8 * kNormMaxVec || dsum == nullptr) return -kErrBadArgument;
  const int grid = stb_rmsnorm_bwd_grid(rows);
  rmsnorm_bwd_kernel<<<grid, kNormThreads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(s_in), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(g), rstd, static_cast<__nv_bfloat16*>(ds), dw_partial, static_cast<int>(rows), H,
      s_stride, g_stride, ds_stride, zero_centered, static_cast<const __nv_bfloat16*>(dsum), dsum_stride);
  if (dw != nullptr)
    rmsnorm_dw_reduce_kernel<<<(H + 31) / 32, 32 * kDwReduceWarps, 0, st>>>(dw_partial, dw, grid, H, accumulate_dw, H);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_qknorm_rope_fwd(const void* qkv, const void* qw, const void* kw, const float* cos_t,
                                   const float* sin_t, const int* pos, void* q_out, void* k_out, float* rstd, int T,
                                   int hq, int hkv, int head_dim, long long qkv_stride, int rot, float eps,
                                   int use_norm, int zero_centered, cudaStream_t st) {
  if (T <= 0) return 0;
  if (head_dim != kHeadDim || (rot & 1) || rot > kHeadDim) return -kErrBadArgument;
  const long long warps = static_cast<long long>(T) * (hq + hkv);
  const long long blocks = (warps + 7) / 8;
  qknorm_rope_fwd_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(qw),
      static_cast<const __nv_bfloat16*>(kw), cos_t, sin_t, pos, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(k_out), rstd, T, hq, hkv, qkv_stride, rot, eps, use_norm, zero_centered);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_qknorm_rope_bwd_grid() { return sm_count() * 4; }

// dw_partial: scratch of stb_qknorm_rope_bwd_grid() * 2 * 128 floats; dqw/dkw fp32 [128] (accumulated when asked).
extern "C" int stb_qknorm_rope_bwd(const void* qkv, const void* qw, const void* kw, const float* cos_t,
                                   const float* sin_t, const int* pos, const void* dq, const void* dk,
                                   const float* rstd, void* dqkv, float* dqw, float* dkw, float* dw_partial, int T,
                                   int hq, int hkv, int head_dim, long long qkv_stride, long long dqkv_stride, int rot,
                                   int use_norm, int zero_centered, int accumulate_dw, cudaStream_t st) {
  if (T <= 0) return 0;
  if (head_dim != kHeadDim || (rot & 1) || rot > kHeadDim) return -kErrBadArgument;
  const int grid = stb_qknorm_rope_bwd_grid();
  qknorm_rope_bwd_kernel<<<grid, 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(qw),
      static_cast<const __nv_bfloat16*>(kw), cos_t, sin_t, pos, static_cast<const __nv_bfloat16*>(dq),
      static_cast<const __nv_bfloat16*>(dk), rstd, static_cast<__nv_bfloat16*>(dqkv), dw_partial, T, hq, hkv,
      qkv_stride, dqkv_stride, rot, use_norm, zero_centered);
  if (use_norm && dqw != nullptr) {
    // partial layout [grid][2][128]: first half of each row -> dqw, second half -> dkw
    rmsnorm_dw_reduce_kernel<<<kHeadDim / 32, 32 * kDwReduceWarps, 0, st>>>(dw_partial, dqw, grid, kHeadDim,
                                                                            accumulate_dw, 2 * kHeadDim);
    rmsnorm_dw_reduce_kernel<<<kHeadDim / 32, 32 * kDwReduceWarps, 0, st>>>(dw_partial + kHeadDim, dkw, grid, kHeadDim,
                                                                            accumulate_dw, 2 * kHeadDim);
  }
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_swiglu_fwd(const void* in, void* out, long long rows, int F, long long in_stride,
                              long long out_stride, float limit, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (F % 8) return -kErrBadArgument;
  swiglu_fwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), rows, F, in_stride, out_stride, limit);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_swiglu_bwd(const void* in, const void* dout, void* din, long long rows, int F, long long in_stride,
                              long long dout_stride, long long din_stride, float limit, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (F % 8) return -kErrBadArgument;
  swiglu_bwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(in), static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(din),
      rows, F, in_stride, dout_stride, din_stride, limit);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_embedding_fwd(const long long* ids, const void* table, void* out, long long T, int H,
                                 long long vocab_start, long long vocab_end, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -kErrBadArgument;
  embedding_fwd_kernel<<<grid_for(T * (H / 8), 256), 256, 0, st>>>(ids, static_cast<const __nv_bfloat16*>(table),
                                                                   static_cast<__nv_bfloat16*>(out), T, H,
                                                                   vocab_start, vocab_end);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_embedding_bwd(const long long* ids, const void* g, float* grad_table, long long T, int H,
                                 long long vocab_start, long long vocab_end, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -kErrBadArgument;
  embedding_bwd_kernel<<<grid_for(T * (H / 8), 256), 256, 0, st>>>(ids, static_cast<const __nv_bfloat16*>(g),
                                                                   grad_table, T, H, vocab_start, vocab_end);
  return -static_cast<int>(cudaGetLastError());
}

extern "C" int stb_add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return -kErrBadArgument;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a),
                                                        static_cast<const __nv_bfloat16*>(b),
                                                        static_cast<__nv_bfloat16*>(out), n / 8);
  return -static_cast<int>(cudaGetLastError());
}

// ============================================================================ entry point that allocates nothing
// See noalloc.h.  RMSNorm backward keeps one row of weight-gradient partials per CTA; the regular entry
// point takes that buffer from its caller, this one keeps it in a fixed array that is part of the loaded
// library image on every device.
namespace stb {
constexpr int kNoAllocMaxParts = 256;   // CTAs (partial rows) used by the no-allocation variant
constexpr int kNoAllocMaxH = 4096;      // widest row it accepts
static __device__ __align__(256) float g_rmsnorm_bwd_partials[kNoAllocMaxParts * kNoAllocMaxH];  // 4 MiB per device
constexpr int kNoAllocMaxDevices = 64;
}  // namespace stb

#include <mutex>

extern "C" int stb_rmsnorm_bwd_noalloc_max_hidden() { return stb::kNoAllocMaxH; }

extern "C" int stb_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* g, const float* rstd, void* dx,
                                       float* dw, long long rows, int H, long long x_stride, long long g_stride,
                                       long long dx_stride, int zero_centered, int add_to_dx, int accumulate_dw,
                                       cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H <= 0 || (H % 8) != 0 || H > stb::kNoAllocMaxH) {
    fprintf(stderr,
            "stb_rmsnorm_bwd_noalloc: hidden size %d is not supported (needs a multiple of 8, at most %d); "
            "use stb_rmsnorm_bwd with caller-provided scratch for wider rows\n",
            H, stb::kNoAllocMaxH);
    return -kErrBadArgument;
  }
  // The array's name is only a host-side handle: the device address has to be asked for, once per
  // device, with that device current.
  static float* scratch_of_device[stb::kNoAllocMaxDevices] = {nullptr};
  static std::mutex setup_lock;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return -static_cast<int>(e);
  if (dev < 0 || dev >= stb::kNoAllocMaxDevices) return -kErrBadArgument;
  float* scratch;
  {
    std::lock_guard<std::mutex> hold(setup_lock);
    scratch = scratch_of_device[dev];
    if (scratch == nullptr) {
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), stb::g_rmsnorm_bwd_partials);
      if (e != cudaSuccess) {
        fprintf(stderr, "stb_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
        return -static_cast<int>(e);
      }
      scratch_of_device[dev] = scratch;
    }
  }
  const int grid = static_cast<int>(rows < stb::kNoAllocMaxParts ? rows : stb::kNoAllocMaxParts);
  // every CTA overwrites its whole partial row, so nothing in the shared array has to start at zero
  rmsnorm_bwd_kernel<<<grid, kNormThreads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(g),
      rstd, static_cast<__nv_bfloat16*>(dx), scratch, static_cast<int>(rows), H, x_stride, g_stride, dx_stride,
      zero_centered, add_to_dx ? static_cast<const __nv_bfloat16*>(dx) : nullptr, dx_stride);
  if (dw != nullptr)
    rmsnorm_dw_reduce_kernel<<<(H + 31) / 32, 32 * kDwReduceWarps, 0, st>>>(scratch, dw, grid, H, accumulate_dw, H);
  return -static_cast<int>(cudaGetLastError());
}
