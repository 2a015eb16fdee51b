// HBM-bound kernels of the LoRA step: embedding gather, RMSNorm forward/backward, RoPE,
// SwiGLU forward/backward, add/scale/bias, masked cross-entropy, sum of squares, AdamW and
// the fused norm -> clip -> AdamW tail.  All arithmetic is f32; rows are read with 128-bit
// loads when alignment allows and reduced with warp shuffles.
#include <stdlib.h>
#include <algorithm>

#include <atomic>

#include "ft_common.cuh"

namespace {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block; every thread receives the result.  `buf` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* buf) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // buf may still be read from a previous reduction
  if (lane == 0) buf[w] = v;
  __syncthreads();
  float r = (lane < nw) ? buf[lane] : 0.f;
  return warp_sum(r);
}
// Two sums with one pair of barriers.  `buf` holds 64 floats.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* buf) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();
  if (lane == 0) { buf[w] = a; buf[32 + w] = b; }
  __syncthreads();
  a = warp_sum((lane < nw) ? buf[lane] : 0.f);
  b = warp_sum((lane < nw) ? buf[32 + lane] : 0.f);
}
__device__ __forceinline__ float block_max(float v, float* buf) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) buf[w] = v;
  __syncthreads();
  float r = (lane < nw) ? buf[lane] : -INFINITY;
  return warp_max(r);
}

__device__ __forceinline__ bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

// Folds a thread's largest written magnitude into the context's amax slot.  Must be reached
// by every lane of the warp.  Non-negative floats order like their bit patterns.
__device__ __forceinline__ void amax_commit(float m, int* slot) {
  if (!slot) return;
  m = warp_max(m);
  // thousands of warps fold into one word: look first, and leave the atomic to the few that
  // would raise it (a stale read only costs an unnecessary atomic)
  if ((threadIdx.x & 31) == 0 && m > 0.f && __float_as_int(m) > *(volatile int*)slot)
    atomicMax(slot, __float_as_int(m));
}
__device__ __forceinline__ float amax4(float m, float4 v) {
  return fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
}

// ------------------------------------------------------------------------------- embedding
__global__ void k_embedding(const float* __restrict__ table, const uint32_t* __restrict__ ids,
                            float* __restrict__ out, int vocab, int hidden) {
  int t = blockIdx.x;
  uint32_t id = ids[t];
  float* o = out + (size_t)t * hidden;
  if (id >= (uint32_t)vocab) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const float* r = table + (size_t)id * hidden;
  if ((hidden & 3) == 0 && aligned16(r) && aligned16(o)) {
    const float4* r4 = (const float4*)r;
    float4* o4 = (float4*)o;
    for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x) o4[i] = r4[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = r[i];
  }
}

// --------------------------------------------------------------------------------- RMSNorm
__global__ void __launch_bounds__(kRowThreads)
k_rms_norm(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out,
           __half* __restrict__ out16, int n, float eps) {
  __shared__ float red[32];
  const float* xr = x + (size_t)blockIdx.x * n;
  float* o = out ? out + (size_t)blockIdx.x * n : nullptr;
  __half* o16 = out16 ? out16 + (size_t)blockIdx.x * n : nullptr;
  bool vec = (n & 3) == 0 && aligned16(xr) && (!o || aligned16(o)) && aligned16(w) &&
             (!o16 || (((uintptr_t)o16) & 7) == 0);
  float ss = 0.f;
  if (vec) {
    const float4* x4 = (const float4*)xr;
    for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
      float4 v = x4[i];
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
  }
  ss = block_sum(ss, red);
  float inv = 1.0f / sqrtf(ss / (float)n + eps);
  if (vec) {
    const float4* x4 = (const float4*)xr;
    const float4* w4 = (const float4*)w;
    float4* o4 = (float4*)o;
    for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
      float4 v = x4[i], g = w4[i];
      float4 r = make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
      if (o) o4[i] = r;
      if (o16) {
        __half2 a = __floats2half2_rn(r.x, r.y), b = __floats2half2_rn(r.z, r.w);
        ((uint2*)o16)[i] = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
      }
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float r = xr[i] * inv * w[i];
      if (o) o[i] = r;
      if (o16) o16[i] = __float2half_rn(r);
    }
  }
}

// gx = g*w*inv - x*inv^3*sum(g*w*x)/n   (optionally added to what gx holds)
__global__ void __launch_bounds__(kRowThreads)
k_rms_norm_bwd(const float* __restrict__ x, const float* __restrict__ w,
               const float* __restrict__ g, float* __restrict__ gx, float* __restrict__ inv_out,
               int n, float eps, int accumulate, int* amax_slot) {
  float am = 0.f;
  __shared__ float red[32];
  size_t off = (size_t)blockIdx.x * n;
  const float* xr = x + off;
  const float* gr = g + off;
  float* o = gx + off;
  bool vec = (n & 3) == 0 && aligned16(xr) && aligned16(gr) && aligned16(o) && aligned16(w);
  float ss = 0.f, gwx = 0.f;
  if (vec) {
    const float4 *x4 = (const float4*)xr, *g4 = (const float4*)gr, *w4 = (const float4*)w;
    for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
      float4 a = x4[i], b = g4[i], c = w4[i];
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      gwx += b.x * c.x * a.x + b.y * c.y * a.y + b.z * c.z * a.z + b.w * c.w * a.w;
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float a = xr[i];
      ss += a * a;
      gwx += gr[i] * w[i] * a;
    }
  }
  ss = block_sum(ss, red);
  gwx = block_sum(gwx, red);
  float inv = 1.0f / sqrtf(ss / (float)n + eps);
  float coef = gwx * inv * inv * inv / (float)n;
  if (vec) {
    const float4 *x4 = (const float4*)xr, *g4 = (const float4*)gr, *w4 = (const float4*)w;
    float4* o4 = (float4*)o;
    for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
      float4 a = x4[i], b = g4[i], c = w4[i];
      float4 r = make_float4(b.x * c.x * inv - a.x * coef, b.y * c.y * inv - a.y * coef,
                             b.z * c.z * inv - a.z * coef, b.w * c.w * inv - a.w * coef);
      if (accumulate) {
        float4 p = o4[i];
        r.x += p.x; r.y += p.y; r.z += p.z; r.w += p.w;
      }
      o4[i] = r;
      am = amax4(am, r);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float r = gr[i] * w[i] * inv - xr[i] * coef;
      r = accumulate ? o[i] + r : r;
      o[i] = r;
      am = fmaxf(am, fabsf(r));
    }
  }
  amax_commit(am, amax_slot);
  if (inv_out && threadIdx.x == 0) inv_out[blockIdx.x] = inv;
}

// Register-resident forms for rows of up to 256 * 4 * NV elements (16-byte aligned, n % 4 == 0):
// every input element is read from memory exactly once.
template <int NV>
__global__ void __launch_bounds__(kRowThreads)
k_rms_norm_reg(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out,
               __half* __restrict__ out16, int n, float eps) {
  ft_pdl_wait();
  ft_pdl_launch();
  __shared__ float red[32];
  const int n4 = n >> 2;
  const float4* x4 = (const float4*)(x + (size_t)blockIdx.x * n);
  float4 xv[NV];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * kRowThreads;
    xv[k] = i < n4 ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += xv[k].x * xv[k].x + xv[k].y * xv[k].y + xv[k].z * xv[k].z + xv[k].w * xv[k].w;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  const float4* w4 = (const float4*)w;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * kRowThreads;
    if (i >= n4) continue;
    const float4 g = w4[i];
    const float4 r = make_float4(xv[k].x * inv * g.x, xv[k].y * inv * g.y, xv[k].z * inv * g.z,
                                 xv[k].w * inv * g.w);
    if (out) ((float4*)(out + (size_t)blockIdx.x * n))[i] = r;
    if (out16) {
      __half2 a = __floats2half2_rn(r.x, r.y), b = __floats2half2_rn(r.z, r.w);
      ((uint2*)(out16 + (size_t)blockIdx.x * n))[i] = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
    }
  }
}

// The same for two rows per CTA (rows 2b and 2b + 1, one pair of barriers for both): twice the
// bytes in flight per CTA while the sums are reduced.
template <int NV>
__global__ void __launch_bounds__(kRowThreads)
k_rms_norm_reg2(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out,
                __half* __restrict__ out16, int rows, int n, float eps) {
  ft_pdl_wait();
  ft_pdl_launch();
  __shared__ float red[64];
  const int n4 = n >> 2;
  const size_t r0 = (size_t)blockIdx.x * 2;
  const bool two = r0 + 1 < (size_t)rows;
  const float4* xa = (const float4*)(x + r0 * n);
  const float4* xb = (const float4*)(x + (two ? r0 + 1 : r0) * n);
  float4 va[NV], vb[NV];
  float sa = 0.f, sb = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * kRowThreads;
    va[k] = i < n4 ? xa[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    vb[k] = i < n4 ? xb[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    sa += va[k].x * va[k].x + va[k].y * va[k].y + va[k].z * va[k].z + va[k].w * va[k].w;
    sb += vb[k].x * vb[k].x + vb[k].y * vb[k].y + vb[k].z * vb[k].z + vb[k].w * vb[k].w;
  }
  block_sum2(sa, sb, red);
  const float ia = 1.0f / sqrtf(sa / (float)n + eps), ib = 1.0f / sqrtf(sb / (float)n + eps);
  const float4* w4 = (const float4*)w;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * kRowThreads;
    if (i >= n4) continue;
    const float4 g = w4[i];
    const float4 ra = make_float4(va[k].x * ia * g.x, va[k].y * ia * g.y, va[k].z * ia * g.z, va[k].w * ia * g.w);
    const float4 rb = make_float4(vb[k].x * ib * g.x, vb[k].y * ib * g.y, vb[k].z * ib * g.z, vb[k].w * ib * g.w);
    if (out) {
      ((float4*)(out + r0 * n))[i] = ra;
      if (two) ((float4*)(out + (r0 + 1) * n))[i] = rb;
    }
    if (out16) {
      __half2 a = __floats2half2_rn(ra.x, ra.y), b = __floats2half2_rn(ra.z, ra.w);
      ((uint2*)(out16 + r0 * n))[i] = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
      if (two) {
        a = __floats2half2_rn(rb.x, rb.y); b = __floats2half2_rn(rb.z, rb.w);
        ((uint2*)(out16 + (r0 + 1) * n))[i] = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
      }
    }
  }
}

template <int NV>
__global__ void __launch_bounds__(kRowThreads)
k_rms_norm_bwd_reg(const float* __restrict__ x, const float* __restrict__ w,
                   const float* __restrict__ g, float* __restrict__ gx, int n, float eps,
                   int accumulate, int* amax_slot, __half* __restrict__ gx16 = nullptr,
                   const int* __restrict__ carry_amax = nullptr, int carry_exp = 0,
                   float* __restrict__ carry_scales = nullptr) {
  ft_pdl_wait();
  ft_pdl_launch();
  __shared__ float red[64];
  const int n4 = n >> 2;
  const size_t off = (size_t)blockIdx.x * n;
  // gx16 = f16(S gx) with S carried from the amax of the previous version of this gradient
  float s16 = 1.0f;
  if (gx16) {
    s16 = ft_scale_from_amax_bits(*carry_amax, carry_exp);
    if (blockIdx.x == 0 && threadIdx.x == 0) ft_publish_scales(carry_scales, s16);
  }
  const float4 *x4 = (const float4*)(x + off), *g4 = (const float4*)(g + off), *w4 = (const float4*)w;
  float4* o4 = (float4*)(gx + off);
  float4 xv[NV], gv[NV], pv[NV];   // gv holds g * w, pv what the result is added to
  float ss = 0.f, gwx = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * kRowThreads;
    if (i < n4) {
      xv[k] = x4[i];
      const float4 b = g4[i], c = w4[i];
      gv[k] = make_float4(b.x * c.x, b.y * c.y, b.z * c.z, b.w * c.w);
      // in flight during the reductions instead of after them
      pv[k] = accumulate ? o4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      xv[k] = gv[k] = pv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    ss += xv[k].x * xv[k].x + xv[k].y * xv[k].y + xv[k].z * xv[k].z + xv[k].w * xv[k].w;
    gwx += gv[k].x * xv[k].x + gv[k].y * xv[k].y + gv[k].z * xv[k].z + gv[k].w * xv[k].w;
  }
  block_sum2(ss, gwx, red);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  const float coef = gwx * inv * inv * inv / (float)n;
  float am = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * kRowThreads;
    if (i >= n4) continue;
    float4 r = make_float4(gv[k].x * inv - xv[k].x * coef, gv[k].y * inv - xv[k].y * coef,
                           gv[k].z * inv - xv[k].z * coef, gv[k].w * inv - xv[k].w * coef);
    r.x += pv[k].x; r.y += pv[k].y; r.z += pv[k].z; r.w += pv[k].w;
    o4[i] = r;
    if (gx16) {
      __half2 a = __floats2half2_rn(r.x * s16, r.y * s16), b = __floats2half2_rn(r.z * s16, r.w * s16);
      ((uint2*)(gx16 + off))[i] = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
    }
    am = amax4(am, r);
  }
  amax_commit(am, amax_slot);
}

// Two rows per CTA for the frozen-norm backward (gx accumulated, f16 copy optional): rows 2b and
// 2b + 1 share one pair of barriers for their four sums.
template <int NV>
__global__ void __launch_bounds__(kRowThreads)
k_rms_norm_bwd_reg2(const float* __restrict__ x, const float* __restrict__ w,
                    const float* __restrict__ g, float* __restrict__ gx, int rows, int n, float eps,
                    int* amax_slot, __half* __restrict__ gx16, const int* __restrict__ carry_amax,
                    int carry_exp, float* __restrict__ carry_scales) {
  ft_pdl_wait();
  ft_pdl_launch();
  __shared__ float red[128];
  const int n4 = n >> 2;
  float s16 = 1.0f;
  if (gx16) {
    s16 = ft_scale_from_amax_bits(*carry_amax, carry_exp);
    if (blockIdx.x == 0 && threadIdx.x == 0) ft_publish_scales(carry_scales, s16);
  }
  const float4* w4 = (const float4*)w;
  float am = 0.f;
  const size_t r0 = (size_t)blockIdx.x * 2;
  const int nr = r0 + 1 < (size_t)rows ? 2 : 1;
  float4 xv[2][NV], gv[2][NV], pv[2][NV];
  float ss[2] = {0.f, 0.f}, gwx[2] = {0.f, 0.f};
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const size_t off = (r0 + (r < nr ? r : 0)) * n;
    const float4 *x4 = (const float4*)(x + off), *g4 = (const float4*)(g + off);
    const float4* o4 = (const float4*)(gx + off);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * kRowThreads;
      if (i < n4) {
        xv[r][k] = x4[i];
        const float4 b = g4[i], c = w4[i];
        gv[r][k] = make_float4(b.x * c.x, b.y * c.y, b.z * c.z, b.w * c.w);
        pv[r][k] = o4[i];
      } else {
        xv[r][k] = gv[r][k] = pv[r][k] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      ss[r] += xv[r][k].x * xv[r][k].x + xv[r][k].y * xv[r][k].y + xv[r][k].z * xv[r][k].z + xv[r][k].w * xv[r][k].w;
      gwx[r] += gv[r][k].x * xv[r][k].x + gv[r][k].y * xv[r][k].y + gv[r][k].z * xv[r][k].z + gv[r][k].w * xv[r][k].w;
    }
  }
  {
    // four sums, one pair of barriers
    const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
#pragma unroll
    for (int r = 0; r < 2; ++r) { ss[r] = warp_sum(ss[r]); gwx[r] = warp_sum(gwx[r]); }
    __syncthreads();
    if (lane == 0) { red[wp] = ss[0]; red[32 + wp] = gwx[0]; red[64 + wp] = ss[1]; red[96 + wp] = gwx[1]; }
    __syncthreads();
    const int nw = kRowThreads >> 5;
    ss[0] = warp_sum(lane < nw ? red[lane] : 0.f);
    gwx[0] = warp_sum(lane < nw ? red[32 + lane] : 0.f);
    ss[1] = warp_sum(lane < nw ? red[64 + lane] : 0.f);
    gwx[1] = warp_sum(lane < nw ? red[96 + lane] : 0.f);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (r >= nr) break;
    const size_t off = (r0 + r) * n;
    float4* o4 = (float4*)(gx + off);
    const float inv = 1.0f / sqrtf(ss[r] / (float)n + eps);
    const float coef = gwx[r] * inv * inv * inv / (float)n;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * kRowThreads;
      if (i >= n4) continue;
      float4 v = make_float4(gv[r][k].x * inv - xv[r][k].x * coef, gv[r][k].y * inv - xv[r][k].y * coef,
                             gv[r][k].z * inv - xv[r][k].z * coef, gv[r][k].w * inv - xv[r][k].w * coef);
      v.x += pv[r][k].x; v.y += pv[r][k].y; v.z += pv[r][k].z; v.w += pv[r][k].w;
      o4[i] = v;
      if (gx16) {
        __half2 a = __floats2half2_rn(v.x * s16, v.y * s16), b = __floats2half2_rn(v.z * s16, v.w * s16);
        ((uint2*)(gx16 + off))[i] = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
      }
      am = amax4(am, v);
    }
  }
  amax_commit(am, amax_slot);
}

// Warp-per-row forms for rows of up to 32 * 4 * NV elements (16-byte aligned, n % 4 == 0), eight
// rows per CTA: no block-wide barrier, so the eight warps of a CTA have their loads in flight
// independently.  Serves the forward norm of the narrow models (hidden 576, 896, 960): 4.6
// against 6.5 ms per step on the 360M workload.  (The backward norm in the same form, three
// register-resident rows per lane, was slower than the two-pass kernel and is not kept; so was
// this forward form at 2048 elements per row against one CTA per row, 11.2 against 10.0 ms.)
constexpr int kWarpRows = 8;
template <int NV>
__global__ void __launch_bounds__(kWarpRows * 32)
k_rms_norm_warp(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out,
                __half* __restrict__ out16, int rows, int n, float eps) {
  ft_pdl_wait();
  ft_pdl_launch();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpRows + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int n4 = n >> 2;
  const float4* x4 = (const float4*)(x + (size_t)row * n);
  float4 xv[NV];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = lane + k * 32;
    xv[k] = i < n4 ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += xv[k].x * xv[k].x + xv[k].y * xv[k].y + xv[k].z * xv[k].z + xv[k].w * xv[k].w;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  const float4* w4 = (const float4*)w;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = lane + k * 32;
    if (i >= n4) continue;
    const float4 g = w4[i];
    const float4 r = make_float4(xv[k].x * inv * g.x, xv[k].y * inv * g.y, xv[k].z * inv * g.z,
                                 xv[k].w * inv * g.w);
    if (out) ((float4*)(out + (size_t)row * n))[i] = r;
    if (out16) {
      __half2 a = __floats2half2_rn(r.x, r.y), b = __floats2half2_rn(r.z, r.w);
      ((uint2*)(out16 + (size_t)row * n))[i] = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
    }
  }
}

// partial[c, i] = sum over the rows of chunk c of g*x*inv ; one thread per feature
__global__ void k_rms_gw_partial(const float* __restrict__ x, const float* __restrict__ g,
                                 const float* __restrict__ inv, float* __restrict__ partial,
                                 int rows, int n, int rows_per_chunk) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int r0 = blockIdx.y * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
  float acc = 0.f;
  for (int r = r0; r < r1; ++r) acc += g[(size_t)r * n + i] * x[(size_t)r * n + i] * inv[r];
  partial[(size_t)blockIdx.y * n + i] = acc;
}
__global__ void k_rms_gw_final(const float* __restrict__ partial, float* __restrict__ gw, int n,
                               int chunks) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0.f;
  for (int c = 0; c < chunks; ++c) acc += partial[(size_t)c * n + i];
  gw[i] = acc;
}

// ------------------------------------------------------------------------------------ RoPE
// One thread per (token, head, pair).  angle = +-f32(position) * powf(theta, -2i/d).
__global__ void k_rope(float* __restrict__ x, long long ld, long long pairs, int heads,
                       int head_dim, int seq_len, int pos0, float theta, int inverse) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= pairs) return;
  int half = head_dim >> 1;
  int i = (int)(idx % half);
  long long th = idx / half;
  int h = (int)(th % heads);
  long long t = th / heads;
  float pos = (float)(pos0 + (int)(t % seq_len));
  float freq = powf(theta, -2.0f * (float)i / (float)head_dim);
  float angle = (inverse ? -1.0f : 1.0f) * pos * freq;
  float s, c;
  sincosf(angle, &s, &c);
  float* p = x + t * ld + (long long)h * head_dim + i;
  float v1 = p[0], v2 = p[half];
  p[0] = v1 * c - v2 * s;
  p[half] = v1 * s + v2 * c;
}

// {cos, sin} of f32(position) * powf(theta, -2i/d): the angle recipe of k_rope, evaluated once
__global__ void k_rope_table(float2* __restrict__ table, int seq_len, int half, int head_dim,
                             float theta) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= seq_len * half) return;
  int pos = idx / half, i = idx % half;
  float freq = powf(theta, -2.0f * (float)i / (float)head_dim);
  float s, c;
  sincosf((float)pos * freq, &s, &c);
  table[idx] = make_float2(c, s);
  // second copy, transposed ([i][pos]): threads that own consecutive rows (positions) of a tile
  // read consecutive addresses
  table[(size_t)seq_len * half + (size_t)i * seq_len + pos] = make_float2(c, s);
}

// sigmoid with the fast exponential and reciprocal (about 2 ulp): the results are rounded to
// f16, whose half ulp is 2^-12
__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// One thread per 8 elements of a q|k|v row with head_dim 64: in the q and k parts the thread
// owns pairs (i..i+3, i+32..i+35) of one head, in the v part 8 consecutive values.
// out = f16(scale * rotate(+-angle)(x)).
__global__ void k_rope_to_f16(const float* __restrict__ src, __half* __restrict__ dst, long long ld,
                              long long tokens, int nq, int nkv, int seq_len,
                              const float2* __restrict__ table, int inverse,
                              const float* __restrict__ scales) {
  ft_pdl_wait();
  ft_pdl_launch();
  const float S = scales ? scales[0] : 1.0f;
  const int per_tok = (nq + 2 * nkv) / 8;
  const long long total = tokens * per_tok;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long st = (long long)gridDim.x * blockDim.x;
  // token, unit within the token and position in the sequence advance without dividing in the loop
  RowWalk w((size_t)idx, (size_t)st, (size_t)per_tok);
  int pos = (int)(w.r % seq_len);
  const int st_pos = w.st_r % seq_len;
  for (; idx < total; idx += st) {
    const long long t = w.r;
    const int u = w.c;
    const int pos_now = pos;
    {
      const long long r_before = w.r;
      w.next();
      pos += st_pos + (int)(w.r - r_before - w.st_r);
      if (pos >= seq_len) pos -= seq_len;
    }
    const float* row = src + t * ld;
    __half* orow = dst + t * ld;
    const int rot_units = (nq + nkv) / 8;
    if (u < rot_units) {
      const int head = u >> 3, i = (u & 7) * 4;      // 8 threads per 64-wide head
      const int c0 = head * 64 + i;
      const float4 lo = *(const float4*)(row + c0), hi = *(const float4*)(row + c0 + 32);
      const float2* tb = table + (size_t)pos_now * 32 + i;
      const float a[4] = {lo.x, lo.y, lo.z, lo.w}, b[4] = {hi.x, hi.y, hi.z, hi.w};
      float o1[4], o2[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 cs = tb[k];
        const float sn = inverse ? -cs.y : cs.y;
        o1[k] = (a[k] * cs.x - b[k] * sn) * S;
        o2[k] = (a[k] * sn + b[k] * cs.x) * S;
      }
      __half2 p0 = __floats2half2_rn(o1[0], o1[1]), p1 = __floats2half2_rn(o1[2], o1[3]);
      __half2 q0 = __floats2half2_rn(o2[0], o2[1]), q1 = __floats2half2_rn(o2[2], o2[3]);
      *(uint2*)(orow + c0) = make_uint2(*(uint32_t*)&p0, *(uint32_t*)&p1);
      *(uint2*)(orow + c0 + 32) = make_uint2(*(uint32_t*)&q0, *(uint32_t*)&q1);
    } else {
      const int c0 = (nq + nkv) + (u - rot_units) * 8;
      const float4 x = *(const float4*)(row + c0), y = *(const float4*)(row + c0 + 4);
      __half2 h0 = __floats2half2_rn(x.x * S, x.y * S), h1 = __floats2half2_rn(x.z * S, x.w * S);
      __half2 h2 = __floats2half2_rn(y.x * S, y.y * S), h3 = __floats2half2_rn(y.z * S, y.w * S);
      *(uint4*)(orow + c0) = make_uint4(*(uint32_t*)&h0, *(uint32_t*)&h1, *(uint32_t*)&h2, *(uint32_t*)&h3);
    }
  }
}

// ------------------------------------------------------------------------- add/scale/bias
__global__ void k_add(const float* __restrict__ a, const float* __restrict__ b,
                      float* __restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += st) out[i] = a[i] + b[i];
}
__global__ void k_add4(const float4* __restrict__ a, const float4* __restrict__ b,
                       float4* __restrict__ out, size_t n4) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  for (; i < n4; i += st) {
    float4 u = a[i], v = b[i];
    out[i] = make_float4(u.x + v.x, u.y + v.y, u.z + v.z, u.w + v.w);
  }
}
__global__ void k_scale(float* __restrict__ x, size_t n, float s) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += st) x[i] *= s;
}
__global__ void k_add_bias(float* __restrict__ y, long long ld, const float* __restrict__ bias,
                           int rows, int n) {
  size_t total = (size_t)rows * n;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += st) {
    size_t r = i / n, c = i % n;
    y[r * ld + c] += bias[c];
  }
}

// ---------------------------------------------------------------------------------- SwiGLU
__global__ void k_silu_gate(const float* __restrict__ a, long long lda,
                            const float* __restrict__ b, long long ldb, float* __restrict__ out,
                            long long ldo, int rows, int n) {
  size_t total = (size_t)rows * n;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += st) {
    size_t r = i / n, c = i % n;
    float x = a[r * lda + c];
    float s = 1.0f / (1.0f + expf(-x));
    out[r * ldo + c] = x * s * b[r * ldb + c];
  }
}
// SwiGLU forward from f16 gate | up rows (the projection wrote them as f16) to the f16 operand
// of the down projection: 8 columns per thread.  With in_amax the largest |gate| or |up| seen is
// folded into that slot: the backward pass bounds its output with it.
// (il: gate and up interleaved in runs of 32 columns, b = a + 32: feature c sits at
// (c / 32) * 64 + c % 32 of either)
__device__ __forceinline__ size_t il_feature(size_t c, int il) {
  return il ? ((c >> 5) << 6) + (c & 31) : c;
}
__global__ void k_silu_gate16h(const __half* __restrict__ a, const __half* __restrict__ b,
                               long long ldab, __half* __restrict__ out, long long ldo, int rows,
                               int n, int* in_amax, int il) {
  ft_pdl_wait();
  ft_pdl_launch();
  const size_t per_row = (size_t)n / 8, total = (size_t)rows * per_row;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t st = (size_t)gridDim.x * blockDim.x;
  RowWalk w(i, st, per_row);
  __half2 am2 = __float2half2_rn(0.f);
  for (; i < total; i += st, w.next()) {
    const size_t c = (size_t)w.c * 8, ci = il_feature(c, il);
    const uint4 xa = *(const uint4*)(a + w.r * ldab + ci), ya = *(const uint4*)(b + w.r * ldab + ci);
    const __half2* xh = (const __half2*)&xa;
    const __half2* yh = (const __half2*)&ya;
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = __half22float2(xh[k]), y = __half22float2(yh[k]);
      const float v0 = x.x * fast_sigmoid(x.x) * y.x, v1 = x.y * fast_sigmoid(x.y) * y.y;
      __half2 h = __floats2half2_rn(v0, v1);
      o[k] = *(uint32_t*)&h;
      am2 = __hmax2(am2, __hmax2(__habs2(xh[k]), __habs2(yh[k])));
    }
    *(uint4*)(out + w.r * ldo + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  const float2 amf = __half22float2(am2);
  amax_commit(fmaxf(amf.x, amf.y), in_amax);
}

// SwiGLU backward from f16 gate | up rows straight to f16 tensor-core operands: out[r, c] =
// S d(gate), out[r, n + c] = S d(up).  No pass over the result is needed to choose S: with
// |silu(x)| <= |x| and |silu'(x)| < 1.1, every result is at most 1.1 * max|g| * max(|gate|, |up|),
// both factors left behind by the kernels that produced those tensors; S is the power of two
// that brings this bound under 2^13.  One thread publishes {S, 1/S, 2^-11/S}.
__global__ void k_silu_gate_bwd16h(const __half* __restrict__ a, const __half* __restrict__ b,
                                   long long ldab, const float* __restrict__ g, long long ldg,
                                   __half* __restrict__ out, long long ldo, int rows, int n,
                                   const int* __restrict__ g_amax, const int* __restrict__ in_amax,
                                   float* __restrict__ scales_out, int il) {
  ft_pdl_wait();
  ft_pdl_launch();
  float S = 1.0f;
  {
    float bound = 1.1f * __int_as_float(*g_amax) * __int_as_float(*in_amax);
    if (bound > 0.f && isfinite(bound)) {
      int e;
      frexpf(bound, &e);
      S = ldexpf(1.0f, 13 - e);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      scales_out[0] = S;
      scales_out[1] = 1.0f / S;
      scales_out[2] = ldexpf(1.0f / S, -11);
    }
  }
  const size_t per_row = (size_t)n / 8, total = (size_t)rows * per_row;
  const size_t up_off = il ? 32 : (size_t)n;   // d(up) relative to d(gate) in an output row
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t st = (size_t)gridDim.x * blockDim.x;
  RowWalk w(i, st, per_row);
  for (; i < total; i += st, w.next()) {
    const long long r = w.r;
    const size_t c = (size_t)w.c * 8, ci = il_feature(c, il);
    const uint4 xa = *(const uint4*)(a + r * ldab + ci), ya = *(const uint4*)(b + r * ldab + ci);
    const float4 g0 = *(const float4*)(g + r * ldg + c), g1 = *(const float4*)(g + r * ldg + c + 4);
    const __half2* xh = (const __half2*)&xa;
    const __half2* yh = (const __half2*)&ya;
    const float gs[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    uint32_t oa[4], ob[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = __half22float2(xh[k]), y = __half22float2(yh[k]);
      const float xs[2] = {x.x, x.y}, ys[2] = {y.x, y.y};
      float va[2], vb[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float s = fast_sigmoid(xs[e]);
        const float gk = gs[2 * k + e] * S;
        vb[e] = gk * (xs[e] * s);
        va[e] = gk * ys[e] * (s * (1.0f + xs[e] * (1.0f - s)));
      }
      __half2 ha = __floats2half2_rn(va[0], va[1]), hb = __floats2half2_rn(vb[0], vb[1]);
      oa[k] = *(uint32_t*)&ha;
      ob[k] = *(uint32_t*)&hb;
    }
    *(uint4*)(out + r * ldo + ci) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
    *(uint4*)(out + r * ldo + up_off + ci) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
  }
}

// The same with the upstream gradient as f16 rows g16 = f16(Sg g) (the down projection's input
// gradient written with a carried scale): g_scales = {Sg, 1/Sg, ..}, g_amax the largest |g|.
__global__ void k_silu_gate_bwd16hh(const __half* __restrict__ a, const __half* __restrict__ b,
                                    long long ldab, const __half* __restrict__ g16, long long ldg,
                                    const float* __restrict__ g_scales,
                                    __half* __restrict__ out, long long ldo, int rows, int n,
                                    const int* __restrict__ g_amax, const int* __restrict__ in_amax,
                                    float* __restrict__ scales_out, int il) {
  ft_pdl_wait();
  ft_pdl_launch();
  float S = 1.0f;
  {
    float bound = 1.1f * __int_as_float(*g_amax) * __int_as_float(*in_amax);
    if (bound > 0.f && isfinite(bound)) {
      int e;
      frexpf(bound, &e);
      S = ldexpf(1.0f, 13 - e);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) ft_publish_scales(scales_out, S);
  }
  const float SG = S * g_scales[1];   // powers of two: exact
  const size_t up_off = il ? 32 : (size_t)n;
  const size_t per_row = (size_t)n / 8, total = (size_t)rows * per_row;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t st = (size_t)gridDim.x * blockDim.x;
  RowWalk w(i, st, per_row);
  for (; i < total; i += st, w.next()) {
    const long long r = w.r;
    const size_t c = (size_t)w.c * 8, ci = il_feature(c, il);
    const uint4 xa = *(const uint4*)(a + r * ldab + ci), ya = *(const uint4*)(b + r * ldab + ci);
    const uint4 ga = *(const uint4*)(g16 + r * ldg + c);
    const __half2* xh = (const __half2*)&xa;
    const __half2* yh = (const __half2*)&ya;
    const __half2* gh = (const __half2*)&ga;
    uint32_t oa[4], ob[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = __half22float2(xh[k]), y = __half22float2(yh[k]), gg = __half22float2(gh[k]);
      const float xs[2] = {x.x, x.y}, ys[2] = {y.x, y.y}, gs[2] = {gg.x, gg.y};
      float va[2], vb[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float s = fast_sigmoid(xs[e]);
        const float gk = gs[e] * SG;
        vb[e] = gk * (xs[e] * s);
        va[e] = gk * ys[e] * (s * (1.0f + xs[e] * (1.0f - s)));
      }
      __half2 ha = __floats2half2_rn(va[0], va[1]), hb = __floats2half2_rn(vb[0], vb[1]);
      oa[k] = *(uint32_t*)&ha;
      ob[k] = *(uint32_t*)&hb;
    }
    *(uint4*)(out + r * ldo + ci) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
    *(uint4*)(out + r * ldo + up_off + ci) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
  }
}

__global__ void k_silu_gate_bwd(const float* __restrict__ a, long long lda,
                                const float* __restrict__ b, long long ldb,
                                const float* __restrict__ g, long long ldg,
                                float* __restrict__ ga, long long ldga, float* __restrict__ gb,
                                long long ldgb, int rows, int n, int* amax_slot) {
  size_t total = (size_t)rows * n;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  float am = 0.f;
  for (; i < total; i += st) {
    size_t r = i / n, c = i % n;
    float x = a[r * lda + c], y = b[r * ldb + c], go = g[r * ldg + c];
    float s = 1.0f / (1.0f + expf(-x));
    float vb = go * (x * s), va = go * y * (s * (1.0f + x * (1.0f - s)));
    gb[r * ldgb + c] = vb;
    ga[r * ldga + c] = va;
    am = fmaxf(am, fmaxf(fabsf(va), fabsf(vb)));
  }
  amax_commit(am, amax_slot);
}

// the same with 4 columns per thread (width and pitches multiples of 4, 16-byte aligned)
__global__ void k_silu_gate_bwd4(const float* __restrict__ a, long long lda,
                                 const float* __restrict__ b, long long ldb,
                                 const float* __restrict__ g, long long ldg,
                                 float* __restrict__ ga, long long ldga, float* __restrict__ gb,
                                 long long ldgb, int rows, int n, int* amax_slot) {
  size_t per_row = (size_t)n / 4, total = (size_t)rows * per_row;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  float am = 0.f;
  for (; i < total; i += st) {
    size_t r = i / per_row, c = (i % per_row) * 4;
    float4 x = *(const float4*)(a + r * lda + c), y = *(const float4*)(b + r * ldb + c);
    float4 go = *(const float4*)(g + r * ldg + c);
    float xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w}, gs[4] = {go.x, go.y, go.z, go.w};
    float va[4], vb[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float s = 1.0f / (1.0f + expf(-xs[k]));
      vb[k] = gs[k] * (xs[k] * s);
      va[k] = gs[k] * ys[k] * (s * (1.0f + xs[k] * (1.0f - s)));
      am = fmaxf(am, fmaxf(fabsf(va[k]), fabsf(vb[k])));
    }
    *(float4*)(ga + r * ldga + c) = make_float4(va[0], va[1], va[2], va[3]);
    *(float4*)(gb + r * ldgb + c) = make_float4(vb[0], vb[1], vb[2], vb[3]);
  }
  amax_commit(am, amax_slot);
}

// ------------------------------------------------------------------- masked cross-entropy
// One block per row.  Pass 1 keeps a running (max, sum) per thread; pass 2 writes the
// gradient.  grad_scale folds the upstream gradient of the loss into the same pass.
// Long rows get 1024 threads: two such blocks per SM keep about 300 rows in flight, which for
// a 49152-entry vocabulary (192 KiB a row) is 58 MB, so the second pass finds its row in L2.
constexpr int kCeThreads = 1024;
__global__ void __launch_bounds__(kCeThreads)
k_masked_ce(const float* logits, const uint32_t* __restrict__ targets,
            const float* __restrict__ weights, float* grad, float* __restrict__ row_loss,
            int vocab, float grad_scale, int* amax_slot, __half* __restrict__ g16 = nullptr,
            long long ld16 = 0, const float* __restrict__ scales16 = nullptr) {
  // `grad` may alias `logits` (in-place use by the fused step): every element is read for
  // the last time by the thread that then overwrites it, after both reductions are done.
  __shared__ float red[32];
  int row = blockIdx.x;
  const float* z = logits + (size_t)row * vocab;
  float* gz = grad ? grad + (size_t)row * vocab : nullptr;
  uint32_t tgt = targets[row];
  bool vec = (vocab & 3) == 0 && aligned16(z) && (!gz || aligned16(gz));
  // optional f16 copy of the gradient, times the power of two scales16[0] (vocab % 4 == 0)
  __half* hz = g16 ? g16 + (size_t)row * ld16 : nullptr;
  const float S16 = hz ? scales16[0] : 1.0f;
  if (tgt == FT_MASKED_CE_SKIP) {
    if (hz)
      for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) ((uint2*)hz)[i] = make_uint2(0u, 0u);
    if (gz) {
      if (vec) {
        float4* g4 = (float4*)gz;
        for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x)
          g4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) gz[i] = 0.f;
      }
    }
    if (threadIdx.x == 0) row_loss[row] = 0.f;
    return;
  }
  // read before the gradient pass: in in-place use that pass overwrites the logits
  const float z_target = (threadIdx.x == 0 && tgt < (uint32_t)vocab) ? z[tgt] : 0.f;
  float m = -3.4e38f, se = 0.f;
  if (vec) {
    // one pass: every thread keeps a running maximum and the sum of exponentials against it
    const float4* z4 = (const float4*)z;
    for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) {
      float4 v = z4[i];
      const float m_new = fmaxf(m, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
      se = se * expf(m - m_new) + (expf(v.x - m_new) + expf(v.y - m_new) + expf(v.z - m_new) + expf(v.w - m_new));
      m = m_new;
    }
    const float m_all = block_max(m, red);
    se = block_sum(se * expf(m - m_all), red);
    m = m_all;
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) m = fmaxf(m, z[i]);
    m = block_max(m, red);
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) se += expf(z[i] - m);
    se = block_sum(se, red);
  }
  float log_z = m + logf(se);
  float inv = weights[row] * grad_scale;
  // |(softmax - onehot) * inv| <= |inv|: a tight bound serves as this row's amax
  if (amax_slot && threadIdx.x == 0 && inv != 0.f) atomicMax(amax_slot, __float_as_int(fabsf(inv)));
  if (hz) {
    const float4* z4 = (const float4*)z;
    const float invs = inv * S16;
    for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) {
      float4 v = z4[i];
      float4 r = make_float4(expf(v.x - log_z) * invs, expf(v.y - log_z) * invs,
                             expf(v.z - log_z) * invs, expf(v.w - log_z) * invs);
      uint32_t base = (uint32_t)i * 4u;
      if (tgt - base < 4u) {
        uint32_t k = tgt - base;
        if (k == 0) r.x -= invs; else if (k == 1) r.y -= invs;
        else if (k == 2) r.z -= invs; else r.w -= invs;
      }
      __half2 h0 = __floats2half2_rn(r.x, r.y), h1 = __floats2half2_rn(r.z, r.w);
      ((uint2*)hz)[i] = make_uint2(*(uint32_t*)&h0, *(uint32_t*)&h1);
    }
  }
  if (gz) {
    if (vec) {
      const float4* z4 = (const float4*)z;
      float4* g4 = (float4*)gz;
      for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) {
        float4 v = z4[i];
        float4 r = make_float4(expf(v.x - log_z) * inv, expf(v.y - log_z) * inv,
                               expf(v.z - log_z) * inv, expf(v.w - log_z) * inv);
        uint32_t base = (uint32_t)i * 4u;
        if (tgt - base < 4u) {
          uint32_t k = tgt - base;
          if (k == 0) r.x -= inv; else if (k == 1) r.y -= inv;
          else if (k == 2) r.z -= inv; else r.w -= inv;
        }
        g4[i] = r;
      }
    } else {
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float gv = expf(z[i] - log_z) * inv;
        if ((uint32_t)i == tgt) gv -= inv;
        gz[i] = gv;
      }
    }
  }
  if (threadIdx.x == 0) row_loss[row] = (tgt < (uint32_t)vocab) ? log_z - z_target : 0.f;
}

// ------------------------------------------------------------------------- optimizer side
// One block per 4096-element chunk; chunk b's f32 sum of squares goes to out[offset + b].
__global__ void __launch_bounds__(kRowThreads)
k_sum_squares(const float* __restrict__ x, size_t n, float* __restrict__ out, size_t offset,
              float pre_scale) {
  __shared__ float red[32];
  size_t start = (size_t)blockIdx.x * FT_SUM_SQUARES_CHUNK;
  size_t end = min(start + (size_t)FT_SUM_SQUARES_CHUNK, n);
  float acc = 0.f;
  for (size_t i = start + threadIdx.x; i < end; i += blockDim.x) {
    float v = x[i] * pre_scale;
    acc += v * v;
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) out[offset + blockIdx.x] = acc;
}

__device__ __forceinline__ void adamw_one(float& w, float g, float& m, float& v, float lr,
                                          float b1, float b2, float eps, float wd, float c1,
                                          float c2) {
  m = m * b1 + (1.0f - b1) * g;
  v = v * b2 + (1.0f - b2) * g * g;
  float m_hat = m / c1, v_hat = v / c2;
  w = w - lr * (m_hat / (sqrtf(v_hat) + eps) + wd * w);
}

__global__ void k_adamw(float* __restrict__ w, const float* __restrict__ g,
                        float* __restrict__ m, float* __restrict__ v, size_t n, FtAdamParams p) {
  float c1 = 1.0f - powf(p.beta1, p.t), c2 = 1.0f - powf(p.beta2, p.t);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += st) {
    float wi = w[i], mi = m[i], vi = v[i];
    adamw_one(wi, g[i], mi, vi, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, c1, c2);
    w[i] = wi; m[i] = mi; v[i] = vi;
  }
}

// norm_out[0] = norm, [1] = 1 if the step is applied, [2] = factor to apply to the raw
// gradient (grad_scale, times the clip factor when clipping).  Chunk sums are added in
// f64 like the reference's host loop, but not in index order: each thread sums a fixed strided
// subset and a fixed shared-memory tree joins them, so the result is identical from run to run
// and can differ from a sequential f64 sum in its last bit.
__global__ void k_norm_finalize(const float* __restrict__ partials, size_t chunks,
                                float grad_scale, float max_norm, float* __restrict__ norm_out) {
  __shared__ double sred[kRowThreads];
  // fixed assignment of chunks to threads and a fixed tree => run-to-run identical
  double acc = 0.0;
  for (size_t i = threadIdx.x; i < chunks; i += blockDim.x) acc += (double)partials[i];
  sred[threadIdx.x] = acc;
  __syncthreads();
  for (int s = blockDim.x / 2; s > 0; s >>= 1) {
    if ((int)threadIdx.x < s) sred[threadIdx.x] += sred[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    float norm = (float)sqrt(sred[0]);
    bool finite = isfinite(norm);
    float factor = grad_scale;
    if (finite && max_norm > 0.f && norm > max_norm) factor *= max_norm / (norm + 1e-6f);
    norm_out[0] = norm;
    norm_out[1] = finite ? 1.f : 0.f;
    norm_out[2] = factor;
  }
}

__global__ void k_adamw_scaled(float* __restrict__ w, const float* __restrict__ g,
                               float* __restrict__ m, float* __restrict__ v, size_t n,
                               FtAdamParams p, const float* __restrict__ norm_out) {
  if (norm_out[1] == 0.f) return;  // non-finite norm: the step is skipped
  float factor = norm_out[2];
  float c1 = 1.0f - powf(p.beta1, p.t), c2 = 1.0f - powf(p.beta2, p.t);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += st) {
    float wi = w[i], mi = m[i], vi = v[i];
    adamw_one(wi, g[i] * factor, mi, vi, p.lr, p.beta1, p.beta2, p.eps, p.weight_decay, c1, c2);
    w[i] = wi; m[i] = mi; v[i] = vi;
  }
}

inline int ew_grid(FtContext* ctx, size_t n, int block = 256, int per_thread = 4) {
  size_t want = (n + (size_t)block * per_thread - 1) / ((size_t)block * per_thread);
  size_t cap = (size_t)ctx->sm_count * 16;
  return (int)std::max<size_t>(1, std::min(want, cap));
}

}  // namespace

// ------------------------------------------------------------------------------- launchers
int ft_k_embedding(FtContext* ctx, const float* table, const uint32_t* ids, float* out,
                   int tokens, int vocab, int hidden) {
  int block = hidden >= 1024 ? 256 : 128;
  FT_LAUNCH(ctx, k_embedding, tokens, block, 0, table, ids, out, vocab, hidden);
  return FT_OK;
}

int ft_k_rms_norm(FtContext* ctx, const float* x, const float* w, float* out, int rows, int n,
                  float eps) {
  int block = n >= 1024 ? kRowThreads : (n >= 256 ? 128 : 32);
  FT_LAUNCH(ctx, k_rms_norm, rows, block, 0, x, w, out, (__half*)nullptr, n, eps);
  return FT_OK;
}

int ft_k_rms_norm16(FtContext* ctx, const float* x, const float* w, float* out, __half* out16,
                    int rows, int n, float eps) {
  const bool al = (n % 4) == 0 && ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)out)) & 15) == 0 &&
                  (((uintptr_t)out16) & 7) == 0;
  if (al && n >= 1024 && n <= 4096) {
    if (n <= 2048)   // two rows per CTA: 9.5 against 10.3 ms per step of the 1.7B workload
      FT_LAUNCH_PDL(ctx, k_rms_norm_reg2<2>, ft_cdiv(rows, 2), kRowThreads, 0, x, w, out, out16, rows, n, eps);
    else
      FT_LAUNCH_PDL(ctx, k_rms_norm_reg<4>, rows, kRowThreads, 0, x, w, out, out16, n, eps);
    return FT_OK;
  }
  if (al && n >= 128 && n < 1024) {
    const int grid = ft_cdiv(rows, kWarpRows);
    if (n <= 512)
      FT_LAUNCH_PDL(ctx, k_rms_norm_warp<4>, grid, kWarpRows * 32, 0, x, w, out, out16, rows, n, eps);
    else
      FT_LAUNCH_PDL(ctx, k_rms_norm_warp<8>, grid, kWarpRows * 32, 0, x, w, out, out16, rows, n, eps);
    return FT_OK;
  }
  int block = n >= 1024 ? kRowThreads : (n >= 256 ? 128 : 32);
  FT_LAUNCH(ctx, k_rms_norm, rows, block, 0, x, w, out, out16, n, eps);
  return FT_OK;
}

int ft_k_rms_norm_bwd(FtContext* ctx, const float* x, const float* w, const float* g, float* gx,
                      float* gw, int rows, int n, float eps, bool accumulate_gx) {
  float* inv = nullptr;
  float* partial = nullptr;
  int chunks = 0, rows_per_chunk = 0;
  if (gw) {
    chunks = std::max(1, std::min(rows, (ctx->sm_count * 8) / std::max(1, ft_cdiv(n, 128))));
    chunks = std::min(chunks, 1024);
    rows_per_chunk = ft_cdiv(rows, chunks);
    chunks = ft_cdiv(rows, rows_per_chunk);
    void* s = nullptr;
    FT_TRY(ft_scratch(ctx, ft_align_up((size_t)rows * 4, 256) + (size_t)chunks * n * 4, &s));
    inv = (float*)s;
    partial = (float*)((char*)s + ft_align_up((size_t)rows * 4, 256));
  }
  int block = n >= 1024 ? kRowThreads : (n >= 256 ? 128 : 32);
  int* am = ctx->amax_out;
  if (am) ctx->amax_ready = true;
  const bool al = (n % 4) == 0 &&
                  ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)g) | ((uintptr_t)gx)) & 15) == 0;
  if (!gw && al && n >= 1024 && n <= 4096) {
    if (n <= 2048)
      FT_LAUNCH_PDL(ctx, k_rms_norm_bwd_reg<2>, rows, kRowThreads, 0, x, w, g, gx, n, eps,
                accumulate_gx ? 1 : 0, am, (__half*)nullptr, (const int*)nullptr, 0, (float*)nullptr);
    else
      FT_LAUNCH_PDL(ctx, k_rms_norm_bwd_reg<4>, rows, kRowThreads, 0, x, w, g, gx, n, eps,
                accumulate_gx ? 1 : 0, am, (__half*)nullptr, (const int*)nullptr, 0, (float*)nullptr);
    return FT_OK;
  }
  FT_LAUNCH(ctx, k_rms_norm_bwd, rows, block, 0, x, w, g, gx, inv, n, eps, accumulate_gx ? 1 : 0, am);
  if (gw) {
    dim3 grid(ft_cdiv(n, 128), chunks);
    FT_LAUNCH(ctx, k_rms_gw_partial, grid, 128, 0, x, g, inv, partial, rows, n, rows_per_chunk);
    FT_LAUNCH(ctx, k_rms_gw_final, ft_cdiv(n, 128), 128, 0, partial, gw, n, chunks);
  }
  return FT_OK;
}

int ft_k_rms_norm_bwd_carry(FtContext* ctx, const float* x, const float* w, const float* g,
                            float* gx, __half* gx16, int rows, int n, float eps,
                            const FtCarry& carry) {
  const bool al = (n % 4) == 0 && (((uintptr_t)gx16) & 7) == 0 &&
                  ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)g) | ((uintptr_t)gx)) & 15) == 0;
  if (!al || n < 1024 || n > 4096 || !carry.amax_in || !carry.scales) return FT_ERR_UNSUPPORTED;
  if (n <= 2048 && g)   // two rows per CTA: 23.8 against 24.7 ms per step of the 1.7B workload
    FT_LAUNCH_PDL(ctx, k_rms_norm_bwd_reg2<2>, ft_cdiv(rows, 2), kRowThreads, 0, x, w, g, gx, rows, n, eps,
                  carry.amax_out, gx16, carry.amax_in, carry.exp, carry.scales);
  else if (n <= 2048)
    FT_LAUNCH_PDL(ctx, k_rms_norm_bwd_reg<2>, rows, kRowThreads, 0, x, w, g, gx, n, eps, 1,
                  carry.amax_out, gx16, carry.amax_in, carry.exp, carry.scales);
  else
    FT_LAUNCH_PDL(ctx, k_rms_norm_bwd_reg<4>, rows, kRowThreads, 0, x, w, g, gx, n, eps, 1,
                  carry.amax_out, gx16, carry.amax_in, carry.exp, carry.scales);
  return FT_OK;
}

// ---------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate.
//
// Some hosts of this library cannot let a call reach cudaMalloc: a runtime that has handed all
// of its device memory to its own pool, or code running where an allocation would serialise or
// fail (inside a latency-critical loop, under a memory cap set by the embedding program).  The
// regular entry point borrows per-row scratch from the context, which grows it with cudaMalloc
// on demand.  This variant keeps that scratch in a fixed array inside the library image
// instead: 2 MiB that every GPU loading the library holds until the process exits.
// ---------------------------------------------------------------------------------------
constexpr size_t kNoAllocFloats = 512 * 1024;  // 2 MiB
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocFloats];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address:
// the address is asked for once per device (with that device current) and cached.
// (A cached address does not survive cudaDeviceReset: a host that resets a device must not
// call this entry point on it afterwards.)
constexpr int kMaxDevices = FT_MAX_DEVICES;
static std::atomic<float*> g_noalloc_ptr[kMaxDevices];

extern "C" int ft_rms_norm_backward_noalloc(FtContext* ctx, const float* x, const float* w,
                                            const float* g, float* gx, float* gw, int rows,
                                            int size, float eps) {
  FT_REQUIRE(ctx && x && w && g && gx, "ft_rms_norm_backward_noalloc: NULL argument");
  FT_REQUIRE(rows >= 0 && size > 0, "ft_rms_norm_backward_noalloc: bad shape");
  if (!rows) return FT_OK;
  // scratch layout: inv[rows] (256-byte aligned), then partial[chunks][size]
  const size_t inv_floats = ft_align_up((size_t)rows, 64);
  FT_REQUIRE(!gw || inv_floats + (size_t)size <= kNoAllocFloats,
             "ft_rms_norm_backward_noalloc: rows (rounded up to 64) + size = %zu floats exceeds the "
             "fixed scratch of %zu floats; use ft_rms_norm_backward",
             inv_floats + (size_t)size, kNoAllocFloats);
  FT_REQUIRE(ctx->device >= 0 && ctx->device < kMaxDevices,
             "ft_rms_norm_backward_noalloc: device ordinal %d out of range", ctx->device);
  float* scratch = g_noalloc_ptr[ctx->device].load(std::memory_order_acquire);
  if (!scratch) {
    // first call on this device: resolve the symbol with that device current (do this before
    // any stream capture), then give the caller its own current device back
    int prev = -1;
    FT_CUDA(cudaGetDevice(&prev));
    if (prev != ctx->device) FT_CUDA(cudaSetDevice(ctx->device));
    void* p = nullptr;
    cudaError_t se = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (prev != ctx->device) cudaSetDevice(prev);
    if (se != cudaSuccess) return ft_cuda_fail(se, "cudaGetSymbolAddress", __FILE__, __LINE__);
    FT_REQUIRE(p != nullptr, "ft_rms_norm_backward_noalloc: symbol address is NULL");
    scratch = (float*)p;
    g_noalloc_ptr[ctx->device].store(scratch, std::memory_order_release);
  }
  float* inv = nullptr;
  float* partial = nullptr;
  int chunks = 0, rows_per_chunk = 0;
  if (gw) {
    const size_t fit = (kNoAllocFloats - inv_floats) / (size_t)size;
    chunks = std::max(1, std::min(rows, (ctx->sm_count * 8) / std::max(1, ft_cdiv(size, 128))));
    chunks = (int)std::min<size_t>((size_t)std::min(chunks, 1024), fit);
    rows_per_chunk = ft_cdiv(rows, chunks);
    chunks = ft_cdiv(rows, rows_per_chunk);
    inv = scratch;
    partial = scratch + inv_floats;
  }
  // every scratch word that is read is written first by these launches: nothing to clear
  int block = size >= 1024 ? kRowThreads : (size >= 256 ? 128 : 32);
  FT_LAUNCH(ctx, k_rms_norm_bwd, rows, block, 0, x, w, g, gx, inv, size, eps, 0, (int*)nullptr);
  if (gw) {
    dim3 grid(ft_cdiv(size, 128), chunks);
    FT_LAUNCH(ctx, k_rms_gw_partial, grid, 128, 0, x, g, inv, partial, rows, size, rows_per_chunk);
    FT_LAUNCH(ctx, k_rms_gw_final, ft_cdiv(size, 128), 128, 0, partial, gw, size, chunks);
  }
  return FT_OK;
}

int ft_k_rope(FtContext* ctx, float* x, long long ld, int tokens, int heads, int head_dim,
              int seq_len, int pos, float theta, bool inverse) {
  long long pairs = (long long)tokens * heads * (head_dim / 2);
  if (pairs == 0) return FT_OK;
  long long blocks = (pairs + 255) / 256;
  FT_REQUIRE(blocks <= 0x7fffffffLL, "rope: too many elements");
  FT_LAUNCH(ctx, k_rope, (unsigned)blocks, 256, 0, x, ld, pairs, heads, head_dim, seq_len, pos,
            theta, inverse ? 1 : 0);
  return FT_OK;
}

int ft_k_rope_table(FtContext* ctx, float* table, int seq_len, int head_dim, float theta) {
  int half = head_dim / 2, n = seq_len * half;
  FT_LAUNCH(ctx, k_rope_table, ft_cdiv(n, 256), 256, 0, (float2*)table, seq_len, half, head_dim, theta);
  return FT_OK;
}

int ft_k_rope_to_f16(FtContext* ctx, const float* src, __half* dst, long long ld, int tokens,
                     int nq, int nkv, int seq_len, const float* table, bool inverse,
                     const float* scales) {
  FT_REQUIRE((nq % 64) == 0 && (nkv % 64) == 0 && (ld % 8) == 0 && ld >= nq + 2 * nkv &&
                 (((uintptr_t)src) & 15) == 0 && (((uintptr_t)dst) & 15) == 0,
             "rope_to_f16: needs head_dim 64 and 16-byte aligned rows");
  size_t total = (size_t)tokens * ((nq + 2 * nkv) / 8);
  FT_LAUNCH_PDL(ctx, k_rope_to_f16, ew_grid(ctx, total, 256, 2), 256, 0, src, dst, ld, (long long)tokens, nq,
            nkv, seq_len, (const float2*)table, inverse ? 1 : 0, scales);
  return FT_OK;
}

int ft_k_add(FtContext* ctx, const float* a, const float* b, float* out, size_t n) {
  if ((n & 3) == 0 && ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)out)) & 15) == 0) {
    FT_LAUNCH(ctx, k_add4, ew_grid(ctx, n / 4, 256, 2), 256, 0, (const float4*)a,
              (const float4*)b, (float4*)out, n / 4);
  } else {
    FT_LAUNCH(ctx, k_add, ew_grid(ctx, n), 256, 0, a, b, out, n);
  }
  return FT_OK;
}

int ft_k_scale(FtContext* ctx, float* x, size_t n, float s) {
  FT_LAUNCH(ctx, k_scale, ew_grid(ctx, n), 256, 0, x, n, s);
  return FT_OK;
}

int ft_k_add_bias(FtContext* ctx, float* y, long long ld, const float* bias, int rows, int n) {
  FT_LAUNCH(ctx, k_add_bias, ew_grid(ctx, (size_t)rows * n), 256, 0, y, ld, bias, rows, n);
  return FT_OK;
}

int ft_k_silu_gate(FtContext* ctx, const float* a, long long lda, const float* b, long long ldb,
                   float* out, long long ldo, int rows, int n) {
  FT_LAUNCH(ctx, k_silu_gate, ew_grid(ctx, (size_t)rows * n), 256, 0, a, lda, b, ldb, out, ldo,
            rows, n);
  return FT_OK;
}

int ft_k_silu_gate16h(FtContext* ctx, const __half* gu, long long ld, __half* out, long long ldo,
                      int rows, int n, int* in_amax, bool il) {
  FT_REQUIRE(!il || (n % 32) == 0, "silu_gate16h: interleaved rows need a width that is a multiple of 32");
  FT_REQUIRE((n % 8) == 0 && (ld % 8) == 0 && (ldo % 8) == 0 && (((uintptr_t)gu) & 15) == 0 &&
                 (((uintptr_t)out) & 15) == 0,
             "silu_gate16h: width and pitches must be multiples of 8");
  FT_LAUNCH_PDL(ctx, k_silu_gate16h, ew_grid(ctx, (size_t)rows * n / 8, 256, 2), 256, 0, gu,
                gu + (il ? 32 : n), ld, out, ldo, rows, n, in_amax, il ? 1 : 0);
  return FT_OK;
}

// Consumes the armed amax of g (left by the product that wrote it) and in_amax (left by
// ft_k_silu_gate16h); *scales_out points at {S, 1/S, 2^-11/S} on the device.
int ft_k_silu_gate_bwd16h(FtContext* ctx, const __half* gu, long long ld, const float* g,
                          long long ldg, __half* out, long long ldo, int rows, int n,
                          const int* in_amax, const float** scales_out, bool il) {
  FT_REQUIRE(!il || (n % 32) == 0, "silu_gate_bwd16h: interleaved rows need a width that is a multiple of 32");
  FT_REQUIRE((n % 8) == 0 && (ld % 8) == 0 && (ldg % 4) == 0 && (ldo % 8) == 0 &&
                 ((((uintptr_t)gu) | ((uintptr_t)g) | ((uintptr_t)out)) & 15) == 0,
             "silu_gate_bwd16h: width and pitches must be multiples of 8");
  FT_REQUIRE(ctx->amax_ready && ctx->amax_out && in_amax,
             "silu_gate_bwd16h: the upstream gradient's amax must have been armed and produced");
  const int* g_amax = ctx->amax_out;
  ctx->amax_out = nullptr;
  ctx->amax_ready = false;
  FT_LAUNCH_PDL(ctx, k_silu_gate_bwd16h, ew_grid(ctx, (size_t)rows * n / 8, 256, 2), 256, 0, gu,
                gu + (il ? 32 : n), ld, g, ldg, out, ldo, rows, n, g_amax, in_amax,
                ctx->scale_buf + 4, il ? 1 : 0);
  *scales_out = ctx->scale_buf + 4;
  return FT_OK;
}

int ft_k_silu_gate_bwd16hh(FtContext* ctx, const __half* gu, long long ld, const __half* g16,
                           long long ldg, const float* g_scales, const int* g_amax, __half* out,
                           long long ldo, int rows, int n, const int* in_amax,
                           const float** scales_out, bool il) {
  FT_REQUIRE(!il || (n % 32) == 0, "silu_gate_bwd16hh: interleaved rows need a width that is a multiple of 32");
  FT_REQUIRE((n % 8) == 0 && (ld % 8) == 0 && (ldg % 8) == 0 && (ldo % 8) == 0 &&
                 ((((uintptr_t)gu) | ((uintptr_t)g16) | ((uintptr_t)out)) & 15) == 0,
             "silu_gate_bwd16hh: width and pitches must be multiples of 8");
  FT_REQUIRE(g_scales && g_amax && in_amax, "silu_gate_bwd16hh: scales and maxima are required");
  FT_LAUNCH_PDL(ctx, k_silu_gate_bwd16hh, ew_grid(ctx, (size_t)rows * n / 8, 256, 2), 256, 0, gu,
                gu + (il ? 32 : n), ld, g16, ldg, g_scales, out, ldo, rows, n, g_amax, in_amax,
                ctx->scale_buf + 4, il ? 1 : 0);
  *scales_out = ctx->scale_buf + 4;
  return FT_OK;
}

int ft_k_silu_gate_bwd(FtContext* ctx, const float* a, long long lda, const float* b,
                       long long ldb, const float* g, long long ldg, float* ga, long long ldga,
                       float* gb, long long ldgb, int rows, int n) {
  int* am = ctx->amax_out;
  if (am) ctx->amax_ready = true;
  const bool vec = (n % 4) == 0 && ((lda | ldb | ldg | ldga | ldgb) % 4) == 0 &&
                   ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)g) | ((uintptr_t)ga) |
                     ((uintptr_t)gb)) & 15) == 0;
  if (vec)
    FT_LAUNCH(ctx, k_silu_gate_bwd4, ew_grid(ctx, (size_t)rows * n / 4, 256, 2), 256, 0, a, lda, b,
              ldb, g, ldg, ga, ldga, gb, ldgb, rows, n, am);
  else
    FT_LAUNCH(ctx, k_silu_gate_bwd, ew_grid(ctx, (size_t)rows * n), 256, 0, a, lda, b, ldb, g, ldg,
              ga, ldga, gb, ldgb, rows, n, am);
  return FT_OK;
}

int ft_k_masked_ce(FtContext* ctx, const float* logits, const uint32_t* targets,
                   const float* weights, float* grad, float* row_loss, int rows, int vocab,
                   float grad_scale) {
  int* am = ctx->amax_out;
  if (am) ctx->amax_ready = true;
  FT_LAUNCH(ctx, k_masked_ce, rows, vocab >= 16384 ? kCeThreads : kRowThreads, 0, logits, targets, weights, grad, row_loss,
            vocab, grad_scale, am, (__half*)nullptr, 0ll, (const float*)nullptr);
  return FT_OK;
}

// {S, 1/S, 2^-11/S} with S the power of two that brings max_r |weights[r] * grad_scale| - a bound
// on every element of the loss gradient, since |softmax - onehot| <= 1 - into [2^7, 2^8)
__global__ void __launch_bounds__(1024)
k_ce_scale(const float* __restrict__ weights, const uint32_t* __restrict__ targets, int rows,
           float grad_scale, float* __restrict__ scales) {
  ft_pdl_wait();
  __shared__ float red[32];
  float m = 0.f;
  for (int i = threadIdx.x; i < rows; i += blockDim.x)
    if (targets[i] != FT_MASKED_CE_SKIP) m = fmaxf(m, fabsf(weights[i] * grad_scale));
  m = block_max(m, red);
  if (threadIdx.x == 0) {
    float S = 1.0f;
    if (m > 0.f && isfinite(m)) {
      int e;
      frexpf(m, &e);
      S = ldexpf(1.0f, 8 - e);
    }
    scales[0] = S;
    scales[1] = 1.0f / S;
    scales[2] = ldexpf(1.0f / S, -11);
  }
}

// Loss rows and the gradient as scaled f16 operands [rows, ld16] (no f32 gradient is written);
// *scales_out points at {S, 1/S, 2^-11/S} on the device.
int ft_k_masked_ce16(FtContext* ctx, const float* logits, const uint32_t* targets,
                     const float* weights, __half* g16, long long ld16, float* row_loss, int rows,
                     int vocab, float grad_scale, const float** scales_out) {
  FT_REQUIRE((vocab % 4) == 0 && (ld16 % 4) == 0 && ld16 >= vocab && (((uintptr_t)logits) & 15) == 0 &&
                 (((uintptr_t)g16) & 7) == 0,
             "masked_ce16: vocabulary and pitch must be multiples of 4");
  ctx->amax_out = nullptr;
  ctx->amax_ready = false;
  FT_LAUNCH(ctx, k_ce_scale, 1, 1024, 0, weights, targets, rows, grad_scale, ctx->scale_buf + 4);
  FT_LAUNCH(ctx, k_masked_ce, rows, vocab >= 16384 ? kCeThreads : kRowThreads, 0, logits, targets, weights, (float*)nullptr, row_loss,
            vocab, grad_scale, (int*)nullptr, g16, ld16, (const float*)(ctx->scale_buf + 4));
  *scales_out = ctx->scale_buf + 4;
  return FT_OK;
}

int ft_k_sum_squares(FtContext* ctx, const float* x, size_t n, float* out, size_t offset) {
  size_t chunks = (n + FT_SUM_SQUARES_CHUNK - 1) / FT_SUM_SQUARES_CHUNK;
  FT_REQUIRE(chunks <= 0x7fffffffull, "sum_squares: too many elements");
  FT_LAUNCH(ctx, k_sum_squares, (unsigned)chunks, kRowThreads, 0, x, n, out, offset, 1.0f);
  return FT_OK;
}

int ft_k_adamw(FtContext* ctx, float* w, const float* g, float* m, float* v, size_t n,
               const FtAdamParams* p) {
  FT_LAUNCH(ctx, k_adamw, ew_grid(ctx, n), 256, 0, w, g, m, v, n, *p);
  return FT_OK;
}

int ft_k_apply_fused(FtContext* ctx, float* w, float* g, float* m, float* v, size_t n,
                     float grad_scale, float max_norm, const FtAdamParams* p, float* partials,
                     float* norm_out) {
  size_t chunks = (n + FT_SUM_SQUARES_CHUNK - 1) / FT_SUM_SQUARES_CHUNK;
  FT_REQUIRE(chunks <= 0x7fffffffull, "apply: too many parameters");
  FT_LAUNCH(ctx, k_sum_squares, (unsigned)chunks, kRowThreads, 0, g, n, partials, 0, grad_scale);
  FT_LAUNCH(ctx, k_norm_finalize, 1, kRowThreads, 0, partials, chunks, grad_scale, max_norm,
            norm_out);
  FT_LAUNCH(ctx, k_adamw_scaled, ew_grid(ctx, n), 256, 0, w, g, m, v, n, *p, norm_out);
  return FT_OK;
}
