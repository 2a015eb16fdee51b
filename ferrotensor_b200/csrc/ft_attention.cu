// Exact f32 attention (CUDA cores): causal / windowed, grouped-query, online softmax.
// Forward saves the log-sum-exp per query row; backward runs in two passes without
// atomics (dQ per query row, then dK/dV per key row summed over the query heads that
// share the KV head), so results are identical from run to run.
//
// Thread layout for all three kernels: a block owns 32 rows (queries or keys) of one head,
// 4 lanes share a row and each lane owns the 16-byte chunks {lane, lane+4, ...} of head_dim,
// so the four lanes of a row read 64 contiguous bytes of a staged tile.
#include <math.h>

#include "ft_common.cuh"

namespace {

constexpr int ROWS = 32;     // rows per block
constexpr int TILE = 32;     // rows of the other side staged per step
constexpr int THREADS = 128;
constexpr float kMaskedLse = 3.0e38f;

__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

__device__ __forceinline__ bool visible(int i, int j, const FtAttnParams& p) {
  int qi = i + (int)p.causal_offset;
  if (p.causal && j > qi) return false;
  if (p.window) {
    int d = qi - j;
    if (d < 0) d = -d;
    if (d >= (int)p.window) return false;
  }
  return true;
}

// number of keys any query of rows [i0, i1) can see (upper bound, for tile skipping)
__device__ __forceinline__ int key_limit(int i1, const FtAttnParams& p) {
  if (!p.causal) return (int)p.seq_k;
  long long lim = (long long)(i1 - 1) + p.causal_offset + 1;
  if (lim < 0) lim = 0;
  return (int)(lim < (long long)p.seq_k ? lim : p.seq_k);
}

// stage `n` rows x nchunks float4 from global (row stride ld) into smem [TILE][nchunks]
__device__ __forceinline__ void stage(float4* dst, const float* src, long long ld, int n,
                                      int nchunks) {
  for (int e = threadIdx.x; e < TILE * nchunks; e += THREADS) {
    int r = e / nchunks, c = e % nchunks;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < n) {
      const float* p = src + (long long)r * ld + c * 4;
      if ((((uintptr_t)p) & 15) == 0) v = *(const float4*)p;
      else v = make_float4(p[0], p[1], p[2], p[3]);
    }
    dst[e] = v;
  }
}

__device__ __forceinline__ float4 ld4(const float* p) {
  if ((((uintptr_t)p) & 15) == 0) return *(const float4*)p;
  return make_float4(p[0], p[1], p[2], p[3]);
}
__device__ __forceinline__ void st4(float* p, float4 v) {
  if ((((uintptr_t)p) & 15) == 0) *(float4*)p = v;
  else { p[0] = v.x; p[1] = v.y; p[2] = v.z; p[3] = v.w; }
}
__device__ __forceinline__ float dot4(float4 a, float4 b) {
  return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
}
__device__ __forceinline__ void fma4(float4& acc, float s, float4 v) {
  acc.x = fmaf(s, v.x, acc.x); acc.y = fmaf(s, v.y, acc.y);
  acc.z = fmaf(s, v.z, acc.z); acc.w = fmaf(s, v.w, acc.w);
}
__device__ __forceinline__ void scale4(float4& a, float s) { a.x *= s; a.y *= s; a.z *= s; a.w *= s; }

// ---------------------------------------------------------------------------------- forward
template <int CPL>
__global__ void __launch_bounds__(THREADS)
k_attn_fwd(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
           float* __restrict__ out, float* __restrict__ stats, long long ldq, long long ldk,
           long long ldv, long long ldo, FtAttnParams p, float scale) {
  extern __shared__ float4 smem[];
  const int d = p.head_dim, nchunks = d >> 2;
  float4* ks = smem;
  float4* vs = smem + TILE * nchunks;
  const int bh = blockIdx.y, b = bh / p.heads, h = bh % p.heads;
  const int kvh = h / (p.heads / p.kv_heads);
  const int lane = threadIdx.x & 3, r = threadIdx.x >> 2;
  const int i0 = blockIdx.x * ROWS, i = i0 + r;
  const bool row_ok = i < (int)p.seq_q;

  float4 qv[CPL], acc[CPL];
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    int ch = lane + 4 * c;
    acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    qv[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row_ok && ch < nchunks) {
      qv[c] = ld4(q + ((long long)b * p.seq_q + i) * ldq + (long long)h * d + ch * 4);
      scale4(qv[c], scale);
    }
  }
  float m = -INFINITY, l = 0.f;
  const int klim = key_limit(min(i0 + ROWS, (int)p.seq_q), p);
  const float* kbase = k + (long long)b * p.seq_k * ldk + (long long)kvh * d;
  const float* vbase = v + (long long)b * p.seq_k * ldv + (long long)kvh * d;
  for (int j0 = 0; j0 < klim; j0 += TILE) {
    int n = min(TILE, klim - j0);
    __syncthreads();
    stage(ks, kbase + (long long)j0 * ldk, ldk, n, nchunks);
    stage(vs, vbase + (long long)j0 * ldv, ldv, n, nchunks);
    __syncthreads();
    for (int jj = 0; jj < n; ++jj) {
      float part = 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        int ch = lane + 4 * c;
        if (ch < nchunks) part += dot4(qv[c], ks[jj * nchunks + ch]);
      }
      float s = quad_sum(part);
      if (row_ok && visible(i, j0 + jj, p)) {
        float m_new = fmaxf(m, s);
        float corr = expf(m - m_new);  // exp(-inf) = 0 on the first visible key
        float pj = expf(s - m_new);
        l = l * corr + pj;
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          int ch = lane + 4 * c;
          if (ch < nchunks) {
            scale4(acc[c], corr);
            fma4(acc[c], pj, vs[jj * nchunks + ch]);
          }
        }
        m = m_new;
      }
    }
  }
  if (!row_ok) return;
  float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    int ch = lane + 4 * c;
    if (ch < nchunks) {
      scale4(acc[c], inv);
      st4(out + ((long long)b * p.seq_q + i) * ldo + (long long)h * d + ch * 4, acc[c]);
    }
  }
  if (stats && lane == 0) {
    size_t row = ((size_t)b * p.heads + h) * p.seq_q + i;
    stats[2 * row + 1] = l > 0.f ? m + logf(l) : kMaskedLse;
  }
}

// ------------------------------------------------------------------------ backward, pass 1
// Per query row: Delta = dO . O, (LSE if not saved), dQ = scale * sum_j dS_ij K_j.
template <int CPL>
__global__ void __launch_bounds__(THREADS)
k_attn_bwd_dq(const float* __restrict__ q, const float* __restrict__ k,
              const float* __restrict__ v, const float* __restrict__ o,
              const float* __restrict__ dout, float* __restrict__ dq, float* __restrict__ stats,
              long long ldq, long long ldk, long long ldv, long long ldo, long long lddo,
              long long lddq, FtAttnParams p, float scale) {
  extern __shared__ float4 smem[];
  const int d = p.head_dim, nchunks = d >> 2;
  float4* ks = smem;
  float4* vs = smem + TILE * nchunks;
  const int bh = blockIdx.y, b = bh / p.heads, h = bh % p.heads;
  const int kvh = h / (p.heads / p.kv_heads);
  const int lane = threadIdx.x & 3, r = threadIdx.x >> 2;
  const int i0 = blockIdx.x * ROWS, i = i0 + r;
  const bool row_ok = i < (int)p.seq_q;
  const size_t row = ((size_t)b * p.heads + h) * p.seq_q + (row_ok ? i : 0);

  float4 qv[CPL], dov[CPL], acc[CPL];
  float dpart = 0.f;
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    int ch = lane + 4 * c;
    acc[c] = qv[c] = dov[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row_ok && ch < nchunks) {
      long long tok = (long long)b * p.seq_q + i;
      qv[c] = ld4(q + tok * ldq + (long long)h * d + ch * 4);
      dov[c] = ld4(dout + tok * lddo + (long long)h * d + ch * 4);
      float4 ov = ld4(o + tok * ldo + (long long)h * d + ch * 4);
      dpart += dot4(dov[c], ov);
    }
  }
  const float delta = quad_sum(dpart);
  const int klim = key_limit(min(i0 + ROWS, (int)p.seq_q), p);
  const float* kbase = k + (long long)b * p.seq_k * ldk + (long long)kvh * d;
  const float* vbase = v + (long long)b * p.seq_k * ldv + (long long)kvh * d;

  float lse;
  if (p.lse_saved) {
    lse = row_ok ? stats[2 * row + 1] : 0.f;
  } else {
    float m = -INFINITY, l = 0.f;
    for (int j0 = 0; j0 < klim; j0 += TILE) {
      int n = min(TILE, klim - j0);
      __syncthreads();
      stage(ks, kbase + (long long)j0 * ldk, ldk, n, nchunks);
      __syncthreads();
      for (int jj = 0; jj < n; ++jj) {
        float part = 0.f;
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          int ch = lane + 4 * c;
          if (ch < nchunks) part += dot4(qv[c], ks[jj * nchunks + ch]);
        }
        float s = quad_sum(part) * scale;
        if (row_ok && visible(i, j0 + jj, p)) {
          float m_new = fmaxf(m, s);
          l = l * expf(m - m_new) + expf(s - m_new);
          m = m_new;
        }
      }
    }
    lse = l > 0.f ? m + logf(l) : kMaskedLse;
  }

  for (int j0 = 0; j0 < klim; j0 += TILE) {
    int n = min(TILE, klim - j0);
    __syncthreads();
    stage(ks, kbase + (long long)j0 * ldk, ldk, n, nchunks);
    stage(vs, vbase + (long long)j0 * ldv, ldv, n, nchunks);
    __syncthreads();
    for (int jj = 0; jj < n; ++jj) {
      float sp = 0.f, dp = 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        int ch = lane + 4 * c;
        if (ch < nchunks) {
          sp += dot4(qv[c], ks[jj * nchunks + ch]);
          dp += dot4(dov[c], vs[jj * nchunks + ch]);
        }
      }
      float s = quad_sum(sp) * scale;
      dp = quad_sum(dp);
      if (row_ok && visible(i, j0 + jj, p)) {
        float pj = expf(s - lse);
        float ds = pj * (dp - delta) * scale;
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          int ch = lane + 4 * c;
          if (ch < nchunks) fma4(acc[c], ds, ks[jj * nchunks + ch]);
        }
      }
    }
  }
  if (!row_ok) return;
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    int ch = lane + 4 * c;
    if (ch < nchunks)
      st4(dq + ((long long)b * p.seq_q + i) * lddq + (long long)h * d + ch * 4, acc[c]);
  }
  if (lane == 0) {
    stats[2 * row] = delta;
    stats[2 * row + 1] = lse;
  }
}

// ------------------------------------------------------------------------ backward, pass 2
// Per key row j of KV head kvh: dV_j = sum_i P_ij dO_i, dK_j = scale * sum_i dS_ij Q_i over
// all queries of all query heads in the group.
template <int CPL>
__global__ void __launch_bounds__(THREADS)
k_attn_bwd_dkv(const float* __restrict__ q, const float* __restrict__ k,
               const float* __restrict__ v, const float* __restrict__ dout,
               float* __restrict__ dk, float* __restrict__ dv, const float* __restrict__ stats,
               long long ldq, long long ldk, long long ldv, long long lddo, long long lddk,
               long long lddv, FtAttnParams p, float scale) {
  extern __shared__ float4 smem[];
  const int d = p.head_dim, nchunks = d >> 2;
  float4* qs = smem;
  float4* dos = smem + TILE * nchunks;
  float* srow = (float*)(smem + 2 * TILE * nchunks);  // [TILE][2]: Delta, LSE
  const int bk = blockIdx.y, b = bk / p.kv_heads, kvh = bk % p.kv_heads;
  const int group = p.heads / p.kv_heads;
  const int lane = threadIdx.x & 3, r = threadIdx.x >> 2;
  const int j0 = blockIdx.x * ROWS, j = j0 + r;
  const bool row_ok = j < (int)p.seq_k;

  float4 kv[CPL], vv[CPL], dka[CPL], dva[CPL];
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    int ch = lane + 4 * c;
    kv[c] = vv[c] = dka[c] = dva[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row_ok && ch < nchunks) {
      long long tok = (long long)b * p.seq_k + j;
      kv[c] = ld4(k + tok * ldk + (long long)kvh * d + ch * 4);
      vv[c] = ld4(v + tok * ldv + (long long)kvh * d + ch * 4);
    }
  }
  // first query that can see key j0 (causal: i + offset >= j0)
  int i_start = 0;
  if (p.causal) {
    long long s = (long long)j0 - p.causal_offset;
    i_start = s > 0 ? (int)(s / TILE) * TILE : 0;
  }
  for (int g = 0; g < group; ++g) {
    const int h = kvh * group + g;
    const float* qbase = q + (long long)b * p.seq_q * ldq + (long long)h * d;
    const float* dobase = dout + (long long)b * p.seq_q * lddo + (long long)h * d;
    const size_t srow0 = ((size_t)b * p.heads + h) * p.seq_q;
    for (int t0 = i_start; t0 < (int)p.seq_q; t0 += TILE) {
      int n = min(TILE, (int)p.seq_q - t0);
      __syncthreads();
      stage(qs, qbase + (long long)t0 * ldq, ldq, n, nchunks);
      stage(dos, dobase + (long long)t0 * lddo, lddo, n, nchunks);
      for (int e = threadIdx.x; e < TILE * 2; e += THREADS)
        srow[e] = (e / 2 < n) ? stats[2 * (srow0 + t0) + e] : 0.f;
      __syncthreads();
      for (int ii = 0; ii < n; ++ii) {
        float sp = 0.f, dp = 0.f;
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
          int ch = lane + 4 * c;
          if (ch < nchunks) {
            sp += dot4(kv[c], qs[ii * nchunks + ch]);
            dp += dot4(vv[c], dos[ii * nchunks + ch]);
          }
        }
        float s = quad_sum(sp) * scale;
        dp = quad_sum(dp);
        if (row_ok && visible(t0 + ii, j, p)) {
          float pj = expf(s - srow[2 * ii + 1]);
          float ds = pj * (dp - srow[2 * ii]) * scale;
#pragma unroll
          for (int c = 0; c < CPL; ++c) {
            int ch = lane + 4 * c;
            if (ch < nchunks) {
              fma4(dva[c], pj, dos[ii * nchunks + ch]);
              fma4(dka[c], ds, qs[ii * nchunks + ch]);
            }
          }
        }
      }
    }
  }
  if (!row_ok) return;
#pragma unroll
  for (int c = 0; c < CPL; ++c) {
    int ch = lane + 4 * c;
    if (ch < nchunks) {
      long long tok = (long long)b * p.seq_k + j;
      st4(dk + tok * lddk + (long long)kvh * d + ch * 4, dka[c]);
      st4(dv + tok * lddv + (long long)kvh * d + ch * 4, dva[c]);
    }
  }
}

inline int pick_cpl(int head_dim) {
  int need = ((head_dim >> 2) + 3) / 4;
  return need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
}

inline float attn_scale(const FtAttnParams& p) {
  return p.scale != 0.f ? p.scale : 1.0f / sqrtf((float)p.head_dim);
}

}  // namespace

#define FT_ATTN_DISPATCH(cpl, KERNEL, ...)                                   \
  switch (cpl) {                                                             \
    case 1: FT_LAUNCH(ctx, KERNEL<1>, grid, THREADS, smem, __VA_ARGS__); break; \
    case 2: FT_LAUNCH(ctx, KERNEL<2>, grid, THREADS, smem, __VA_ARGS__); break; \
    case 4: FT_LAUNCH(ctx, KERNEL<4>, grid, THREADS, smem, __VA_ARGS__); break; \
    default: FT_LAUNCH(ctx, KERNEL<8>, grid, THREADS, smem, __VA_ARGS__); break; \
  }

int ft_k_attention_fwd(FtContext* ctx, const FtAttnLaunch& a) {
  const FtAttnParams& p = a.p;
  FT_REQUIRE((long long)p.batch * p.heads <= 65535, "attention: batch*heads exceeds 65535");
  dim3 grid(ft_cdiv(p.seq_q, ROWS), p.batch * p.heads);
  size_t smem = (size_t)2 * TILE * (p.head_dim / 4) * sizeof(float4);
  float scale = attn_scale(p);
  FT_ATTN_DISPATCH(pick_cpl(p.head_dim), k_attn_fwd, a.q, a.k, a.v, a.out, a.stats, a.ldq, a.ldk,
                   a.ldv, a.ldo, p, scale);
  return FT_OK;
}

int ft_k_attention_bwd(FtContext* ctx, const FtAttnBwdLaunch& a) {
  FtAttnParams p = a.p;
  FT_REQUIRE((long long)p.batch * p.heads <= 65535, "attention: batch*heads exceeds 65535");
  float* stats = a.stats;
  if (!stats) {
    void* s = nullptr;
    FT_TRY(ft_scratch(ctx, (size_t)p.batch * p.heads * p.seq_q * 2 * sizeof(float), &s));
    stats = (float*)s;
    p.lse_saved = 0;
  }
  float scale = attn_scale(p);
  int cpl = pick_cpl(p.head_dim);
  {
    dim3 grid(ft_cdiv(p.seq_q, ROWS), p.batch * p.heads);
    size_t smem = (size_t)2 * TILE * (p.head_dim / 4) * sizeof(float4);
    FT_ATTN_DISPATCH(cpl, k_attn_bwd_dq, a.q, a.k, a.v, a.out, a.dout, a.dq, stats, a.ldq, a.ldk,
                     a.ldv, a.ldo, a.lddo, a.lddq, p, scale);
  }
  {
    dim3 grid(ft_cdiv(p.seq_k, ROWS), p.batch * p.kv_heads);
    size_t smem = (size_t)2 * TILE * (p.head_dim / 4) * sizeof(float4) + TILE * 2 * sizeof(float);
    FT_ATTN_DISPATCH(cpl, k_attn_bwd_dkv, a.q, a.k, a.v, a.dout, a.dk, a.dv, stats, a.ldq, a.ldk,
                     a.ldv, a.lddo, a.lddk, a.lddv, p, scale);
  }
  return FT_OK;
}
