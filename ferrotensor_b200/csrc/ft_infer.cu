// Decode-time kernels (one token against a KV cache): matrix-vector products, attention for a
// single query, greedy argmax.  All are HBM-bound: the design goal is to have every SM
// streaming and to read every weight / cache byte exactly once.
//
//   k_matvec_partial / k_matvec_reduce   out[N] = x[K] . W[K, N] (W f32 or f16, row-major), the
//       shape of every linear when one token is decoded (reference: matmul.rs:394-424,
//       matvec.wgsl).  A block covers 256 columns x one K slice, a thread 8 columns (one
//       16-byte load of f16 weights per k); slices are summed in a fixed order by a second
//       tiny kernel, so results do not depend on scheduling.
//   k_attn_decode_partial / k_attn_decode_combine   softmax(q K^T / sqrt(D)) V for seq_q = 1
//       (reference: attention.rs:205-224, flash_attention_v2.wgsl:284-382): keys are split over
//       blocks (batch*heads alone would leave most SMs idle), each block keeps a running
//       (max, sum, acc[D]) over its keys, the combine kernel merges the splits in order.
//   k_argmax_rows   index of the largest value per row in f32::total_cmp order, the last index
//       winning ties (reference: misc.rs:20-34, kernels.wgsl:251-296); bit-exact.
#include <math.h>

#include "ft_common.cuh"

namespace {

// ----------------------------------------------------------------------------- matvec
template <typename W>
__device__ __forceinline__ void load8(const W* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
  const uint4 a = *(const uint4*)p;
  const __half2* h = (const __half2*)&a;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

constexpr int MV_COLS = 256;     // columns per block (32 lanes x 8)
constexpr int MV_SLICES = 8;     // warps per block, each taking every 8th k of the block's range

// part[split][n] = sum over the block's K range of x[k] * w[k, n]
template <typename W>
__global__ void __launch_bounds__(256)
k_matvec_partial(const float* __restrict__ x, const W* __restrict__ w, float* __restrict__ part,
                 int K, int N, int k_per_split) {
  __shared__ float red[MV_SLICES][MV_COLS + 8];
  const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int col = blockIdx.x * MV_COLS + lane * 8;
  const int k0 = blockIdx.y * k_per_split, k1 = min(K, k0 + k_per_split);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const bool vec = col + 8 <= N && (N % 8) == 0;
  if (col < N) {
    if (vec) {
#pragma unroll 4
      for (int k = k0 + slice; k < k1; k += MV_SLICES) {
        float v[8];
        load8<W>(w + (size_t)k * N + col, v);
        const float xv = x[k];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(xv, v[e], acc[e]);
      }
    } else {
      for (int k = k0 + slice; k < k1; k += MV_SLICES) {
        const float xv = x[k];
        for (int e = 0; e < 8 && col + e < N; ++e)
          acc[e] = fmaf(xv, (float)w[(size_t)k * N + col + e], acc[e]);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[slice][lane * 8 + e] = acc[e];
  __syncthreads();
  // slices added in index order
  const int c = threadIdx.x;
  if (blockIdx.x * MV_COLS + c < N) {
    float s = 0.f;
#pragma unroll
    for (int sl = 0; sl < MV_SLICES; ++sl) s += red[sl][c];
    part[(size_t)blockIdx.y * N + blockIdx.x * MV_COLS + c] = s;
  }
}

__global__ void k_matvec_reduce(const float* __restrict__ part, float* __restrict__ out, int N, int splits) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float s = 0.f;
  for (int sp = 0; sp < splits; ++sp) s += part[(size_t)sp * N + n];
  out[n] = s;
}

// ----------------------------------------------------------------------------- decode attention
constexpr int DEC_THREADS = 128;   // keys per tile = threads
constexpr int DEC_MAX_D = 128;
constexpr float DEC_MASKED = -3.0e38f;

__device__ __forceinline__ bool dec_visible(const FtAttnParams& p, int kp) {
  const long long qa = (long long)p.causal_offset;   // the single query sits at this position
  if (kp >= (int)p.seq_k) return false;
  if (p.causal && kp > qa) return false;
  if (p.window) {
    const long long dist = qa >= kp ? qa - kp : kp - qa;
    if (dist >= (long long)p.window) return false;
  }
  return true;
}

__device__ __forceinline__ float dec_block_reduce(float v, bool take_max, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = take_max ? fmaxf(v, t) : v + t;
  }
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int i = 1; i < DEC_THREADS / 32; ++i) r = take_max ? fmaxf(r, red[i]) : r + red[i];
  return r;
}

// One block per (key split, batch*head).  Writes {m, l} and acc[D] of its key range.
__global__ void __launch_bounds__(DEC_THREADS)
k_attn_decode_partial(const float* __restrict__ q, const float* __restrict__ k,
                      const float* __restrict__ v, float* __restrict__ part, FtAttnParams p,
                      int keys_per_split, float scale) {
  __shared__ float qs[DEC_MAX_D];
  __shared__ float wts[DEC_THREADS];
  __shared__ float red[DEC_THREADS / 32];
  const int D = (int)p.head_dim, lid = threadIdx.x;
  const int bh = blockIdx.y, b = bh / (int)p.heads, h = bh % (int)p.heads;
  const int kvh = h / ((int)p.heads / (int)p.kv_heads);
  const float* qrow = q + (size_t)bh * D;
  if (lid < D) qs[lid] = qrow[lid] * scale;
  __syncthreads();
  const int k_begin = blockIdx.x * keys_per_split;
  const int k_end = min((int)p.seq_k, k_begin + keys_per_split);
  float m_run = DEC_MASKED, l_run = 0.f;
  float acc[DEC_MAX_D / 32] = {0.f, 0.f, 0.f, 0.f};
  for (int ks = k_begin; ks < k_end; ks += DEC_THREADS) {
    const int kp = ks + lid;
    float sc = DEC_MASKED;
    if (kp < k_end && dec_visible(p, kp)) {
      const float* kr = k + (((size_t)b * p.seq_k + kp) * p.kv_heads + kvh) * D;
      float dot = 0.f;
      if ((D & 3) == 0) {
        for (int c = 0; c < D; c += 4) {
          const float4 kk = *(const float4*)(kr + c);
          dot = fmaf(qs[c], kk.x, dot); dot = fmaf(qs[c + 1], kk.y, dot);
          dot = fmaf(qs[c + 2], kk.z, dot); dot = fmaf(qs[c + 3], kk.w, dot);
        }
      } else {
        for (int c = 0; c < D; ++c) dot = fmaf(qs[c], kr[c], dot);
      }
      sc = dot;
    }
    const float m_new = fmaxf(m_run, dec_block_reduce(sc, true, red));
    const float corr = expf(m_run - m_new);
    const float pj = sc > DEC_MASKED ? expf(sc - m_new) : 0.f;
    wts[lid] = pj;
    l_run = l_run * corr + dec_block_reduce(pj, false, red);   // (its barriers publish wts too)
    // P V: warp g takes keys g, g + 4, ... of the tile, lane l the dimensions l, l + 32, ...
    // (one coalesced row segment per load); the four warps are added once, after the last tile
    {
      const int g = lid >> 5, l = lid & 31;
      const int keys = min(DEC_THREADS, k_end - ks);
      const size_t stride = (size_t)p.kv_heads * D;
      const float* vr = v + (((size_t)b * p.seq_k + ks) * p.kv_heads + kvh) * D;
#pragma unroll
      for (int i = 0; i < DEC_MAX_D / 32; ++i) acc[i] *= corr;
#pragma unroll 4
      for (int j = g; j < keys; j += 4) {
        const float wj = wts[j];
        const float* row = vr + (size_t)j * stride;
#pragma unroll
        for (int i = 0; i < DEC_MAX_D / 32; ++i)
          if (l + 32 * i < D) acc[i] = fmaf(wj, row[l + 32 * i], acc[i]);
      }
    }
    m_run = m_new;
    __syncthreads();
  }
  // add the four warps' partial outputs in warp order
  __shared__ float accs[4][DEC_MAX_D];
  {
    const int g = lid >> 5, l = lid & 31;
#pragma unroll
    for (int i = 0; i < DEC_MAX_D / 32; ++i)
      if (l + 32 * i < D) accs[g][l + 32 * i] = acc[i];
  }
  __syncthreads();
  float* o = part + ((size_t)bh * gridDim.x + blockIdx.x) * (DEC_MAX_D + 2);
  if (lid == 0) { o[0] = m_run; o[1] = l_run; }
  if (lid < D) o[2 + lid] = ((accs[0][lid] + accs[1][lid]) + accs[2][lid]) + accs[3][lid];
}

// out[bh, d] = sum_s exp(m_s - M) acc_s[d] / sum_s exp(m_s - M) l_s, splits taken in order
__global__ void k_attn_decode_combine(const float* __restrict__ part, float* __restrict__ out, int D,
                                      int splits) {
  const int bh = blockIdx.x, d = threadIdx.x;
  const float* base = part + (size_t)bh * splits * (DEC_MAX_D + 2);
  float M = DEC_MASKED;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, base[(size_t)s * (DEC_MAX_D + 2)]);
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* ps = base + (size_t)s * (DEC_MAX_D + 2);
    const float w = ps[1] > 0.f ? expf(ps[0] - M) : 0.f;
    l += w * ps[1];
    if (d < D) acc += w * ps[2 + d];
  }
  if (d < D) out[(size_t)bh * D + d] = l > 0.f ? acc / l : 0.f;
}

// ----------------------------------------------------------------------------- argmax
// A key whose unsigned order is f32::total_cmp's order of the bits.
__device__ __forceinline__ uint32_t order_key(uint32_t bits) {
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__global__ void __launch_bounds__(256)
k_argmax_rows(const uint32_t* __restrict__ bits, uint32_t* __restrict__ out, int len) {
  __shared__ uint32_t skey[256], sidx[256];
  const uint32_t* row = bits + (size_t)blockIdx.x * len;
  // a thread with no elements keeps (0, 0): the lowest key, and on equal keys the larger
  // index wins, so it never beats a real element
  uint32_t key = 0u, idx = 0u;
  for (int i = threadIdx.x; i < len; i += 256) {
    const uint32_t ki = order_key(row[i]);
    if (ki >= key) { key = ki; idx = (uint32_t)i; }
  }
  skey[threadIdx.x] = key;
  sidx[threadIdx.x] = idx;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if ((int)threadIdx.x < s) {
      const uint32_t ok = skey[threadIdx.x + s], oi = sidx[threadIdx.x + s];
      if (ok > skey[threadIdx.x] || (ok == skey[threadIdx.x] && oi > sidx[threadIdx.x])) {
        skey[threadIdx.x] = ok;
        sidx[threadIdx.x] = oi;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) out[blockIdx.x] = sidx[0];
}

}  // namespace

// out[N] = x[K] . W[K, N]; W is f32 or f16.  Two launches (K slices, then their ordered sum).
int ft_k_matvec(FtContext* ctx, const float* x, const void* w, FtDType w_type, float* out, int K, int N) {
  FT_REQUIRE(w_type == FT_F32 || w_type == FT_F16, "matvec: weights must be f32 or f16");
  FT_REQUIRE(K > 0 && N > 0, "matvec: empty product");
  const int col_blocks = ft_cdiv(N, MV_COLS);
  // enough blocks to keep every SM streaming, each slice at least 64 rows deep
  int splits = std::max(1, std::min(ft_cdiv(4 * ctx->sm_count, col_blocks), ft_cdiv(K, 64)));
  const int per = ft_cdiv(K, splits);
  splits = ft_cdiv(K, per);
  void* s = nullptr;
  FT_TRY(ft_scratch(ctx, (size_t)splits * N * sizeof(float), &s));
  dim3 grid(col_blocks, splits);
  const bool aligned = (((uintptr_t)w) & 15) == 0;
  FT_REQUIRE(aligned, "matvec: weights must be 16-byte aligned");
  if (w_type == FT_F16)
    FT_LAUNCH(ctx, k_matvec_partial<__half>, grid, 256, 0, x, (const __half*)w, (float*)s, K, N, per);
  else
    FT_LAUNCH(ctx, k_matvec_partial<float>, grid, 256, 0, x, (const float*)w, (float*)s, K, N, per);
  FT_LAUNCH(ctx, k_matvec_reduce, ft_cdiv(N, 256), 256, 0, (const float*)s, out, N, splits);
  return FT_OK;
}

// Attention for one query per (batch, head): q [batch, 1, heads, D], k/v [batch, seq_k, kv_heads, D],
// out [batch, 1, heads, D]; causal with the query at position causal_offset, optional window.
int ft_k_attention_decode(FtContext* ctx, const float* q, const float* k, const float* v, float* out,
                          const FtAttnParams& p) {
  FT_REQUIRE(p.seq_q == 1 && p.head_dim >= 1 && p.head_dim <= DEC_MAX_D,
             "attention decode: one query, head_dim at most %d", DEC_MAX_D);
  const int bh = (int)(p.batch * p.heads);
  FT_REQUIRE(bh > 0 && bh <= 65535, "attention decode: batch*heads must be in 1..65535");
  const int tiles = ft_cdiv((long long)p.seq_k, DEC_THREADS);
  // about eight blocks per SM keep enough loads in flight to stream the cache
  int splits = std::max(1, std::min(tiles, ft_cdiv(8 * ctx->sm_count, bh)));
  const int per = ft_cdiv(tiles, splits) * DEC_THREADS;
  splits = ft_cdiv((long long)p.seq_k, per);
  void* s = nullptr;
  FT_TRY(ft_scratch(ctx, (size_t)bh * splits * (DEC_MAX_D + 2) * sizeof(float), &s));
  const float scale = p.scale != 0.f ? p.scale : 1.0f / sqrtf((float)p.head_dim);
  FT_LAUNCH(ctx, k_attn_decode_partial, dim3(splits, bh), DEC_THREADS, 0, q, k, v, (float*)s, p, per, scale);
  FT_LAUNCH(ctx, k_attn_decode_combine, bh, DEC_MAX_D, 0, (const float*)s, out, (int)p.head_dim, splits);
  return FT_OK;
}

int ft_k_argmax_rows(FtContext* ctx, const float* x, uint32_t* out, int rows, int len) {
  FT_REQUIRE(rows > 0 && len > 0, "argmax_rows: empty input");
  FT_LAUNCH(ctx, k_argmax_rows, rows, 256, 0, (const uint32_t*)x, out, len);
  return FT_OK;
}
