// Exact f32 matmul on CUDA cores: C[m,n] (+)= alpha * sum_k A(m,k) * B(k,n) for operands
// with arbitrary element strides (covers a.b, a.b^T and a^T.b) and B stored as f32 or
// binary16.  Products and sums are f32 FMA; this is the parity path and the fallback for
// shapes the tensor-core kernel does not take.
#include "ft_common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename T>
__device__ __forceinline__ float ldval(const T* p);
template <>
__device__ __forceinline__ float ldval<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldval<__half>(const __half* p) { return __half2float(*p); }

template <typename TB>
__global__ void __launch_bounds__(256)
k_gemm_simt(const float* __restrict__ a, long long sam, long long sak, const TB* __restrict__ b,
            long long sbk, long long sbn, float* __restrict__ c, long long ldc, int M, int N,
            int K, float alpha, int accumulate, int k_chunk) {
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Bs[BK][BN + PAD];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int kb = blockIdx.z * k_chunk, ke = min(K, kb + k_chunk);
  const bool a_kfast = (sak == 1);
  const bool b_nfast = (sbn == 1);
  float acc[4][4] = {};

  for (int k0 = kb; k0 < ke; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int e = tid + i * 256;
      int m, k;
      if (a_kfast) { k = e & 15; m = e >> 4; } else { m = e & 63; k = e >> 6; }
      int gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < M && gk < ke) ? a[(long long)gm * sam + (long long)gk * sak] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int e = tid + i * 256;
      int n, k;
      if (b_nfast) { n = e & 63; k = e >> 6; } else { k = e & 15; n = e >> 4; }
      int gn = n0 + n, gk = k0 + k;
      Bs[k][n] = (gn < N && gk < ke) ? ldval<TB>(b + (long long)gk * sbk + (long long)gn * sbn) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float4 av = *(const float4*)&As[k][ty * 4];
      float4 bv = *(const float4*)&Bs[k][tx * 4];
      float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
    }
    __syncthreads();
  }
  // split-K partials go to slab blockIdx.z of c (the caller reduces them in order)
  float* cz = c + (size_t)blockIdx.z * (size_t)M * (size_t)ldc * (gridDim.z > 1 ? 1 : 0);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = alpha * acc[i][j];
      float* p = cz + (long long)gm * ldc + gn;
      *p = accumulate ? *p + v : v;
    }
  }
}

// c[m,n] (+)= sum over slabs, in slab order (deterministic)
__global__ void k_splitk_reduce(const float* __restrict__ part, int slabs, float* __restrict__ c,
                                long long ldc, int M, int N, int accumulate) {
  size_t total = (size_t)M * N;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += st) {
    float acc = 0.f;
    for (int s = 0; s < slabs; ++s) acc += part[(size_t)s * total + i];
    size_t m = i / N, n = i % N;
    float* p = c + m * ldc + n;
    *p = accumulate ? *p + acc : acc;
  }
}

}  // namespace

int ft_gemm_simt(FtContext* ctx, const float* a, long long sam, long long sak, const void* b,
                 FtDType b_type, long long sbk, long long sbn, float* c, long long ldc, int M,
                 int N, int K, float alpha, bool accumulate) {
  FT_REQUIRE(b_type == FT_F32 || b_type == FT_F16, "gemm_simt: B must be f32 or f16");
  dim3 grid(ft_cdiv(N, BN), ft_cdiv(M, BM), 1);
  FT_REQUIRE(grid.y <= 65535, "gemm_simt: M too large");
  // A long reduction with few output tiles (the LoRA weight gradients: K = tokens) is split
  // along K into slabs that are then summed in a fixed order.
  int tiles = (int)(grid.x * grid.y);
  int slabs = 1;
  if (tiles < ctx->sm_count && K >= 2048) {
    slabs = std::min(std::min(ft_cdiv(2 * ctx->sm_count, tiles), K / 512), 64);
    if (slabs < 1) slabs = 1;
  }
  if (slabs == 1) {
    if (b_type == FT_F32)
      FT_LAUNCH(ctx, k_gemm_simt<float>, grid, 256, 0, a, sam, sak, (const float*)b, sbk, sbn, c,
                ldc, M, N, K, alpha, accumulate ? 1 : 0, K);
    else
      FT_LAUNCH(ctx, k_gemm_simt<__half>, grid, 256, 0, a, sam, sak, (const __half*)b, sbk, sbn,
                c, ldc, M, N, K, alpha, accumulate ? 1 : 0, K);
    return FT_OK;
  }
  int k_chunk = ft_cdiv(ft_cdiv(K, slabs), BK) * BK;
  slabs = ft_cdiv(K, k_chunk);
  void* s = nullptr;
  FT_TRY(ft_scratch(ctx, (size_t)slabs * M * N * sizeof(float), &s));
  grid.z = slabs;
  if (b_type == FT_F32)
    FT_LAUNCH(ctx, k_gemm_simt<float>, grid, 256, 0, a, sam, sak, (const float*)b, sbk, sbn,
              (float*)s, (long long)N, M, N, K, alpha, 0, k_chunk);
  else
    FT_LAUNCH(ctx, k_gemm_simt<__half>, grid, 256, 0, a, sam, sak, (const __half*)b, sbk, sbn,
              (float*)s, (long long)N, M, N, K, alpha, 0, k_chunk);
  size_t total = (size_t)M * N;
  int rg = (int)std::min<size_t>((total + 255) / 256, (size_t)ctx->sm_count * 8);
  FT_LAUNCH(ctx, k_splitk_reduce, rg, 256, 0, (const float*)s, slabs, c, ldc, M, N,
            accumulate ? 1 : 0);
  return FT_OK;
}
