// Context, error reporting, tensor plumbing and the per-operator C ABI wrappers.
// Each wrapper validates what the reference asserts, then calls the internal kernel.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "ft_common.cuh"

static thread_local char g_error[512] = "";

void ft_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int ft_cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
  ft_set_error("CUDA error %d (%s) at %s:%d in %s", (int)e, cudaGetErrorString(e), file, line,
               what);
  return FT_ERR_CUDA;
}

extern "C" const char* ft_last_error(void) { return g_error; }

extern "C" const char* ft_build_info(void) {
  return "arch: sm_100a\n"
         "gemm_simt_f32\n"
         "gemm_tcgen05_f16 (TMA + TMEM)\n"
         "attention_fwd_simt_f32\nattention_bwd_simt_f32\n"
         "rms_norm\nrms_norm_backward\nrope\nsilu_gate\nmasked_cross_entropy\n"
         "sum_squares\nadamw\napply_fused\nembedding_gather\n";
}

extern "C" int ft_ctx_create(int device, void* stream, FtContext** out) {
  FT_REQUIRE(out != nullptr, "ft_ctx_create: out is NULL");
  int count = 0;
  FT_CUDA(cudaGetDeviceCount(&count));
  FT_REQUIRE(device >= 0 && device < count && device < FT_MAX_DEVICES,
             "ft_ctx_create: device %d of %d", device, count);
  FT_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  FT_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    ft_set_error("ft_ctx_create: device %d is sm_%d%d; this library holds sm_100a code only",
                 device, prop.major, prop.minor);
    return FT_ERR_UNSUPPORTED;
  }
  FtContext* ctx = new FtContext();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  if (stream) {
    ctx->stream = (cudaStream_t)stream;
  } else {
    FT_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
    ctx->own_stream = true;
  }
  FT_CUDA(cudaHostAlloc((void**)&ctx->status_host, sizeof(int) * 16, cudaHostAllocMapped));
  memset(ctx->status_host, 0, sizeof(int) * 16);
  const char* dbg = getenv("FT_GEMM_DEBUG");
  ctx->debug_markers = dbg && dbg[0] == '1';
  if (const char* tm = getenv("FT_GEMM_TILE_M")) ctx->tile_m_override = atoi(tm);
  if (const char* pd = getenv("FT_PDL")) ctx->pdl = atoi(pd) != 0;
  FT_CUDA(cudaHostGetDevicePointer((void**)&ctx->status_dev, ctx->status_host, 0));
  FT_CUDA(cudaMalloc((void**)&ctx->scale_buf, 8 * sizeof(float)));
  FT_CUDA(cudaMalloc((void**)&ctx->pre_flags, FT_PRE_FLAGS * sizeof(int)));
  FT_CUDA(cudaMalloc((void**)&ctx->amax_ring, FT_AMAX_RING * sizeof(int)));
  {
    const float init[8] = {0.f, 1.0f / 2048.0f, 0.f, 0.f, 1.f, 1.f, 1.0f / 2048.0f, 0.f};
    FT_CUDA(cudaMemcpy(ctx->scale_buf, init, sizeof(init), cudaMemcpyHostToDevice));
  }
  cudaDriverEntryPointQueryResult qres;
  void* fn = nullptr;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) ctx->encode_tiled = fn;
  *out = ctx;
  return FT_OK;
}

// Flags and amax slots must be zero when a launch starts to use them.  Instead of one memset in
// front of every such launch (a stream operation that also keeps the launch from overlapping
// with its predecessor), launches take consecutive stretches of a larger array that is zeroed as
// a whole when it has been used up; by stream order every earlier user has finished by then.
int ft_take_pre_flags(FtContext* ctx, int count, int** flags) {
  FT_REQUIRE(count > 0 && count <= FT_PRE_FLAGS, "pre-tile flags: %d row blocks exceed %d", count,
             FT_PRE_FLAGS);
  if (ctx->pre_flag_pos + count > FT_PRE_FLAGS) {
    FT_CUDA(cudaMemsetAsync(ctx->pre_flags, 0, FT_PRE_FLAGS * sizeof(int), ctx->stream));
    ctx->pre_flag_pos = 0;
  }
  *flags = ctx->pre_flags + ctx->pre_flag_pos;
  ctx->pre_flag_pos += count;
  return FT_OK;
}
int ft_take_amax_slot(FtContext* ctx, int** slot) {
  if (ctx->amax_pos >= FT_AMAX_RING) {
    FT_CUDA(cudaMemsetAsync(ctx->amax_ring, 0, FT_AMAX_RING * sizeof(int), ctx->stream));
    ctx->amax_pos = 0;
  }
  *slot = ctx->amax_ring + ctx->amax_pos++;
  return FT_OK;
}

extern "C" int ft_ctx_destroy(FtContext* ctx) {
  if (!ctx) return FT_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->scale_buf) cudaFree(ctx->scale_buf);
  if (ctx->pre_flags) cudaFree(ctx->pre_flags);
  if (ctx->amax_ring) cudaFree(ctx->amax_ring);
  for (cudaEvent_t e : ctx->prof_events) cudaEventDestroy(e);
  if (ctx->status_host) cudaFreeHost(ctx->status_host);
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return FT_OK;
}

extern "C" int ft_ctx_flush(FtContext* ctx) {
  FT_REQUIRE(ctx, "ft_ctx_flush: ctx is NULL");
  return FT_OK;
}

extern "C" int ft_ctx_synchronize(FtContext* ctx) {
  FT_REQUIRE(ctx, "ft_ctx_synchronize: ctx is NULL");
  FT_CUDA(cudaStreamSynchronize(ctx->stream));
  if (ctx->status_host[0] != 0) {
    ft_set_error("device status %d: a kernel's bounded wait ran out (detail %d, %d)",
                 ctx->status_host[0], ctx->status_host[1], ctx->status_host[2]);
    return FT_ERR_DEVICE;
  }
  return FT_OK;
}

extern "C" int ft_ctx_status(FtContext* ctx, int* s) {
  FT_REQUIRE(ctx && s, "ft_ctx_status: NULL argument");
  *s = ctx->status_host[0];
  return FT_OK;
}

extern "C" int ft_ctx_debug_words(FtContext* ctx, int* out16) {
  FT_REQUIRE(ctx && out16, "ft_ctx_debug_words: NULL argument");
  for (int i = 0; i < 16; ++i) out16[i] = ctx->status_host[i];
  return FT_OK;
}

void ft_prof_begin(FtContext* ctx, const char* name) {
  FtContext::ProfRec r;
  r.name = name;
  cudaEvent_t* ev[2] = {&r.e0, &r.e1};
  for (auto* e : ev) {
    if (ctx->prof_pool.empty()) {
      cudaEventCreate(e);
    } else {
      *e = ctx->prof_pool.back();
      ctx->prof_pool.pop_back();
    }
  }
  cudaEventRecord(r.e0, ctx->stream);
  ctx->prof_recs.push_back(r);
}

void ft_prof_end(FtContext* ctx) { cudaEventRecord(ctx->prof_recs.back().e1, ctx->stream); }

extern "C" int ft_ctx_profile(FtContext* ctx, int enable) {
  FT_REQUIRE(ctx, "ft_ctx_profile: ctx is NULL");
  ctx->profile = enable == 1;
  ctx->profile_all = enable == 2;
  return FT_OK;
}

// Text table "kernel launches total_ms" of everything launched while ft_ctx_profile(ctx, 2)
// was on; waits for the stream and resets the records.
extern "C" int ft_ctx_profile_report(FtContext* ctx, char* buf, size_t cap) {
  FT_REQUIRE(ctx && buf && cap > 0, "ft_ctx_profile_report: bad argument");
  FT_CUDA(cudaStreamSynchronize(ctx->stream));
  struct Agg { const char* name; int n; double ms; };
  std::vector<Agg> agg;
  for (auto& r : ctx->prof_recs) {
    float t = 0.f;
    cudaEventElapsedTime(&t, r.e0, r.e1);
    bool found = false;
    for (auto& a : agg)
      if (!strcmp(a.name, r.name)) { a.n++; a.ms += t; found = true; break; }
    if (!found) agg.push_back({r.name, 1, (double)t});
    ctx->prof_pool.push_back(r.e0);
    ctx->prof_pool.push_back(r.e1);
  }
  ctx->prof_recs.clear();
  size_t off = 0;
  buf[0] = 0;
  for (auto& a : agg) {
    int w = snprintf(buf + off, cap - off, "%s %d %.4f\n", a.name, a.n, a.ms);
    if (w < 0 || (size_t)w >= cap - off) break;
    off += (size_t)w;
  }
  return FT_OK;
}

extern "C" int ft_ctx_profile_read(FtContext* ctx, double* gemm_ms, double* gemm_flops,
                                   uint64_t* gemm_launches) {
  FT_REQUIRE(ctx && gemm_ms && gemm_flops && gemm_launches, "ft_ctx_profile_read: NULL argument");
  FT_CUDA(cudaStreamSynchronize(ctx->stream));
  double ms = 0.0;
  for (size_t i = 0; i + 1 < ctx->prof_used; i += 2) {
    float t = 0.f;
    FT_CUDA(cudaEventElapsedTime(&t, ctx->prof_events[i], ctx->prof_events[i + 1]));
    ms += t;
  }
  *gemm_ms = ms;
  *gemm_flops = ctx->prof_flops;
  *gemm_launches = ctx->prof_launches;
  ctx->prof_used = 0;
  ctx->prof_flops = 0.0;
  ctx->prof_fused_flops = 0.0;
  ctx->prof_launches = 0;
  return FT_OK;
}

extern "C" int ft_ctx_profile_read_fused(FtContext* ctx, double* ms_out, double* flops_out,
                                         uint64_t* launches_out) {
  FT_REQUIRE(ctx && ms_out && flops_out && launches_out, "ft_ctx_profile_read_fused: NULL argument");
  FT_CUDA(cudaStreamSynchronize(ctx->stream));
  double ms = 0.0;
  uint64_t n = 0;
  for (size_t i = 0; i + 1 < ctx->prof_used; i += 2) {
    if (i / 2 >= ctx->prof_fused.size() || !ctx->prof_fused[i / 2]) continue;
    float t = 0.f;
    FT_CUDA(cudaEventElapsedTime(&t, ctx->prof_events[i], ctx->prof_events[i + 1]));
    ms += t;
    ++n;
  }
  *ms_out = ms;
  *flops_out = ctx->prof_fused_flops;
  *launches_out = n;
  return FT_OK;
}

extern "C" int ft_ctx_profile_bytes(FtContext* ctx, double* gemm_bytes) {
  FT_REQUIRE(ctx && gemm_bytes, "ft_ctx_profile_bytes: NULL argument");
  *gemm_bytes = ctx->prof_bytes;
  ctx->prof_bytes = 0.0;
  return FT_OK;
}

extern "C" int ft_ctx_set_gemm_mode(FtContext* ctx, int mode) {
  FT_REQUIRE(ctx, "ft_ctx_set_gemm_mode: ctx is NULL");
  FT_REQUIRE(mode == FT_GEMM_F32 || mode == FT_GEMM_F16 || mode == FT_GEMM_F16X2,
             "ft_ctx_set_gemm_mode: unknown mode %d", mode);
  ctx->gemm_mode = mode;
  return FT_OK;
}

extern "C" int ft_ctx_set_gemm_tile_m(FtContext* ctx, int rows) {
  FT_REQUIRE(ctx, "ft_ctx_set_gemm_tile_m: ctx is NULL");
  FT_REQUIRE(rows == 0 || rows == 128 || rows == 256 || rows == 512,
             "ft_ctx_set_gemm_tile_m: 0, 128, 256 or 512 (CTA pairs)");
  ctx->tile_m_override = rows;
  return FT_OK;
}

extern "C" int ft_ctx_launch_count(FtContext* ctx, uint64_t* n) {
  FT_REQUIRE(ctx && n, "ft_ctx_launch_count: NULL argument");
  *n = ctx->launches;
  return FT_OK;
}

int ft_scratch(FtContext* ctx, size_t bytes, void** out) {
  if (bytes > ctx->scratch_bytes) {
    FT_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch) FT_CUDA(cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    size_t want = ft_align_up(bytes + bytes / 4, 1 << 20);
    FT_CUDA(cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
  }
  *out = ctx->scratch;
  return FT_OK;
}

// ---------------------------------------------------------------------------------------
// tensors
// ---------------------------------------------------------------------------------------
extern "C" int ft_tensor_alloc(FtContext* ctx, size_t bytes, void** p) {
  FT_REQUIRE(ctx && p, "ft_tensor_alloc: NULL argument");
  FT_CUDA(cudaMalloc(p, bytes ? bytes : 4));
  return FT_OK;
}

extern "C" int ft_tensor_free(FtContext* ctx, void* p) {
  FT_REQUIRE(ctx, "ft_tensor_free: ctx is NULL");
  if (!p) return FT_OK;
  FT_CUDA(cudaStreamSynchronize(ctx->stream));
  FT_CUDA(cudaFree(p));
  return FT_OK;
}

extern "C" int ft_tensor_zero(FtContext* ctx, void* p, size_t bytes) {
  FT_REQUIRE(ctx && (p || !bytes), "ft_tensor_zero: NULL argument");
  FT_CUDA(cudaMemsetAsync(p, 0, bytes, ctx->stream));
  return FT_OK;
}

extern "C" int ft_upload(FtContext* ctx, void* dst, const void* src, size_t bytes) {
  FT_REQUIRE(ctx && (dst || !bytes) && (src || !bytes), "ft_upload: NULL argument");
  FT_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  FT_CUDA(cudaStreamSynchronize(ctx->stream));  // the host buffer may be reused on return
  return FT_OK;
}

extern "C" int ft_download(FtContext* ctx, void* dst, const void* src, size_t bytes) {
  FT_REQUIRE(ctx && (dst || !bytes) && (src || !bytes), "ft_download: NULL argument");
  FT_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return ft_ctx_synchronize(ctx);
}

__global__ void k_f32_to_f16(const float* __restrict__ src, __half* __restrict__ dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = __float2half_rn(src[i]);
}

// dst[c, r] = src[r, c] through a padded shared tile; T = float or __half
template <typename T>
__global__ void k_transpose(const float* __restrict__ src, T* __restrict__ dst, size_t rows,
                            size_t cols) {
  __shared__ float tile[32][33];
  size_t c0 = (size_t)blockIdx.x * 32, r0 = (size_t)blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    size_t r = r0 + j, c = c0 + threadIdx.x;
    tile[j][threadIdx.x] = (r < rows && c < cols) ? src[r * cols + c] : 0.f;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    size_t c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) {
      float v = tile[threadIdx.x][j];
      if constexpr (sizeof(T) == 2)
        dst[c * rows + r] = __float2half_rn(v);
      else
        dst[c * rows + r] = v;
    }
  }
}

extern "C" int ft_convert_f32_to_f16(FtContext* ctx, const float* src, void* dst, size_t n) {
  FT_REQUIRE(ctx && (src || !n) && (dst || !n), "ft_convert_f32_to_f16: NULL argument");
  if (!n) return FT_OK;
  int grid = (int)std::min<size_t>((n + 255) / 256, (size_t)ctx->sm_count * 16);
  FT_LAUNCH(ctx, k_f32_to_f16, grid, 256, 0, src, (__half*)dst, n);
  return FT_OK;
}

extern "C" int ft_transpose_f32(FtContext* ctx, const float* src, void* dst, size_t rows,
                                size_t cols, int as_f16) {
  FT_REQUIRE(ctx && src && dst, "ft_transpose_f32: NULL argument");
  if (!rows || !cols) return FT_OK;
  FT_REQUIRE((cols + 31) / 32 <= 0x7fffffff && (rows + 31) / 32 <= 65535 * 32,
             "ft_transpose_f32: matrix too large");
  dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
  FT_REQUIRE(grid.y <= 65535, "ft_transpose_f32: more than 65535*32 rows");
  dim3 block(32, 8);
  if (as_f16)
    FT_LAUNCH(ctx, k_transpose<__half>, grid, block, 0, src, (__half*)dst, rows, cols);
  else
    FT_LAUNCH(ctx, k_transpose<float>, grid, block, 0, src, (float*)dst, rows, cols);
  return FT_OK;
}

extern "C" int ft_upload_f32_as_f16(FtContext* ctx, void* dst, const float* src, size_t n) {
  FT_REQUIRE(ctx && (src || !n) && (dst || !n), "ft_upload_f32_as_f16: NULL argument");
  if (!n) return FT_OK;
  void* stage = nullptr;
  FT_TRY(ft_scratch(ctx, n * sizeof(float), &stage));
  FT_CUDA(cudaMemcpyAsync(stage, src, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  FT_TRY(ft_convert_f32_to_f16(ctx, (const float*)stage, dst, n));
  FT_CUDA(cudaStreamSynchronize(ctx->stream));
  return FT_OK;
}

extern "C" int ft_upload_f32_transposed(FtContext* ctx, void* dst, const float* src,
                                        size_t rows, size_t cols, int as_f16) {
  FT_REQUIRE(ctx && src && dst, "ft_upload_f32_transposed: NULL argument");
  size_t n = rows * cols;
  if (!n) return FT_OK;
  void* stage = nullptr;
  FT_TRY(ft_scratch(ctx, n * sizeof(float), &stage));
  FT_CUDA(cudaMemcpyAsync(stage, src, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  FT_TRY(ft_transpose_f32(ctx, (const float*)stage, dst, rows, cols, as_f16));
  FT_CUDA(cudaStreamSynchronize(ctx->stream));
  return FT_OK;
}

// ---------------------------------------------------------------------------------------
// matmul family
// ---------------------------------------------------------------------------------------
static int check_mm(const char* who, FtContext* ctx, const void* a, const void* b, void* out,
                    int M, int K, int N) {
  FT_REQUIRE(ctx && a && b && out, "%s: NULL argument", who);
  FT_REQUIRE(M > 0 && K > 0 && N > 0, "%s: dimensions must be positive (M=%d K=%d N=%d)", who, M,
             K, N);
  return FT_OK;
}

// Dense products go to the tensor cores when the context asks for it and the shape allows;
// otherwise (and always in FT_GEMM_F32 mode) to the exact f32 kernel.
static int mm_dispatch(FtContext* ctx, const float* a, long long sam, long long sak,
                       const void* b, FtDType bt, long long sbk, long long sbn, float* out, int M,
                       int N, int K) {
  // one row against a row-major [K, N] matrix: the matrix-vector kernel, as the reference
  // routes it (matmul.rs:328-331)
  if (M == 1 && sak == 1 && sbn == 1 && sbk == N && (((uintptr_t)b) & 15) == 0)
    return ft_k_matvec(ctx, a, b, bt, out, K, N);
  if (ctx->gemm_mode != FT_GEMM_F32 && sak == 1 && sbk == 1 && bt == FT_F16 && (K % 8) == 0 &&
      M >= 128 && N >= 64 && K >= 64) {
    // A[M,K] row-major f32 -> f16 scratch (auto-scaled: the caller's data may be gradients);
    // B[N,K] K-contiguous f16 is used as stored.
    size_t kp = ft_align_up((size_t)K, 8);
    size_t bytes = ft_align_up((size_t)M * kp * sizeof(__half), 256);
    void* s = nullptr;
    FT_TRY(ft_scratch(ctx, bytes * 2, &s));
    int r = ft_gemm_tc_f32a(ctx, a, sam, (__half*)s, (__half*)((char*)s + bytes), b, sbn, out, N,
                            M, N, K, false, true);
    if (r != FT_ERR_UNSUPPORTED) return r;
  }
  return ft_gemm_simt(ctx, a, sam, sak, b, bt, sbk, sbn, out, N, M, N, K, 1.f, false);
}

extern "C" int ft_matmul(FtContext* ctx, const float* a, const float* b, float* out, int M, int K,
                         int N) {
  FT_TRY(check_mm("ft_matmul", ctx, a, b, out, M, K, N));
  return mm_dispatch(ctx, a, K, 1, b, FT_F32, N, 1, out, M, N, K);
}
extern "C" int ft_matmul_bt(FtContext* ctx, const float* a, const float* b, float* out, int M,
                            int K, int N) {
  FT_TRY(check_mm("ft_matmul_bt", ctx, a, b, out, M, K, N));
  return mm_dispatch(ctx, a, K, 1, b, FT_F32, 1, K, out, M, N, K);
}
extern "C" int ft_matmul_at(FtContext* ctx, const float* a, const float* b, float* out, int M,
                            int K, int N) {
  FT_TRY(check_mm("ft_matmul_at", ctx, a, b, out, M, K, N));
  return mm_dispatch(ctx, a, 1, M, b, FT_F32, N, 1, out, M, N, K);
}
extern "C" int ft_matmul_f16b(FtContext* ctx, const float* a, const void* b, float* out, int M,
                              int K, int N) {
  FT_TRY(check_mm("ft_matmul_f16b", ctx, a, b, out, M, K, N));
  return mm_dispatch(ctx, a, K, 1, b, FT_F16, N, 1, out, M, N, K);
}
extern "C" int ft_matmul_bt_f16b(FtContext* ctx, const float* a, const void* b, float* out, int M,
                                 int K, int N) {
  FT_TRY(check_mm("ft_matmul_bt_f16b", ctx, a, b, out, M, K, N));
  return mm_dispatch(ctx, a, K, 1, b, FT_F16, 1, K, out, M, N, K);
}

// ---------------------------------------------------------------------------------------
// the remaining operators
// ---------------------------------------------------------------------------------------
extern "C" int ft_rope_theta(FtContext* ctx, float* x, size_t n, int head_dim, int seq_len,
                             int heads, int pos, float theta, int inverse) {
  FT_REQUIRE(ctx && x, "ft_rope_theta: NULL argument");
  FT_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "ft_rope_theta: head_dim %d must be even",
             head_dim);
  FT_REQUIRE(heads > 0 && seq_len > 0 && pos >= 0, "ft_rope_theta: bad heads/seq_len/pos");
  size_t per_token = (size_t)heads * head_dim;
  FT_REQUIRE(n % per_token == 0, "ft_rope_theta: %zu elements is not a multiple of heads*head_dim",
             n);
  return ft_k_rope(ctx, x, (long long)per_token, (int)(n / per_token), heads, head_dim, seq_len,
                   pos, theta, inverse != 0);
}

extern "C" int ft_rms_norm_eps(FtContext* ctx, const float* x, const float* w, float* out,
                               int rows, int size, float eps) {
  FT_REQUIRE(ctx && x && w && out, "ft_rms_norm_eps: NULL argument");
  FT_REQUIRE(rows >= 0 && size > 0, "ft_rms_norm_eps: bad shape");
  if (!rows) return FT_OK;
  return ft_k_rms_norm(ctx, x, w, out, rows, size, eps);
}

extern "C" int ft_rms_norm_backward(FtContext* ctx, const float* x, const float* w,
                                    const float* g, float* gx, float* gw, int rows, int size,
                                    float eps) {
  FT_REQUIRE(ctx && x && w && g && gx, "ft_rms_norm_backward: NULL argument");
  FT_REQUIRE(rows >= 0 && size > 0, "ft_rms_norm_backward: bad shape");
  if (!rows) return FT_OK;
  return ft_k_rms_norm_bwd(ctx, x, w, g, gx, gw, rows, size, eps, false);
}

extern "C" int ft_add(FtContext* ctx, const float* a, const float* b, float* out, size_t n) {
  FT_REQUIRE(ctx && (n == 0 || (a && b && out)), "ft_add: NULL argument");
  return n ? ft_k_add(ctx, a, b, out, n) : FT_OK;
}

extern "C" int ft_add_backward(FtContext* ctx, const float* g, float* ga, float* gb, size_t n) {
  FT_REQUIRE(ctx && (n == 0 || (g && ga && gb)), "ft_add_backward: NULL argument");
  if (!n) return FT_OK;
  FT_CUDA(cudaMemcpyAsync(ga, g, n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  FT_CUDA(cudaMemcpyAsync(gb, g, n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  return FT_OK;
}

extern "C" int ft_gradient_scale(FtContext* ctx, float* x, size_t n, float s) {
  FT_REQUIRE(ctx && (n == 0 || x), "ft_gradient_scale: NULL argument");
  return n ? ft_k_scale(ctx, x, n, s) : FT_OK;
}

extern "C" int ft_clip_grad_by_norm(FtContext* ctx, float* g, size_t n, float s) {
  FT_REQUIRE(ctx && (n == 0 || g), "ft_clip_grad_by_norm: NULL argument");
  return n ? ft_k_scale(ctx, g, n, s) : FT_OK;
}

extern "C" int ft_copy(FtContext* ctx, const void* src, void* dst, size_t off, size_t bytes) {
  FT_REQUIRE(ctx && (bytes == 0 || (src && dst)), "ft_copy: NULL argument");
  if (!bytes) return FT_OK;
  FT_CUDA(cudaMemcpyAsync((char*)dst + off, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return FT_OK;
}

extern "C" int ft_silu_gate_fused(FtContext* ctx, const float* a, const float* b, float* out,
                                  size_t n) {
  FT_REQUIRE(ctx && (n == 0 || (a && b && out)), "ft_silu_gate_fused: NULL argument");
  if (!n) return FT_OK;
  FT_REQUIRE(n <= 0x7fffffffull * 1024, "ft_silu_gate_fused: too many elements");
  // a flat buffer is one row of n columns, folded into rows of 1024 when it divides evenly
  int cols = (n % 1024 == 0) ? 1024 : (int)std::min<size_t>(n, 0x7fffffff);
  FT_REQUIRE(n % cols == 0, "ft_silu_gate_fused: unsupported element count %zu", n);
  int rows = (int)(n / cols);
  return ft_k_silu_gate(ctx, a, cols, b, cols, out, cols, rows, cols);
}

extern "C" int ft_silu_gate_backward(FtContext* ctx, const float* a, const float* b,
                                     const float* g, float* ga, float* gb, size_t n) {
  FT_REQUIRE(ctx && (n == 0 || (a && b && g && ga && gb)), "ft_silu_gate_backward: NULL argument");
  if (!n) return FT_OK;
  int cols = (n % 1024 == 0) ? 1024 : (int)std::min<size_t>(n, 0x7fffffff);
  FT_REQUIRE(n % cols == 0, "ft_silu_gate_backward: unsupported element count %zu", n);
  int rows = (int)(n / cols);
  return ft_k_silu_gate_bwd(ctx, a, cols, b, cols, g, cols, ga, cols, gb, cols, rows, cols);
}

static int check_attn(const char* who, const FtAttnParams* p, const float* mask) {
  FT_REQUIRE(p, "%s: params is NULL", who);
  FT_REQUIRE(p->batch > 0 && p->heads > 0 && p->kv_heads > 0 && p->seq_q > 0 && p->seq_k > 0,
             "%s: empty dimension", who);
  FT_REQUIRE(p->heads % p->kv_heads == 0, "%s: heads %u not a multiple of kv_heads %u", who,
             p->heads, p->kv_heads);
  FT_REQUIRE(p->head_dim >= 4 && p->head_dim <= 128 && p->head_dim % 4 == 0,
             "%s: head_dim %u must be a multiple of 4 in [4,128]", who, p->head_dim);
  FT_REQUIRE(p->dropout_prob >= 0.f && p->dropout_prob < 1.f, "%s: dropout_prob %g is outside [0, 1)",
             who, (double)p->dropout_prob);
  (void)mask;
  return FT_OK;
}
// masks and dropout are served by the exact f32 kernels only
static inline bool attn_plain(const FtAttnParams* p, const float* mask) {
  return mask == nullptr && p->dropout_prob == 0.f;
}

extern "C" int ft_flash_attention_v2(FtContext* ctx, const float* q, const float* k,
                                     const float* v, float* out, float* stats, const float* mask,
                                     const FtAttnParams* p) {
  FT_REQUIRE(ctx && q && k && v && out, "ft_flash_attention_v2: NULL argument");
  FT_TRY(check_attn("ft_flash_attention_v2", p, mask));
  // one query and no stats: the decode kernel, whose blocks split the keys (attention.rs:205-224)
  const bool plain = attn_plain(p, mask);
  if (plain && p->seq_q == 1 && !stats && p->head_dim <= 128) return ft_k_attention_decode(ctx, q, k, v, out, *p);
  if (plain && ctx->gemm_mode == FT_GEMM_F16 && p->head_dim == 64 && p->causal && !p->causal_offset &&
      !p->window && p->seq_q == p->seq_k && p->seq_q >= 64) {
    // tensor-core form: q, k, v are rounded to f16 side by side, one row per token
    const int nq = p->heads * 64, nkv = p->kv_heads * 64, ld = nq + 2 * nkv;
    const int T = (int)(p->batch * p->seq_q);
    void* s = nullptr;
    FT_TRY(ft_scratch(ctx, (size_t)T * ld * sizeof(__half), &s));
    __half* qkv16 = (__half*)s;
    FT_TRY(ft_to_f16(ctx, q, nq, qkv16, nullptr, ld, T, nq, false, nullptr));
    FT_TRY(ft_to_f16(ctx, k, nkv, qkv16 + nq, nullptr, ld, T, nkv, false, nullptr));
    FT_TRY(ft_to_f16(ctx, v, nkv, qkv16 + nq + nkv, nullptr, ld, T, nkv, false, nullptr));
    int r = ft_attention_fwd_tc(ctx, qkv16, ld, 0, nq, nq + nkv, nullptr, 0, out, nq, stats,
                                (int)p->batch, (int)p->seq_q, (int)p->heads, (int)p->kv_heads, 64);
    if (r != FT_ERR_UNSUPPORTED) return r;
  }
  FtAttnLaunch a;
  a.q = q; a.k = k; a.v = v; a.out = out; a.stats = stats; a.mask = mask; a.p = *p;
  a.ldq = a.ldo = (long long)p->heads * p->head_dim;
  a.ldk = a.ldv = (long long)p->kv_heads * p->head_dim;
  return ft_k_attention_fwd(ctx, a);
}

extern "C" int ft_flash_attention_v2_backward(FtContext* ctx, const float* q, const float* k,
                                              const float* v, const float* out,
                                              const float* dout, float* dq, float* dk, float* dv,
                                              float* stats, const float* mask,
                                              const FtAttnParams* p) {
  FT_REQUIRE(ctx && q && k && v && out && dout && dq && dk && dv,
             "ft_flash_attention_v2_backward: NULL argument");
  FT_TRY(check_attn("ft_flash_attention_v2_backward", p, mask));
  if (attn_plain(p, mask) && ctx->gemm_mode == FT_GEMM_F16 && p->head_dim == 64 && p->causal && !p->causal_offset &&
      !p->window && p->seq_q == p->seq_k && p->seq_q >= 64 && stats && p->lse_saved) {
    // tensor-core form: operands rounded to f16 (dout after a power-of-two scale)
    const int nq = p->heads * 64, nkv = p->kv_heads * 64, ld = nq + 2 * nkv;
    const int T = (int)(p->batch * p->seq_q);
    void* s = nullptr;
    const size_t n_qkv = ft_align_up((size_t)T * ld * sizeof(__half), 256);
    const size_t n_o = ft_align_up((size_t)T * nq * sizeof(__half), 256);
    FT_TRY(ft_scratch(ctx, n_qkv + 2 * n_o, &s));
    __half* qkv16 = (__half*)s;
    __half* o16 = (__half*)((char*)s + n_qkv);
    __half* do16 = (__half*)((char*)s + n_qkv + n_o);
    FT_TRY(ft_to_f16(ctx, q, nq, qkv16, nullptr, ld, T, nq, false, nullptr));
    FT_TRY(ft_to_f16(ctx, k, nkv, qkv16 + nq, nullptr, ld, T, nkv, false, nullptr));
    FT_TRY(ft_to_f16(ctx, v, nkv, qkv16 + nq + nkv, nullptr, ld, T, nkv, false, nullptr));
    FT_TRY(ft_to_f16(ctx, out, nq, o16, nullptr, nq, T, nq, false, nullptr));
    const float* scales = nullptr;
    FT_TRY(ft_to_f16(ctx, dout, nq, do16, nullptr, nq, T, nq, true, &scales, 8));
    int r = ft_attention_bwd_tc(ctx, qkv16, ld, 0, nq, nq + nkv, o16, nq, do16, nq, dq, nq, dk, dv,
                                nkv, stats, scales + 1, (int)p->batch, (int)p->seq_q,
                                (int)p->heads, (int)p->kv_heads, 64);
    if (r != FT_ERR_UNSUPPORTED) return r;
  }
  FtAttnBwdLaunch a;
  a.q = q; a.k = k; a.v = v; a.out = out; a.dout = dout; a.dq = dq; a.dk = dk; a.dv = dv;
  a.stats = stats; a.mask = mask; a.p = *p;
  a.ldq = a.ldo = a.lddo = a.lddq = (long long)p->heads * p->head_dim;
  a.ldk = a.ldv = a.lddk = a.lddv = (long long)p->kv_heads * p->head_dim;
  return ft_k_attention_bwd(ctx, a);
}

extern "C" int ft_masked_cross_entropy_weighted(FtContext* ctx, const float* logits,
                                                const uint32_t* targets, const float* weights,
                                                float* grad, float* row_loss, int rows,
                                                int vocab) {
  FT_REQUIRE(ctx && logits && targets && weights && grad && row_loss,
             "ft_masked_cross_entropy_weighted: NULL argument");
  FT_REQUIRE(rows >= 0 && vocab > 0, "ft_masked_cross_entropy_weighted: bad shape");
  if (!rows) return FT_OK;
  return ft_k_masked_ce(ctx, logits, targets, weights, grad, row_loss, rows, vocab, 1.f);
}

extern "C" int ft_sum_squares_partial(FtContext* ctx, const float* x, size_t n, float* out,
                                      size_t offset, size_t* chunks) {
  FT_REQUIRE(ctx && out && (x || !n), "ft_sum_squares_partial: NULL argument");
  size_t c = (n + FT_SUM_SQUARES_CHUNK - 1) / FT_SUM_SQUARES_CHUNK;
  if (chunks) *chunks = c;
  return c ? ft_k_sum_squares(ctx, x, n, out, offset) : FT_OK;
}

extern "C" int ft_adamw_update(FtContext* ctx, float* w, const float* g, float* m, float* v,
                               size_t n, const FtAdamParams* p) {
  FT_REQUIRE(ctx && p && (n == 0 || (w && g && m && v)), "ft_adamw_update: NULL argument");
  return n ? ft_k_adamw(ctx, w, g, m, v, n, p) : FT_OK;
}

extern "C" int ft_argmax_rows(FtContext* ctx, const float* x, uint32_t* out_idx, int rows, int len) {
  FT_REQUIRE(ctx && x && out_idx, "ft_argmax_rows: NULL argument");
  return ft_k_argmax_rows(ctx, x, out_idx, rows, len);
}

extern "C" int ft_embedding_gather(FtContext* ctx, const float* table, const uint32_t* ids,
                                   float* out, int tokens, int vocab, int hidden) {
  FT_REQUIRE(ctx && table && ids && out, "ft_embedding_gather: NULL argument");
  FT_REQUIRE(tokens >= 0 && vocab > 0 && hidden > 0, "ft_embedding_gather: bad shape");
  return tokens ? ft_k_embedding(ctx, table, ids, out, tokens, vocab, hidden) : FT_OK;
}
