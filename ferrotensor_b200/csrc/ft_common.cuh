// Shared declarations of libft_cuda: context object, error reporting, launch helpers and
// the internal (strided, typed) forms of the kernels that both the per-op C ABI and the
// fused step driver call.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <vector>

#include "../../include/ft_cuda.h"

struct FtContext {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int sm_count = 148;
  int gemm_mode = FT_GEMM_F32;
  uint64_t launches = 0;
  // scratch owned by the context; grown on demand (never inside a captured region)
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  // status word written by kernels whose bounded waits ran out (pinned, device-mapped)
  int* status_host = nullptr;   // 16 words: [0..3] status, [4..15] progress markers
  int* status_dev = nullptr;
  bool debug_markers = false;   // FT_GEMM_DEBUG=1: kernels record progress markers
  // device floats: [0] amax bits, [1] the constant 2^-11, [4..6] {S, 1/S, 2^-11/S} of the
  // operand being converted (consumed by the GEMM that follows in stream order)
  float* scale_buf = nullptr;
  // "amax in the producer": while armed, kernels that support it fold the largest magnitude
  // of what they write into scale_buf[0] (atomicMax), and the next auto-scaled conversion
  // uses it instead of making its own pass over the tensor.
  bool pdl = true;   // programmatic dependent launch for the kernels that support it
  int* pre_flags = nullptr;   // FT_PRE_FLAGS per-row-block flags of the adapter pre-tiles: each
                              // launch takes the next unused stretch, the array is zeroed again
                              // (one memset) when it has been used up
  int pre_flag_pos = 1 << 30; // first unused flag; past the end = zero the array first
  int* amax_ring = nullptr;   // FT_AMAX_RING slots for armed maxima, handed out and zeroed the same way
  int amax_pos = 1 << 30;
  int* amax_out = nullptr;
  bool amax_ready = false;
  int tile_m_override = 0;   // FT_GEMM_TILE_M: 128 or 256 forces the GEMM tile height
  // optional timing of the tensor-core GEMM launches (CUDA events on the launch stream)
  bool profile = false;
  std::vector<cudaEvent_t> prof_events;  // start/stop pairs, reused
  size_t prof_used = 0;                  // events handed out since the last read
  double prof_flops = 0.0;
  double next_launch_bytes = 0.0;
  double prof_bytes = 0.0;   // algorithmic bytes (operands once, results once) of the timed GEMM launches
  uint64_t prof_launches = 0;
  // the same for the subset of those launches whose epilogue also does elementwise work of the
  // step (RoPE, SwiGLU forward or backward): marks parallel to the event pairs
  std::vector<uint8_t> prof_fused;
  double prof_fused_flops = 0.0;
  bool next_launch_fused = false;
  // optional timing of EVERY launch by kernel name (ft_ctx_profile(ctx, 2))
  bool profile_all = false;
  struct ProfRec { const char* name; cudaEvent_t e0, e1; };
  std::vector<ProfRec> prof_recs;
  std::vector<cudaEvent_t> prof_pool;
  // cuTensorMapEncodeTiled, resolved through the runtime (no link against libcuda)
  void* encode_tiled = nullptr;
};

void ft_set_error(const char* fmt, ...);
int ft_cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define FT_CUDA(expr)                                                        \
  do {                                                                       \
    cudaError_t _e = (expr);                                                 \
    if (_e != cudaSuccess) return ft_cuda_fail(_e, #expr, __FILE__, __LINE__); \
  } while (0)

#define FT_REQUIRE(cond, ...)   \
  do {                          \
    if (!(cond)) {              \
      ft_set_error(__VA_ARGS__); \
      return FT_ERR_INVALID;    \
    }                           \
  } while (0)

#define FT_TRY(expr)             \
  do {                           \
    int _r = (expr);             \
    if (_r != FT_OK) return _r;  \
  } while (0)

void ft_prof_begin(FtContext* ctx, const char* name);
void ft_prof_end(FtContext* ctx);

constexpr int FT_MAX_DEVICES = 64;   // per-device launch state is kept in arrays of this size
constexpr int FT_PRE_FLAGS = 4096;
constexpr int FT_AMAX_RING = 1024;

// Launch on the context's stream, count the launch and surface launch errors.
#define FT_LAUNCH(ctx, kernel, grid, block, smem, ...)                          \
  do {                                                                          \
    if ((ctx)->profile_all) ft_prof_begin((ctx), #kernel);                      \
    kernel<<<(grid), (block), (smem), (ctx)->stream>>>(__VA_ARGS__);            \
    if ((ctx)->profile_all) ft_prof_end((ctx));                                 \
    (ctx)->launches++;                                                          \
    cudaError_t _e = cudaPeekAtLastError();                                     \
    if (_e != cudaSuccess) return ft_cuda_fail(_e, #kernel, __FILE__, __LINE__); \
  } while (0)

// Programmatic dependent launch.  A kernel launched through FT_LAUNCH_PDL may start while the
// kernel before it in the stream is still draining; it must call ft_pdl_wait() before it
// touches global memory (what ran before is complete and visible from then on) and may call
// ft_pdl_launch() to let its own successor start early.  Both are no-ops in a plain launch.
#ifdef __CUDACC__
__device__ __forceinline__ void ft_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void ft_pdl_launch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
template <typename... KArgs, typename... Args>
inline cudaError_t ft_launch_ex(FtContext* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                size_t smem, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess && ctx->pdl) {
    // the attribute is refused on this stream or driver: drop it for good and launch plainly
    (void)cudaGetLastError();
    ctx->pdl = false;
    cfg.numAttrs = 0;
    e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  }
  return e;
}
#define FT_LAUNCH_PDL(ctx, kernel, grid, block, smem, ...)                       \
  do {                                                                          \
    if ((ctx)->profile_all) ft_prof_begin((ctx), #kernel);                      \
    cudaError_t _e = ft_launch_ex((ctx), kernel, (grid), (block), (smem), __VA_ARGS__); \
    if ((ctx)->profile_all) ft_prof_end((ctx));                                 \
    (ctx)->launches++;                                                          \
    if (_e == cudaSuccess) _e = cudaPeekAtLastError();                          \
    if (_e != cudaSuccess) return ft_cuda_fail(_e, #kernel, __FILE__, __LINE__); \
  } while (0)
#endif

// Scratch of at least `bytes`, 256-byte aligned.  Stream order makes reuse by consecutive
// calls safe; growth synchronises the stream before the old block is released.
int ft_scratch(FtContext* ctx, size_t bytes, void** out);

static inline size_t ft_align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static inline int ft_cdiv(long long a, long long b) { return (int)((a + b - 1) / b); }

// ----- internal kernels (definitions in the .cu files named on the right) -----------------

// B operand element type of a matmul
enum FtDType { FT_F32 = 0, FT_F16 = 1, FT_BF16 = 2 };

// C[m,n] (+)= alpha * sum_k A(m,k) B(k,n) with arbitrary element strides; f32 FMA.
// A is f32; B is f32 or f16.                                         (ft_matmul_simt.cu)
int ft_gemm_simt(FtContext* ctx, const float* a, long long sam, long long sak, const void* b,
                 FtDType b_type, long long sbk, long long sbn, float* c, long long ldc, int M,
                 int N, int K, float alpha, bool accumulate);

// tcgen05 GEMM: C[M,N] f32 (ldc) (=|+=) alpha * A[M,K] (lda) . B[N,K]^T (ldb), A and B both
// f16 or both bf16, K contiguous.  alpha_ptr (device, may be NULL = 1) is read by the
// epilogue.  Returns FT_ERR_UNSUPPORTED when the shape breaks a TMA rule.  (ft_gemm_tc.cu)
int ft_gemm_tc(FtContext* ctx, const void* a, long long lda, const void* b, FtDType ab_type,
               long long ldb, float* c, long long ldc, int M, int N, int K, bool accumulate,
               const float* alpha_ptr);
// General form: C[M,N] = alpha_dev * alpha * (A[M,K].B[N,K]^T + A2[M,K2].B2[N,K2]^T)
//                         (+ bias[col]) (+ residual[row, col]), written as f32 and/or f16.
// The optional second operand pair extends the contraction (how the rank-r adapter product
// rides in the same accumulator as the frozen projection).
struct FtGemmArgs {
  const void* a = nullptr; long long lda = 0;
  const void* b = nullptr; long long ldb = 0;
  const void* a2 = nullptr; long long lda2 = 0;
  const void* b2 = nullptr; long long ldb2 = 0;
  int K2 = 0;
  int k2_used = 0;   // > 0: only the first k2_used columns of the second pair are non-zero
  FtDType ab_type = FT_F16;
  int M = 0, N = 0, K = 0;
  float* c = nullptr; long long ldc = 0;
  __half* c16 = nullptr; long long ldc16 = 0;
  const float* alpha_ptr = nullptr; float alpha = 1.f;
  const float* bias = nullptr;
  const float* residual = nullptr; long long ldr = 0;
  bool want_amax = false;   // contribute the output's largest magnitude to an armed amax slot
  int* amax_slot = nullptr; // ... or to this slot (zero before the launch), armed or not
  // carried scale: the f16 result is multiplied by the power of two that would bring
  // *carry_amax (the largest magnitude of an EARLIER tensor of the same kind, e.g. the same
  // gradient one block later in the backward pass) into [2^(carry_exp-1), 2^carry_exp); one
  // thread publishes {S, 1/S, 2^-11/S} to carry_scales.  CTA-pair launches only
  // (ft_gemm_tc_pair_eligible); amax_slot still receives the UNSCALED magnitude.
  const int* carry_amax = nullptr;
  int carry_exp = 0;
  float* carry_scales = nullptr;
  // rotary epilogue of a q|k|v projection (CTA-pair launches, f16 result only): the columns
  // are heads of 64; those below rope_cols are rotated by the angles of the row's position
  // (row % rope_seq) from rope_table ({cos, sin} transposed: [32, rope_seq] f32), after the bias
  const float* rope_table = nullptr;
  int rope_seq = 0, rope_cols = 0;
  // SwiGLU inside the epilogue (CTA-pair launches; gate|up columns interleaved in runs of 32).
  // Forward (gate|up projection): beside c16 = gate|up, swi_f16[row, 32 per 64-column run] =
  // silu(gate) * up; amax_slot receives the largest |gate| or |up|.
  __half* swi_f16 = nullptr; long long swi_ldf = 0;
  // Backward (down projection's input gradient, N = features): no f32/f16 result of its own;
  // with the saved gate|up rows swi_gu16 it writes S * (d gate | d up) to swi_dgu16, S from the
  // bound 1.1 * *carry_amax * *swi_gu_amax (published to swi_scales); amax_slot receives the
  // largest magnitude of the input gradient itself.
  const __half* swi_gu16 = nullptr; long long swi_ldgu = 0;
  __half* swi_dgu16 = nullptr; long long swi_lddgu = 0;
  const int* swi_gu_amax = nullptr;
  float* swi_scales = nullptr;
  // adapter pre-tiles: when pre_b is set, the launch first computes
  //   pre_c16[M, 64] (f16, pitch pre_ldc16) = pre_alpha * A . pre_b^T   (pre_b [64, K], f16)
  // which is normally the very buffer a2 points at (the K-concatenated tail operand)
  const void* pre_b = nullptr; long long pre_ldb = 0;
  __half* pre_c16 = nullptr; long long pre_ldc16 = 0;
  float pre_alpha = 1.f;
};
int ft_gemm_tc_ex(FtContext* ctx, const FtGemmArgs& g);
// whether a product of this size runs on CTA pairs (the kernel with the carried-scale epilogue)
bool ft_gemm_tc_pair_eligible(const FtContext* ctx, int M, int N);
// S = 2^(target_exp - e) for amax = f * 2^e, f in [0.5, 1); 1 when amax is zero or not finite
#ifdef __CUDACC__
__device__ __forceinline__ float ft_scale_from_amax_bits(int bits, int target_exp) {
  const float amax = __int_as_float(bits);
  if (!(amax > 0.f) || !isfinite(amax)) return 1.0f;
  int e;
  frexpf(amax, &e);
  return ldexpf(1.0f, target_exp - e);
}
__device__ __forceinline__ void ft_publish_scales(float* scales, float S) {
  scales[0] = S;
  scales[1] = 1.0f / S;
  scales[2] = ldexpf(1.0f / S, -11);
}
#endif
// One problem of a token-reduction launch: P[M, N<=64] = sum_t A[t, m] B[t, n]; the reduction
// launch adds it into up to three segments out[(m - m0) * som + (n - n0) * son].
struct FtKoSeg {
  float* out = nullptr;
  int m0 = 0, mcount = 0, n0 = 0, ncount = 0;
  long long som = 0, son = 0;
  // >= 0: the segment's rows are interleaved in runs of 32 with another segment's: its row m is
  // row (m / 32) * 64 + il_off + m % 32 of the product (m0 is not used then)
  int il_off = -1;
};
struct FtKoProblem {
  const void* a = nullptr; long long lda = 0;
  const void* b = nullptr; long long ldb = 0;
  int M = 0, N = 0;
  int nseg = 0;
  FtKoSeg seg[3];
  float* slabs = nullptr;   // set by the call: [nslabs][M][64]
  int nslabs = 0;
};
int ft_gemm_tc_kouter_pair(FtContext* ctx, int nprob, FtKoProblem* prob, int T);
int ft_slab_reduce_problems(FtContext* ctx, int nprob, const FtKoProblem* prob,
                            const float* alpha_ptr, float alpha, bool accumulate);
// f32 [rows, cols] (ld) -> f16 [rows, ldo]; `lo` (optional) receives the rounding remainder
// x 2^11.  auto_scale first multiplies by the power of two that brings the largest magnitude
// to [2^11, 2^12) (gradients are far below f16's normal range otherwise); *scales_out then
// points at device floats {S, 1/S, 2^-11/S}, else it is NULL.
int ft_to_f16(FtContext* ctx, const float* src, long long ld, __half* hi, __half* lo,
              long long ldo, int rows, int cols, bool auto_scale, const float** scales_out,
              int target_exp = 12);
// Arms the producer-side amax (see FtContext::amax_out): zeroes the slot; the kernels launched
// until the next auto-scaled ft_to_f16 contribute to it.
int ft_amax_arm(FtContext* ctx);
int ft_scales_from_amax_or_pass(FtContext* ctx, const float* src, long long ld, int rows, int cols,
                                int target_exp, const float** scales_out);
// conversion + one (FT_GEMM_F16) or two (FT_GEMM_F16X2) tensor-core passes
int ft_gemm_tc_f32a(FtContext* ctx, const float* a, long long lda_f32, __half* stage_hi,
                    __half* stage_lo, const void* b_f16, long long ldb, float* c, long long ldc,
                    int M, int N, int K, bool accumulate, bool auto_scale);

// elementwise / norm / loss / optimizer kernels with leading dimensions (ft_kernels.cu)
int ft_k_embedding(FtContext* ctx, const float* table, const uint32_t* ids, float* out,
                   int tokens, int vocab, int hidden);
int ft_k_rms_norm(FtContext* ctx, const float* x, const float* w, float* out, int rows, int n,
                  float eps);
// same, writing f32 (out, may be NULL) and/or f16 (out16, may be NULL)
int ft_k_rms_norm16(FtContext* ctx, const float* x, const float* w, float* out, __half* out16,
                    int rows, int n, float eps);
int ft_k_rms_norm_bwd(FtContext* ctx, const float* x, const float* w, const float* g, float* gx,
                      float* gw, int rows, int n, float eps, bool accumulate_gx);
// A carried scale (see FtGemmArgs::carry_amax) for a kernel that also writes its result as f16.
struct FtCarry {
  const int* amax_in = nullptr;   // largest magnitude of the earlier tensor
  int exp = 0;
  float* scales = nullptr;        // {S, 1/S, 2^-11/S} published by one thread
  int* amax_out = nullptr;        // receives this result's largest magnitude (zero before)
};
// frozen-norm backward (gw == NULL, gx accumulated) that also writes gx16 = f16(S gx); rows of
// 1024..4096 elements, 16-byte aligned.  Returns FT_ERR_UNSUPPORTED for other shapes.
int ft_k_rms_norm_bwd_carry(FtContext* ctx, const float* x, const float* w, const float* g,
                            float* gx, __half* gx16, int rows, int n, float eps,
                            const FtCarry& carry);
// in place on x[t*ld + h*head_dim + i]; position of token t = pos + t % seq_len
int ft_k_rope(FtContext* ctx, float* x, long long ld, int tokens, int heads, int head_dim,
              int seq_len, int pos, float theta, bool inverse);
// RoPE for the tensor-core path.  table: float2 {cos, sin} [seq_len, head_dim/2] built with the
// same f32 recipe as ft_k_rope, followed by the same values transposed ([head_dim/2, seq_len]):
// 2 * seq_len * head_dim floats in all.  ft_k_rope_to_f16 reads the first form; the epilogues
// that rotate (FtGemmArgs::rope_table, FtAttnBwdOut16::table) take a pointer to the second.  forward: f32 q|k|v rows -> f16 rows (q, k rotated, v copied).
// backward: f32 gradient rows -> f16 rows times the scale in `scales[0]`, q, k parts rotated
// by the negated angle.  Rows are [tokens, nq + 2 nkv], head_dim 64.
int ft_k_rope_table(FtContext* ctx, float* table, int seq_len, int head_dim, float theta);
int ft_k_rope_to_f16(FtContext* ctx, const float* src, __half* dst, long long ld, int tokens,
                     int nq, int nkv, int seq_len, const float* table, bool inverse,
                     const float* scales);
int ft_k_add(FtContext* ctx, const float* a, const float* b, float* out, size_t n);
int ft_k_scale(FtContext* ctx, float* x, size_t n, float s);
// 2-D SwiGLU: out[t, j] = silu(a[t*lda + j]) * b[t*ldb + j], j < n
int ft_k_silu_gate(FtContext* ctx, const float* a, long long lda, const float* b, long long ldb,
                   float* out, long long ldo, int rows, int n);
// gu rows hold gate | up as two halves of n columns each, or (il) interleaved in runs of 32:
// gate 0..31, up 0..31, gate 32..63, ...; the backward forms write d gate | d up the same way
int ft_k_silu_gate16h(FtContext* ctx, const __half* gu, long long ld, __half* out, long long ldo,
                      int rows, int n, int* in_amax, bool il = false);
int ft_k_silu_gate_bwd16h(FtContext* ctx, const __half* gu, long long ld, const float* g,
                          long long ldg, __half* out, long long ldo, int rows, int n,
                          const int* in_amax, const float** scales_out, bool il = false);
// the same with the upstream gradient as f16 rows carrying the scale g_scales[0]; g_amax is the
// largest magnitude of the UNSCALED upstream gradient
int ft_k_silu_gate_bwd16hh(FtContext* ctx, const __half* gu, long long ld, const __half* g16,
                           long long ldg, const float* g_scales, const int* g_amax, __half* out,
                           long long ldo, int rows, int n, const int* in_amax,
                           const float** scales_out, bool il = false);
int ft_k_silu_gate_bwd(FtContext* ctx, const float* a, long long lda, const float* b,
                       long long ldb, const float* g, long long ldg, float* ga, long long ldga,
                       float* gb, long long ldgb, int rows, int n);
// y[t, j] += bias[j]
int ft_k_add_bias(FtContext* ctx, float* y, long long ld, const float* bias, int rows, int n);
// decode-time kernels                                               (ft_infer.cu)
int ft_k_matvec(FtContext* ctx, const float* x, const void* w, FtDType w_type, float* out, int K, int N);
int ft_k_attention_decode(FtContext* ctx, const float* q, const float* k, const float* v, float* out,
                          const FtAttnParams& p);
int ft_k_argmax_rows(FtContext* ctx, const float* x, uint32_t* out, int rows, int len);
int ft_k_masked_ce16(FtContext* ctx, const float* logits, const uint32_t* targets,
                     const float* weights, __half* g16, long long ld16, float* row_loss, int rows,
                     int vocab, float grad_scale, const float** scales_out);
int ft_k_masked_ce(FtContext* ctx, const float* logits, const uint32_t* targets,
                   const float* weights, float* grad, float* row_loss, int rows, int vocab,
                   float grad_scale);
int ft_k_sum_squares(FtContext* ctx, const float* x, size_t n, float* out, size_t offset);
int ft_k_adamw(FtContext* ctx, float* w, const float* g, float* m, float* v, size_t n,
               const FtAdamParams* p);
// norm (from chunk partials) -> skip/clip -> AdamW, all on the device
int ft_k_apply_fused(FtContext* ctx, float* w, float* g, float* m, float* v, size_t n,
                     float grad_scale, float max_norm, const FtAdamParams* p, float* partials,
                     float* norm_out);

// data parallelism (ft_comm.cu): in-place sum over the ranks on the context's stream
int ft_comm_allreduce_f32(FtComm* c, float* buf, size_t n);
int ft_comm_world(const FtComm* c);
FtContext* ft_comm_ctx(const FtComm* c);

// A flat index i = r * per_row + c walked with stride st without dividing in the loop:
// (r, c) advance by (st / per_row, st % per_row) with a carry.
struct RowWalk {
  long long r;
  int c, st_r, st_c, per_row;
  __device__ __forceinline__ RowWalk(size_t i, size_t st, size_t per_row_)
      : r((long long)(i / per_row_)), c((int)(i % per_row_)), st_r((int)(st / per_row_)),
        st_c((int)(st % per_row_)), per_row((int)per_row_) {}
  __device__ __forceinline__ void next() {
    r += st_r;
    c += st_c;
    if (c >= per_row) { c -= per_row; ++r; }
  }
};

// attention with token strides (elements between consecutive tokens)   (ft_attention.cu)
// the next `count` zeroed pre-tile flags / the next zeroed amax slot of the context's rings
int ft_take_pre_flags(FtContext* ctx, int count, int** flags);
int ft_take_amax_slot(FtContext* ctx, int** slot);

struct FtAttnLaunch {
  const float *q, *k, *v;
  long long ldq, ldk, ldv;  // elements between tokens
  float* out;
  long long ldo;
  float* stats;             // [b*h*sq*2] or nullptr
  const float* mask = nullptr;   // additive, strides in p.mask_stride
  FtAttnParams p;
};
int ft_k_attention_fwd(FtContext* ctx, const FtAttnLaunch& a);
struct FtAttnBwdLaunch {
  const float *q, *k, *v, *out, *dout;
  long long ldq, ldk, ldv, ldo, lddo;
  float *dq, *dk, *dv;
  long long lddq, lddk, lddv;
  float* stats;
  const float* mask = nullptr;
  FtAttnParams p;
};
int ft_k_attention_bwd(FtContext* ctx, const FtAttnBwdLaunch& a);

// Causal attention on the tensor cores (head_dim 64).  qkv16: f16 rows [tokens, ld] holding
// q at column q_col0, k at k_col0, v at v_col0 (RoPE applied); writes f16 and/or f32 output
// rows [tokens, heads*64] and the log-sum-exp of every row into stats[2*row+1].
// FT_ERR_UNSUPPORTED when the shape is outside the kernel's domain.   (ft_attention_tc.cu)
int ft_attention_fwd_tc(FtContext* ctx, const __half* qkv16, long long ld, int q_col0, int k_col0,
                        int v_col0, __half* out16, long long ldo16, float* out32, long long ldo32,
                        float* stats, int batch, int seq, int heads, int kv_heads, int head_dim);
// Backward: o16 = forward output (f16), do16 = output gradient (f16, times the power-of-two
// scale whose inverse is the device scalar *inv_scale, NULL = 1); stats must hold the forward
// log-sum-exp at [2*row+1] and receives Delta at [2*row].  dq [tokens, lddq]; dk, dv [tokens, ldd].
// With out16 the results are written instead as f16 rows in the operands' q|k|v column layout,
// dq and dk rotated back by the rotary angles of `table` ({cos, sin} transposed: [32, seq] f32) and all
// times the power of two carried from *carry_amax (see FtGemmArgs::carry_amax); the armed amax
// slot still receives the largest unrotated, unscaled magnitude.
struct FtAttnBwdOut16 {
  __half* rows = nullptr; long long ld = 0;
  const float* table = nullptr;
  const int* carry_amax = nullptr; int carry_exp = 0;
  float* carry_scales = nullptr;
};
int ft_attention_bwd_tc(FtContext* ctx, const __half* qkv16, long long ld, int q_col0, int k_col0,
                        int v_col0, const __half* o16, long long ldo, const __half* do16,
                        long long lddo, float* dq, long long lddq, float* dk, float* dv,
                        long long ldd, float* stats, const float* inv_scale, int batch, int seq,
                        int heads, int kv_heads, int head_dim, const FtAttnBwdOut16* out16 = nullptr);
