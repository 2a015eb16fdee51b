/*
 * ft_cuda.h - C ABI of libft_cuda.so, the sm_100a `cuda` device for ferrotensor's
 * LoRA fine-tuning step.
 *
 * Every entry point below replaces one method of the reference's operator surface,
 * `ferrotensor_backend::ComputeEngine` (plus the tensor/context plumbing it needs), and
 * keeps that method's argument meaning:
 *   - buffers are plain device pointers owned by the caller; shapes are row-major, dense,
 *     outermost first, and passed as explicit sizes;
 *   - outputs are pre-allocated by the caller and OVERWRITTEN, never accumulated, except
 *     for the methods the reference documents as in place;
 *   - calls enqueue work on the context's stream in program order and return at once;
 *     only ft_ctx_synchronize / ft_download* wait for the device;
 *   - arithmetic is f32; "f16b" weights are IEEE binary16, two per little-endian 32-bit
 *     word, element 2i in the low half (the reference's FP16 storage format).
 * Where the reference panics on a precondition these functions return non-zero and
 * ft_last_error() describes the failure.  A kernel never traps: device-side problems
 * (a bounded wait that ran out) are reported through ft_ctx_status().
 *
 * Paths cited are relative to the reference repository.
 */
#ifndef FT_CUDA_H
#define FT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FT_OK 0
#define FT_ERR_INVALID 1   /* precondition violated (the reference would panic)     */
#define FT_ERR_CUDA 2      /* a CUDA runtime call failed                            */
#define FT_ERR_UNSUPPORTED 3
#define FT_ERR_DEVICE 4    /* a kernel reported a failed bounded wait               */
#define FT_ERR_COMM 5      /* NCCL missing or failed, or a rank did not answer in time */

/* ferrotensor-backend/src/engine/training.rs:7,11 */
#define FT_MASKED_CE_SKIP 0xffffffffu
#define FT_SUM_SQUARES_CHUNK 4096u

/* How the dense contractions round their operands (accumulation is always f32).
 *   FT_GEMM_F32   exact f32 FMA on CUDA cores - the parity path
 *   FT_GEMM_F16   activations (and their gradients, after a power-of-two scale) rounded to
 *                 f16, f16 weights exact, tcgen05 tensor cores, one pass
 *   FT_GEMM_F16X2 activations split into two f16 halves (22 significant bits), two passes */
#define FT_GEMM_F32 0
#define FT_GEMM_F16 1
#define FT_GEMM_F16X2 2

typedef struct FtContext FtContext;

/* ---- context: ferrotensor-backend/src/context.rs:164-237 (new), :373-397 (flush,
 * synchronize).  `stream` is a cudaStream_t to enqueue on (cudaStreamLegacy, handle value 1,
 * names the legacy default stream), or NULL for a stream the context creates.  One context
 * per device, as in the reference; a process may hold contexts on several devices (kernel
 * attributes and occupancy limits are kept per device). */
int ft_ctx_create(int device_ordinal, void* stream, FtContext** out);
int ft_ctx_destroy(FtContext* ctx);
int ft_ctx_flush(FtContext* ctx);        /* no-op: a stream needs no submit            */
int ft_ctx_synchronize(FtContext* ctx);  /* waits; returns FT_ERR_DEVICE if a kernel failed */
int ft_ctx_status(FtContext* ctx, int* device_status); /* non-blocking read of the status word */
/* Diagnostics: the 16 status words kernels write to pinned host memory ([0..3] status of a
 * failed bounded wait; [4..15] progress markers, recorded only by a library built with
 * -DFT_DEBUG_MARKERS and with FT_GEMM_DEBUG=1 in the environment at context creation).
 * Makes no CUDA call, so it works after a device fault. */
int ft_ctx_debug_words(FtContext* ctx, int* out16);
/* Timing of the tensor-core GEMM launches with CUDA events on the launch stream.  While
 * enabled every launch is bracketed by two events; ft_ctx_profile_read waits for the stream,
 * returns the summed kernel time, the algorithmic FLOPs (2 M N K per launch) and the launch
 * count since the previous read, and resets them. */
int ft_ctx_profile(FtContext* ctx, int enable);   /* 0 off, 1 GEMM launches, 2 every launch by name */
/* After ft_ctx_profile(ctx, 2): one line "kernel launches total_ms" per kernel name for all
 * launches since the last report (CUDA events on the launch stream); waits for the stream. */
int ft_ctx_profile_report(FtContext* ctx, char* buf, size_t cap);
int ft_ctx_profile_read(FtContext* ctx, double* gemm_ms, double* gemm_flops,
                        uint64_t* gemm_launches);
/* The part of that interval spent in GEMM launches whose epilogue also does elementwise work of
 * the step (RoPE of q|k|v, SwiGLU forward or backward): time, FLOPs and count; call it before
 * ft_ctx_profile_read, which closes the interval. */
int ft_ctx_profile_read_fused(FtContext* ctx, double* ms, double* flops, uint64_t* launches);
/* Algorithmic bytes (operands read once, results written once) of the GEMM launches timed since
 * the last call; call it before ft_ctx_profile_read, which closes the same interval. */
int ft_ctx_profile_bytes(FtContext* ctx, double* gemm_bytes);
int ft_ctx_set_gemm_mode(FtContext* ctx, int mode);    /* FT_GEMM_*; default FT_GEMM_F32 */
/* Tuning/diagnostics: force the tensor-core GEMM's output tile height (128 or 256 rows, 512 = 256 x 256
 * tiles on CTA pairs;
 * 0 = choose per shape, the default; FT_GEMM_TILE_M in the environment sets the initial value). */
int ft_ctx_set_gemm_tile_m(FtContext* ctx, int rows);
int ft_ctx_launch_count(FtContext* ctx, uint64_t* kernels_launched);
const char* ft_last_error(void);
/* Lists, one name per line, every kernel family compiled into the library. */
const char* ft_build_info(void);

/* ---- tensors: ferrotensor-backend/src/tensor.rs:157-406 (UnifiedTensor::{new, empty,
 * zeros, from_f32_as_f16, from_f32_transposed, to_vec, write_data}). */
int ft_tensor_alloc(FtContext* ctx, size_t bytes, void** dev_ptr);
int ft_tensor_free(FtContext* ctx, void* dev_ptr);
int ft_tensor_zero(FtContext* ctx, void* dev_ptr, size_t bytes);
int ft_upload(FtContext* ctx, void* dst_dev, const void* src_host, size_t bytes);
int ft_download(FtContext* ctx, void* dst_host, const void* src_dev, size_t bytes);
/* n f32 values on the host -> packed binary16 (round to nearest even) on the device. */
int ft_upload_f32_as_f16(FtContext* ctx, void* dst_dev, const float* src_host, size_t n);
/* host f32 [rows, cols] -> device [cols, rows]; as_f16 != 0 also rounds to binary16
 * (tensor.rs:385-406: how a Hugging Face [out, in] weight becomes the [in, out] operand). */
int ft_upload_f32_transposed(FtContext* ctx, void* dst_dev, const float* src_host,
                             size_t rows, size_t cols, int as_f16);
/* device-side forms of the two conversions (src already on the device, f32) */
int ft_convert_f32_to_f16(FtContext* ctx, const float* src, void* dst, size_t n);
int ft_transpose_f32(FtContext* ctx, const float* src, void* dst, size_t rows, size_t cols,
                     int as_f16);

/* ---- matmul: ferrotensor-backend/src/engine/matmul.rs:94-156.
 * out[M,N] = a[M,K] b[K,N] | a[M,K] b[N,K]^T | a[K,M]^T b[K,N]; *_f16b: b is packed f16. */
int ft_matmul(FtContext* ctx, const float* a, const float* b, float* out, int M, int K, int N);
int ft_matmul_bt(FtContext* ctx, const float* a, const float* b, float* out, int M, int K, int N);
int ft_matmul_at(FtContext* ctx, const float* a, const float* b, float* out, int M, int K, int N);
int ft_matmul_f16b(FtContext* ctx, const float* a, const void* b_f16, float* out, int M, int K,
                   int N);
int ft_matmul_bt_f16b(FtContext* ctx, const float* a, const void* b_f16, float* out, int M,
                      int K, int N);

/* ---- rope: engine/attention.rs:21-83, shaders/kernels.wgsl:45-73.  In place on
 * n_elems f32 laid out [tokens, heads, head_dim]; token t sits at position
 * pos + (t % seq_len); pairs (x[i], x[i + head_dim/2]); inverse != 0 rotates by the
 * negated angle (the backward pass). */
int ft_rope_theta(FtContext* ctx, float* x, size_t n_elems, int head_dim, int seq_len,
                  int heads, int pos, float theta, int inverse);

/* ---- RMSNorm: engine/norm.rs:20-99, kernels.wgsl:76-151. */
int ft_rms_norm_eps(FtContext* ctx, const float* x, const float* w, float* out, int rows,
                    int size, float eps);
/* gx[rows,size] and gw[size] are both written (gw may be NULL when the norm is frozen). */
int ft_rms_norm_backward(FtContext* ctx, const float* x, const float* w, const float* g,
                         float* gx, float* gw, int rows, int size, float eps);

/* No counterpart in the reference.  ft_rms_norm_backward for hosts that cannot allocate
 * device memory during a call (all memory already handed to their own pool, an embedding
 * program's memory cap, a loop where a cudaMalloc stall is not acceptable): same arguments,
 * results equal to ft_rms_norm_backward's to rounding (the kernel choice can differ), but the
 * per-row scratch lives in a fixed 2 MiB array inside the library image
 * (held by every GPU that loads the library until the process exits) and the call makes no
 * cudaMalloc/cudaFree.  Limit: with gw != NULL, rows rounded up to 64 plus size must not
 * exceed 524288 floats; larger shapes are rejected with FT_ERR_INVALID.  The first call on a
 * device resolves the array's address - make that call before any stream capture.  All
 * calls share the one array, which keeps the previous call's contents (every word read is
 * first rewritten, so nothing needs clearing); calls that overlap on the GPU (different
 * streams or contexts of one device) race on it. */
int ft_rms_norm_backward_noalloc(FtContext* ctx, const float* x, const float* w, const float* g,
                                 float* gx, float* gw, int rows, int size, float eps);

/* ---- elementwise: engine/elementwise.rs:8-17,57-75,183-215; engine/training.rs:189-205;
 * engine/mod.rs:399-428 (copy_tensor). */
int ft_add(FtContext* ctx, const float* a, const float* b, float* out, size_t n);
int ft_add_backward(FtContext* ctx, const float* g, float* ga, float* gb, size_t n);
int ft_gradient_scale(FtContext* ctx, float* x, size_t n, float scale);
int ft_copy(FtContext* ctx, const void* src, void* dst, size_t dst_offset_bytes, size_t bytes);
/* out = silu(a) * b: the FIRST operand passes through SiLU (the model passes the gate
 * projection first, ferrotensor-graph/src/lib.rs:504-510). */
int ft_silu_gate_fused(FtContext* ctx, const float* a, const float* b, float* out, size_t n);
int ft_silu_gate_backward(FtContext* ctx, const float* a, const float* b, const float* g,
                          float* ga, float* gb, size_t n);

/* ---- attention: engine/attention.rs:139-255 (forward, with stats), :312-441 (backward),
 * :515-594 (parameter block and AttentionOptions).  q, out, dout, dq are
 * [batch, seq_q, heads, head_dim]; k, v, dk, dv are [batch, seq_k, kv_heads, head_dim].
 * stats (may be NULL) has 2 f32 per (batch, head, query) row: element 2*row+1 receives
 * the row's log-sum-exp in the forward pass, element 2*row is backward scratch (Delta).
 * The backward pass recomputes the log-sum-exp when stats is NULL or lse_saved == 0.
 * mask (may be NULL) is added to the scaled score of every visible (query, key) pair:
 * element b*mask_stride[0] + h*mask_stride[1] + q*mask_stride[2] + k*mask_stride[3], a stride
 * of 0 broadcasting that dimension (attention.rs:596-620); a score at or below -1e30 after the
 * addition counts as hidden (flash_attention_v2.wgsl:32-33).
 * dropout_prob > 0 multiplies the weight of pair (b*heads + h, q, k) by 0 or 1/(1 - p), decided
 * by the hash of flash_attention_v2.wgsl:68-104 on the 64-bit seed; the log-sum-exp stays that
 * of the undropped scores and the backward pass regenerates the same decisions.  Masks and
 * dropout run on the exact f32 kernels whatever the GEMM mode. */
typedef struct FtAttnParams {
  uint32_t batch, heads, seq_q, seq_k, head_dim, kv_heads;
  uint32_t causal;        /* hide keys after the query's absolute position           */
  uint32_t causal_offset; /* absolute position of query 0                            */
  uint32_t window;        /* sliding window in tokens; 0 = unlimited                 */
  float scale;            /* 0 => 1/sqrt(head_dim)                                   */
  float dropout_prob;     /* 0 = none                                                */
  uint32_t lse_saved;     /* backward only: stats already holds the forward's LSE    */
  uint32_t seed_lo, seed_hi;   /* the two halves of the 64-bit dropout seed           */
  uint32_t mask_stride[4];     /* elements per step of batch, head, query, key        */
} FtAttnParams;
int ft_flash_attention_v2(FtContext* ctx, const float* q, const float* k, const float* v,
                          float* out, float* stats, const float* mask, const FtAttnParams* p);
int ft_flash_attention_v2_backward(FtContext* ctx, const float* q, const float* k,
                                   const float* v, const float* out, const float* dout,
                                   float* dq, float* dk, float* dv, float* stats,
                                   const float* mask, const FtAttnParams* p);

/* ---- loss: engine/training.rs:207-258, kernels.wgsl:672-711.  Per row:
 * row_loss = logZ - logit[target]; grad = (softmax - onehot) * weights[row];
 * target == FT_MASKED_CE_SKIP => zero loss and gradient. */
int ft_masked_cross_entropy_weighted(FtContext* ctx, const float* logits,
                                     const uint32_t* targets, const float* weights, float* grad,
                                     float* row_loss, int rows, int vocab);

/* ---- optimizer side: engine/training.rs:15-32,54-77,161-171,263-290;
 * kernels.wgsl:355-387,661-670,713-735. */
typedef struct FtAdamParams {
  float lr, beta1, beta2, eps, weight_decay, t;
  float _pad[2];
} FtAdamParams;
/* writes ceil(n/4096) chunk sums to out[offset ...]; *chunks_written receives that count */
int ft_sum_squares_partial(FtContext* ctx, const float* x, size_t n, float* out, size_t offset,
                           size_t* chunks_written);
int ft_clip_grad_by_norm(FtContext* ctx, float* g, size_t n, float scale);
int ft_adamw_update(FtContext* ctx, float* w, const float* g, float* m, float* v, size_t n,
                    const FtAdamParams* p);

/* engine/misc.rs:20-34 argmax_rows: for each of `rows` rows of `len` f32 values, the index of
 * the largest in f32::total_cmp order, the last index winning ties (a greedy token). */
int ft_argmax_rows(FtContext* ctx, const float* x, uint32_t* out_idx, int rows, int len);

/* ---- embedding rows: ferrotensor-autograd/src/lib.rs:1159-1179 (a host loop in the
 * reference).  out[t,:] = table[ids[t],:]; ids[t] >= vocab gives a zero row. */
int ft_embedding_gather(FtContext* ctx, const float* table, const uint32_t* ids, float* out,
                        int tokens, int vocab, int hidden);

/* =====================================================================================
 * Fused step: one object that runs the reference's whole LoRA step
 * (ferrotensor-trainer/src/lib.rs:426-502 train_chunk, :296-360 apply_gradients;
 * ferrotensor-graph/src/lfm.rs:116-139,597-623; ferrotensor-graph/src/lib.rs:112-142)
 * as a fixed sequence of the kernels above plus fused forms of them.  It has no
 * counterpart function in the reference: it is the composition its autograd tape
 * performs, with the same results.
 * ===================================================================================== */
typedef struct FtLoraModel FtLoraModel;

/* indices of the seven block linears, in the reference's order */
enum { FT_Q = 0, FT_K, FT_V, FT_O, FT_GATE, FT_UP, FT_DOWN, FT_LINEARS };

typedef struct FtModelConfig {
  int vocab, hidden, layers, heads, kv_heads, head_dim, ffn;
  float eps, theta;
  int qkv_bias;          /* q/k/v projections carry a bias (Qwen2)                     */
  int lora_rank;         /* 0 = no adapters                                            */
  float lora_alpha;
  int lora_mask;         /* bit i set => block linear i carries an adapter             */
  int lora_head;         /* lm_head carries an adapter                                 */
  int f16_base;          /* frozen linears and the head are stored as f16              */
  int checkpoint_blocks; /* keep only block inputs, replay each block in backward      */
  float attention_dropout; /* config.json attention_dropout (model_builder.rs:541); > 0
                            * keeps attention on the exact f32 kernels                  */
} FtModelConfig;

int ft_model_create(FtContext* ctx, const FtModelConfig* cfg, FtLoraModel** out);
int ft_model_destroy(FtLoraModel* m);
/* Number of trainable f32 values, and the offset of each adapter tensor inside the flat
 * parameter / gradient / moment buffers.  Order: sorted by the reference's parameter name
 * is NOT used; the flat order is layer-major, then linear index, A before B, then lm_head.
 * layer == -1 addresses the lm_head adapter. */
int ft_model_trainable_count(FtLoraModel* m, size_t* n);
int ft_model_adapter_offset(FtLoraModel* m, int layer, int linear, int which_b, size_t* offset,
                            int* rows, int* cols);
/* Frozen weights.  `embed` f32 [vocab, hidden]; norms f32; every linear is given in the
 * reference's device layout [in, out] (f32, or packed f16 when cfg.f16_base); biases f32.
 * head may alias nothing: for tied models pass the separate [hidden, vocab] copy the
 * reference's builder makes (model_builder.rs:653-689).  Pointers are borrowed. */
int ft_model_set_embedding(FtLoraModel* m, const float* embed, const float* final_norm,
                           const void* head_in_out);
int ft_model_set_layer(FtLoraModel* m, int layer, const float* norm1, const float* norm2,
                       const void* const linears_in_out[FT_LINEARS],
                       const float* const biases[3]);
/* Flat trainable state, each `trainable_count` f32: parameters, gradients, m, v. */
int ft_model_set_state(FtLoraModel* m, float* params, float* grads, float* adam_m,
                       float* adam_v);
/* Called once after the weights are set (and again if they change): builds the operand
 * copies the tensor-core path wants (transposed f16 weights, fused q|k|v and gate|up). */
int ft_model_prepare(FtLoraModel* m);
/* Tell the model that the caller wrote the flat parameter buffer directly (loading an
 * adapter): derived operand copies are rebuilt before the next micro-batch. */
int ft_model_params_changed(FtLoraModel* m);
/* Bytes of activation workspace a micro-batch of `sequences` x `seq_len` needs. */
int ft_model_workspace_bytes(FtLoraModel* m, int sequences, int seq_len, size_t* bytes);
int ft_model_set_workspace(FtLoraModel* m, void* dev_ptr, size_t bytes);

/* One micro-batch: embedding, blocks, head, masked CE, backward; LoRA gradients are ADDED
 * into the flat gradient buffer (zero it with ft_model_zero_grad at the window start).
 *   ids      u32 [sequences*seq_len] device
 *   targets  u32 [rows] device, FT_MASKED_CE_SKIP for unsupervised rows
 *   weights  f32 [rows] device, 1/tokens(sequence) or 0   (trainer/lib.rs:689-716)
 *   seed     upstream gradient of the loss, 1/grad_accum_steps (trainer/lib.rs:474)
 *   row_loss f32 [rows] device, receives each row's loss (0 for skipped rows)
 *   logits   f32 [rows, vocab] device or NULL; when given the logits are materialised
 *            there as the reference does, otherwise the head and the loss are fused. */
int ft_model_forward_backward(FtLoraModel* m, const uint32_t* ids, const uint32_t* targets,
                              const float* weights, int sequences, int seq_len, float seed,
                              float* row_loss, float* logits);
/* The seed of the next training pass's attention-dropout masks (models with
 * attention_dropout > 0; ferrotensor-trainer/src/lib.rs:185-197, :452-456).  Layer l draws its
 * masks from derive_seed([step_seed, l]) (ferrotensor-graph/src/dropout.rs:28-38); the backward
 * pass and a checkpointed block's replay regenerate them.  Evaluation applies no dropout. */
int ft_model_set_dropout_seed(FtLoraModel* m, uint64_t step_seed);
/* The forward half of ft_model_forward_backward: row losses (and logits when asked for) with
 * the same arguments, gradients untouched - what the reference's `evaluate` computes under
 * `no_grad` (ferrotensor-cli/src/main.rs:1111-1137). */
int ft_model_forward_loss(FtLoraModel* m, const uint32_t* ids, const uint32_t* targets,
                          const float* weights, int sequences, int seq_len, float* row_loss,
                          float* logits);
int ft_model_zero_grad(FtLoraModel* m);
/* After the (optional) cross-rank sum of the gradient buffer: g *= grad_scale (1/world),
 * global L2 norm on the device (4096-element f32 partials, summed in f64), skip when
 * non-finite, clip with max_norm/(norm + 1e-6) when norm > max_norm (max_norm <= 0: no
 * clipping), AdamW.  norm_out: device f32[4] (or NULL) = {norm, applied (1) or skipped (0), factor
 * applied to the raw gradient, unused}. */
int ft_model_apply_gradients(FtLoraModel* m, float grad_scale, float max_norm,
                             const FtAdamParams* p, float* norm_out);

/* =====================================================================================
 * Data parallelism: ferrotensor-trainer/src/distributed.rs:17-69 (FileGradSyncConfig: world
 * size, rank, max_wait), :107-185 (average_grads_file_sync), called from
 * Trainer::apply_gradients (ferrotensor-trainer/src/lib.rs:318-328) before the norm, the clip
 * and the optimizer.  The reference exchanges gradient files in a shared directory; here one
 * NCCL all-reduce of the model's flat gradient buffer runs on the context's stream over
 * NVLink.  NCCL is bound at run time (libnccl.so.2, or the path in FT_NCCL_LIB); a world of
 * one needs no NCCL.  Nothing here hangs the host: communicators are non-blocking and every
 * wait has a deadline, after which the communicator is aborted, the call returns FT_ERR_COMM
 * and every later call on it fails the same way (the reference returns "timed out waiting
 * for ..." after max_wait).
 * ===================================================================================== */
#define FT_COMM_ID_BYTES 128
typedef struct FtComm FtComm;
/* Rank 0 makes the 128-byte identifier of a new communicator and hands it to the other ranks
 * by any host-side channel (a file in the sync directory, a TCP store, an environment variable). */
int ft_comm_unique_id(void* id_out);
/* Joins `rank` of `world_size` (one process per GPU; ctx's device is the rank's GPU).  Rejects
 * world_size == 0 and rank >= world_size with the reference's messages (distributed.rs:36-44).
 * timeout_ms bounds this call and each later collective's set-up.  id may be NULL when
 * world_size == 1. */
int ft_comm_create(FtContext* ctx, int world_size, int rank, const void* id, int timeout_ms,
                   FtComm** out);
int ft_comm_destroy(FtComm* comm);
int ft_comm_info(FtComm* comm, int* world_size, int* rank);
/* buf[i] = sum over ranks of buf[i], n f32 on the device, enqueued on the context's stream. */
int ft_comm_allreduce_sum(FtComm* comm, float* buf, size_t n);
/* Waits (host) until the last collective enqueued has finished on the device, at most
 * timeout_ms (0 = the communicator's own limit).  On expiry the communicator is aborted, which
 * ends the waiting kernel, and FT_ERR_COMM is returned: how a rank learns that a peer never
 * entered the collective. */
int ft_comm_wait(FtComm* comm, int timeout_ms);
/* Trainer::apply_gradients for `world_size` ranks (lib.rs:318-358): sum of the flat gradient
 * buffer over the ranks, then ft_model_apply_gradients with grad_scale = 1/world_size, so every
 * rank performs the identical update.  comm == NULL means a single rank. */
int ft_model_allreduce_apply_gradients(FtLoraModel* m, FtComm* comm, float max_norm,
                                       const FtAdamParams* p, float* norm_out);

#ifdef __cplusplus
}
#endif
#endif /* FT_CUDA_H */
