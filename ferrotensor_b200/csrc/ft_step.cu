// The LoRA step driver: embedding -> blocks -> head -> masked CE -> backward -> LoRA
// gradients, and the norm/clip/AdamW tail, as one fixed kernel sequence on the context's
// stream.  It performs the composition the reference's autograd tape performs
// (ferrotensor-graph/src/lfm.rs:116-139,597-623; ferrotensor-graph/src/lib.rs:112-142;
// ferrotensor-autograd/src/lib.rs:256-290,509-595,725-749,1328-1390;
// ferrotensor-trainer/src/lib.rs:296-360,426-502) without a tape: frozen base weights get
// an input gradient only, adapters get dA/dB added into one flat gradient buffer.
//
// Linears that share an input are computed as a group into one wide buffer
// (q|k|v -> [T, nq+2nkv], gate|up -> [T, 2F]); attention, RoPE and SwiGLU read their slices
// through leading dimensions, so no slice is ever copied.
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "ft_common.cuh"

namespace {

struct Linear {
  int in = 0, out = 0;
  const void* w_io = nullptr;  // [in, out] f32 or f16 (borrowed)
  const float* bias = nullptr;
  bool lora = false;
  size_t a_off = 0, b_off = 0; // offsets of A [in, r] and B [r, out] in the flat buffers
};

struct Group {
  int in = 0, n = 0;           // input width, total output width
  int nlin = 0;
  Linear* lin[3] = {nullptr, nullptr, nullptr};
  int col_off[3] = {0, 0, 0};
  int r_off[3] = {0, 0, 0};
  int R = 0;                   // total adapter rank in the group
  // operand copies for the tensor-core path (owned unless they alias w_io)
  __half* w_nk = nullptr;      // [n, in]   forward operand, K = in contiguous
  __half* w_kn = nullptr;      // [in, n]   input-gradient operand, K = n contiguous
  bool own_kn = false;
  // f16 operand forms of the group's adapters, rebuilt whenever the parameters change.
  // RP = 64: the group's total rank padded to one 128-byte swizzle row.
  __half* a_catT16 = nullptr;  // [64, in]  (x . A) product:        N = 64, K = in
  __half* b_bdT16 = nullptr;   // [n, 64]   forward tail operand:   N = n,  K = 64 (block diagonal)
  __half* b_bd16 = nullptr;    // [64, n]   (dY . B^T) product:     N = 64, K = n
  __half* a_cat16 = nullptr;   // [in, 64]  backward tail operand:  N = in, K = 64
  float* bias_cat = nullptr;   // [n] concatenated biases, or NULL
  bool tc_lora = false;        // adapters ride on the tensor-core path
  // gate|up on the fused path: the group's columns are interleaved in runs of 32 (gate 0..31,
  // up 0..31, gate 32..63, ...), so that a thread of a GEMM epilogue, which holds 64 adjacent
  // columns of a row, has the gate and the up value of 32 features: SwiGLU and its backward run
  // inside the projections' epilogues.  Column c of linear j sits at (c / 32) * 64 + 32 j + c % 32.
  // The interleaved operand copies exist beside the plain ones (which the unfused modes use).
  bool il = false;
  __half* w_nk_il = nullptr;   // [n, in] rows interleaved
  __half* w_kn_il = nullptr;   // [in, n] columns interleaved
  const __half* fwd_w() const { return il ? w_nk_il : w_nk; }
  const __half* bwd_w() const { return il ? w_kn_il : w_kn; }
};

constexpr int RP = 64;

struct Layer {
  const float* norm1 = nullptr;
  const float* norm2 = nullptr;
  Linear lin[FT_LINEARS];
  Group qkv, o, gu, down;
};

// activations one block keeps for its backward pass
struct BlockActs {
  float *h1, *qkv, *attn, *stats, *x1, *h2, *gu, *f;
  float *xa_qkv, *xa_o, *xa_gu, *xa_down;
  // fused tensor-core path: GEMM inputs are kept as f16 only
  __half *h1_16, *qkv16, *attn16, *h2_16, *f_16, *gu16;
  __half *xa16_qkv, *xa16_o, *xa16_gu, *xa16_down;
};

struct Bump {
  char* base;
  size_t off = 0;
  bool dry;
  template <typename T>
  T* take(size_t count) {
    size_t bytes = ft_align_up(count * sizeof(T), 256);
    T* p = dry ? nullptr : (T*)(base + off);
    off += bytes;
    return p;
  }
};

}  // namespace

struct FtLoraModel {
  FtContext* ctx = nullptr;
  FtModelConfig cfg;
  int nq = 0, nkv = 0;
  float scale = 0.f;  // alpha / rank
  const float* embed = nullptr;
  const float* final_norm = nullptr;
  Linear head_lin;
  Group head;
  std::vector<Layer> layers;
  size_t trainable = 0;
  float *params = nullptr, *grads = nullptr, *adam_m = nullptr, *adam_v = nullptr;
  bool prepared = false;
  std::vector<void*> owned;  // operand copies to free
  void* ws = nullptr;
  size_t ws_bytes = 0;
  float* apply_scratch = nullptr;  // partials + norm_out (owned)

  // planned pointers of the current micro-batch
  int T = 0, sequences = 0, seq_len = 0, head_chunk = 0;
  std::vector<float*> x;           // layers+1 residual-stream buffers
  std::vector<BlockActs> acts;     // one per layer, or a single shared one when checkpointing
  float *hN = nullptr, *xa_head = nullptr, *logit_chunk = nullptr;
  float *dx = nullptr, *dh = nullptr, *dqkv = nullptr, *dattn = nullptr, *dgu = nullptr,
        *df = nullptr, *g = nullptr;
  __half *cvt_hi = nullptr, *cvt_lo = nullptr;
  size_t cvt_elems = 0;
  bool plan_fused = false;         // the planned workspace is the fused tensor-core layout
  __half *hN16 = nullptr, *xa16_head = nullptr, *g16 = nullptr;
  bool packs_dirty = true;         // adapter operand forms must be rebuilt before use
  void* pack_jobs = nullptr;       // device table of the groups' packing jobs (k_pack_adapters)
  int n_pack_jobs = 0;
  size_t pack_most = 0;            // elements of the largest operand form
  bool tc_attention = false;       // head_dim 64: attention and RoPE take the tensor-core route
  uint64_t dropout_step_seed = 0;  // seed of the coming forward pass (ft_model_set_dropout_seed)
  bool dropout_on = false;         // training pass of a model with attention dropout
  float* rope_table = nullptr;     // {cos, sin} [seq_len, 32], then transposed [32, seq_len], in the workspace
  const float* rope_tableT() const { return rope_table + (size_t)seq_len * cfg.head_dim; }
  int table_seq = 0;
  int* gu_amax = nullptr;          // per layer: largest |gate| or |up| of the forward pass
  // Carried scales of the backward pass.  A gradient that a kernel writes as f16 needs its
  // power-of-two scale BEFORE its largest magnitude is known; it takes the scale from the
  // largest magnitude of the same gradient one step earlier in the pass (the residual-stream
  // gradient from its previous version, a block's df / dattn / dq|dk|dv from the block above),
  // which leaves 2^(16 - kCarryExp) of growth before f16 overflows (an overflow makes the
  // gradient norm non-finite and the step is skipped, never silently wrong).  The first of
  // each kind takes the two-pass route (f32 result, conversion with its own amax).
  // Slots: amax ints and {S, 1/S, 2^-11/S} floats, zeroed at the start of every backward pass.
  int* carry_amax = nullptr;
  float* carry_scales = nullptr;
  bool rope_in_gemm = false;       // the q|k|v projection's epilogue applies RoPE (FT_CARRY bit 16)
  int carry_mask = 0;              // FT_CARRY bits: 1 residual stream, 2 df, 4 dattn, 8 dq|dk|dv,
                                   // 128 SwiGLU backward / 256 SwiGLU forward in GEMM epilogues
  __half *dx16 = nullptr, *df16 = nullptr, *dattn16 = nullptr, *dgu16 = nullptr;
  int carry_slots() const { return 6 * cfg.layers + 1; }
  int slot_dgu(int l) const { return 5 * cfg.layers + 1 + l; }   // scales only
  int slot_dx(int k) const { return k; }                                  // k = 0 .. 2L
  int slot_df(int l) const { return 2 * cfg.layers + 1 + l; }
  int slot_dattn(int l) const { return 3 * cfg.layers + 1 + l; }
  int slot_dqkv(int l) const { return 4 * cfg.layers + 1 + l; }
  int* camax(int slot) const { return carry_amax + slot; }
  float* cscales(int slot) const { return carry_scales + 4 * (size_t)slot; }
};
constexpr int kCarryExp = 7;   // carried scales aim the earlier amax at [2^6, 2^7)

namespace {

FtDType base_type(const FtLoraModel* m) { return m->cfg.f16_base ? FT_F16 : FT_F32; }
bool use_tc(const FtLoraModel* m) { return m->ctx->gemm_mode != FT_GEMM_F32 && m->cfg.f16_base; }
// The fused path (f16 activations, adapters inside the GEMMs) needs every group on the tensor
// cores; the split mode keeps the unfused route, which holds activations in f32.
bool use_fused(const FtLoraModel* m) {
  if (m->ctx->gemm_mode != FT_GEMM_F16 || !m->cfg.f16_base) return false;
  for (const auto& ly : m->layers)
    for (const Group* g : {&ly.qkv, &ly.o, &ly.gu, &ly.down})
      if (!g->w_nk || (g->R > 0 && !g->tc_lora)) return false;
  return m->head.w_nk && (m->head.R == 0 || m->head.tc_lora) && (m->cfg.ffn % 8) == 0;
}

void setup_group(Group& g, std::initializer_list<Linear*> lins, int rank) {
  g = Group();
  int col = 0, r = 0;
  for (Linear* l : lins) {
    g.lin[g.nlin] = l;
    g.col_off[g.nlin] = col;
    g.r_off[g.nlin] = r;
    col += l->out;
    if (l->lora) r += rank;
    g.in = l->in;
    g.nlin++;
  }
  g.n = col;
  g.R = r;
}

// ---- plan the workspace: the same walk sizes it (dry) and assigns pointers ----------------
size_t plan(FtLoraModel* m, int sequences, int seq_len, bool dry, void* base) {
  const FtModelConfig& c = m->cfg;
  const size_t T = (size_t)sequences * seq_len;
  Bump b{(char*)base, 0, dry};
  const int L = c.layers;
  const int nqkv = m->nq + 2 * m->nkv;
  const bool fused = use_fused(m);
  // (attention dropout is served by the exact f32 kernels only)
  const bool tc_attention = fused && c.head_dim == 64 && (nqkv % 8) == 0 && (m->nq % 64) == 0 &&
                            (long long)sequences * c.heads <= 65535 && c.attention_dropout == 0.f;
  std::vector<float*> x(L + 1);
  for (int l = 0; l <= L; ++l) x[l] = b.take<float>(T * c.hidden);
  // with attention on the tensor cores only the f16 q|k|v rows are kept per block: the f32
  // projection output is a scratch shared by all blocks and the f32 attention output is gone
  float* qkv_shared = tc_attention ? b.take<float>(T * nqkv) : nullptr;
  const int nact = c.checkpoint_blocks ? 1 : L;
  std::vector<BlockActs> acts(nact);
  for (int i = 0; i < nact; ++i) {
    const Layer& ly = m->layers[c.checkpoint_blocks ? 0 : i];
    BlockActs& a = acts[i];
    memset(&a, 0, sizeof(a));
    if (fused) {
      a.h1_16 = b.take<__half>(T * c.hidden);
      a.qkv = tc_attention ? qkv_shared : b.take<float>(T * nqkv);
      a.qkv16 = b.take<__half>(T * nqkv);
      a.attn = tc_attention ? nullptr : b.take<float>(T * m->nq);
      a.attn16 = b.take<__half>(T * m->nq);
      a.stats = b.take<float>((size_t)sequences * c.heads * seq_len * 2);
      a.x1 = b.take<float>(T * c.hidden);
      a.h2_16 = b.take<__half>(T * c.hidden);
      a.gu16 = b.take<__half>(T * 2 * c.ffn);   // gate | up kept as f16 only
      a.f_16 = b.take<__half>(T * c.ffn);
      a.xa16_qkv = b.take<__half>(T * RP);
      a.xa16_o = b.take<__half>(T * RP);
      a.xa16_gu = b.take<__half>(T * RP);
      a.xa16_down = b.take<__half>(T * RP);
      continue;
    }
    a.h1 = b.take<float>(T * c.hidden);
    a.qkv = b.take<float>(T * nqkv);
    a.attn = b.take<float>(T * m->nq);
    a.stats = b.take<float>((size_t)sequences * c.heads * seq_len * 2);
    a.x1 = b.take<float>(T * c.hidden);
    a.h2 = b.take<float>(T * c.hidden);
    a.gu = b.take<float>(T * 2 * c.ffn);
    a.f = b.take<float>(T * c.ffn);
    // adapter ranks are the same in every layer (one lora_mask for the model)
    a.xa_qkv = b.take<float>(T * std::max(1, ly.qkv.R));
    a.xa_o = b.take<float>(T * std::max(1, ly.o.R));
    a.xa_gu = b.take<float>(T * std::max(1, ly.gu.R));
    a.xa_down = b.take<float>(T * std::max(1, ly.down.R));
  }
  float* hN = b.take<float>(T * c.hidden);
  // head + loss run in row chunks so that [rows, vocab] never exceeds ~1 GiB
  size_t per_row = (size_t)c.vocab * sizeof(float);
  size_t chunk = std::max<size_t>(128, ((size_t)1 << 30) / per_row / 128 * 128);
  chunk = std::min(chunk, T);
  float* xa_head = b.take<float>(T * std::max(1, m->head.R));
  float* logit_chunk = b.take<float>(chunk * c.vocab);
  float* dx = b.take<float>(T * c.hidden);
  float* dh = b.take<float>(T * c.hidden);
  float* dqkv = b.take<float>(T * nqkv);
  float* dattn = b.take<float>(T * m->nq);
  // (the fused path writes the gate|up gradient straight to f16)
  float* dgu = fused ? nullptr : b.take<float>(T * 2 * c.ffn);
  float* df = b.take<float>(T * c.ffn);
  int rmax = std::max({m->layers[0].qkv.R, m->layers[0].o.R, m->layers[0].gu.R,
                       m->layers[0].down.R, m->head.R, 1});
  float* g = b.take<float>(T * rmax);
  // f16 staging of a GEMM's activation operand (widest: gate|up gradient or vocab chunk)
  size_t widest = std::max<size_t>({(size_t)c.hidden, (size_t)nqkv, (size_t)2 * c.ffn});
  size_t cvt = std::max(T * ft_align_up(widest, 8), chunk * ft_align_up((size_t)c.vocab, 8));
  __half* hi = b.take<__half>(cvt);
  __half* lo = fused ? nullptr : b.take<__half>(cvt);
  float* rope_table = fused ? b.take<float>(2 * (size_t)seq_len * c.head_dim) : nullptr;
  __half* hN16 = fused ? b.take<__half>(T * c.hidden) : nullptr;
  __half* xa16_head = fused ? b.take<__half>(T * RP) : nullptr;
  __half* g16 = fused ? b.take<__half>(T * RP) : nullptr;
  int* gu_amax = fused ? b.take<int>((size_t)L) : nullptr;
  int carry_mask = 0;
  if (tc_attention) {
    // FT_CARRY=<bits> (read whenever a workspace is planned) switches kinds off: 0 = every
    // gradient takes the two-pass route
    const char* env = getenv("FT_CARRY");
    const int env_mask = env ? atoi(env) : 511;
    if ((env_mask & 16) && ft_gemm_tc_pair_eligible(m->ctx, (int)T, nqkv) && (nqkv % 64) == 0 &&
        ((m->nq + m->nkv) % 64) == 0)
      carry_mask |= 16;
    if (c.hidden >= 1024 && c.hidden <= 4096 && (c.hidden % 8) == 0) carry_mask |= 1;
    if (ft_gemm_tc_pair_eligible(m->ctx, (int)T, c.ffn)) carry_mask |= 2;
    if (ft_gemm_tc_pair_eligible(m->ctx, (int)T, m->nq)) carry_mask |= 4 | 8;
    if (m->layers[0].gu.il && ft_gemm_tc_pair_eligible(m->ctx, (int)T, c.ffn)) carry_mask |= 128;
    if (m->layers[0].gu.il && ft_gemm_tc_pair_eligible(m->ctx, (int)T, 2 * c.ffn)) carry_mask |= 256;
    carry_mask &= env_mask;
  }
  int* carry_amax = fused ? b.take<int>((size_t)m->carry_slots()) : nullptr;
  float* carry_scales = fused ? b.take<float>(4 * (size_t)m->carry_slots()) : nullptr;
  __half* dx16 = (carry_mask & 1) ? b.take<__half>(T * c.hidden) : nullptr;
  __half* df16 = (carry_mask & 2) ? b.take<__half>(T * c.ffn) : nullptr;
  __half* dattn16 = (carry_mask & 4) ? b.take<__half>(T * m->nq) : nullptr;
  __half* dgu16 = (carry_mask & 128) ? b.take<__half>(T * 2 * c.ffn) : nullptr;
  if (!dry) {
    m->carry_amax = carry_amax; m->carry_scales = carry_scales; m->carry_mask = carry_mask;
    m->rope_in_gemm = (carry_mask & 16) != 0;
    m->dx16 = dx16; m->df16 = df16; m->dattn16 = dattn16; m->dgu16 = dgu16;
    m->gu_amax = gu_amax;
    m->plan_fused = fused; m->hN16 = hN16; m->xa16_head = xa16_head; m->g16 = g16;
    m->rope_table = rope_table; m->table_seq = 0;
    m->tc_attention = tc_attention;
    m->T = (int)T; m->sequences = sequences; m->seq_len = seq_len; m->head_chunk = (int)chunk;
    m->x = x; m->acts = acts; m->hN = hN; m->xa_head = xa_head; m->logit_chunk = logit_chunk;
    m->dx = dx; m->dh = dh; m->dqkv = dqkv; m->dattn = dattn; m->dgu = dgu; m->df = df; m->g = g;
    m->cvt_hi = hi; m->cvt_lo = lo; m->cvt_elems = cvt;
  }
  return b.off;
}

// ---- dense product through the selected path ---------------------------------------------
// Y[T, n] (ldy) = X[T, in] (ldx) . W for a whole group
int group_matmul_fwd(FtLoraModel* m, const Group& g, const float* X, long long ldx, float* Y,
                     long long ldy, int T) {
  FtContext* ctx = m->ctx;
  if (use_tc(m) && g.w_nk) {
    // activations are O(1): f16 holds them without scaling
    int r = ft_gemm_tc_f32a(ctx, X, ldx, m->cvt_hi, m->cvt_lo, g.w_nk, g.in, Y, ldy, T, g.n, g.in,
                            false, false);
    if (r != FT_ERR_UNSUPPORTED) return r;
  }
  for (int j = 0; j < g.nlin; ++j) {
    const Linear& l = *g.lin[j];
    FT_TRY(ft_gemm_simt(ctx, X, ldx, 1, l.w_io, base_type(m), l.out, 1, Y + g.col_off[j], ldy, T,
                        l.out, l.in, 1.f, false));
  }
  return FT_OK;
}

// dX[T, in] (=|+=) dY[T, n] (lddy) . W^T for a whole group
int group_matmul_bwd(FtLoraModel* m, const Group& g, const float* dY, long long lddy, float* dX,
                     long long lddx, int T, bool accumulate) {
  FtContext* ctx = m->ctx;
  if (use_tc(m) && g.w_kn) {
    // gradients are many orders of magnitude below f16's normal range: scale by a power of two
    int r = ft_gemm_tc_f32a(ctx, dY, lddy, m->cvt_hi, m->cvt_lo, g.w_kn, g.n, dX, lddx, T, g.in,
                            g.n, accumulate, true);
    if (r != FT_ERR_UNSUPPORTED) return r;
  }
  for (int j = 0; j < g.nlin; ++j) {
    const Linear& l = *g.lin[j];
    // B(k = output feature, n = input feature) = W[n, k]
    FT_TRY(ft_gemm_simt(ctx, dY + g.col_off[j], lddy, 1, l.w_io, base_type(m), 1, l.out, dX, lddx,
                        T, l.in, l.out, 1.f, accumulate || j > 0));
  }
  return FT_OK;
}

// Y = X W + (alpha/r) (X A) B + bias, for every linear of the group; xa keeps (alpha/r) X A
int linear_fwd(FtLoraModel* m, const Group& g, const float* X, long long ldx, float* Y,
               long long ldy, float* xa, int T) {
  FtContext* ctx = m->ctx;
  const int r = m->cfg.lora_rank;
  FT_TRY(group_matmul_fwd(m, g, X, ldx, Y, ldy, T));
  for (int j = 0; j < g.nlin; ++j) {
    const Linear& l = *g.lin[j];
    if (l.lora) {
      const float* A = m->params + l.a_off;
      const float* B = m->params + l.b_off;
      float* xaj = xa + g.r_off[j];
      FT_TRY(ft_gemm_simt(ctx, X, ldx, 1, A, FT_F32, r, 1, xaj, g.R, T, r, l.in, m->scale, false));
      FT_TRY(ft_gemm_simt(ctx, xaj, g.R, 1, B, FT_F32, l.out, 1, Y + g.col_off[j], ldy, T, l.out,
                          r, 1.f, true));
    }
    if (l.bias) FT_TRY(ft_k_add_bias(ctx, Y + g.col_off[j], ldy, l.bias, T, l.out));
  }
  return FT_OK;
}

// Adapter gradients (added into the flat buffer) and, when dX != NULL, the input gradient
// dX (=|+=) dY W^T + (alpha/r) (dY B^T) A^T.
int linear_bwd(FtLoraModel* m, const Group& g, const float* X, long long ldx, const float* dY,
               long long lddy, const float* xa, float* dX, long long lddx, int T,
               bool accumulate_dx) {
  FtContext* ctx = m->ctx;
  const int r = m->cfg.lora_rank;
  if (dX) FT_TRY(group_matmul_bwd(m, g, dY, lddy, dX, lddx, T, accumulate_dx));
  for (int j = 0; j < g.nlin; ++j) {
    const Linear& l = *g.lin[j];
    if (!l.lora) continue;
    const float* A = m->params + l.a_off;
    const float* B = m->params + l.b_off;
    const float* dYj = dY + g.col_off[j];
    const float* xaj = xa + g.r_off[j];
    float* gj = m->g;  // [T, r], pitch r
    // G = (alpha/r) dY B^T        B operand (k = out, n = r) = B[n, k]
    FT_TRY(ft_gemm_simt(ctx, dYj, lddy, 1, B, FT_F32, 1, l.out, gj, r, T, r, l.out, m->scale, false));
    // dB += ((alpha/r) X A)^T dY   [r, out], reduction over tokens
    FT_TRY(ft_gemm_simt(ctx, xaj, 1, g.R, dYj, FT_F32, lddy, 1, m->grads + l.b_off, l.out, r, l.out,
                        T, 1.f, true));
    // dA += X^T G                  [in, r], reduction over tokens
    FT_TRY(ft_gemm_simt(ctx, X, 1, ldx, gj, FT_F32, r, 1, m->grads + l.a_off, r, l.in, r, T, 1.f,
                        true));
    // dX += G A^T                  B operand (k = r, n = in) = A[n, k]
    if (dX)
      FT_TRY(ft_gemm_simt(ctx, gj, r, 1, A, FT_F32, 1, r, dX, lddx, T, l.in, r, 1.f, true));
  }
  return FT_OK;
}

// SplitMix64's finaliser and the seed of layer l for one forward pass
// (ferrotensor-graph/src/dropout.rs:17-38): derive_seed([step_seed, l]).
inline uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
inline uint64_t layer_seed(uint64_t step_seed, int l) {
  uint64_t acc = mix64(2);
  acc = mix64(acc ^ mix64(step_seed));
  return mix64(acc ^ mix64((uint64_t)l));
}
// training passes of a model with attention dropout: the layer's probability and seed
inline void fill_dropout(const FtLoraModel* m, int l, FtAttnParams& p) {
  if (!m->dropout_on) return;
  const uint64_t s = layer_seed(m->dropout_step_seed, l);
  p.dropout_prob = m->cfg.attention_dropout;
  p.seed_lo = (uint32_t)s;
  p.seed_hi = (uint32_t)(s >> 32);
}

int block_forward(FtLoraModel* m, int l, const float* x_in, float* x_out, BlockActs& a) {
  FtContext* ctx = m->ctx;
  const FtModelConfig& c = m->cfg;
  Layer& ly = m->layers[l];
  const int T = m->T, h = c.hidden, nq = m->nq, nkv = m->nkv, nqkv = nq + 2 * nkv, F = c.ffn;
  FT_TRY(ft_k_rms_norm(ctx, x_in, ly.norm1, a.h1, T, h, c.eps));
  FT_TRY(linear_fwd(m, ly.qkv, a.h1, h, a.qkv, nqkv, a.xa_qkv, T));
  FT_TRY(ft_k_rope(ctx, a.qkv, nqkv, T, c.heads, c.head_dim, m->seq_len, 0, c.theta, false));
  FT_TRY(ft_k_rope(ctx, a.qkv + nq, nqkv, T, c.kv_heads, c.head_dim, m->seq_len, 0, c.theta, false));
  FtAttnLaunch at;
  at.q = a.qkv; at.k = a.qkv + nq; at.v = a.qkv + nq + nkv;
  at.ldq = at.ldk = at.ldv = nqkv;
  at.out = a.attn; at.ldo = nq; at.stats = a.stats;
  memset(&at.p, 0, sizeof(at.p));
  at.p.batch = m->sequences; at.p.heads = c.heads; at.p.kv_heads = c.kv_heads;
  at.p.seq_q = at.p.seq_k = m->seq_len; at.p.head_dim = c.head_dim; at.p.causal = 1;
  fill_dropout(m, l, at.p);
  FT_TRY(ft_k_attention_fwd(ctx, at));
  FT_TRY(linear_fwd(m, ly.o, a.attn, nq, a.x1, h, a.xa_o, T));
  FT_TRY(ft_k_add(ctx, x_in, a.x1, a.x1, (size_t)T * h));
  FT_TRY(ft_k_rms_norm(ctx, a.x1, ly.norm2, a.h2, T, h, c.eps));
  FT_TRY(linear_fwd(m, ly.gu, a.h2, h, a.gu, 2 * F, a.xa_gu, T));
  FT_TRY(ft_k_silu_gate(ctx, a.gu, 2 * F, a.gu + F, 2 * F, a.f, F, T, F));
  FT_TRY(linear_fwd(m, ly.down, a.f, F, x_out, h, a.xa_down, T));
  FT_TRY(ft_k_add(ctx, a.x1, x_out, x_out, (size_t)T * h));
  return FT_OK;
}

// on entry m->dx = dL/d(x_out); on exit m->dx = dL/d(x_in) (undefined for layer 0)
int block_backward(FtLoraModel* m, int l, const float* x_in, BlockActs& a) {
  FtContext* ctx = m->ctx;
  const FtModelConfig& c = m->cfg;
  Layer& ly = m->layers[l];
  const int T = m->T, h = c.hidden, nq = m->nq, nkv = m->nkv, nqkv = nq + 2 * nkv, F = c.ffn;
  // x_out = x1 + down(f)
  FT_TRY(linear_bwd(m, ly.down, a.f, F, m->dx, h, a.xa_down, m->df, F, T, false));
  FT_TRY(ft_k_silu_gate_bwd(ctx, a.gu, 2 * F, a.gu + F, 2 * F, m->df, F, m->dgu, 2 * F,
                            m->dgu + F, 2 * F, T, F));
  FT_TRY(linear_bwd(m, ly.gu, a.h2, h, m->dgu, 2 * F, a.xa_gu, m->dh, h, T, false));
  FT_TRY(ft_k_rms_norm_bwd(ctx, a.x1, ly.norm2, m->dh, m->dx, nullptr, T, h, c.eps, true));
  // x1 = x_in + o(attn)
  FT_TRY(linear_bwd(m, ly.o, a.attn, nq, m->dx, h, a.xa_o, m->dattn, nq, T, false));
  FtAttnBwdLaunch ab;
  ab.q = a.qkv; ab.k = a.qkv + nq; ab.v = a.qkv + nq + nkv;
  ab.ldq = ab.ldk = ab.ldv = nqkv;
  ab.out = a.attn; ab.ldo = nq; ab.dout = m->dattn; ab.lddo = nq;
  ab.dq = m->dqkv; ab.dk = m->dqkv + nq; ab.dv = m->dqkv + nq + nkv;
  ab.lddq = ab.lddk = ab.lddv = nqkv;
  ab.stats = a.stats;
  memset(&ab.p, 0, sizeof(ab.p));
  ab.p.batch = m->sequences; ab.p.heads = c.heads; ab.p.kv_heads = c.kv_heads;
  ab.p.seq_q = ab.p.seq_k = m->seq_len; ab.p.head_dim = c.head_dim; ab.p.causal = 1;
  ab.p.lse_saved = 1;
  fill_dropout(m, l, ab.p);
  FT_TRY(ft_k_attention_bwd(ctx, ab));
  FT_TRY(ft_k_rope(ctx, m->dqkv, nqkv, T, c.heads, c.head_dim, m->seq_len, 0, c.theta, true));
  FT_TRY(ft_k_rope(ctx, m->dqkv + nq, nqkv, T, c.kv_heads, c.head_dim, m->seq_len, 0, c.theta, true));
  // The embedding output is frozen: layer 0 needs adapter gradients only.
  const bool need_dx = l > 0;
  FT_TRY(linear_bwd(m, ly.qkv, a.h1, h, m->dqkv, nqkv, a.xa_qkv, need_dx ? m->dh : nullptr, h, T,
                    false));
  if (need_dx)
    FT_TRY(ft_k_rms_norm_bwd(ctx, x_in, ly.norm1, m->dh, m->dx, nullptr, T, h, c.eps, true));
  return FT_OK;
}


// ======================================================================================
// Fused tensor-core path
// ======================================================================================

struct PackMeta {
  int nlin, in, n, r;
  int il;   // columns interleaved in runs of 32 (Group::il)
  int col_off[3], out[3], r_off[3], lora[3];
  unsigned long long a_off[3], b_off[3];
};

struct PackJob {
  PackMeta g;
  __half* out[4];  // a_catT16, b_bdT16, b_bd16, a_cat16
};

// Writes the four f16 operand forms of every group's adapters in one launch: blockIdx.z selects
// the group, blockIdx.y the form.
__global__ void k_pack_adapters(const float* __restrict__ params, const PackJob* __restrict__ jobs) {
  const PackJob& job = jobs[blockIdx.z];
  const PackMeta& g = job.g;
  const int which = blockIdx.y;
  __half* __restrict__ dst = job.out[which];
  const size_t total = (size_t)RP * (which == 0 || which == 3 ? g.in : g.n);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += st) {
    int rr, other;  // rr = padded rank index, other = input feature or output column
    if (which == 0 || which == 2) { rr = (int)(i / (which == 0 ? g.in : g.n)); other = (int)(i % (which == 0 ? g.in : g.n)); }
    else { other = (int)(i / RP); rr = (int)(i % RP); }
    float v = 0.f;
    if (which == 0 || which == 3) {
      for (int j = 0; j < g.nlin; ++j)
        if (g.lora[j] && rr >= g.r_off[j] && rr < g.r_off[j] + g.r)
          v = params[g.a_off[j] + (size_t)other * g.r + (rr - g.r_off[j])];
    } else if (g.il) {
      // interleaved group column -> (linear, its column)
      const int j = (other >> 5) & 1, col = ((other >> 6) << 5) + (other & 31);
      if (g.lora[j] && col < g.out[j] && rr >= g.r_off[j] && rr < g.r_off[j] + g.r)
        v = params[g.b_off[j] + (size_t)(rr - g.r_off[j]) * g.out[j] + col];
    } else {
      for (int j = 0; j < g.nlin; ++j)
        if (g.lora[j] && other >= g.col_off[j] && other < g.col_off[j] + g.out[j] &&
            rr >= g.r_off[j] && rr < g.r_off[j] + g.r)
          v = params[g.b_off[j] + (size_t)(rr - g.r_off[j]) * g.out[j] + (other - g.col_off[j])];
    }
    dst[i] = __float2half_rn(v);
  }
}

void pack_job_of(const FtLoraModel* m, const Group& g, PackJob* job) {
  memset(job, 0, sizeof(*job));
  PackMeta& pm = job->g;
  pm.nlin = g.nlin; pm.in = g.in; pm.n = g.n; pm.r = m->cfg.lora_rank;
  pm.il = g.il ? 1 : 0;
  for (int j = 0; j < g.nlin; ++j) {
    pm.col_off[j] = g.col_off[j]; pm.out[j] = g.lin[j]->out; pm.r_off[j] = g.r_off[j];
    pm.lora[j] = g.lin[j]->lora ? 1 : 0;
    pm.a_off[j] = g.lin[j]->a_off; pm.b_off[j] = g.lin[j]->b_off;
  }
  job->out[0] = g.a_catT16; job->out[1] = g.b_bdT16; job->out[2] = g.b_bd16; job->out[3] = g.a_cat16;
}

// The job table of all groups that keep f16 adapter forms, on the device (after prepare_group).
int build_pack_jobs(FtLoraModel* m) {
  std::vector<PackJob> jobs;
  size_t most = 0;
  auto add = [&](const Group& g) {
    if (!g.tc_lora) return;
    jobs.emplace_back();
    pack_job_of(m, g, &jobs.back());
    most = std::max(most, (size_t)RP * std::max(g.in, g.n));
  };
  for (auto& ly : m->layers) { add(ly.qkv); add(ly.o); add(ly.gu); add(ly.down); }
  add(m->head);
  m->pack_jobs = nullptr;
  m->n_pack_jobs = (int)jobs.size();
  m->pack_most = most;
  if (jobs.empty()) return FT_OK;
  FT_REQUIRE(jobs.size() <= 65535, "prepare: too many adapter groups");
  void* p = nullptr;
  FT_CUDA(cudaMalloc(&p, jobs.size() * sizeof(PackJob)));
  m->owned.push_back(p);
  FT_CUDA(cudaMemcpy(p, jobs.data(), jobs.size() * sizeof(PackJob), cudaMemcpyHostToDevice));
  m->pack_jobs = p;
  return FT_OK;
}

int pack_all(FtLoraModel* m) {
  if (m->n_pack_jobs > 0) {
    dim3 grid((unsigned)std::min<size_t>((m->pack_most + 255) / 256, 256), 4, (unsigned)m->n_pack_jobs);
    FT_LAUNCH(m->ctx, k_pack_adapters, grid, 256, 0, m->params, (const PackJob*)m->pack_jobs);
  }
  m->packs_dirty = false;
  return FT_OK;
}

// Y[T, n] = X16 . W + (alpha/r)(X16 . A) . B (+ bias) (+ residual); keeps xa16 = (alpha/r) X16 . A
int linear_fwd_fused(FtLoraModel* m, const Group& g, const __half* X16, float* Y, long long ldy,
                     __half* xa16, const float* residual, long long ldr, int T,
                     __half* Y16 = nullptr, const float* rope_table = nullptr, int rope_seq = 0,
                     int rope_cols = 0, __half* swi_f16 = nullptr, long long swi_ldf = 0,
                     int* amax_slot = nullptr) {
  FtContext* ctx = m->ctx;
  FtGemmArgs a;
  a.a = X16; a.lda = g.in; a.b = g.fwd_w(); a.ldb = g.in;
  a.M = T; a.N = g.n; a.K = g.in;
  if (g.R > 0) {
    // xa16 = (alpha/r) X16 . A is made by pre-tiles of the same launch
    a.a2 = xa16; a.lda2 = RP; a.b2 = g.b_bdT16; a.ldb2 = RP; a.K2 = RP; a.k2_used = g.R;
    a.pre_b = g.a_catT16; a.pre_ldb = g.in; a.pre_c16 = xa16; a.pre_ldc16 = RP; a.pre_alpha = m->scale;
  }
  a.c = Y; a.ldc = ldy; a.c16 = Y16; a.ldc16 = ldy;   // Y16: the result as f16 (pitch ldy)
  a.bias = g.bias_cat; a.residual = residual; a.ldr = ldr;
  a.rope_table = rope_table; a.rope_seq = rope_seq; a.rope_cols = rope_cols;
  a.swi_f16 = swi_f16; a.swi_ldf = swi_ldf; a.amax_slot = amax_slot;
  return ft_gemm_tc_ex(ctx, a);
}

// Adapter gradients (added to the flat buffer) and dX (=|+ residual) = dY W^T + G A^T.
// dY is rounded to f16 after a power-of-two scale S chosen from its largest magnitude; S is
// carried through G and removed by the epilogues (1/S is a device scalar).
// When dY16 is given, dY has already been converted (pitch lddy, scale in scales16).  With
// amax_on_dx the dX product also reports its largest magnitude for the conversion that follows.
// Where the input gradient's largest magnitude goes, and (with dX16) the f16 form that
// replaces the f32 result, written with a carried scale.
struct DxOut {
  int* amax_out = nullptr;
  __half* dX16 = nullptr; long long ld16 = 0;
  const int* carry_in = nullptr;
  float* carry_scales = nullptr;
  // SwiGLU backward inside the epilogue (FtGemmArgs::swi_dgu16): no input gradient is stored
  const __half* swi_gu16 = nullptr; long long swi_ldgu = 0;
  __half* swi_dgu16 = nullptr; long long swi_lddgu = 0;
  const int* swi_gu_amax = nullptr;
  float* swi_scales = nullptr;
  bool stores_f16() const { return dX16 != nullptr || swi_dgu16 != nullptr; }
};
// the next producer's largest magnitude goes to `slot` (zero since the pass began)
void arm_at(FtContext* ctx, int* slot) {
  ctx->amax_out = slot;
  ctx->amax_ready = false;
}

int linear_bwd_fused(FtLoraModel* m, const Group& g, const __half* X16, const float* dY,
                     long long lddy, const __half* xa16, float* dX, long long lddx,
                     const float* residual, long long ldr, int T, const __half* dY16 = nullptr,
                     const float* scales16 = nullptr, bool amax_on_dx = false,
                     const DxOut* dxo = nullptr) {
  FtContext* ctx = m->ctx;
  const int r = m->cfg.lora_rank;
  long long np = (long long)ft_align_up((size_t)g.n, 8);
  const float* scales = scales16;
  if (dY16) {
    np = lddy;
  } else {
    FT_TRY(ft_to_f16(ctx, dY, lddy, m->cvt_hi, nullptr, np, T, g.n, true, &scales, 8));
    dY16 = m->cvt_hi;
  }
  const float* inv_s = scales + 1;
  if (g.R > 0 && !dX && !(dxo && dxo->stores_f16())) {
    FtGemmArgs a;   // G16 = (alpha/r) * (S dY) . B^T
    a.a = dY16; a.lda = np; a.b = g.b_bd16; a.ldb = g.n;
    a.M = T; a.N = RP; a.K = g.n;
    a.c16 = m->g16; a.ldc16 = RP; a.alpha = m->scale;
    FT_TRY(ft_gemm_tc_ex(ctx, a));
  }
  if (dX || (dxo && dxo->stores_f16())) {
    FtGemmArgs a;
    a.a = dY16; a.lda = np; a.b = g.bwd_w(); a.ldb = g.n;
    a.M = T; a.N = g.in; a.K = g.n;
    if (g.R > 0) {
      // G16 = (alpha/r) * (S dY) . B^T is made by pre-tiles of the same launch
      a.a2 = m->g16; a.lda2 = RP; a.b2 = g.a_cat16; a.ldb2 = RP; a.K2 = RP; a.k2_used = g.R;
      a.pre_b = g.b_bd16; a.pre_ldb = g.n; a.pre_c16 = m->g16; a.pre_ldc16 = RP; a.pre_alpha = m->scale;
    }
    a.c = dX; a.ldc = lddx; a.alpha_ptr = inv_s; a.residual = residual; a.ldr = ldr;
    if (dxo) {
      a.amax_slot = dxo->amax_out;
      if (dxo->swi_dgu16) {
        a.c = nullptr;
        a.swi_gu16 = dxo->swi_gu16; a.swi_ldgu = dxo->swi_ldgu;
        a.swi_dgu16 = dxo->swi_dgu16; a.swi_lddgu = dxo->swi_lddgu;
        a.swi_gu_amax = dxo->swi_gu_amax; a.swi_scales = dxo->swi_scales;
        a.carry_amax = dxo->carry_in;
      } else if (dxo->dX16) {
        a.c = nullptr;
        a.c16 = dxo->dX16; a.ldc16 = dxo->ld16;
        a.carry_amax = dxo->carry_in; a.carry_exp = kCarryExp; a.carry_scales = dxo->carry_scales;
      }
    } else if (amax_on_dx) {
      FT_TRY(ft_amax_arm(ctx));
      a.want_amax = true;
    }
    FT_TRY(ft_gemm_tc_ex(ctx, a));
  }
  if (g.R > 0) {
    // one launch for both adapter gradients, each reduced over tokens:
    //   dB^T [n, 64] = (S dY)^T . xa16      dA [in, 64] = X16^T . G16
    // the slabs of the K splits are summed inside the launch and added to the flat buffer
    FtKoProblem pr[2];
    pr[0].a = dY16; pr[0].lda = np; pr[0].b = xa16; pr[0].ldb = RP; pr[0].M = g.n; pr[0].N = RP;
    pr[1].a = X16; pr[1].lda = g.in; pr[1].b = m->g16; pr[1].ldb = RP; pr[1].M = g.in; pr[1].N = RP;
    for (int j = 0; j < g.nlin; ++j) {
      const Linear& l = *g.lin[j];
      if (!l.lora) continue;
      FtKoSeg& sb = pr[0].seg[pr[0].nseg++];   // lora_b [r, out]
      sb.il_off = g.il ? 32 * j : -1;
      sb.out = m->grads + l.b_off; sb.m0 = g.col_off[j]; sb.mcount = l.out;
      sb.n0 = g.r_off[j]; sb.ncount = r; sb.som = 1; sb.son = l.out;
      FtKoSeg& sa = pr[1].seg[pr[1].nseg++];   // lora_a [in, r]
      sa.out = m->grads + l.a_off; sa.m0 = 0; sa.mcount = l.in;
      sa.n0 = g.r_off[j]; sa.ncount = r; sa.som = r; sa.son = 1;
    }
    // (summing the slabs inside the launch, by the last warp to finish each piece, was
    // measured slower than this second small launch: a long serial tail on few warps)
    FT_TRY(ft_gemm_tc_kouter_pair(ctx, 2, pr, T));
    FT_TRY(ft_slab_reduce_problems(ctx, 2, pr, inv_s, 1.f, true));
  }
  return FT_OK;
}

int attention_launch(FtLoraModel* m, int l, BlockActs& a, bool backward) {
  const FtModelConfig& c = m->cfg;
  const int nq = m->nq, nkv = m->nkv, nqkv = nq + 2 * nkv;
  FtAttnParams p;
  memset(&p, 0, sizeof(p));
  p.batch = m->sequences; p.heads = c.heads; p.kv_heads = c.kv_heads;
  p.seq_q = p.seq_k = m->seq_len; p.head_dim = c.head_dim; p.causal = 1;
  fill_dropout(m, l, p);
  if (!backward) {
    FtAttnLaunch at;
    at.q = a.qkv; at.k = a.qkv + nq; at.v = a.qkv + nq + nkv;
    at.ldq = at.ldk = at.ldv = nqkv;
    at.out = a.attn; at.ldo = nq; at.stats = a.stats; at.p = p;
    return ft_k_attention_fwd(m->ctx, at);
  }
  FtAttnBwdLaunch ab;
  ab.q = a.qkv; ab.k = a.qkv + nq; ab.v = a.qkv + nq + nkv;
  ab.ldq = ab.ldk = ab.ldv = nqkv;
  ab.out = a.attn; ab.ldo = nq; ab.dout = m->dattn; ab.lddo = nq;
  ab.dq = m->dqkv; ab.dk = m->dqkv + nq; ab.dv = m->dqkv + nq + nkv;
  ab.lddq = ab.lddk = ab.lddv = nqkv;
  ab.stats = a.stats;
  p.lse_saved = 1;
  ab.p = p;
  return ft_k_attention_bwd(m->ctx, ab);
}

int block_forward_fused(FtLoraModel* m, int l, const float* x_in, float* x_out, BlockActs& a) {
  FtContext* ctx = m->ctx;
  const FtModelConfig& c = m->cfg;
  Layer& ly = m->layers[l];
  const int T = m->T, h = c.hidden, nq = m->nq, nkv = m->nkv, nqkv = nq + 2 * nkv, F = c.ffn;
  FT_TRY(ft_k_rms_norm16(ctx, x_in, ly.norm1, nullptr, a.h1_16, T, h, c.eps));
  if (m->tc_attention && m->rope_in_gemm) {
    // the projection's epilogue rotates and rounds: no f32 q|k|v rows, no pass over them
    FT_TRY(linear_fwd_fused(m, ly.qkv, a.h1_16, nullptr, nqkv, a.xa16_qkv, nullptr, 0, T, a.qkv16,
                            m->rope_tableT(), m->seq_len, nq + nkv));
  } else {
    FT_TRY(linear_fwd_fused(m, ly.qkv, a.h1_16, a.qkv, nqkv, a.xa16_qkv, nullptr, 0, T));
  }
  if (m->tc_attention) {
    // RoPE (from the table) and the f16 rounding in one pass; attention on the tensor cores
    if (!m->rope_in_gemm)
      FT_TRY(ft_k_rope_to_f16(ctx, a.qkv, a.qkv16, nqkv, T, nq, nkv, m->seq_len, m->rope_table, false,
                              nullptr));
    FT_TRY(ft_attention_fwd_tc(ctx, a.qkv16, nqkv, 0, nq, nq + nkv, a.attn16, nq, nullptr, 0, a.stats,
                               m->sequences, m->seq_len, c.heads, c.kv_heads, c.head_dim));
  } else {
    FT_TRY(ft_k_rope(ctx, a.qkv, nqkv, T, c.heads, c.head_dim, m->seq_len, 0, c.theta, false));
    FT_TRY(ft_k_rope(ctx, a.qkv + nq, nqkv, T, c.kv_heads, c.head_dim, m->seq_len, 0, c.theta, false));
    FT_TRY(attention_launch(m, l, a, false));
    FT_TRY(ft_to_f16(ctx, a.attn, nq, a.attn16, nullptr, nq, T, nq, false, nullptr));
  }
  // x1 = x_in + o(attn): the residual rides in the GEMM epilogue
  FT_TRY(linear_fwd_fused(m, ly.o, a.attn16, a.x1, h, a.xa16_o, x_in, h, T));
  FT_TRY(ft_k_rms_norm16(ctx, a.x1, ly.norm2, nullptr, a.h2_16, T, h, c.eps));
  if (m->carry_mask & 256) {
    // SwiGLU in the gate|up projection's epilogue: gate|up and silu(gate) * up leave together
    FT_TRY(linear_fwd_fused(m, ly.gu, a.h2_16, nullptr, 2 * F, a.xa16_gu, nullptr, 0, T, a.gu16, nullptr,
                            0, 0, a.f_16, F, m->gu_amax + l));
  } else {
    FT_TRY(linear_fwd_fused(m, ly.gu, a.h2_16, nullptr, 2 * F, a.xa16_gu, nullptr, 0, T, a.gu16));
    FT_TRY(ft_k_silu_gate16h(ctx, a.gu16, 2 * F, a.f_16, F, T, F, m->gu_amax + l, ly.gu.il));
  }
  FT_TRY(linear_fwd_fused(m, ly.down, a.f_16, x_out, h, a.xa16_down, a.x1, h, T));
  return FT_OK;
}

int block_backward_fused(FtLoraModel* m, int l, const float* x_in, BlockActs& a) {
  FtContext* ctx = m->ctx;
  const FtModelConfig& c = m->cfg;
  Layer& ly = m->layers[l];
  const int T = m->T, h = c.hidden, nq = m->nq, nkv = m->nkv, nqkv = nq + 2 * nkv, F = c.ffn;
  const int L = c.layers;
  const bool top = l == L - 1;
  // m->dx is version k0 of the residual-stream gradient (0 = what the final norm left).  With
  // carried scales every later version also exists as f16 rows in m->dx16; version 0 is
  // converted by a pass of its own, from the amax its producer left in slot_dx(0).
  const int k0 = 2 * (L - 1 - l);
  const bool cdx = (m->carry_mask & 1) != 0;
  const bool cdf = (m->carry_mask & 2) != 0 && !top;
  const bool cda = (m->carry_mask & 4) != 0 && !top && m->tc_attention;
  auto dx16_of = [&](int k) { return cdx && k > 0 ? m->dx16 : nullptr; };
  auto dxs_of = [&](int k) { return cdx && k > 0 ? m->cscales(m->slot_dx(k)) : nullptr; };
  // norm backward producing version k + 1 from version k
  auto norm_bwd = [&](const float* x, const float* w, int k) -> int {
    if (cdx) {
      FtCarry cy;
      cy.amax_in = m->camax(m->slot_dx(k)); cy.exp = kCarryExp;
      cy.scales = m->cscales(m->slot_dx(k + 1)); cy.amax_out = m->camax(m->slot_dx(k + 1));
      return ft_k_rms_norm_bwd_carry(ctx, x, w, m->dh, m->dx, m->dx16, T, h, c.eps, cy);
    }
    arm_at(ctx, m->camax(m->slot_dx(k + 1)));
    return ft_k_rms_norm_bwd(ctx, x, w, m->dh, m->dx, nullptr, T, h, c.eps, true);
  };
  // The down projection's input gradient reports its amax; SwiGLU's backward bounds its own
  // output with it and writes the gate|up gradient as f16 operands in the same pass.
  const bool cswi = (m->carry_mask & 128) != 0 && !top;
  DxOut od;
  od.amax_out = m->camax(m->slot_df(l));
  if (cswi) {
    // SwiGLU's backward runs in this product's epilogue: d gate | d up leave as f16 operands,
    // the gradient of the SwiGLU output itself is never stored
    od.swi_gu16 = a.gu16; od.swi_ldgu = 2 * F;
    od.swi_dgu16 = m->dgu16; od.swi_lddgu = 2 * F;
    od.swi_gu_amax = m->gu_amax + l;
    od.swi_scales = m->cscales(m->slot_dgu(l));
    od.carry_in = m->camax(m->slot_df(l + 1));
  } else if (cdf) {
    od.dX16 = m->df16; od.ld16 = F;
    od.carry_in = m->camax(m->slot_df(l + 1)); od.carry_scales = m->cscales(m->slot_df(l));
  }
  FT_TRY(linear_bwd_fused(m, ly.down, a.f_16, dx16_of(k0) ? nullptr : m->dx, h, a.xa16_down, m->df, F,
                          nullptr, 0, T, dx16_of(k0), dxs_of(k0), false, &od));
  const float* gu_scales = nullptr;
  const __half* dgu16 = m->cvt_hi;
  if (cswi) {
    gu_scales = od.swi_scales;
    dgu16 = m->dgu16;
  } else if (cdf) {
    FT_TRY(ft_k_silu_gate_bwd16hh(ctx, a.gu16, 2 * F, m->df16, F, m->cscales(m->slot_df(l)),
                                  m->camax(m->slot_df(l)), m->cvt_hi, 2 * F, T, F, m->gu_amax + l,
                                  &gu_scales, ly.gu.il));
  } else {
    ctx->amax_out = m->camax(m->slot_df(l));
    ctx->amax_ready = true;
    FT_TRY(ft_k_silu_gate_bwd16h(ctx, a.gu16, 2 * F, m->df, F, m->cvt_hi, 2 * F, T, F, m->gu_amax + l,
                                 &gu_scales, ly.gu.il));
  }
  FT_TRY(linear_bwd_fused(m, ly.gu, a.h2_16, nullptr, 2 * F, a.xa16_gu, m->dh, h, nullptr, 0, T,
                          dgu16, gu_scales));
  FT_TRY(norm_bwd(a.x1, ly.norm2, k0));
  const bool need_dx = l > 0;
  const int k1 = k0 + 1;
  if (m->tc_attention) {
    // the o projection's input gradient reports its amax; attention consumes it as f16
    DxOut oa;
    oa.amax_out = m->camax(m->slot_dattn(l));
    const __half* do16 = m->cvt_hi;
    const float* scales = nullptr;
    if (cda) {
      oa.dX16 = m->dattn16; oa.ld16 = nq;
      oa.carry_in = m->camax(m->slot_dattn(l + 1)); oa.carry_scales = m->cscales(m->slot_dattn(l));
    }
    FT_TRY(linear_bwd_fused(m, ly.o, a.attn16, dx16_of(k1) ? nullptr : m->dx, h, a.xa16_o, m->dattn, nq,
                            nullptr, 0, T, dx16_of(k1), dxs_of(k1), false, &oa));
    if (cda) {
      do16 = m->dattn16;
      scales = m->cscales(m->slot_dattn(l));
    } else {
      ctx->amax_out = m->camax(m->slot_dattn(l));
      ctx->amax_ready = true;
      FT_TRY(ft_to_f16(ctx, m->dattn, nq, m->cvt_hi, nullptr, nq, T, nq, true, &scales, 8));
    }
    arm_at(ctx, m->camax(m->slot_dqkv(l)));
    // (a rotation grows a component by at most sqrt(2), hence target exponents one below the
    // usual ones for dq | dk | dv)
    if (cda && (m->carry_mask & 8)) {
      // the attention kernels write the rotated-back, scaled f16 rows themselves; m->cvt_hi is
      // free here because the output gradient arrived in m->dattn16
      FtAttnBwdOut16 o16;
      o16.rows = m->cvt_hi; o16.ld = nqkv; o16.table = m->rope_tableT();
      o16.carry_amax = m->camax(m->slot_dqkv(l + 1)); o16.carry_exp = kCarryExp - 1;
      o16.carry_scales = m->cscales(m->slot_dqkv(l));
      FT_TRY(ft_attention_bwd_tc(ctx, a.qkv16, nqkv, 0, nq, nq + nkv, a.attn16, nq, do16, nq,
                                 nullptr, 0, nullptr, nullptr, 0, a.stats, scales + 1, m->sequences,
                                 m->seq_len, c.heads, c.kv_heads, c.head_dim, &o16));
      ctx->amax_out = nullptr;
      ctx->amax_ready = false;
      scales = o16.carry_scales;
    } else {
      FT_TRY(ft_attention_bwd_tc(ctx, a.qkv16, nqkv, 0, nq, nq + nkv, a.attn16, nq, do16, nq,
                                 m->dqkv, nqkv, m->dqkv + nq, m->dqkv + nq + nkv, nqkv, a.stats,
                                 scales + 1, m->sequences, m->seq_len, c.heads, c.kv_heads,
                                 c.head_dim));
      // inverse RoPE + f16 rounding in one pass
      FT_TRY(ft_scales_from_amax_or_pass(ctx, m->dqkv, nqkv, T, nqkv, 7, &scales));
      FT_TRY(ft_k_rope_to_f16(ctx, m->dqkv, m->cvt_hi, nqkv, T, nq, nkv, m->seq_len, m->rope_table, true,
                              scales));
    }
    FT_TRY(linear_bwd_fused(m, ly.qkv, a.h1_16, nullptr, nqkv, a.xa16_qkv, need_dx ? m->dh : nullptr,
                            h, nullptr, 0, T, m->cvt_hi, scales));
  } else {
    FT_TRY(linear_bwd_fused(m, ly.o, a.attn16, m->dx, h, a.xa16_o, m->dattn, nq, nullptr, 0, T));
    FT_TRY(attention_launch(m, l, a, true));
    FT_TRY(ft_k_rope(ctx, m->dqkv, nqkv, T, c.heads, c.head_dim, m->seq_len, 0, c.theta, true));
    FT_TRY(ft_k_rope(ctx, m->dqkv + nq, nqkv, T, c.kv_heads, c.head_dim, m->seq_len, 0, c.theta, true));
    FT_TRY(linear_bwd_fused(m, ly.qkv, a.h1_16, m->dqkv, nqkv, a.xa16_qkv, need_dx ? m->dh : nullptr,
                            h, nullptr, 0, T));
  }
  if (need_dx) FT_TRY(norm_bwd(x_in, ly.norm1, k1));
  return FT_OK;
}

// il_off >= 0: source column c goes to the interleaved column (c / 32) * 64 + il_off + c % 32
__device__ __forceinline__ long long il_col(long long c, int il_off) {
  return il_off < 0 ? c : ((c >> 5) << 6) + il_off + (c & 31);
}
__global__ void k_copy_f16_2d(const __half* __restrict__ src, long long lds, __half* __restrict__ dst,
                              long long ldd, int rows, int cols, int il_off) {
  size_t total = (size_t)rows * cols;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += st) {
    size_t r = i / cols, c = i % cols;
    dst[r * ldd + il_col((long long)c, il_off)] = src[r * lds + c];
  }
}
// dst[c, r] (pitch ldd) = src[r, c] (pitch lds); with il_off >= 0 row c of dst is il_col(c)
__global__ void k_transpose_f16(const __half* __restrict__ src, long long lds,
                                __half* __restrict__ dst, long long ldd, int rows, int cols,
                                int il_off) {
  __shared__ __half tile[32][34];
  int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = r0 + j, c = c0 + threadIdx.x;
    tile[j][threadIdx.x] = (r < rows && c < cols) ? src[(long long)r * lds + c] : __half(0.f);
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[il_col(c, il_off) * ldd + r] = tile[threadIdx.x][j];
  }
}

int prepare_group(FtLoraModel* m, Group& g) {
  FtContext* ctx = m->ctx;
  if (!m->cfg.f16_base) return FT_OK;  // tensor-core operands exist for f16 bases only
  if ((g.in % 8) || (g.n % 8)) return FT_OK;  // TMA pitch rule not met: exact path serves it
  void* p = nullptr;
  FT_CUDA(cudaMalloc(&p, (size_t)g.n * g.in * sizeof(__half)));
  m->owned.push_back(p);
  g.w_nk = (__half*)p;
  if (g.nlin == 1) {
    g.w_kn = (__half*)g.lin[0]->w_io;  // [in, out] as the reference stores it
    g.own_kn = false;
  } else {
    FT_CUDA(cudaMalloc(&p, (size_t)g.n * g.in * sizeof(__half)));
    m->owned.push_back(p);
    g.w_kn = (__half*)p;
    g.own_kn = true;
  }
  bool any_bias = false;
  for (int j = 0; j < g.nlin; ++j) any_bias |= g.lin[j]->bias != nullptr;
  if (g.il && (any_bias || g.nlin != 2 || g.lin[0]->out != g.lin[1]->out || (g.lin[0]->out % 32)))
    g.il = false;
  if (g.il) {
    for (__half** slot : {&g.w_nk_il, &g.w_kn_il}) {
      FT_CUDA(cudaMalloc(&p, (size_t)g.n * g.in * sizeof(__half)));
      m->owned.push_back(p);
      *slot = (__half*)p;
    }
  }
  if (any_bias) {
    FT_CUDA(cudaMalloc(&p, (size_t)g.n * sizeof(float)));
    m->owned.push_back(p);
    g.bias_cat = (float*)p;
    FT_CUDA(cudaMemsetAsync(p, 0, (size_t)g.n * sizeof(float), ctx->stream));
    for (int j = 0; j < g.nlin; ++j)
      if (g.lin[j]->bias)
        FT_CUDA(cudaMemcpyAsync(g.bias_cat + g.col_off[j], g.lin[j]->bias,
                                (size_t)g.lin[j]->out * sizeof(float), cudaMemcpyDeviceToDevice,
                                ctx->stream));
  }
  if (g.R > 0 && g.R <= RP) {
    __half** slots[4] = {&g.a_catT16, &g.b_bdT16, &g.b_bd16, &g.a_cat16};
    size_t sizes[4] = {(size_t)RP * g.in, (size_t)g.n * RP, (size_t)RP * g.n, (size_t)g.in * RP};
    for (int k = 0; k < 4; ++k) {
      FT_CUDA(cudaMalloc(&p, sizes[k] * sizeof(__half)));
      m->owned.push_back(p);
      *slots[k] = (__half*)p;
    }
    g.tc_lora = true;
  }
  for (int j = 0; j < g.nlin; ++j) {
    const Linear& l = *g.lin[j];
    const __half* w = (const __half*)l.w_io;  // [in, out]
    dim3 grid(ft_cdiv(l.out, 32), ft_cdiv(l.in, 32)), block(32, 8);
    FT_REQUIRE(grid.y <= 65535, "prepare: input width too large");
    FT_LAUNCH(ctx, k_transpose_f16, grid, block, 0, w, (long long)l.out,
              g.w_nk + (size_t)g.col_off[j] * g.in, (long long)g.in, l.in, l.out, -1);
    const int cg = (int)std::min<size_t>(((size_t)l.in * l.out + 255) / 256, (size_t)ctx->sm_count * 16);
    if (g.own_kn)
      FT_LAUNCH(ctx, k_copy_f16_2d, cg, 256, 0, w, (long long)l.out, g.w_kn + g.col_off[j],
                (long long)g.n, l.in, l.out, -1);
    if (g.il) {
      FT_LAUNCH(ctx, k_transpose_f16, grid, block, 0, w, (long long)l.out, g.w_nk_il,
                (long long)g.in, l.in, l.out, 32 * j);
      FT_LAUNCH(ctx, k_copy_f16_2d, cg, 256, 0, w, (long long)l.out, g.w_kn_il, (long long)g.n, l.in,
                l.out, 32 * j);
    }
  }
  return FT_OK;
}

}  // namespace

// =========================================================================================
extern "C" int ft_model_create(FtContext* ctx, const FtModelConfig* cfg, FtLoraModel** out) {
  FT_REQUIRE(ctx && cfg && out, "ft_model_create: NULL argument");
  FT_REQUIRE(cfg->vocab > 0 && cfg->hidden > 0 && cfg->layers > 0 && cfg->heads > 0 &&
                 cfg->kv_heads > 0 && cfg->head_dim > 0 && cfg->ffn > 0,
             "ft_model_create: empty dimension");
  FT_REQUIRE(cfg->heads % cfg->kv_heads == 0, "ft_model_create: heads %% kv_heads != 0");
  FT_REQUIRE(cfg->head_dim % 4 == 0 && cfg->head_dim <= 128,
             "ft_model_create: head_dim must be a multiple of 4, at most 128");
  FT_REQUIRE(cfg->lora_rank >= 0, "ft_model_create: negative rank");
  FT_REQUIRE(cfg->attention_dropout >= 0.f && cfg->attention_dropout < 1.f,
             "ft_model_create: attention_dropout %g is outside [0, 1)", (double)cfg->attention_dropout);
  FtLoraModel* m = new FtLoraModel();
  m->ctx = ctx;
  m->cfg = *cfg;
  m->nq = cfg->heads * cfg->head_dim;
  m->nkv = cfg->kv_heads * cfg->head_dim;
  m->scale = cfg->lora_rank ? cfg->lora_alpha / (float)cfg->lora_rank : 0.f;
  m->layers.resize(cfg->layers);
  const int h = cfg->hidden, F = cfg->ffn, r = cfg->lora_rank;
  const int ins[FT_LINEARS] = {h, h, h, m->nq, h, h, F};
  const int outs[FT_LINEARS] = {m->nq, m->nkv, m->nkv, h, F, F, h};
  size_t off = 0;
  for (int l = 0; l < cfg->layers; ++l) {
    Layer& ly = m->layers[l];
    for (int i = 0; i < FT_LINEARS; ++i) {
      Linear& li = ly.lin[i];
      li.in = ins[i];
      li.out = outs[i];
      li.lora = r > 0 && ((cfg->lora_mask >> i) & 1);
      if (li.lora) {
        li.a_off = off; off += (size_t)li.in * r;
        li.b_off = off; off += (size_t)r * li.out;
      }
    }
    setup_group(ly.qkv, {&ly.lin[FT_Q], &ly.lin[FT_K], &ly.lin[FT_V]}, r);
    setup_group(ly.o, {&ly.lin[FT_O]}, r);
    setup_group(ly.gu, {&ly.lin[FT_GATE], &ly.lin[FT_UP]}, r);
    {
      // FT_CARRY bit 64 (read when the model is created): interleaved gate|up operands
      const char* env = getenv("FT_CARRY");
      ly.gu.il = cfg->f16_base && ((env ? atoi(env) : 127) & 64) != 0;
    }
    setup_group(ly.down, {&ly.lin[FT_DOWN]}, r);
  }
  m->head_lin.in = h;
  m->head_lin.out = cfg->vocab;
  m->head_lin.lora = r > 0 && cfg->lora_head;
  if (m->head_lin.lora) {
    m->head_lin.a_off = off; off += (size_t)h * r;
    m->head_lin.b_off = off; off += (size_t)r * cfg->vocab;
  }
  setup_group(m->head, {&m->head_lin}, r);
  m->trainable = off;
  *out = m;
  return FT_OK;
}

extern "C" int ft_model_destroy(FtLoraModel* m) {
  if (!m) return FT_OK;
  cudaStreamSynchronize(m->ctx->stream);
  for (void* p : m->owned) cudaFree(p);
  if (m->apply_scratch) cudaFree(m->apply_scratch);
  delete m;
  return FT_OK;
}

extern "C" int ft_model_trainable_count(FtLoraModel* m, size_t* n) {
  FT_REQUIRE(m && n, "ft_model_trainable_count: NULL argument");
  *n = m->trainable;
  return FT_OK;
}

extern "C" int ft_model_adapter_offset(FtLoraModel* m, int layer, int linear, int which_b,
                                       size_t* offset, int* rows, int* cols) {
  FT_REQUIRE(m && offset && rows && cols, "ft_model_adapter_offset: NULL argument");
  const Linear* li;
  if (layer < 0) {
    li = &m->head_lin;
  } else {
    FT_REQUIRE(layer < m->cfg.layers && linear >= 0 && linear < FT_LINEARS,
               "ft_model_adapter_offset: layer %d linear %d out of range", layer, linear);
    li = &m->layers[layer].lin[linear];
  }
  FT_REQUIRE(li->lora, "ft_model_adapter_offset: that linear carries no adapter");
  const int r = m->cfg.lora_rank;
  if (which_b) { *offset = li->b_off; *rows = r; *cols = li->out; }
  else { *offset = li->a_off; *rows = li->in; *cols = r; }
  return FT_OK;
}

extern "C" int ft_model_set_embedding(FtLoraModel* m, const float* embed, const float* final_norm,
                                      const void* head) {
  FT_REQUIRE(m && embed && final_norm && head, "ft_model_set_embedding: NULL argument");
  m->embed = embed;
  m->final_norm = final_norm;
  m->head_lin.w_io = head;
  m->prepared = false;
  return FT_OK;
}

extern "C" int ft_model_set_layer(FtLoraModel* m, int layer, const float* norm1,
                                  const float* norm2, const void* const linears[FT_LINEARS],
                                  const float* const biases[3]) {
  FT_REQUIRE(m && norm1 && norm2 && linears, "ft_model_set_layer: NULL argument");
  FT_REQUIRE(layer >= 0 && layer < m->cfg.layers, "ft_model_set_layer: layer %d out of range",
             layer);
  Layer& ly = m->layers[layer];
  ly.norm1 = norm1;
  ly.norm2 = norm2;
  for (int i = 0; i < FT_LINEARS; ++i) {
    FT_REQUIRE(linears[i], "ft_model_set_layer: linear %d is NULL", i);
    ly.lin[i].w_io = linears[i];
  }
  if (m->cfg.qkv_bias) {
    FT_REQUIRE(biases && biases[0] && biases[1] && biases[2],
               "ft_model_set_layer: q/k/v biases required by the config");
    for (int i = 0; i < 3; ++i) ly.lin[i].bias = biases[i];
  }
  m->prepared = false;
  return FT_OK;
}

extern "C" int ft_model_set_state(FtLoraModel* m, float* params, float* grads, float* adam_m,
                                  float* adam_v) {
  FT_REQUIRE(m, "ft_model_set_state: model is NULL");
  FT_REQUIRE(m->trainable == 0 || (params && grads && adam_m && adam_v),
             "ft_model_set_state: NULL buffer");
  m->params = params; m->grads = grads; m->adam_m = adam_m; m->adam_v = adam_v;
  m->packs_dirty = true;
  return FT_OK;
}

extern "C" int ft_model_prepare(FtLoraModel* m) {
  FT_REQUIRE(m, "ft_model_prepare: model is NULL");
  FT_REQUIRE(m->embed && m->head_lin.w_io, "ft_model_prepare: embedding/head not set");
  for (auto& ly : m->layers)
    FT_REQUIRE(ly.norm1 && ly.lin[0].w_io, "ft_model_prepare: a layer has no weights");
  cudaStreamSynchronize(m->ctx->stream);
  for (void* p : m->owned) cudaFree(p);
  m->owned.clear();
  for (auto& ly : m->layers) {
    FT_TRY(prepare_group(m, ly.qkv));
    FT_TRY(prepare_group(m, ly.o));
    FT_TRY(prepare_group(m, ly.gu));
    FT_TRY(prepare_group(m, ly.down));
  }
  FT_TRY(prepare_group(m, m->head));
  FT_TRY(build_pack_jobs(m));
  if (!m->apply_scratch) {
    size_t chunks = (m->trainable + FT_SUM_SQUARES_CHUNK - 1) / FT_SUM_SQUARES_CHUNK;
    FT_CUDA(cudaMalloc((void**)&m->apply_scratch, (chunks + 8) * sizeof(float)));
  }
  m->prepared = true;
  m->packs_dirty = true;
  m->T = 0;  // the workspace layout depends on which groups reached the tensor cores
  return FT_OK;
}

extern "C" int ft_model_params_changed(FtLoraModel* m) {
  FT_REQUIRE(m, "ft_model_params_changed: model is NULL");
  m->packs_dirty = true;
  return FT_OK;
}

extern "C" int ft_model_workspace_bytes(FtLoraModel* m, int sequences, int seq_len,
                                        size_t* bytes) {
  FT_REQUIRE(m && bytes && sequences > 0 && seq_len > 0, "ft_model_workspace_bytes: bad argument");
  *bytes = plan(m, sequences, seq_len, true, nullptr);
  return FT_OK;
}

extern "C" int ft_model_set_workspace(FtLoraModel* m, void* p, size_t bytes) {
  FT_REQUIRE(m && p, "ft_model_set_workspace: NULL argument");
  FT_REQUIRE((((uintptr_t)p) & 255) == 0, "ft_model_set_workspace: pointer must be 256-byte aligned");
  m->ws = p;
  m->ws_bytes = bytes;
  m->T = 0;
  return FT_OK;
}

extern "C" int ft_model_zero_grad(FtLoraModel* m) {
  FT_REQUIRE(m, "ft_model_zero_grad: model is NULL");
  if (m->trainable)
    FT_CUDA(cudaMemsetAsync(m->grads, 0, m->trainable * sizeof(float), m->ctx->stream));
  return FT_OK;
}

static int step_impl(FtLoraModel* m, const uint32_t* ids, const uint32_t* targets,
                     const float* weights, int sequences, int seq_len, float seed, float* row_loss,
                     float* logits, bool backward);

extern "C" int ft_model_forward_backward(FtLoraModel* m, const uint32_t* ids,
                                         const uint32_t* targets, const float* weights,
                                         int sequences, int seq_len, float seed, float* row_loss,
                                         float* logits) {
  return step_impl(m, ids, targets, weights, sequences, seq_len, seed, row_loss, logits, true);
}

extern "C" int ft_model_set_dropout_seed(FtLoraModel* m, uint64_t step_seed) {
  FT_REQUIRE(m, "ft_model_set_dropout_seed: NULL model");
  m->dropout_step_seed = step_seed;
  return FT_OK;
}

extern "C" int ft_model_forward_loss(FtLoraModel* m, const uint32_t* ids, const uint32_t* targets,
                                     const float* weights, int sequences, int seq_len,
                                     float* row_loss, float* logits) {
  return step_impl(m, ids, targets, weights, sequences, seq_len, 0.f, row_loss, logits, false);
}

static int step_impl(FtLoraModel* m, const uint32_t* ids, const uint32_t* targets,
                     const float* weights, int sequences, int seq_len, float seed, float* row_loss,
                     float* logits, bool backward) {
  FT_REQUIRE(m && ids && targets && weights && row_loss, "ft_model_forward_backward: NULL argument");
  FT_REQUIRE(m->prepared, "ft_model_forward_backward: call ft_model_prepare first");
  FT_REQUIRE(sequences > 0 && seq_len > 0, "ft_model_forward_backward: empty batch");
  FT_REQUIRE(m->trainable == 0 || m->params, "ft_model_forward_backward: state not set");
  FtContext* ctx = m->ctx;
  const FtModelConfig& c = m->cfg;
  const bool fused = use_fused(m);
  if (m->sequences != sequences || m->seq_len != seq_len || m->T == 0 || m->plan_fused != fused) {
    size_t need = plan(m, sequences, seq_len, true, nullptr);
    FT_REQUIRE(m->ws && need <= m->ws_bytes,
               "ft_model_forward_backward: workspace of %zu bytes needed, %zu given", need,
               m->ws_bytes);
    plan(m, sequences, seq_len, false, m->ws);
  }
  const int T = m->T, h = c.hidden, L = c.layers, V = c.vocab;
  const bool ckpt = c.checkpoint_blocks != 0;
  m->dropout_on = backward && c.attention_dropout > 0.f;   // evaluation drops nothing
  if (fused && m->packs_dirty) FT_TRY(pack_all(m));
  if (fused && m->tc_attention && m->table_seq != seq_len) {
    FT_TRY(ft_k_rope_table(ctx, m->rope_table, seq_len, c.head_dim, c.theta));
    m->table_seq = seq_len;
  }

  // ---- forward
  if (fused) FT_CUDA(cudaMemsetAsync(m->gu_amax, 0, sizeof(int) * (size_t)L, ctx->stream));
  FT_TRY(ft_k_embedding(ctx, m->embed, ids, m->x[0], T, V, h));
  for (int l = 0; l < L; ++l) {
    BlockActs& a = m->acts[ckpt ? 0 : l];
    FT_TRY(fused ? block_forward_fused(m, l, m->x[l], m->x[l + 1], a)
                 : block_forward(m, l, m->x[l], m->x[l + 1], a));
  }
  if (fused)
    FT_TRY(ft_k_rms_norm16(ctx, m->x[L], m->final_norm, nullptr, m->hN16, T, h, c.eps));
  else
    FT_TRY(ft_k_rms_norm(ctx, m->x[L], m->final_norm, m->hN, T, h, c.eps));

  // ---- head + loss + head backward, in row chunks; m->dh collects dL/d(hN)
  for (int r0 = 0; r0 < T; r0 += m->head_chunk) {
    const int rows = std::min(m->head_chunk, T - r0);
    float* z = logits ? logits + (size_t)r0 * V : m->logit_chunk;
    if (fused) {
      const __half* X16 = m->hN16 + (size_t)r0 * h;
      __half* xa16 = m->xa16_head + (size_t)r0 * RP;
      FT_TRY(linear_fwd_fused(m, m->head, X16, z, V, xa16, nullptr, 0, rows));
      if (!backward) {
        FT_TRY(ft_k_masked_ce(ctx, z, targets + r0, weights + r0, nullptr, row_loss + r0, rows, V, seed));
      } else if ((V % 8) == 0) {
        // the loss kernel writes its gradient as scaled f16 operands: its magnitude is bounded
        // by the row weights, so the scale is known before the first element is written
        const float* ce_scales = nullptr;
        FT_TRY(ft_k_masked_ce16(ctx, z, targets + r0, weights + r0, m->cvt_hi, V, row_loss + r0, rows,
                                V, seed, &ce_scales));
        FT_TRY(linear_bwd_fused(m, m->head, X16, nullptr, V, xa16, m->dh + (size_t)r0 * h, h,
                                nullptr, 0, rows, m->cvt_hi, ce_scales));
      } else {
        FT_TRY(ft_amax_arm(ctx));   // the loss kernel reports the gradient's amax
        FT_TRY(ft_k_masked_ce(ctx, z, targets + r0, weights + r0, m->logit_chunk, row_loss + r0, rows,
                              V, seed));
        FT_TRY(linear_bwd_fused(m, m->head, X16, m->logit_chunk, V, xa16, m->dh + (size_t)r0 * h, h,
                                nullptr, 0, rows));
      }
    } else {
      const float* X = m->hN + (size_t)r0 * h;
      float* xa = m->xa_head + (size_t)r0 * std::max(1, m->head.R);
      FT_TRY(linear_fwd(m, m->head, X, h, z, V, xa, rows));
      FT_TRY(ft_k_masked_ce(ctx, z, targets + r0, weights + r0, backward ? m->logit_chunk : nullptr,
                            row_loss + r0, rows, V, seed));
      if (backward)
        FT_TRY(linear_bwd(m, m->head, X, h, m->logit_chunk, V, xa, m->dh + (size_t)r0 * h, h, rows,
                          false));
    }
  }
  if (!backward) return FT_OK;   // evaluation: the loss rows are all the caller wants
  if (fused) {
    // the pass's amax slots start from zero; the final norm's result reports into the first
    FT_CUDA(cudaMemsetAsync(m->carry_amax, 0, sizeof(int) * (size_t)m->carry_slots(), ctx->stream));
    arm_at(ctx, m->camax(m->slot_dx(0)));
  }
  FT_TRY(ft_k_rms_norm_bwd(ctx, m->x[L], m->final_norm, m->dh, m->dx, nullptr, T, h, c.eps, false));

  // ---- blocks, last to first
  for (int l = L - 1; l >= 0; --l) {
    BlockActs& a = m->acts[ckpt ? 0 : l];
    if (ckpt)  // replay; rewrites x[l+1] with the same values
      FT_TRY(fused ? block_forward_fused(m, l, m->x[l], m->x[l + 1], a)
                   : block_forward(m, l, m->x[l], m->x[l + 1], a));
    FT_TRY(fused ? block_backward_fused(m, l, m->x[l], a) : block_backward(m, l, m->x[l], a));
  }
  return FT_OK;
}

extern "C" int ft_model_apply_gradients(FtLoraModel* m, float grad_scale, float max_norm,
                                        const FtAdamParams* p, float* norm_out) {
  FT_REQUIRE(m && p, "ft_model_apply_gradients: NULL argument");
  FT_REQUIRE(m->prepared, "ft_model_apply_gradients: call ft_model_prepare first");
  if (!m->trainable) return FT_OK;
  size_t chunks = (m->trainable + FT_SUM_SQUARES_CHUNK - 1) / FT_SUM_SQUARES_CHUNK;
  float* partials = m->apply_scratch;
  float* nout = norm_out ? norm_out : m->apply_scratch + chunks;
  m->packs_dirty = true;  // the adapters change: their f16 operand forms are stale
  return ft_k_apply_fused(m->ctx, m->params, m->grads, m->adam_m, m->adam_v, m->trainable,
                          grad_scale, max_norm, p, partials, nout);
}

extern "C" int ft_model_allreduce_apply_gradients(FtLoraModel* m, FtComm* comm, float max_norm,
                                                  const FtAdamParams* p, float* norm_out) {
  FT_REQUIRE(m && p, "ft_model_allreduce_apply_gradients: NULL argument");
  FT_REQUIRE(!comm || ft_comm_ctx(comm) == m->ctx,
             "ft_model_allreduce_apply_gradients: the communicator belongs to another context");
  const int world = ft_comm_world(comm);
  if (world > 1 && m->trainable) FT_TRY(ft_comm_allreduce_f32(comm, m->grads, m->trainable));
  return ft_model_apply_gradients(m, 1.0f / (float)world, max_norm, p, norm_out);
}
