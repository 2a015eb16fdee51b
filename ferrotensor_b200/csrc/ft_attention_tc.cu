// Forward of causal flash attention on the Blackwell tensor cores (head_dim 64, f16 operands,
// f32 accumulation and softmax), grouped-query; the backward kernels are in
// ft_attention_bwd_tc.cu.  Operands are read straight from the fused q|k|v buffer
// [tokens, nq + 2 nkv] (f16, RoPE already applied) with TMA.
//
// A persistent CTA walks (128 queries, head) tiles over 64-key blocks:
//   S = Q K^T      tcgen05.mma 128 x 64 x 64 into one of two tensor-memory accumulators
//   softmax        4 warps, thread t owns query row t (= TMEM lane t): tcgen05.ld the row,
//                  exp2 against a lazily raised maximum, P written to shared memory as f16 in
//                  the 128-byte-swizzled K-major form the next product wants
//   O += P [V|1]   tcgen05.mma 128 x 80 x 64, V used in place as an N-major operand; the
//                  ones column makes column 64 of the accumulator the softmax denominator
// One warp issues the products, another the TMA loads (each behind elect.sync, which keeps
// descriptors in uniform registers: 13 instead of 71 cycles per tcgen05.mma issued); the S
// product of block j+1 is issued as soon as the softmax warps have read block j, so it overlaps
// with their arithmetic and with P V.
// (Measured and not kept: eight softmax warps with a half-row maximum exchange; paired f16
// exponentials; a quarter of the exponentials as a polynomial on the FMA pipe.  Cycle counts
// inside this kernel: of about 2600 cycles per 64-key block, 1100 are the exponentials (two
// CTAs share the SM's special-function unit), the rest are barrier operations of 100-200 cycles
// each, the shared-memory hand-over of P, and per-tile work.
// Also built and measured against this kernel, on 8 x 1024 x 32 heads / 8 x 4096 x 14:2 heads
// (this kernel: 92.6 / 412 us): one CTA per SM with 128-key blocks and P kept in tensor memory as
// the A operand of P V, as the backward kernels do it - (a) two query tiles per CTA sharing K/V,
// P over the tile's single S buffer: 105 / 440 us, the tile's next scores wait for its P V;
// (b) one tile, S double-buffered, four softmax warps with the row in registers: 98 / 466 us, one
// warp per scheduler reaches 10 of the SM's 16 exponentials per cycle; (c) the same with eight
// warps and a half-row maximum exchange: 97 / 461 us - 1150 of 2100 cycles per block are the
// exponentials at 14 per cycle, the rest (loads, maxima, waits, stores) does not overlap with
// them because the two warps of a scheduler move in step.  Halving the K/V bytes loaded changed
// nothing: L2 bandwidth is not the limit.  Two CTAs per SM, whose warps drift apart, remain the
// better way to keep the special-function unit busy.)
// All waits are bounded (see ft_tc.cuh).
#include <math.h>
#include <stdlib.h>

#include "ft_tc.cuh"

namespace {

using namespace ft_tc;

constexpr int AT_Q = 128;        // queries per CTA
constexpr int AT_KV = 128;       // keys per block
constexpr int AT_D = 64;         // head_dim
constexpr int AT_THREADS = 192;  // forward: warps 0..3 softmax, warp 4 MMA issuer, warp 5 loads
constexpr int TILE_BYTES = 128 * 64 * 2;  // one 128 x 64 f16 tile = 16 KiB

constexpr int HALF_TILE = 64 * 64 * 2;  // 64 x 64 f16 tile = 8 KiB

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnSmem {
  static constexpr int KV_STAGES = 3;
  static constexpr int Q_OFF = 0;                                   // 128 x 64
  static constexpr int K_OFF = Q_OFF + TILE_BYTES;                  // 3 stages of 64 keys x 64
  static constexpr int V_OFF = K_OFF + KV_STAGES * HALF_TILE;       // 3 stages of 64 keys x 64
  static constexpr int ONES_OFF = V_OFF + KV_STAGES * HALF_TILE;    // 64 keys x 64: column 0 = 1
  static constexpr int P_OFF = ONES_OFF + HALF_TILE;                // 2 x (128 q x 64 keys), K-major
  static constexpr int BAR_OFF = P_OFF + 2 * TILE_BYTES;
  // q_full, kv_full[3], s_full[2], s_free[2], p_full[2], o_full[2], o_read, kv_free[3], q_free
  static constexpr int NBAR = 17;
  static constexpr int TOTAL = BAR_OFF + NBAR * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

// Forward.  64-key blocks; S is double-buffered in tensor memory so the product of block j+1
// runs while the softmax warps work on block j.  The output stays in tensor memory for the
// whole row of blocks: P V accumulates there, and an extra all-ones column appended to V makes
// column 64 of the accumulator the running sum of P, i.e. the softmax denominator, rounded
// exactly as the numerator is.  The running maximum is only raised (and the accumulator
// rescaled, by the softmax warps themselves) when a block exceeds it by more than 2^8: until
// then exp2(s - m) <= 256 is harmless in f16 and the final O / l is unchanged.  Exponentials
// use the f32 special-function unit; the scale-and-shift before them is a packed pair FMA.
//
// The kernel is persistent: a CTA walks the (128-query tile, head) pairs t = blockIdx.x,
// blockIdx.x + gridDim.x, ..., late (long) query tiles first, and its key/value ring, score
// and P buffers and barrier phases run on across tile boundaries, counted in blocks since the
// CTA started.  The loads of the next tile's first key/value blocks are therefore issued two
// blocks ahead like any others, the next Q tile is fetched as soon as the last S product of
// the current tile has finished, and S of the next tile's first block is computed while the
// softmax warps normalise and store the current tile; tensor memory, barriers and the ones
// block are set up once per CTA instead of once per tile.
// Tile t of a persistent CTA's round `it`: CTAs take the tiles of even rounds in index order and
// of odd rounds in reverse, so a CTA that got the heaviest tile of one round (tiles are sorted
// heavy first) gets the lightest of the next; the per-CTA totals then differ by a few percent
// instead of the 12 % of plain round-robin.
__device__ __forceinline__ int snake_tile(int it) {
  const int c = (it & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
  return it * (int)gridDim.x + c;
}
struct FwdTile {
  int q0, nblk, b, h, kvh, tok0;
};
__device__ __forceinline__ bool fwd_tile(int t, int total, int nq, int bh_count, int heads, int kv_heads,
                                         int seq, FwdTile& w) {
  if (t >= total) return false;
  const int qblk = nq - 1 - t / bh_count;   // heavy (late) query tiles first
  const int bh = t % bh_count;
  w.b = bh / heads;
  w.h = bh % heads;
  w.kvh = w.h / (heads / kv_heads);
  w.q0 = qblk * AT_Q;
  w.nblk = min((w.q0 + AT_Q) / 64, (seq + 63) / 64);   // 64-key blocks at or below the diagonal
  w.tok0 = w.b * seq;
  return true;
}
// a position in the CTA's sequence of (tile, block) pairs
struct FwdCursor {
  int it, j;       // tile iteration of this CTA, block within the tile
  bool has;
  FwdTile w;
};

__global__ void __launch_bounds__(AT_THREADS, 2)
k_attn_fwd_tc(const __grid_constant__ CUtensorMap map_q128, const __grid_constant__ CUtensorMap map_kv64,
              __half* __restrict__ out16, long long ldo16, float* __restrict__ out32,
              long long ldo32, float* __restrict__ stats, int seq, int heads, int kv_heads,
              int bh_count, int q_col0, int k_col0, int v_col0, float scale_log2e, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  const uint32_t bar0 = base + AttnSmem::BAR_OFF;
  const uint32_t bar_q = bar0, bar_kv = bar0 + 8, bar_sfull = bar0 + 32, bar_sfree = bar0 + 48,
                 bar_pfull = bar0 + 64, bar_ofull = bar0 + 80, bar_oread = bar0 + 96,
                 bar_kvfree = bar0 + 104, bar_qfree = bar0 + 128;
  uint32_t* tmem_slot = (uint32_t*)(gbase + AttnSmem::BAR_OFF + AttnSmem::NBAR * 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (seq + AT_Q - 1) / AT_Q, total = nq * bh_count;
  constexpr uint32_t TMEM_COLS = 256;  // S0 [0,64), S1 [64,128), O [128,192), sum of P at 192
  constexpr int O_COLS = 80;           // 64 outputs + the ones column, padded to a multiple of 16

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 3; ++s) mbar_init(bar_kv + s * 8, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_sfull + s * 8, 1);
      mbar_init(bar_sfree + s * 8, 4);
      mbar_init(bar_pfull + s * 8, 4);
      mbar_init(bar_ofull + s * 8, 1);
    }
    mbar_init(bar_oread, 4);
    for (int st = 0; st < 3; ++st) mbar_init(bar_kvfree + st * 8, 1);
    mbar_init(bar_qfree, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else if (warp < 4) {
    // the ones block: same swizzled layout as a V tile (row = key, 128 bytes = 64 columns; the
    // 16-byte chunk c of row k sits at chunk c ^ (k & 7)): column 0 of every key row is 1, the
    // rest 0.  Thread t writes half a row.
    uint8_t* ones = gbase + AttnSmem::ONES_OFF;
    const int t = threadIdx.x, k = t >> 1, hf = t & 1;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = 4 * hf + i;
      *(uint4*)(ones + k * 128 + c * 16) = make_uint4(c == (k & 7) ? 0x3C00u : 0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128;
  ft_pdl_wait();
  ft_pdl_launch();

  auto start_cursor = [&](FwdCursor& c) {
    c.it = 0;
    c.j = 0;
    c.has = fwd_tile((int)blockIdx.x, total, nq, bh_count, heads, kv_heads, seq, c.w);
  };
  auto advance = [&](FwdCursor& c) {
    if (++c.j < c.w.nblk) return;
    c.j = 0;
    ++c.it;
    c.has = fwd_tile(snake_tile(c.it), total, nq, bh_count, heads, kv_heads, seq, c.w);
  };

  if (warp == 5) {
    // ------------------------------------------------------------------ TMA loads
    // One thread keeps the K/V ring and the Q tile filled, so that the thread that issues the
    // products never spends its time on load instructions (about 75 cycles each) or on waiting
    // for a stage to come free.
    if (elect_one()) {
      const uint32_t sq = base + AttnSmem::Q_OFF, sk = base + AttnSmem::K_OFF, sv = base + AttnSmem::V_OFF;
      uint32_t gl = 0;     // key/value blocks loaded since the CTA started
      bool ok = true;
      FwdTile w;
      for (int it = 0; ok && fwd_tile(snake_tile(it), total, nq, bh_count, heads, kv_heads, seq, w); ++it) {
        if (it >= 1) {
          // the Q tile is free once the previous tile's last S product has finished
          ok = mbar_wait(bar_qfree, (it - 1) & 1, abort_flag, status, 16);
          if (!ok) break;
        }
        mbar_expect_tx(bar_q, TILE_BYTES);
        tma_load_2d(sq, &map_q128, bar_q, q_col0 + w.h * AT_D, w.tok0 + w.q0);
        for (int j = 0; j < w.nblk; ++j, ++gl) {
          const uint32_t st = gl % 3;
          if (gl >= 3) {
            // stage st held block gl - 3: free once P V of that block has run (the stage's own
            // barrier: its next completion needs this very load, so the phase cannot run ahead)
            ok = mbar_wait(bar_kvfree + st * 8, (gl / 3 - 1) & 1, abort_flag, status, 17);
            if (!ok) break;
          }
          mbar_expect_tx(bar_kv + st * 8, 2 * HALF_TILE);
          tma_load_2d(sk + st * HALF_TILE, &map_kv64, bar_kv + st * 8, k_col0 + w.kvh * AT_D, w.tok0 + j * 64);
          tma_load_2d(sv + st * HALF_TILE, &map_kv64, bar_kv + st * 8, v_col0 + w.kvh * AT_D, w.tok0 + j * 64);
        }
      }
    }
    __syncwarp();
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t sq = base + AttnSmem::Q_OFF, sk = base + AttnSmem::K_OFF,
                     sv = base + AttnSmem::V_OFF, sp = base + AttnSmem::P_OFF;
      const uint32_t idesc_s = make_idesc(128, 64, 0, 0);                      // Q, K both K-major
      const uint32_t idesc_o = make_idesc(128, O_COLS, 0, 0) | (1u << 16);     // V is N-major
      // two cursors over the same sequence of blocks: S runs one block ahead of P V; gs, gp
      // count blocks since the CTA started
      FwdCursor S, P;
      start_cursor(S);
      start_cursor(P);
      uint32_t gs = 0, gp = 0;
      bool ok = true;
      // S of block gs: the tile's Q and the block's keys must have landed and its accumulator
      // (last used by block gs-2) must have been read
      auto issue_s = [&]() -> bool {
        if (S.j == 0 && !mbar_wait(bar_q, S.it & 1, abort_flag, status, 11)) return false;
        if (!mbar_wait(bar_kv + (gs % 3) * 8, (gs / 3) & 1, abort_flag, status, 13)) return false;
        if (gs >= 2 && !mbar_wait(bar_sfree + (gs & 1) * 8, ((gs - 2) >> 1) & 1, abort_flag, status, 14))
          return false;
        tc_fence_after();
        const uint64_t da = make_desc_sw128(sq), db = make_desc_sw128(sk + (gs % 3) * HALF_TILE);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_f16(tmem_base + (gs & 1) * 64, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s,
                     k > 0 ? 1u : 0u);
        tc_commit(bar_sfull + (gs & 1) * 8);
        if (S.j == S.w.nblk - 1) tc_commit(bar_qfree);   // the tile's last S product: Q may be replaced
        advance(S);
        ++gs;
        return true;
      };
      if (P.has) ok = issue_s();
      while (ok && P.has) {
        // the next S product first when it belongs to the same tile; across a tile boundary the
        // current tile's last P V goes first (the next Q tile is still on its way)
        const bool next_tile = S.has && S.j == 0;
        if (S.has && !next_tile) {
          ok = issue_s();
          if (!ok) break;
        }
        ok = mbar_wait(bar_pfull + (gp & 1) * 8, (gp >> 1) & 1, abort_flag, status, 15);
        if (ok && P.j == 0 && P.it >= 1)   // the previous tile's output must have left tensor memory
          ok = mbar_wait(bar_oread, (P.it - 1) & 1, abort_flag, status, 18);
        if (!ok) break;
        tc_fence_after();
        {
          // O += P[128 q x 64 keys] . [V | 1][64 keys x 80]: V in place as an N-major operand,
          // its second 64-column block is the ones block
          const uint32_t vs = sv + (gp % 3) * HALF_TILE;
          const uint64_t dp = make_desc_sw128(sp + (gp & 1) * TILE_BYTES);
          const uint64_t dv = make_desc_mn_sw128(vs, (base + AttnSmem::ONES_OFF) - vs);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f16(tmem_o, dp + (uint64_t)(k * 2), dv + (uint64_t)(k * 128), idesc_o,
                       (P.j > 0 || k > 0) ? 1u : 0u);
          tc_commit(bar_ofull + (gp & 1) * 8);
          tc_commit(bar_kvfree + (gp % 3) * 8);
        }
        advance(P);
        ++gp;
        if (next_tile) ok = issue_s();
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax warps
    const int row = warp * 32 + lane;          // query row in the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    uint8_t* rowp = gbase + AttnSmem::P_OFF + (row >> 3) * 1024 + (row & 7) * 128;
    uint32_t g0 = 0;                           // blocks of the tiles before this one
    bool ok = true;
    FwdTile w;
    for (int it = 0; ok && fwd_tile(snake_tile(it), total, nq, bh_count, heads,
                                    kv_heads, seq, w); ++it) {
      const int q0 = w.q0, nblk = w.nblk;
      const int qi = q0 + row;                 // position in the sequence
      float m_st = -INFINITY;   // the maximum the exponentials are taken against (log2 domain)
      for (int j = 0; ok && j < nblk; ++j) {
        const uint32_t g = g0 + (uint32_t)j;
        const int sb = (int)(g & 1);
        ok = mbar_wait(bar_sfull + sb * 8, (g >> 1) & 1, abort_flag, status, 21);
        if (!ok) break;
        tc_fence_after();
        uint32_t r0[32], r1[32];
        tc_ld32(tmem_base + lane_addr + sb * 64, r0);
        tc_ld32(tmem_base + lane_addr + sb * 64 + 32, r1);
        tc_wait_ld();
        // the scores are in registers: this accumulator may be overwritten
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sfree + sb * 8);
        const int key0 = j * 64;
        if (key0 + 63 > q0) {                     // the block touches the diagonal for some row
          const int lim = qi - key0;              // keys [0, lim] of the block are visible
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c > lim) r0[c] = 0xff800000u;     // -inf
            if (c + 32 > lim) r1[c] = 0xff800000u;
          }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < 32; ++c)
          mx = fmaxf(mx, fmaxf(__uint_as_float(r0[c]), __uint_as_float(r1[c])));
        const float mxs = mx * scale_log2e;
        if (j == 0) {
          m_st = mxs;   // key 0 is visible to every row, so this is finite
        } else {
          const bool need = mxs > m_st + 8.0f;
          if (__any_sync(0xffffffffu, need)) {
            // raise the maximum and rescale the accumulator (rows that do not need it use 1);
            // P V(j-1) must have finished, P V(j) cannot start before this warp publishes P(j)
            const float m_new = need ? mxs : m_st;
            const float corr = ex2(m_st - m_new);
            ok = mbar_wait(bar_ofull + ((g - 1) & 1) * 8, ((g - 1) >> 1) & 1, abort_flag, status, 22);
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            tc_fence_after();
            uint32_t a[32];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              tc_ld32(tmem_o + lane_addr + hh * 32, a);
              tc_wait_ld();
#pragma unroll
              for (int c = 0; c < 32; ++c) a[c] = __float_as_uint(__uint_as_float(a[c]) * corr);
              tc_st32(tmem_o + lane_addr + hh * 32, a);
            }
            uint32_t s16[16];
            tc_ld16(tmem_o + lane_addr + 64, s16);
            tc_wait_ld();
#pragma unroll
            for (int c = 0; c < 16; ++c) s16[c] = __float_as_uint(__uint_as_float(s16[c]) * corr);
            tc_st16(tmem_o + lane_addr + 64, s16);
            tc_wait_st();
            m_st = m_new;
          }
        }
        // P = exp2(s * scale - m)
        const float nm = -m_st;
        uint32_t packed[32];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float x0, x1, y0, y1;
          ffma2(x0, x1, __uint_as_float(r0[c]), __uint_as_float(r0[c + 1]), scale_log2e, scale_log2e, nm, nm);
          ffma2(y0, y1, __uint_as_float(r1[c]), __uint_as_float(r1[c + 1]), scale_log2e, scale_log2e, nm, nm);
          packed[c >> 1] = pack_h2(ex2(x0), ex2(x1));
          packed[16 + (c >> 1)] = pack_h2(ex2(y0), ex2(y1));
        }
        // This P buffer was last read by P V of block g-2.  That product has finished: the issuer
        // thread issued it before S(g), and the commit that completed sfull(g) above covers every
        // tcgen05 operation the thread had issued before it.
        uint8_t* rp = rowp + sb * TILE_BYTES;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *(uint4*)(rp + ((q ^ (row & 7)) << 4)) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        tc_fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pfull + sb * 8);
      }
      if (!ok) break;
      const uint32_t gl_ = g0 + (uint32_t)nblk - 1;   // the tile's last block
      ok = mbar_wait(bar_ofull + (gl_ & 1) * 8, (gl_ >> 1) & 1, abort_flag, status, 24);
      if (!ok) break;
      tc_fence_after();
      uint32_t a0[32], a1[32], s16[16];
      tc_ld32(tmem_o + lane_addr, a0);
      tc_ld32(tmem_o + lane_addr + 32, a1);
      tc_ld16(tmem_o + lane_addr + 64, s16);
      tc_wait_ld();
      // the accumulator is in registers: the next tile's first P V may overwrite it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_oread);
      if (qi < seq) {
        const float l = __uint_as_float(s16[0]);
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        float o_acc[AT_D];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          o_acc[c] = __uint_as_float(a0[c]) * inv;
          o_acc[32 + c] = __uint_as_float(a1[c]) * inv;
        }
        const long long tok = (long long)w.tok0 + qi;
        if (out16) {
          __half* o = out16 + tok * ldo16 + (long long)w.h * AT_D;
#pragma unroll
          for (int i = 0; i < AT_D; i += 8)
            *(uint4*)(o + i) = make_uint4(pack_h2(o_acc[i], o_acc[i + 1]), pack_h2(o_acc[i + 2], o_acc[i + 3]),
                                          pack_h2(o_acc[i + 4], o_acc[i + 5]), pack_h2(o_acc[i + 6], o_acc[i + 7]));
        }
        if (out32) {
          float* o = out32 + tok * ldo32 + (long long)w.h * AT_D;
#pragma unroll
          for (int i = 0; i < AT_D; i += 4)
            *(float4*)(o + i) = make_float4(o_acc[i], o_acc[i + 1], o_acc[i + 2], o_acc[i + 3]);
        }
        if (stats) {
          const size_t srow = ((size_t)w.b * heads + w.h) * seq + qi;
          // natural-log LSE of the scaled scores
          stats[2 * srow + 1] = l > 0.f ? (m_st + log2f(l)) * 0.6931471805599453f : 3.0e38f;
        }
      }
      g0 += (uint32_t)nblk;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 4) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

}  // namespace

// Forward on f16 q|k|v rows (RoPE applied): writes f16 and/or f32 output rows [tokens, heads*64]
// and the per-row log-sum-exp into stats[2*row+1].
int ft_attention_fwd_tc(FtContext* ctx, const __half* qkv16, long long ld, int q_col0, int k_col0,
                        int v_col0, __half* out16, long long ldo16, float* out32, long long ldo32,
                        float* stats, int batch, int seq, int heads, int kv_heads, int head_dim) {
  if (head_dim != AT_D || (ld % 8) || (((uintptr_t)qkv16) & 15) || (q_col0 % 8) || (k_col0 % 8) ||
      (v_col0 % 8) || (out16 && ((ldo16 % 8) || (((uintptr_t)out16) & 15))) ||
      (out32 && ((ldo32 % 4) || (((uintptr_t)out32) & 15))))
    return FT_ERR_UNSUPPORTED;
  FT_REQUIRE((long long)batch * heads <= 65535, "attention: batch*heads exceeds 65535");
  CUtensorMap q128, kv64;
  FT_TRY(ft_tc::make_map(ctx, &q128, qkv16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (uint64_t)ld,
                         (uint64_t)batch * seq, (uint64_t)ld, 64, 128));
  FT_TRY(ft_tc::make_map(ctx, &kv64, qkv16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (uint64_t)ld,
                         (uint64_t)batch * seq, (uint64_t)ld, 64, 64));
  static bool configured[FT_MAX_DEVICES] = {};   // function attributes are per device
  if (!configured[ctx->device]) {
    FT_CUDA(cudaFuncSetAttribute(k_attn_fwd_tc, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 AttnSmem::DYN_BYTES));
    configured[ctx->device] = true;
  }
  // persistent: two CTAs per SM walk the (query tile, head) pairs
  const int tiles = ft_cdiv(seq, AT_Q) * batch * heads;
  const int grid = std::min(tiles, 2 * ctx->sm_count);
  const float scale_log2e = (1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
  FT_LAUNCH_PDL(ctx, k_attn_fwd_tc, grid, AT_THREADS, AttnSmem::DYN_BYTES, q128, kv64, out16, ldo16,
                out32, ldo32, stats, seq, heads, kv_heads, batch * heads, q_col0, k_col0, v_col0,
                scale_log2e, ctx->status_dev);
  return FT_OK;
}
