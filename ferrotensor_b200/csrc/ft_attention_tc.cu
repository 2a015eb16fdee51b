// Causal flash attention on the Blackwell tensor cores (head_dim 64, f16 operands, f32
// accumulation and softmax), grouped-query.  Operands are read straight from the fused
// q|k|v buffer [tokens, nq + 2 nkv] (f16, RoPE already applied) with TMA: one 128 x 64 box
// shape serves the query, key and value tiles.
//
// Forward, one CTA per (128 queries, head), over 64-key blocks:
//   S = Q K^T      tcgen05.mma 128 x 64 x 64 into one of two tensor-memory accumulators
//   softmax        4 warps, thread t owns query row t (= TMEM lane t): tcgen05.ld the row,
//                  exp2 against a lazily raised maximum, P written to shared memory as f16 in
//                  the 128-byte-swizzled K-major form the next product wants
//   O += P [V|1]   tcgen05.mma 128 x 80 x 64, V used in place as an N-major operand; the
//                  ones column makes column 64 of the accumulator the softmax denominator
// One extra warp issues all TMA loads and MMAs; the S product of block j+1 is issued as soon
// as the softmax warps have read block j, so it overlaps with their arithmetic and with P V.
// (Measured and not kept: eight softmax warps with a half-row maximum exchange; paired f16
// exponentials; a quarter of the exponentials as a polynomial on the FMA pipe; releasing S / dP to the next product before the arithmetic in the backward
// kernels - per block the time goes to the hand-offs between the warps and the tensor pipe,
// not to the arithmetic; a separate loader warp in the backward kernels (8 % slower, while the
// same split made the forward kernel 10 % faster); the backward kernels made persistent like the forward one - the dQ
// kernel ran as before, the dK / dV kernel 20 % slower.  Cycle counts inside the forward kernel:
// of about 2600 cycles per 64-key block, 1100 are the exponentials (two CTAs share the SM's
// special-function unit), the rest are barrier operations of 100-200 cycles each, the
// shared-memory hand-over of P, and per-tile work; one tcgen05.mma costs the issuing thread
// about 55 cycles, a TMA load about 75.)
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
constexpr int BW_THREADS = 288;  // backward: warps 0..7 arithmetic, warp 8 issuer
constexpr int BW_ISSUER = 8;
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

// =========================================================================================
// Backward.  Two kernels, no atomics (results are identical from run to run):
//   k_attn_bwd_dq_tc   one CTA per (128 queries, head): over 64-key blocks,
//                      S = Q K^T, dP = dO V^T (tensor memory), dS = P (dP - Delta) in registers
//                      -> f16 shared tile, dQ += dS K accumulated in tensor memory.
//                      Also computes Delta = dO . O per query row and stores it for pass 2.
//   k_attn_bwd_dkv_tc  one CTA per (128 keys, KV head): over the query heads of the group and
//                      64-query blocks at or below the diagonal, S^T = K Q^T, dP^T = V dO^T,
//                      dV += P^T dO, dK += dS^T Q, both accumulated in tensor memory.
// dO arrives as f16 after a power-of-two scale S (gradients are far below f16's normal
// range); everything downstream is linear in dO, so the epilogues multiply by 1/S.
// =========================================================================================

struct BwdQSmem {
  static constexpr int Q_OFF = 0;                         // 128 x 64
  static constexpr int DO_OFF = Q_OFF + TILE_BYTES;       // 128 x 64
  static constexpr int K_OFF = DO_OFF + TILE_BYTES;       // 2 stages of 64 x 64
  static constexpr int V_OFF = K_OFF + 2 * HALF_TILE;     // 2 stages of 64 x 64
  static constexpr int DS_OFF = V_OFF + 2 * HALF_TILE;    // 128 q x 64 keys, K-major
  static constexpr int BAR_OFF = DS_OFF + TILE_BYTES;
  static constexpr int NBAR = 8;  // q_full, kv_full[2], sp_full, sp_free, ds_full, dq_done, spare
  static constexpr int TOTAL = BAR_OFF + NBAR * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

__global__ void __launch_bounds__(BW_THREADS, 2)
k_attn_bwd_dq_tc(const __grid_constant__ CUtensorMap map_q128, const __grid_constant__ CUtensorMap map_kv64,
                 const __grid_constant__ CUtensorMap map_do128, const __half* __restrict__ do16,
                 long long lddo, const __half* __restrict__ o16, long long ldo,
                 float* __restrict__ dq, long long lddq, float* __restrict__ stats, int seq,
                 int heads, int kv_heads, int q_col0, int k_col0, int v_col0, float scale,
                 const float* __restrict__ inv_scale_ptr, int* amax_slot, int* status) {
  ft_pdl_wait();
  ft_pdl_launch();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  const uint32_t bar0 = base + BwdQSmem::BAR_OFF;
  const uint32_t bar_q = bar0, bar_kv = bar0 + 8, bar_spfull = bar0 + 24, bar_spfree = bar0 + 32,
                 bar_dsfull = bar0 + 40, bar_dqdone = bar0 + 48;
  uint32_t* tmem_slot = (uint32_t*)(gbase + BwdQSmem::BAR_OFF + BwdQSmem::NBAR * 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblk = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int kvh = h / (heads / kv_heads);
  const int q0 = qblk * AT_Q;
  const int nblk = min((q0 + AT_Q) / 64, (seq + 63) / 64);  // 64-key blocks at or below the diagonal
  const int tok0 = b * seq;
  constexpr uint32_t TMEM_COLS = 256;  // S [0,64), dP [64,128), dQ [128,192)

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_kv, 1);
    mbar_init(bar_kv + 8, 1);
    mbar_init(bar_spfull, 1);
    mbar_init(bar_spfree, 8);
    mbar_init(bar_dsfull, 8);
    mbar_init(bar_dqdone, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == BW_ISSUER) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + 64, tmem_dq = tmem_base + 128;

  if (warp == BW_ISSUER) {
    if (lane == 0) {
      const uint32_t sq = base + BwdQSmem::Q_OFF, sdo = base + BwdQSmem::DO_OFF,
                     sk = base + BwdQSmem::K_OFF, sv = base + BwdQSmem::V_OFF,
                     sds = base + BwdQSmem::DS_OFF;
      const uint32_t idesc_kk = make_idesc(128, 64, 0, 0);              // both K-major
      const uint32_t idesc_kn = make_idesc(128, 64, 0, 0) | (1u << 16); // B N-major
      auto load_kv = [&](int j) {
        const int s = j & 1;
        mbar_expect_tx(bar_kv + s * 8, 2 * HALF_TILE);
        tma_load_2d(sk + s * HALF_TILE, &map_kv64, bar_kv + s * 8, k_col0 + kvh * AT_D, tok0 + j * 64);
        tma_load_2d(sv + s * HALF_TILE, &map_kv64, bar_kv + s * 8, v_col0 + kvh * AT_D, tok0 + j * 64);
      };
      auto mma_sp = [&](int j) {
        const int s = j & 1;
        const uint64_t dq_ = make_desc_sw128(sq), ddo = make_desc_sw128(sdo);
        const uint64_t dk_ = make_desc_sw128(sk + s * HALF_TILE), dv_ = make_desc_sw128(sv + s * HALF_TILE);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_f16(tmem_s, dq_ + (uint64_t)(k * 2), dk_ + (uint64_t)(k * 2), idesc_kk, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_f16(tmem_dp, ddo + (uint64_t)(k * 2), dv_ + (uint64_t)(k * 2), idesc_kk, k > 0 ? 1u : 0u);
        tc_commit(bar_spfull);
      };
      mbar_expect_tx(bar_q, 2 * TILE_BYTES);
      tma_load_2d(sq, &map_q128, bar_q, q_col0 + h * AT_D, tok0 + q0);
      tma_load_2d(sdo, &map_do128, bar_q, h * AT_D, tok0 + q0);
      load_kv(0);
      if (nblk > 1) load_kv(1);
      bool ok = mbar_wait(bar_q, 0, abort_flag, status, 31) &&
                mbar_wait(bar_kv, 0, abort_flag, status, 32);
      if (ok) {
        tc_fence_after();
        mma_sp(0);
      }
      for (int j = 0; ok && j < nblk; ++j) {
        if (j + 1 < nblk) {
          ok = mbar_wait(bar_kv + ((j + 1) & 1) * 8, ((j + 1) >> 1) & 1, abort_flag, status, 33) &&
               mbar_wait(bar_spfree, j & 1, abort_flag, status, 34);
          if (!ok) break;
          tc_fence_after();
          mma_sp(j + 1);
        }
        ok = mbar_wait(bar_dsfull, j & 1, abort_flag, status, 35);
        if (!ok) break;
        tc_fence_after();
        {
          // dQ += dS[128 q x 64 keys] . K[64 keys x 64 d]: K tile in place as an N-major operand
          const uint64_t da = make_desc_sw128(sds);
          const uint64_t db = make_desc_mn_sw128(sk + (j & 1) * HALF_TILE, HALF_TILE);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f16(tmem_dq, da + (uint64_t)(k * 2), db + (uint64_t)(k * 128), idesc_kn,
                       (j > 0 || k > 0) ? 1u : 0u);
          tc_commit(bar_dqdone);
        }
        if (j + 2 < nblk) {
          ok = mbar_wait(bar_dqdone, j & 1, abort_flag, status, 36);
          if (!ok) break;
          load_kv(j + 2);
        }
      }
    }
    __syncwarp();
  } else {
    // eight warps: warp w works on the 32 query rows of TMEM quadrant w % 4 and on the 32-key
    // half w / 4 of every block
    const int quad = warp & 3, hc = warp >> 2;
    const int row = quad * 32 + lane;
    const int qi = q0 + row;
    const bool row_ok = qi < seq;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    uint8_t* ds_smem = gbase + BwdQSmem::DS_OFF;
    const size_t srow = ((size_t)b * heads + h) * seq + (row_ok ? qi : 0);
    // Delta = dO . O for this row (both f16 in global memory)
    float delta = 0.f, lse2 = 0.f;
    if (row_ok) {
      const long long tok = (long long)tok0 + qi;
      const uint4* pd = (const uint4*)(do16 + tok * lddo + (long long)h * AT_D);
      const uint4* po = (const uint4*)(o16 + tok * ldo + (long long)h * AT_D);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint4 a = pd[i], c = po[i];
        const __half2* ha = (const __half2*)&a;
        const __half2* hc = (const __half2*)&c;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float2 fa = __half22float2(ha[t]), fc = __half22float2(hc[t]);
          delta += fa.x * fc.x + fa.y * fc.y;
        }
      }
      lse2 = stats[2 * srow + 1] * 1.4426950408889634f;
      if (hc == 0) stats[2 * srow] = delta;
    }
    const float c2 = scale * 1.4426950408889634f;
    bool ok = true;
    for (int j = 0; ok && j < nblk; ++j) {
      ok = mbar_wait(bar_spfull, j & 1, abort_flag, status, 41);
      if (!ok) break;
      tc_fence_after();
      const bool need_mask = (j * 64 + 63) > q0;  // block touches the diagonal
      uint32_t packed[16];
      {
        uint32_t rs[32], rp[32];
        tc_ld32(tmem_s + lane_addr + hc * 32, rs);
        tc_ld32(tmem_dp + lane_addr + hc * 32, rp);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float v[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = j * 64 + hc * 32 + c + e;
            float p = ex2(fmaf(__uint_as_float(rs[c + e]), c2, -lse2));
            if (!row_ok || (need_mask && key > qi)) p = 0.f;
            v[e] = p * (__uint_as_float(rp[c + e]) - delta);
          }
          packed[c >> 1] = pack_h2(v[0], v[1]);
        }
      }
      // S and dP are in registers: the next pair of products may overwrite them
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_spfree);
      // the previous dQ product must have finished reading the dS tile
      if (j > 0) {
        ok = mbar_wait(bar_dqdone, (j - 1) & 1, abort_flag, status, 42);
        if (!ok) break;
      }
      uint8_t* rowp = ds_smem + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
      for (int q = 0; q < 4; ++q)
        *(uint4*)(rowp + (((hc * 4 + q) ^ (row & 7)) << 4)) =
            make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_dsfull);
    }
    if (ok) ok = mbar_wait(bar_dqdone, (nblk - 1) & 1, abort_flag, status, 43);
    if (ok) {
      tc_fence_after();
      const float alpha = scale * (inv_scale_ptr ? *inv_scale_ptr : 1.0f);
      float am = 0.f;
      {
        const int cb = hc;
        uint32_t r[32];
        tc_ld32(tmem_dq + lane_addr + cb * 32, r);
        tc_wait_ld();
        if (row_ok) {
          float* o = dq + ((long long)tok0 + qi) * lddq + (long long)h * AT_D + cb * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 v = make_float4(alpha * __uint_as_float(r[i]), alpha * __uint_as_float(r[i + 1]),
                                   alpha * __uint_as_float(r[i + 2]), alpha * __uint_as_float(r[i + 3]));
            *(float4*)(o + i) = v;
            am = fmaxf(am, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
          }
        }
      }
      if (amax_slot) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        if (lane == 0 && am > 0.f && __float_as_int(am) > *(volatile int*)amax_slot)
          atomicMax(amax_slot, __float_as_int(am));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == BW_ISSUER) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

struct BwdKSmem {
  static constexpr int K_OFF = 0;                         // 128 keys x 64
  static constexpr int V_OFF = K_OFF + TILE_BYTES;        // 128 keys x 64
  static constexpr int Q_OFF = V_OFF + TILE_BYTES;        // 2 stages of 64 q x 64
  static constexpr int DO_OFF = Q_OFF + 2 * HALF_TILE;    // 2 stages of 64 q x 64
  static constexpr int PT_OFF = DO_OFF + 2 * HALF_TILE;   // 128 keys x 64 q, K-major
  static constexpr int DST_OFF = PT_OFF + TILE_BYTES;     // 128 keys x 64 q, K-major
  static constexpr int ROW_OFF = DST_OFF + TILE_BYTES;    // per warp: 32 x {delta, lse2}
  static constexpr int BAR_OFF = ROW_OFF + 8 * 32 * 2 * 4;
  static constexpr int NBAR = 8;  // kv_full, qd_full[2], sp_full, sp_free, ds_full, acc_done, spare
  static constexpr int TOTAL = BAR_OFF + NBAR * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

__global__ void __launch_bounds__(BW_THREADS, 2)
k_attn_bwd_dkv_tc(const __grid_constant__ CUtensorMap map_kv128, const __grid_constant__ CUtensorMap map_q64,
                  const __grid_constant__ CUtensorMap map_do64, float* __restrict__ dk,
                  float* __restrict__ dv, long long ldd, const float* __restrict__ stats, int seq,
                  int heads, int kv_heads, int q_col0, int k_col0, int v_col0, float scale,
                  const float* __restrict__ inv_scale_ptr, int* amax_slot, int* status) {
  ft_pdl_wait();
  ft_pdl_launch();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  const uint32_t bar0 = base + BwdKSmem::BAR_OFF;
  const uint32_t bar_kv = bar0, bar_qd = bar0 + 8, bar_spfull = bar0 + 24, bar_spfree = bar0 + 32,
                 bar_dsfull = bar0 + 40, bar_acc = bar0 + 48;
  uint32_t* tmem_slot = (uint32_t*)(gbase + BwdKSmem::BAR_OFF + BwdKSmem::NBAR * 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblk = blockIdx.x;  // early key blocks see the most queries and run first
  const int bk = blockIdx.y, b = bk / kv_heads, kvh = bk % kv_heads;
  const int group = heads / kv_heads;
  const int k0 = kblk * AT_KV;
  const int nqb = (seq - k0 + 63) / 64;    // 64-query blocks from the diagonal to the end
  const int niter = group * nqb;
  const int tok0 = b * seq;
  constexpr uint32_t TMEM_COLS = 256;  // S^T [0,64), dP^T [64,128), dK [128,192), dV [192,256)

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(bar_qd, 1);
    mbar_init(bar_qd + 8, 1);
    mbar_init(bar_spfull, 1);
    mbar_init(bar_spfree, 8);
    mbar_init(bar_dsfull, 8);
    mbar_init(bar_acc, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == BW_ISSUER) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_st = tmem_base, tmem_dpt = tmem_base + 64, tmem_dk = tmem_base + 128,
                 tmem_dv = tmem_base + 192;

  if (warp == BW_ISSUER) {
    if (lane == 0) {
      const uint32_t sk = base + BwdKSmem::K_OFF, sv = base + BwdKSmem::V_OFF,
                     sq = base + BwdKSmem::Q_OFF, sdo = base + BwdKSmem::DO_OFF,
                     spt = base + BwdKSmem::PT_OFF, sdst = base + BwdKSmem::DST_OFF;
      const uint32_t idesc_kk = make_idesc(128, 64, 0, 0);
      const uint32_t idesc_kn = make_idesc(128, 64, 0, 0) | (1u << 16);
      auto load_qd = [&](int it) {
        const int s = it & 1, g = it / nqb, i = it % nqb, h = kvh * group + g;
        mbar_expect_tx(bar_qd + s * 8, 2 * HALF_TILE);
        tma_load_2d(sq + s * HALF_TILE, &map_q64, bar_qd + s * 8, q_col0 + h * AT_D, tok0 + k0 + i * 64);
        tma_load_2d(sdo + s * HALF_TILE, &map_do64, bar_qd + s * 8, h * AT_D, tok0 + k0 + i * 64);
      };
      auto mma_sp = [&](int it) {
        const int s = it & 1;
        const uint64_t dk_ = make_desc_sw128(sk), dv_ = make_desc_sw128(sv);
        const uint64_t dq_ = make_desc_sw128(sq + s * HALF_TILE), ddo = make_desc_sw128(sdo + s * HALF_TILE);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_f16(tmem_st, dk_ + (uint64_t)(k * 2), dq_ + (uint64_t)(k * 2), idesc_kk, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_f16(tmem_dpt, dv_ + (uint64_t)(k * 2), ddo + (uint64_t)(k * 2), idesc_kk, k > 0 ? 1u : 0u);
        tc_commit(bar_spfull);
      };
      mbar_expect_tx(bar_kv, 2 * TILE_BYTES);
      tma_load_2d(sk, &map_kv128, bar_kv, k_col0 + kvh * AT_D, tok0 + k0);
      tma_load_2d(sv, &map_kv128, bar_kv, v_col0 + kvh * AT_D, tok0 + k0);
      load_qd(0);
      if (niter > 1) load_qd(1);
      bool ok = mbar_wait(bar_kv, 0, abort_flag, status, 51) &&
                mbar_wait(bar_qd, 0, abort_flag, status, 52);
      if (ok) {
        tc_fence_after();
        mma_sp(0);
      }
      for (int it = 0; ok && it < niter; ++it) {
        if (it + 1 < niter) {
          ok = mbar_wait(bar_qd + ((it + 1) & 1) * 8, ((it + 1) >> 1) & 1, abort_flag, status, 53) &&
               mbar_wait(bar_spfree, it & 1, abort_flag, status, 54);
          if (!ok) break;
          tc_fence_after();
          mma_sp(it + 1);
        }
        ok = mbar_wait(bar_dsfull, it & 1, abort_flag, status, 55);
        if (!ok) break;
        tc_fence_after();
        {
          const int s = it & 1;
          const uint64_t dpt = make_desc_sw128(spt), ddst = make_desc_sw128(sdst);
          const uint64_t bdo = make_desc_mn_sw128(sdo + s * HALF_TILE, HALF_TILE);
          const uint64_t bq = make_desc_mn_sw128(sq + s * HALF_TILE, HALF_TILE);
#pragma unroll
          for (int k = 0; k < 4; ++k)   // dV += P^T[128 keys x 64 q] . dO[64 q x 64 d]
            tc_mma_f16(tmem_dv, dpt + (uint64_t)(k * 2), bdo + (uint64_t)(k * 128), idesc_kn,
                       (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 4; ++k)   // dK += dS^T . Q
            tc_mma_f16(tmem_dk, ddst + (uint64_t)(k * 2), bq + (uint64_t)(k * 128), idesc_kn,
                       (it > 0 || k > 0) ? 1u : 0u);
          tc_commit(bar_acc);
        }
        if (it + 2 < niter) {
          ok = mbar_wait(bar_acc, it & 1, abort_flag, status, 56);
          if (!ok) break;
          load_qd(it + 2);
        }
      }
    }
    __syncwarp();
  } else {
    // eight warps: warp w works on the 32 key rows of TMEM quadrant w % 4 and on the 32-query
    // half w / 4 of every block
    const int quad = warp & 3, hc = warp >> 2;
    const int row = quad * 32 + lane;       // key row in the tile
    const int kj = k0 + row;
    const bool row_ok = kj < seq;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    uint8_t* pt_smem = gbase + BwdKSmem::PT_OFF;
    uint8_t* dst_smem = gbase + BwdKSmem::DST_OFF;
    const float c2 = scale * 1.4426950408889634f;
    bool ok = true;
    for (int it = 0; ok && it < niter; ++it) {
      const int g = it / nqb, i = it % nqb, h = kvh * group + g;
      const int qs = k0 + i * 64;
      // per-query {Delta, LSE in the log2 domain} of this warp's 32 queries: every key row needs
      // the same pairs, so each warp stages its own copy in shared memory (no cross-warp barrier)
      float2* qi_s = (float2*)(gbase + BwdKSmem::ROW_OFF) + warp * 32;
      {
        const float2* qinfo = (const float2*)(stats + 2 * (((size_t)b * heads + h) * seq));
        __syncwarp();
        float2 dl = qinfo[min(qs + hc * 32 + lane, seq - 1)];
        dl.y *= 1.4426950408889634f;
        qi_s[lane] = dl;
        __syncwarp();
      }
      ok = mbar_wait(bar_spfull, it & 1, abort_flag, status, 61);
      if (!ok) break;
      tc_fence_after();
      const bool need_mask = qs < k0 + AT_KV - 1 || qs + 64 > seq;
      uint32_t pk_p[16], pk_ds[16];
      {
        uint32_t rs[32], rp[32];
        tc_ld32(tmem_st + lane_addr + hc * 32, rs);
        tc_ld32(tmem_dpt + lane_addr + hc * 32, rp);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float pv[2], dsv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int qq = qs + hc * 32 + c + e;
            const float2 dl = qi_s[c + e];   // x = Delta, y = LSE (log2 domain)
            float p = ex2(fmaf(__uint_as_float(rs[c + e]), c2, -dl.y));
            if (!row_ok || (need_mask && (kj > qq || qq >= seq))) p = 0.f;
            pv[e] = p;
            dsv[e] = p * (__uint_as_float(rp[c + e]) - dl.x);
          }
          pk_p[c >> 1] = pack_h2(pv[0], pv[1]);
          pk_ds[c >> 1] = pack_h2(dsv[0], dsv[1]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_spfree);
      if (it > 0) {
        ok = mbar_wait(bar_acc, (it - 1) & 1, abort_flag, status, 62);
        if (!ok) break;
      }
      const int off = (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int sw = (((hc * 4 + q) ^ (row & 7)) << 4);
        *(uint4*)(pt_smem + off + sw) = make_uint4(pk_p[4 * q], pk_p[4 * q + 1], pk_p[4 * q + 2], pk_p[4 * q + 3]);
        *(uint4*)(dst_smem + off + sw) = make_uint4(pk_ds[4 * q], pk_ds[4 * q + 1], pk_ds[4 * q + 2], pk_ds[4 * q + 3]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_dsfull);
    }
    if (ok) ok = mbar_wait(bar_acc, (niter - 1) & 1, abort_flag, status, 63);
    if (ok) {
      tc_fence_after();
      const float inv_s = inv_scale_ptr ? *inv_scale_ptr : 1.0f;
      const float ak = scale * inv_s, av = inv_s;
      float am = 0.f;
      {
        const int cb = hc;
        uint32_t rk[32], rv[32];
        tc_ld32(tmem_dk + lane_addr + cb * 32, rk);
        tc_ld32(tmem_dv + lane_addr + cb * 32, rv);
        tc_wait_ld();
        if (row_ok) {
          const long long tok = (long long)tok0 + kj;
          float* ok_ = dk + tok * ldd + (long long)kvh * AT_D + cb * 32;
          float* ov_ = dv + tok * ldd + (long long)kvh * AT_D + cb * 32;
#pragma unroll
          for (int i2 = 0; i2 < 32; i2 += 4) {
            *(float4*)(ok_ + i2) = make_float4(ak * __uint_as_float(rk[i2]), ak * __uint_as_float(rk[i2 + 1]),
                                               ak * __uint_as_float(rk[i2 + 2]), ak * __uint_as_float(rk[i2 + 3]));
            *(float4*)(ov_ + i2) = make_float4(av * __uint_as_float(rv[i2]), av * __uint_as_float(rv[i2 + 1]),
                                               av * __uint_as_float(rv[i2 + 2]), av * __uint_as_float(rv[i2 + 3]));
#pragma unroll
            for (int e = 0; e < 4; ++e)
              am = fmaxf(am, fmaxf(fabsf(ak * __uint_as_float(rk[i2 + e])), fabsf(av * __uint_as_float(rv[i2 + e]))));
          }
        }
      }
      if (amax_slot) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        if (lane == 0 && am > 0.f && __float_as_int(am) > *(volatile int*)amax_slot)
          atomicMax(amax_slot, __float_as_int(am));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == BW_ISSUER) {
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

// Backward on f16 operands: qkv16 rows (RoPE applied), o16 = forward output, do16 = output
// gradient times the power-of-two scale whose inverse is *inv_scale (device scalar, may be
// NULL = 1).  stats holds the forward log-sum-exp at [2*row+1]; [2*row] receives Delta.
// Writes dq [tokens, lddq] (heads*64 columns from dq), dk and dv [tokens, ldd] (kv_heads*64).
int ft_attention_bwd_tc_v1(FtContext* ctx, const __half* qkv16, long long ld, int q_col0, int k_col0,
                        int v_col0, const __half* o16, long long ldo, const __half* do16,
                        long long lddo, float* dq, long long lddq, float* dk, float* dv,
                        long long ldd, float* stats, const float* inv_scale, int batch, int seq,
                        int heads, int kv_heads, int head_dim) {
  auto bad16 = [](const void* p, long long l) { return (l % 8) || (((uintptr_t)p) & 15); };
  auto bad32 = [](const void* p, long long l) { return (l % 4) || (((uintptr_t)p) & 15); };
  if (head_dim != AT_D || bad16(qkv16, ld) || bad16(o16, ldo) || bad16(do16, lddo) ||
      bad32(dq, lddq) || bad32(dk, ldd) || bad32(dv, ldd) || (q_col0 % 8) || (k_col0 % 8) ||
      (v_col0 % 8) || !stats)
    return FT_ERR_UNSUPPORTED;
  FT_REQUIRE((long long)batch * heads <= 65535, "attention: batch*heads exceeds 65535");
  const uint64_t T = (uint64_t)batch * seq;
  CUtensorMap q128, kv64, do128, do64;
  FT_TRY(ft_tc::make_map(ctx, &q128, qkv16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (uint64_t)ld, T, (uint64_t)ld, 64, 128));
  FT_TRY(ft_tc::make_map(ctx, &kv64, qkv16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (uint64_t)ld, T, (uint64_t)ld, 64, 64));
  FT_TRY(ft_tc::make_map(ctx, &do128, do16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (uint64_t)lddo, T, (uint64_t)lddo, 64, 128));
  FT_TRY(ft_tc::make_map(ctx, &do64, do16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (uint64_t)lddo, T, (uint64_t)lddo, 64, 64));
  static bool configured[FT_MAX_DEVICES] = {};   // function attributes are per device
  if (!configured[ctx->device]) {
    FT_CUDA(cudaFuncSetAttribute(k_attn_bwd_dq_tc, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 BwdQSmem::DYN_BYTES));
    FT_CUDA(cudaFuncSetAttribute(k_attn_bwd_dkv_tc, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 BwdKSmem::DYN_BYTES));
    configured[ctx->device] = true;
  }
  const float scale = 1.0f / sqrtf((float)head_dim);
  int* am = ctx->amax_out;   // armed: the gradients' largest magnitude goes to the amax slot
  if (am) ctx->amax_ready = true;
  {
    dim3 grid(ft_cdiv(seq, AT_Q), batch * heads);
    FT_LAUNCH_PDL(ctx, k_attn_bwd_dq_tc, grid, BW_THREADS, BwdQSmem::DYN_BYTES, q128, kv64, do128, do16,
              lddo, o16, ldo, dq, lddq, stats, seq, heads, kv_heads, q_col0, k_col0, v_col0, scale,
              inv_scale, am, ctx->status_dev);
  }
  {
    dim3 grid(ft_cdiv(seq, AT_KV), batch * kv_heads);
    FT_LAUNCH_PDL(ctx, k_attn_bwd_dkv_tc, grid, BW_THREADS, BwdKSmem::DYN_BYTES, q128, kv64, do64, dk, dv,
              ldd, stats, seq, heads, kv_heads, q_col0, k_col0, v_col0, scale, inv_scale, am,
              ctx->status_dev);
  }
  return FT_OK;
}
