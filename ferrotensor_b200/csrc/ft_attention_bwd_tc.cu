// Backward of causal flash attention on the Blackwell tensor cores (head_dim 64, f16 operands,
// f32 accumulation), grouped-query.  Arithmetic to match:
// ferrotensor-backend/src/shaders/flash_attention_v2_backward.wgsl:212-460
// (P = exp(s - LSE), dS = P (dP - Delta), dQ = scale dS K, dK = scale dS^T Q, dV = P^T dO).
//
// Two persistent kernels, no atomics on results (identical from run to run):
//   k_attn_bwd_dq_tc2   a CTA walks (128 queries, head) tiles; per 128-key block
//                       S = Q K^T and dP = dO V^T land in tensor memory, eight warps turn them
//                       into dS = P (dP - Delta) (thread = query row x 64 keys), write it BACK
//                       to tensor memory as packed f16 over the S columns it came from, and
//                       dQ += dS K runs with its A operand read from tensor memory.  Delta =
//                       dO . O per row is made by a warp of its own from the dO and O tiles in
//                       shared memory, one tile ahead, and stored for the second kernel.
//   k_attn_bwd_dkv_tc2  a CTA walks (128 keys, KV head) tiles; per query head of the group and
//                       128-query block at or below the diagonal S^T = K Q^T, dP^T = V dO^T,
//                       then dV += P^T dO and dK += dS^T Q with P^T and dS^T as tensor-memory
//                       A operands.
// Nothing goes through shared memory between the softmax arithmetic and the products that
// consume it, S is double-buffered (the products of block j+1 run under the arithmetic of
// block j), and one CTA per SM owns all 512 tensor-memory columns.  A loader warp keeps a
// three-deep ring of streamed tiles and the next tile's resident operands in flight; barrier
// phases run on across tiles, counted in blocks since the CTA started.  What a tile costs
// besides its blocks is kept off the math warps' path: the accumulators of a finished tile
// are read and stored only after the first block of the next tile (its products run
// meanwhile), per-row inputs are fetched a tile or a block ahead, and the largest magnitude
// is folded once per kernel.
// Measured on B200: a tcgen05.mma 128 x 128 x 16 occupies the tensor pipe for 64 cycles, a
// 128 x 64 x 16 for 46-48 (operands in shared or tensor memory alike), so one 128 x 128 block
// is about 800 cycles of products in the dQ kernel and 1270 in the dK/dV kernel; the
// exponentials (16 per cycle and SM) take 1024.
// dO arrives as f16 after a power-of-two scale (gradients are far below f16's normal range);
// everything downstream is linear in dO, so the epilogues multiply by 1/scale.
// All waits are bounded (ft_tc.cuh).
#include <math.h>
#include <stdlib.h>

#include "ft_tc.cuh"

namespace {

using namespace ft_tc;

constexpr int BT = 128;                  // queries per tile, keys per block (and vice versa)
constexpr int BD = 64;                   // head_dim
constexpr int TILE = BT * BD * 2;        // one 128 x 64 f16 tile = 16 KiB
constexpr int NWARP_MATH = 8;
constexpr int W_MMA = 8, W_LOAD = 9, W_DELTA = 10;
constexpr int DQ_THREADS = 352;          // math 0..7, products 8, loads 9, Delta 10
constexpr int DKV_THREADS = 320;         // math 0..7, products 8, loads 9
constexpr int RING = 3;                  // streamed tiles in flight
constexpr uint32_t TMEM_ALL = 512;
constexpr float LOG2E = 1.4426950408889634f;

// Cycle accounting (builds with -DFT_ATTN_TIMING only): TSTAMP(k) adds the cycles since the
// previous stamp to accumulator k, kept in registers and written out once when the warp is done.
#ifdef FT_ATTN_TIMING
__device__ long long g_bwd_timing[64];
#define TSTAMP_DECL long long _acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long _t0 = clock64()
#define TSTAMP(k) do { const long long _t1 = clock64(); _acc[k] += _t1 - _t0; _t0 = _t1; } while (0)
#define TSTAMP_FLUSH(base) do { if (blockIdx.x == 0) for (int _i = 0; _i < 8; ++_i) g_bwd_timing[(base) + _i] = _acc[_i]; } while (0)
#else
#define TSTAMP_DECL do { } while (0)
#define TSTAMP(k) do { } while (0)
#define TSTAMP_FLUSH(base) do { } while (0)
#endif

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// CTAs take the tiles of even rounds in index order and of odd rounds in reverse (tiles are
// sorted heavy first), which evens out the per-CTA totals.
__device__ __forceinline__ int snake(int it) {
  const int c = (it & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
  return it * (int)gridDim.x + c;
}

struct Smem {
  // resident operands (Q, dO, O | K, V), double-buffered by tile parity; streamed ring of two
  // operands (K, V | Q, dO)
  static constexpr int RES_A = 0;                       // 2 x 16 KiB
  static constexpr int RES_B = RES_A + 2 * TILE;        // 2 x 16 KiB
  static constexpr int RES_C = RES_B + 2 * TILE;        // 2 x 16 KiB (dQ kernel: the O tile)
  static constexpr int RING_A = RES_C + 2 * TILE;       // RING x 16 KiB
  static constexpr int RING_B = RING_A + RING * TILE;   // RING x 16 KiB
  static constexpr int INFO = RING_B + RING * TILE;     // dQ kernel: 2 x 128 x {Delta, LSE}
  static constexpr int ROW = INFO + 2 * BT * 8;         // dK/dV kernel: per warp 64 x {Delta, LSE}
  static constexpr int BAR = ROW + NWARP_MATH * 64 * 8;
  static constexpr int NBAR = 24;
  static constexpr int TOTAL = BAR + NBAR * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

// barrier indices
enum {
  B_RES_FULL = 0,   // [2]
  B_RES_FREE = 2,   // [2]
  B_RING_FULL = 4,  // [RING]
  B_RING_FREE = 7,  // [RING]
  B_S_FULL = 10,    // [2]
  B_DP_FULL = 12,
  B_DP_FREE = 13,
  B_DS_FULL = 14,   // [2]: by block parity, so a waiter can never fall two completions behind
  B_ACC_DONE = 16,
  B_ACC_READ = 17,
  B_INFO_FULL = 18, // [2]
  B_INFO_FREE = 20, // [2]
};

struct Common {
  uint32_t base, bar0, tmem;
  uint8_t* gbase;
  volatile int* abort_flag;
  int* status;
  __device__ __forceinline__ uint32_t bar(int i) const { return bar0 + 8u * (uint32_t)i; }
  __device__ __forceinline__ bool wait(int i, uint32_t parity, int where) const {
    return mbar_wait(bar(i), parity & 1u, abort_flag, status, where);
  }
};

// Barriers, tensor memory and the abort flag; every thread of the CTA calls this.
// res_free_count: arrivals that free a resident buffer (the last product that reads it, plus
// the Delta warp in the dQ kernel).
__device__ __forceinline__ void cta_setup(Common& c, uint8_t* smem_raw, int* status, int res_free_count) {
  const uint32_t raw = smem_u32(smem_raw);
  c.base = (raw + 1023u) & ~1023u;
  c.gbase = smem_raw + (c.base - raw);
  c.bar0 = c.base + Smem::BAR;
  c.status = status;
  uint32_t* tmem_slot = (uint32_t*)(c.gbase + Smem::BAR + Smem::NBAR * 8);
  c.abort_flag = (volatile int*)(tmem_slot + 1);
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(c.bar(B_RES_FULL + i), 1);
      mbar_init(c.bar(B_RES_FREE + i), res_free_count);
      mbar_init(c.bar(B_S_FULL + i), 1);
      mbar_init(c.bar(B_DS_FULL + i), NWARP_MATH);
      mbar_init(c.bar(B_INFO_FULL + i), 1);
      mbar_init(c.bar(B_INFO_FREE + i), NWARP_MATH);
    }
    for (int i = 0; i < RING; ++i) {
      mbar_init(c.bar(B_RING_FULL + i), 1);
      mbar_init(c.bar(B_RING_FREE + i), 1);
    }
    mbar_init(c.bar(B_DP_FULL), 1);
    mbar_init(c.bar(B_DP_FREE), NWARP_MATH);
    mbar_init(c.bar(B_ACC_DONE), 1);
    mbar_init(c.bar(B_ACC_READ), NWARP_MATH);
    *c.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == W_MMA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(TMEM_ALL)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem = *tmem_slot;
}

__device__ __forceinline__ void cta_teardown(const Common& c) {
  tc_fence_before();
  __syncthreads();
  if (*c.abort_flag) {
    // a bounded wait ran out: let copies and products in flight land before the memory goes
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if ((threadIdx.x >> 5) == W_MMA) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(c.tmem), "r"(TMEM_ALL)
                 : "memory");
  }
}

// D[128 x N] = A[128 x 64] . B[N x 64]^T, both operands K-major 128-byte-swizzled tiles
__device__ __forceinline__ void mma_kk(uint32_t d, uint32_t sa, uint32_t sb, uint32_t idesc) {
  const uint64_t da = make_desc_sw128(sa), db = make_desc_sw128(sb);
#pragma unroll
  for (int k = 0; k < 4; ++k)
    tc_mma_f16(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, k > 0 ? 1u : 0u);
}
// D[128 x 64] (+)= A[128 x 128] . B[128 x 64]: A = packed f16 pairs in tensor memory, 8 columns
// per 16-deep step; step k of the contraction sits at a_col(k).  B = a [128 rows x 64] tile used
// in place with the rows as the contraction index (two 8-row atoms = 2048 bytes per step).
template <typename ColFn>
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a_base, ColFn a_col, uint32_t sb,
                                       uint32_t idesc, bool accumulate) {
  const uint64_t db = make_desc_mn_sw128(sb, TILE / 2);
#pragma unroll
  for (int k = 0; k < 8; ++k)
    tc_mma_f16_ts(d, a_base + (uint32_t)a_col(k), db + (uint64_t)(k * 128), idesc,
                  (accumulate || k > 0) ? 1u : 0u);
}

// the largest magnitude this warp has written -> the armed amax slot, once per kernel
__device__ __forceinline__ void fold_amax(float am, int* amax_slot, int lane) {
  if (!amax_slot) return;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  if (lane == 0 && am > 0.f) atomicMax(amax_slot, __float_as_int(am));
}

// Optional f16 form of the results: rows [tokens, ld] of S * (dq | dk | dv) with the inverse
// rotary rotation applied to dq and dk (angles from `table`, {cos, sin} transposed: [32, seq]); S is the
// power of two carried from *carry_amax (the largest magnitude of the same gradient in the block
// processed before this one).  When `rows` is set the f32 results are not written.
struct Out16 {
  __half* rows;
  long long ld;
  const float2* table;
  const int* carry_amax;
  int carry_exp;
  float* carry_scales;
};

// Sixteen of a thread's 32 components of a gradient row (half `hc` of the 64), rotated back by
// the angles of one position and scaled: ra = raw accumulator words of components c..c+15,
// rb = of components 32+c..32+c+15, f their factor, tcol = the position's {cos, sin} of component
// c in the transposed table ([32][seq]: the next component is `seq` entries further; lanes own
// consecutive positions, so the warp's loads are contiguous); writes 16 halves to dst.
__device__ __forceinline__ void store_rot16(__half* dst, const uint32_t (&ra)[16], const uint32_t (&rb)[16],
                                            float f, int hc, const float2* __restrict__ tcol, size_t seq,
                                            float S, float& am) {
  uint32_t w[8];
  const float fs = f * S;   // S is a power of two: exact
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const float2 c0 = tcol[0], c1 = tcol[seq];
    tcol += 2 * seq;
    const float a0 = __uint_as_float(ra[i]), a1 = __uint_as_float(ra[i + 1]);
    const float b0 = __uint_as_float(rb[i]), b1 = __uint_as_float(rb[i + 1]);
    float o0, o1;
    if (hc == 0) {   // first half: a cos + b sin
      o0 = a0 * c0.x + b0 * c0.y;
      o1 = a1 * c1.x + b1 * c1.y;
      am = fmaxf(am, fmaxf(fabsf(a0), fabsf(a1)));
    } else {         // second half: b cos - a sin
      o0 = b0 * c0.x - a0 * c0.y;
      o1 = b1 * c1.x - a1 * c1.y;
      am = fmaxf(am, fmaxf(fabsf(b0), fabsf(b1)));
    }
    w[i >> 1] = pack_h2(o0 * fs, o1 * fs);
  }
  *(uint4*)dst = make_uint4(w[0], w[1], w[2], w[3]);
  *(uint4*)(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
}
__device__ __forceinline__ void store_plain16(__half* dst, const uint32_t (&r)[16], float f, float S,
                                              float& am) {
  uint32_t w[8];
  const float fs = f * S;
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const float v0 = __uint_as_float(r[i]), v1 = __uint_as_float(r[i + 1]);
    am = fmaxf(am, fmaxf(fabsf(v0), fabsf(v1)));
    w[i >> 1] = pack_h2(v0 * fs, v1 * fs);
  }
  *(uint4*)dst = make_uint4(w[0], w[1], w[2], w[3]);
  *(uint4*)(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
}

// The dK/dV kernel's f16 epilogue of one thread (kept out of line: the kernel's main loop
// needs every register it can have, and this runs once per tile).  dK rotated back (component
// i pairs with i + 32), then dV, sixteen components at a time; arrives on `bar_read` once the
// accumulators have been read; returns the largest magnitude written, before the carried scale.
__device__ __noinline__ float dkv_store16(uint32_t t_dk_lane, uint32_t t_dv_half, int hc, __half* k16,
                                          __half* v16, const float2* __restrict__ tcol, size_t seq, float ak,
                                          float av, float s16, uint32_t bar_read, int lane) {
  float amk = 0.f, amv = 0.f;
  uint32_t ra[16], rb[16];
  tc_ld16(t_dk_lane, ra);
  tc_ld16(t_dk_lane + 32, rb);
  tc_wait_ld();
  if (k16) store_rot16(k16, ra, rb, ak, hc, tcol, seq, s16, amk);
  tc_ld16(t_dk_lane + 16, ra);
  tc_ld16(t_dk_lane + 48, rb);
  tc_wait_ld();
  if (k16) store_rot16(k16 + 16, ra, rb, ak, hc, tcol + 16 * seq, seq, s16, amk);
  tc_ld16(t_dv_half, ra);
  tc_ld16(t_dv_half + 16, rb);
  tc_wait_ld();
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar_read);
  if (v16) {
    store_plain16(v16, ra, av, s16, amv);
    store_plain16(v16 + 16, rb, av, s16, amv);
  }
  return fmaxf(ak * amk, av * amv);
}

// =========================================================================================
// dQ
// =========================================================================================
struct QTile {
  int q0, nblk, b, h, kvh, tok0;
};
__device__ __forceinline__ bool q_tile(int t, int total, int nqt, int bh_count, int heads, int kv_heads,
                                       int seq, QTile& w) {
  if (t >= total) return false;
  const int qblk = nqt - 1 - t / bh_count;   // late (long) query tiles first
  const int bh = t % bh_count;
  w.b = bh / heads;
  w.h = bh % heads;
  w.kvh = w.h / (heads / kv_heads);
  w.q0 = qblk * BT;
  w.nblk = qblk + 1;                         // 128-key blocks at or below the diagonal
  w.tok0 = w.b * seq;
  return true;
}

__global__ void __launch_bounds__(DQ_THREADS, 1)
k_attn_bwd_dq_tc2(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do,
                  const __grid_constant__ CUtensorMap map_o, float* __restrict__ dq, long long lddq,
                  float* __restrict__ stats, int seq, int heads, int kv_heads, int bh_count, int q_col0,
                  int k_col0, int v_col0, float scale, const float* __restrict__ inv_scale_ptr,
                  int* amax_slot, int* status, Out16 o16) {
  extern __shared__ uint8_t smem_raw[];
  Common c;
  cta_setup(c, smem_raw, status, 2);
  ft_pdl_wait();
  ft_pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqt = (seq + BT - 1) / BT, total = nqt * bh_count;
  // tensor memory: S0 [0,128) S1 [128,256) dP [256,384) dQ [384,448)
  const uint32_t t_s = c.tmem, t_dp = c.tmem + 256, t_dq = c.tmem + 384;
  const uint32_t s_q = c.base + Smem::RES_A, s_do = c.base + Smem::RES_B, s_o = c.base + Smem::RES_C,
                 s_k = c.base + Smem::RING_A, s_v = c.base + Smem::RING_B;

  if (warp == W_LOAD) {
    if (elect_one()) {
      uint32_t g = 0;
      bool ok = true;
      QTile w;
      for (int it = 0; ok && q_tile(snake(it), total, nqt, bh_count, heads, kv_heads, seq, w); ++it) {
        const int rb = it & 1;
        if (it >= 2) {
          ok = c.wait(B_RES_FREE + rb, (uint32_t)((it >> 1) - 1), 71);
          if (!ok) break;
        }
        mbar_expect_tx(c.bar(B_RES_FULL + rb), 3 * TILE);
        tma_load_2d(s_q + rb * TILE, &map_qkv, c.bar(B_RES_FULL + rb), q_col0 + w.h * BD, w.tok0 + w.q0);
        tma_load_2d(s_do + rb * TILE, &map_do, c.bar(B_RES_FULL + rb), w.h * BD, w.tok0 + w.q0);
        tma_load_2d(s_o + rb * TILE, &map_o, c.bar(B_RES_FULL + rb), w.h * BD, w.tok0 + w.q0);
        for (int j = 0; j < w.nblk; ++j, ++g) {
          const uint32_t st = g % RING;
          if (g >= RING) {
            ok = c.wait(B_RING_FREE + st, g / RING - 1, 72);
            if (!ok) break;
          }
          mbar_expect_tx(c.bar(B_RING_FULL + st), 2 * TILE);
          tma_load_2d(s_k + st * TILE, &map_qkv, c.bar(B_RING_FULL + st), k_col0 + w.kvh * BD, w.tok0 + j * BT);
          tma_load_2d(s_v + st * TILE, &map_qkv, c.bar(B_RING_FULL + st), v_col0 + w.kvh * BD, w.tok0 + j * BT);
        }
      }
    }
    __syncwarp();
  } else if (warp == W_DELTA) {
    // Delta = dO . O of the tile's 128 rows from the two tiles in shared memory (the swizzle
    // permutes the 16-byte pieces of a row identically in both, so piece i meets piece i), the
    // rows' log-sum-exp from global memory; both go to shared memory for the math warps, Delta
    // also to `stats` for the second kernel.  Runs up to a tile ahead of the math warps.
    bool ok = true;
    QTile w;
    for (int it = 0; ok && q_tile(snake(it), total, nqt, bh_count, heads, kv_heads, seq, w); ++it) {
      const int rb = it & 1;
      float lse[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int qi = w.q0 + lane + 32 * i;
        lse[i] = qi < seq ? stats[2 * (((size_t)w.b * heads + w.h) * seq + qi) + 1] * LOG2E : 0.f;
      }
      ok = c.wait(B_RES_FULL + rb, (uint32_t)(it >> 1), 78);
      if (ok && it >= 2) ok = c.wait(B_INFO_FREE + rb, (uint32_t)((it >> 1) - 1), 79);
      if (!ok) break;
      float2* info = (float2*)(c.gbase + Smem::INFO) + rb * BT;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = lane + 32 * i;
        const uint8_t* pd = c.gbase + Smem::RES_B + rb * TILE + r * 128;
        const uint8_t* po = c.gbase + Smem::RES_C + rb * TILE + r * 128;
        float delta = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int piece = ((k + lane) & 7) * 16;   // lanes start at different pieces: no bank conflict
          const uint4 a = *(const uint4*)(pd + piece), o = *(const uint4*)(po + piece);
          const __half2* ha = (const __half2*)&a;
          const __half2* ho = (const __half2*)&o;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 fa = __half22float2(ha[t]), fo = __half22float2(ho[t]);
            delta = fmaf(fa.x, fo.x, fmaf(fa.y, fo.y, delta));
          }
        }
        info[r] = make_float2(delta, lse[i]);
        const int qi = w.q0 + r;
        if (qi < seq) stats[2 * (((size_t)w.b * heads + w.h) * seq + qi)] = delta;
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(c.bar(B_INFO_FULL + rb));
        mbar_arrive(c.bar(B_RES_FREE + rb));   // this warp is done with the dO and O tiles
      }
    }
  } else if (warp == W_MMA) {
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc(128, 128, 0, 0);               // both operands K-major
      const uint32_t idesc_o = make_idesc(128, 64, 0, 0) | (1u << 16);   // B: rows = contraction
      // two cursors over the CTA's sequence of (tile, block) pairs: the S / dP products run one
      // block ahead of the dQ product
      struct Cur { int it, j; bool has; QTile w; };
      auto start = [&](Cur& u) { u.it = 0; u.j = 0; u.has = q_tile(snake(0), total, nqt, bh_count, heads, kv_heads, seq, u.w); };
      auto advance = [&](Cur& u) {
        if (++u.j < u.w.nblk) return;
        u.j = 0; ++u.it;
        u.has = q_tile(snake(u.it), total, nqt, bh_count, heads, kv_heads, seq, u.w);
      };
      Cur A, D;           // A: block whose S and dP are issued next; D: block whose dQ is next
      start(A); start(D);
      uint32_t ga = 0, gd = 0;
      bool ok = true;
      auto issue_s = [&]() -> bool {
        if (A.j == 0 && !c.wait(B_RES_FULL + (A.it & 1), (uint32_t)(A.it >> 1), 73)) return false;
        if (!c.wait(B_RING_FULL + ga % RING, ga / RING, 74)) return false;
        tc_fence_after();
        mma_kk(t_s + (ga & 1) * 128, s_q + (A.it & 1) * TILE, s_k + (ga % RING) * TILE, idesc_s);
        tc_commit(c.bar(B_S_FULL + (ga & 1)));
        return true;
      };
      auto issue_dp = [&]() {
        mma_kk(t_dp, s_do + (A.it & 1) * TILE, s_v + (ga % RING) * TILE, idesc_s);
        tc_commit(c.bar(B_DP_FULL));
        if (A.j == A.w.nblk - 1) tc_commit(c.bar(B_RES_FREE + (A.it & 1)));   // last product on Q, dO
        advance(A);
        ++ga;
      };
      if (D.has) {
        ok = issue_s();
        if (ok) issue_dp();
      }
      TSTAMP_DECL;
      while (ok && D.has) {
        if (A.has) {
          // S of the next block goes into the other S buffer; dP has one buffer, which the math
          // warps must have read first
          ok = issue_s();
          TSTAMP(0);
          ok = ok && c.wait(B_DP_FREE, gd, 75);
          if (!ok) break;
          TSTAMP(1);
          tc_fence_after();
          issue_dp();
          TSTAMP(2);
        }
        ok = c.wait(B_DS_FULL + (gd & 1), gd >> 1, 76);
        // a tile's first dQ product overwrites the accumulator: the previous tile's must have
        // been read (the math warps do that right after this tile's first block)
        if (ok && D.j == 0 && D.it >= 1) ok = c.wait(B_ACC_READ, (uint32_t)(D.it - 1), 77);
        if (!ok) break;
        tc_fence_after();
        // dQ += dS[128 q x 128 keys] . K[128 keys x 64]; warp half h left its 64 keys as 32
        // columns at h * 64 of the S buffer
        TSTAMP(3);
        mma_ts(t_dq, t_s + (gd & 1) * 128, [](int k) { return (k >> 2) * 64 + (k & 3) * 8; },
               s_k + (gd % RING) * TILE, idesc_o, D.j > 0);
        tc_commit(c.bar(B_RING_FREE + gd % RING));
        if (D.j == D.w.nblk - 1) tc_commit(c.bar(B_ACC_DONE));
        advance(D);
        ++gd;
        TSTAMP(4);
      }
#ifdef FT_ATTN_TIMING
      _acc[5] = gd;
#endif
      TSTAMP_FLUSH(8);
    }
    __syncwarp();
  } else {
    // eight math warps: warp w works on the 32 query rows of lane quadrant w % 4 and on the
    // 64-key half w / 4 of every block
    const int quad = warp & 3, hc = warp >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const float c2 = scale * LOG2E;
    const float alpha = scale * (inv_scale_ptr ? *inv_scale_ptr : 1.0f);
    float am = 0.f;
    uint32_t g = 0;
    bool ok = true;
    TSTAMP_DECL;
    // a finished tile whose accumulator has not been stored yet
    bool pend = false;
    int pend_it = 0;
    float* pend_out = nullptr;
    __half* pend16 = nullptr;
    int pend_pos = 0;
    float s16 = 1.0f;
    if (o16.rows) {
      s16 = ft_scale_from_amax_bits(*o16.carry_amax, o16.carry_exp);
      if (blockIdx.x == 0 && threadIdx.x == 0) ft_publish_scales(o16.carry_scales, s16);
    }
    auto flush = [&]() -> bool {
      if (!pend) return true;
      pend = false;
      if (!c.wait(B_ACC_DONE, (uint32_t)pend_it, 83)) return false;
      tc_fence_after();
      if (o16.rows) {
        // the rotation pairs component i with i + 32: sixteen components of either half at a
        // time (magnitudes are folded raw and scaled by alpha once)
        float amr = 0.f;
        const float2* tcol = o16.table + pend_pos;   // transposed table: [32][seq]
        uint32_t ra[16], rb[16];
        tc_ld16(t_dq + lane_addr, ra);
        tc_ld16(t_dq + lane_addr + 32, rb);
        tc_wait_ld();
        if (pend16) store_rot16(pend16, ra, rb, alpha, hc, tcol, (size_t)seq, s16, amr);
        tc_ld16(t_dq + lane_addr + 16, ra);
        tc_ld16(t_dq + lane_addr + 48, rb);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(c.bar(B_ACC_READ));
        if (pend16) store_rot16(pend16 + 16, ra, rb, alpha, hc, tcol + 16 * (size_t)seq, (size_t)seq, s16, amr);
        am = fmaxf(am, alpha * amr);
        return true;
      }
      uint32_t r[32];
      tc_ld32(t_dq + lane_addr + hc * 32, r);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(c.bar(B_ACC_READ));
      if (pend_out) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 v = make_float4(alpha * __uint_as_float(r[i]), alpha * __uint_as_float(r[i + 1]),
                                       alpha * __uint_as_float(r[i + 2]), alpha * __uint_as_float(r[i + 3]));
          *(float4*)(pend_out + i) = v;
          am = fmaxf(am, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
      }
      return true;
    };
    QTile w;
    for (int it = 0; ok && q_tile(snake(it), total, nqt, bh_count, heads, kv_heads, seq, w); ++it) {
      const int qi = w.q0 + row;
      const bool row_ok = qi < seq;
      ok = c.wait(B_INFO_FULL + (it & 1), (uint32_t)(it >> 1), 80);
      if (!ok) break;
      const float2 dl = ((const float2*)(c.gbase + Smem::INFO))[(it & 1) * BT + row];
      __syncwarp();
      if (lane == 0) mbar_arrive(c.bar(B_INFO_FREE + (it & 1)));
      const float delta = dl.x, lse2 = dl.y;
      const bool tile_ragged = w.q0 + BT > seq;   // some rows of the tile lie past the sequence
      TSTAMP(0);
      for (int j = 0; ok && j < w.nblk; ++j, ++g) {
        const uint32_t sb = t_s + (g & 1) * 128 + lane_addr + hc * 64;
        ok = c.wait(B_S_FULL + (g & 1), g >> 1, 81) && c.wait(B_DP_FULL, g, 82);
        if (!ok) break;
        TSTAMP(1);
        tc_fence_after();
        const bool diag = j == w.nblk - 1;
        const int key0 = j * BT + hc * 64;
        // dP first and whole: its one buffer is what the next block's products wait for
        uint32_t rp[2][32];
        tc_ld32(t_dp + lane_addr + hc * 64, rp[0]);
        tc_ld32(t_dp + lane_addr + hc * 64 + 32, rp[1]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(c.bar(B_DP_FREE));
        TSTAMP(2);
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          uint32_t rs[32], packed[16];
          tc_ld32(sb + sub * 32, rs);
          tc_wait_ld();
          TSTAMP(3);
          if (diag || tile_ragged) {
            // the block on the diagonal, or a tile that runs past the sequence: per-element mask
#pragma unroll
            for (int cc = 0; cc < 32; cc += 2) {
              float v[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                float p = ex2(fmaf(__uint_as_float(rs[cc + e]), c2, -lse2));
                if (!row_ok || key0 + sub * 32 + cc + e > qi) p = 0.f;
                v[e] = p * (__uint_as_float(rp[sub][cc + e]) - delta);
              }
              packed[cc >> 1] = pack_h2(v[0], v[1]);
            }
          } else {
            // everything visible: packed pair arithmetic, three instructions for two elements
            // beside the exponentials and the rounding
            const float nl = -lse2, nd = -delta;
#pragma unroll
            for (int cc = 0; cc < 32; cc += 2) {
              float x0, x1, t0, t1, v0, v1;
              ffma2(x0, x1, __uint_as_float(rs[cc]), __uint_as_float(rs[cc + 1]), c2, c2, nl, nl);
              fadd2(t0, t1, __uint_as_float(rp[sub][cc]), __uint_as_float(rp[sub][cc + 1]), nd, nd);
              fmul2(v0, v1, ex2(x0), ex2(x1), t0, t1);
              packed[cc >> 1] = pack_h2(v0, v1);
            }
          }
          // dS replaces the S columns this thread has just read (16 columns per 32 keys)
          tc_st16(sb + sub * 16, packed);
          TSTAMP(4);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(c.bar(B_DS_FULL + (g & 1)));
        TSTAMP(5);
        // the previous tile's dQ: its last product has long finished, and this tile's first
        // one waits for exactly this read
        if (j == 0) {
          ok = flush();
          TSTAMP(6);
        }
      }
      if (!ok) break;
      pend = true;
      pend_it = it;
      if (o16.rows) {
        pend16 = row_ok ? o16.rows + ((long long)w.tok0 + qi) * o16.ld + q_col0 + (long long)w.h * BD + hc * 32
                        : nullptr;
        pend_pos = qi;
      } else {
        pend_out = row_ok ? dq + ((long long)w.tok0 + qi) * lddq + (long long)w.h * BD + hc * 32 : nullptr;
      }
      TSTAMP(7);
    }
    if (ok) ok = flush();
    fold_amax(am, amax_slot, lane);
    if (threadIdx.x == 0) TSTAMP_FLUSH(0);
  }
  cta_teardown(c);
}

// =========================================================================================
// dK, dV
// =========================================================================================
struct KTile {
  int k0, nqb, niter, b, kvh, tok0;
};
__device__ __forceinline__ bool k_tile(int t, int total, int nkt, int bk_count, int group, int kv_heads,
                                       int seq, KTile& w) {
  if (t >= total) return false;
  const int kblk = t / bk_count;             // early key tiles see the most queries: first
  const int bk = t % bk_count;
  w.b = bk / kv_heads;
  w.kvh = bk % kv_heads;
  w.k0 = kblk * BT;
  w.nqb = nkt - kblk;                        // 128-query blocks from the diagonal to the end
  w.niter = group * w.nqb;
  w.tok0 = w.b * seq;
  return true;
}

__global__ void __launch_bounds__(DKV_THREADS, 1)
k_attn_bwd_dkv_tc2(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do,
                   float* __restrict__ dk, float* __restrict__ dv, long long ldd,
                   const float* __restrict__ stats, int seq, int heads, int kv_heads, int bk_count,
                   int q_col0, int k_col0, int v_col0, float scale,
                   const float* __restrict__ inv_scale_ptr, int* amax_slot, int* status, Out16 o16) {
  extern __shared__ uint8_t smem_raw[];
  Common c;
  cta_setup(c, smem_raw, status, 1);
  ft_pdl_wait();
  ft_pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = heads / kv_heads;
  const int nkt = (seq + BT - 1) / BT, total = nkt * bk_count;
  // tensor memory: S^T 0 [0,128) S^T 1 [128,256) dP^T [256,384) dK [384,448) dV [448,512)
  const uint32_t t_s = c.tmem, t_dp = c.tmem + 256, t_dk = c.tmem + 384, t_dv = c.tmem + 448;
  const uint32_t s_k = c.base + Smem::RES_A, s_v = c.base + Smem::RES_B,
                 s_q = c.base + Smem::RING_A, s_do = c.base + Smem::RING_B;

  if (warp == W_LOAD) {
    if (elect_one()) {
      uint32_t g = 0;
      bool ok = true;
      KTile w;
      for (int it = 0; ok && k_tile(snake(it), total, nkt, bk_count, group, kv_heads, seq, w); ++it) {
        const int rb = it & 1;
        if (it >= 2) {
          ok = c.wait(B_RES_FREE + rb, (uint32_t)((it >> 1) - 1), 91);
          if (!ok) break;
        }
        mbar_expect_tx(c.bar(B_RES_FULL + rb), 2 * TILE);
        tma_load_2d(s_k + rb * TILE, &map_qkv, c.bar(B_RES_FULL + rb), k_col0 + w.kvh * BD, w.tok0 + w.k0);
        tma_load_2d(s_v + rb * TILE, &map_qkv, c.bar(B_RES_FULL + rb), v_col0 + w.kvh * BD, w.tok0 + w.k0);
        for (int i = 0; i < w.niter; ++i, ++g) {
          const uint32_t st = g % RING;
          if (g >= RING) {
            ok = c.wait(B_RING_FREE + st, g / RING - 1, 92);
            if (!ok) break;
          }
          const int h = w.kvh * group + i / w.nqb, qs = w.k0 + (i % w.nqb) * BT;
          mbar_expect_tx(c.bar(B_RING_FULL + st), 2 * TILE);
          tma_load_2d(s_q + st * TILE, &map_qkv, c.bar(B_RING_FULL + st), q_col0 + h * BD, w.tok0 + qs);
          tma_load_2d(s_do + st * TILE, &map_do, c.bar(B_RING_FULL + st), h * BD, w.tok0 + qs);
        }
      }
    }
    __syncwarp();
  } else if (warp == W_MMA) {
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc(128, 128, 0, 0);
      const uint32_t idesc_o = make_idesc(128, 64, 0, 0) | (1u << 16);
      struct Cur { int it, j; bool has; KTile w; };
      auto start = [&](Cur& u) { u.it = 0; u.j = 0; u.has = k_tile(snake(0), total, nkt, bk_count, group, kv_heads, seq, u.w); };
      auto advance = [&](Cur& u) {
        if (++u.j < u.w.niter) return;
        u.j = 0; ++u.it;
        u.has = k_tile(snake(u.it), total, nkt, bk_count, group, kv_heads, seq, u.w);
      };
      Cur A, D;
      start(A); start(D);
      uint32_t ga = 0, gd = 0;
      bool ok = true;
      auto issue_s = [&]() -> bool {
        if (A.j == 0 && !c.wait(B_RES_FULL + (A.it & 1), (uint32_t)(A.it >> 1), 93)) return false;
        if (!c.wait(B_RING_FULL + ga % RING, ga / RING, 94)) return false;
        tc_fence_after();
        // S^T[128 keys x 128 q] = K . Q^T
        mma_kk(t_s + (ga & 1) * 128, s_k + (A.it & 1) * TILE, s_q + (ga % RING) * TILE, idesc_s);
        tc_commit(c.bar(B_S_FULL + (ga & 1)));
        return true;
      };
      auto issue_dp = [&]() {
        // dP^T[128 keys x 128 q] = V . dO^T
        mma_kk(t_dp, s_v + (A.it & 1) * TILE, s_do + (ga % RING) * TILE, idesc_s);
        tc_commit(c.bar(B_DP_FULL));
        if (A.j == A.w.niter - 1) tc_commit(c.bar(B_RES_FREE + (A.it & 1)));   // last product on K, V
        advance(A);
        ++ga;
      };
      if (D.has) {
        ok = issue_s();
        if (ok) issue_dp();
      }
      while (ok && D.has) {
        if (A.has) {
          ok = issue_s() && c.wait(B_DP_FREE, gd, 95);
          if (!ok) break;
          tc_fence_after();
          issue_dp();
        }
        ok = c.wait(B_DS_FULL + (gd & 1), gd >> 1, 96);
        if (ok && D.j == 0 && D.it >= 1) ok = c.wait(B_ACC_READ, (uint32_t)(D.it - 1), 97);
        if (!ok) break;
        tc_fence_after();
        // Each math warp replaced its 64 S^T columns by [P (16) | dS (16)] for its first 32
        // queries and the same for the next 32: contraction step k (16 queries) of P^T sits at
        // column (k / 2) * 32 + (k % 2) * 8, of dS^T 16 columns further on.
        const uint32_t ab = t_s + (gd & 1) * 128;
        mma_ts(t_dv, ab, [](int k) { return (k >> 1) * 32 + (k & 1) * 8; },
               s_do + (gd % RING) * TILE, idesc_o, D.j > 0);                    // dV += P^T dO
        mma_ts(t_dk, ab, [](int k) { return (k >> 1) * 32 + 16 + (k & 1) * 8; },
               s_q + (gd % RING) * TILE, idesc_o, D.j > 0);                     // dK += dS^T Q
        tc_commit(c.bar(B_RING_FREE + gd % RING));
        if (D.j == D.w.niter - 1) tc_commit(c.bar(B_ACC_DONE));
        advance(D);
        ++gd;
      }
    }
    __syncwarp();
  } else {
    // eight math warps: warp w works on the 32 key rows of lane quadrant w % 4 and on the
    // 64-query half w / 4 of every block
    const int quad = warp & 3, hc = warp >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const float c2 = scale * LOG2E;
    const float inv_s = inv_scale_ptr ? *inv_scale_ptr : 1.0f;
    const float ak = scale * inv_s, av = inv_s;
    float am = 0.f;
    // per-query {Delta, LSE in the log2 domain} of this warp's 64 queries: every key row needs
    // the same pairs, so each warp stages its own copy in shared memory (no cross-warp barrier)
    float* nl_s = (float*)(c.gbase + Smem::ROW) + warp * 128;   // -LSE (log2 domain) of 64 queries
    float* nd_s = nl_s + 64;                                    // -Delta of the same queries
    uint32_t g = 0;
    bool ok = true;
    bool pend = false;
    int pend_it = 0;
    float *pend_k = nullptr, *pend_v = nullptr;
    __half *pend_k16 = nullptr, *pend_v16 = nullptr;
    int pend_pos = 0;
    const float s16 = o16.rows ? ft_scale_from_amax_bits(*o16.carry_amax, o16.carry_exp) : 1.0f;
    auto flush = [&]() -> bool {
      if (!pend) return true;
      pend = false;
      if (!c.wait(B_ACC_DONE, (uint32_t)pend_it, 103)) return false;
      tc_fence_after();
      if (o16.rows) {
        am = fmaxf(am, dkv_store16(t_dk + lane_addr, t_dv + lane_addr + hc * 32, hc, pend_k16, pend_v16,
                                   o16.table + pend_pos, (size_t)seq, ak, av, s16, c.bar(B_ACC_READ),
                                   lane));
        return true;
      }
      uint32_t rk[32], rv[32];
      tc_ld32(t_dk + lane_addr + hc * 32, rk);
      tc_ld32(t_dv + lane_addr + hc * 32, rv);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(c.bar(B_ACC_READ));
      if (pend_k) {
#pragma unroll
        for (int i2 = 0; i2 < 32; i2 += 4) {
          const float4 a = make_float4(ak * __uint_as_float(rk[i2]), ak * __uint_as_float(rk[i2 + 1]),
                                       ak * __uint_as_float(rk[i2 + 2]), ak * __uint_as_float(rk[i2 + 3]));
          const float4 b = make_float4(av * __uint_as_float(rv[i2]), av * __uint_as_float(rv[i2 + 1]),
                                       av * __uint_as_float(rv[i2 + 2]), av * __uint_as_float(rv[i2 + 3]));
          *(float4*)(pend_k + i2) = a;
          *(float4*)(pend_v + i2) = b;
          am = fmaxf(am, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
          am = fmaxf(am, fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
        }
      }
      return true;
    };
    // {Delta, LSE} of query block i of tile u for this warp's lanes (two queries per lane)
    auto fetch_info = [&](const KTile& u, int i, float2& a, float2& b) {
      const int h = u.kvh * group + i / u.nqb, qs = u.k0 + (i % u.nqb) * BT;
      const float2* qinfo = (const float2*)(stats + 2 * (((size_t)u.b * heads + h) * seq));
      a = qinfo[min(qs + hc * 64 + lane, seq - 1)];
      b = qinfo[min(qs + hc * 64 + 32 + lane, seq - 1)];
    };
    KTile w, wn;
    bool has = k_tile(snake(0), total, nkt, bk_count, group, kv_heads, seq, w);
    float2 na = make_float2(0.f, 0.f), nb = na;
    if (has) fetch_info(w, 0, na, nb);
    for (int it = 0; ok && has; ++it) {
      const int kj = w.k0 + row;
      const bool row_ok = kj < seq;
      const bool tile_ragged = w.k0 + BT > seq;   // some key rows of the tile lie past the sequence
      const bool has_next = k_tile(snake(it + 1), total, nkt, bk_count, group, kv_heads, seq, wn);
      for (int i = 0; ok && i < w.niter; ++i, ++g) {
        const int qs = w.k0 + (i % w.nqb) * BT;
        __syncwarp();
        nd_s[lane] = -na.x;
        nl_s[lane] = -na.y * LOG2E;
        nd_s[32 + lane] = -nb.x;
        nl_s[32 + lane] = -nb.y * LOG2E;
        __syncwarp();
        // the next block's pairs (of the next tile after the last block) travel under this
        // block's arithmetic
        if (i + 1 < w.niter) fetch_info(w, i + 1, na, nb);
        else if (has_next) fetch_info(wn, 0, na, nb);
        const uint32_t sb = t_s + (g & 1) * 128 + lane_addr + hc * 64;
        ok = c.wait(B_S_FULL + (g & 1), g >> 1, 101) && c.wait(B_DP_FULL, g, 102);
        if (!ok) break;
        tc_fence_after();
        const bool need_mask = (i % w.nqb) == 0 || qs + BT > seq;
        // dP^T first and whole: its one buffer is what the next block's products wait for
        uint32_t rp[2][32];
        tc_ld32(t_dp + lane_addr + hc * 64, rp[0]);
        tc_ld32(t_dp + lane_addr + hc * 64 + 32, rp[1]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(c.bar(B_DP_FREE));
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          uint32_t rs[32], pk_p[16], pk_ds[16];
          tc_ld32(sb + sub * 32, rs);
          tc_wait_ld();
          if (need_mask || tile_ragged) {
#pragma unroll
            for (int cc = 0; cc < 32; cc += 2) {
              float pv[2], dsv[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int qq = qs + hc * 64 + sub * 32 + cc + e;
                float p = ex2(fmaf(__uint_as_float(rs[cc + e]), c2, nl_s[sub * 32 + cc + e]));
                if (!row_ok || kj > qq || qq >= seq) p = 0.f;
                pv[e] = p;
                dsv[e] = p * (__uint_as_float(rp[sub][cc + e]) + nd_s[sub * 32 + cc + e]);
              }
              pk_p[cc >> 1] = pack_h2(pv[0], pv[1]);
              pk_ds[cc >> 1] = pack_h2(dsv[0], dsv[1]);
            }
          } else {
            // everything visible: packed pair arithmetic on two queries at a time
#pragma unroll
            for (int cc = 0; cc < 32; cc += 2) {
              const float2 nl = *(const float2*)(nl_s + sub * 32 + cc);
              const float2 nd = *(const float2*)(nd_s + sub * 32 + cc);
              float x0, x1, t0, t1, d0, d1;
              ffma2(x0, x1, __uint_as_float(rs[cc]), __uint_as_float(rs[cc + 1]), c2, c2, nl.x, nl.y);
              fadd2(t0, t1, __uint_as_float(rp[sub][cc]), __uint_as_float(rp[sub][cc + 1]), nd.x, nd.y);
              const float p0 = ex2(x0), p1 = ex2(x1);
              fmul2(d0, d1, p0, p1, t0, t1);
              pk_p[cc >> 1] = pack_h2(p0, p1);
              pk_ds[cc >> 1] = pack_h2(d0, d1);
            }
          }
          // the 32 S^T columns just read become [P (16) | dS (16)]
          tc_st16(sb + sub * 32, pk_p);
          tc_st16(sb + sub * 32 + 16, pk_ds);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(c.bar(B_DS_FULL + (g & 1)));
        // the previous tile's dK and dV: their last products have long finished, and this
        // tile's first ones wait for exactly this read
        if (i == 0) ok = flush();
      }
      if (!ok) break;
      pend = true;
      pend_it = it;
      const long long tok = (long long)w.tok0 + kj;
      if (o16.rows) {
        pend_k16 = row_ok ? o16.rows + tok * o16.ld + k_col0 + (long long)w.kvh * BD + hc * 32 : nullptr;
        pend_v16 = row_ok ? o16.rows + tok * o16.ld + v_col0 + (long long)w.kvh * BD + hc * 32 : nullptr;
        pend_pos = kj;
      } else {
        pend_k = row_ok ? dk + tok * ldd + (long long)w.kvh * BD + hc * 32 : nullptr;
        pend_v = row_ok ? dv + tok * ldd + (long long)w.kvh * BD + hc * 32 : nullptr;
      }
      w = wn;
      has = has_next;
    }
    if (ok) ok = flush();
    fold_amax(am, amax_slot, lane);
  }
  cta_teardown(c);
}

}  // namespace

#ifdef FT_ATTN_TIMING
// Reads the cycle counters CTA 0 left (timing builds only).
extern "C" int ft_debug_attn_timing(long long* out64) {
  FT_CUDA(cudaDeviceSynchronize());
  FT_CUDA(cudaMemcpyFromSymbol(out64, g_bwd_timing, sizeof(long long) * 64));
  return FT_OK;
}
#endif

// Backward on f16 operands: qkv16 rows (RoPE applied), o16 = forward output, do16 = output
// gradient times the power-of-two scale whose inverse is *inv_scale (device scalar, may be
// NULL = 1).  stats holds the forward log-sum-exp at [2*row+1]; [2*row] receives Delta.
// Writes dq [tokens, lddq] (heads*64 columns from dq), dk and dv [tokens, ldd] (kv_heads*64).
int ft_attention_bwd_tc(FtContext* ctx, const __half* qkv16, long long ld, int q_col0, int k_col0,
                        int v_col0, const __half* o16, long long ldo, const __half* do16,
                        long long lddo, float* dq, long long lddq, float* dk, float* dv,
                        long long ldd, float* stats, const float* inv_scale, int batch, int seq,
                        int heads, int kv_heads, int head_dim, const FtAttnBwdOut16* out16) {
  auto bad16 = [](const void* p, long long l) { return (l % 8) || (((uintptr_t)p) & 15); };
  auto bad32 = [](const void* p, long long l) { return (l % 4) || (((uintptr_t)p) & 15); };
  Out16 o;
  memset(&o, 0, sizeof(o));
  if (out16 && out16->rows) {
    // the f16 rows share the q|k|v column layout of the operands
    if (bad16(out16->rows, out16->ld) || !out16->table || !out16->carry_amax || !out16->carry_scales ||
        (((uintptr_t)out16->table) & 15))
      return FT_ERR_UNSUPPORTED;
    o.rows = out16->rows; o.ld = out16->ld; o.table = (const float2*)out16->table;
    o.carry_amax = out16->carry_amax; o.carry_exp = out16->carry_exp; o.carry_scales = out16->carry_scales;
  } else if (bad32(dq, lddq) || bad32(dk, ldd) || bad32(dv, ldd)) {
    return FT_ERR_UNSUPPORTED;
  }
  if (head_dim != BD || bad16(qkv16, ld) || bad16(o16, ldo) || bad16(do16, lddo) ||
      (q_col0 % 8) || (k_col0 % 8) || (v_col0 % 8) || !stats)
    return FT_ERR_UNSUPPORTED;
  const uint64_t T = (uint64_t)batch * seq;
  CUtensorMap m_qkv, m_do, m_o;
  FT_TRY(ft_tc::make_map(ctx, &m_qkv, qkv16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (uint64_t)ld, T, (uint64_t)ld, 64, 128));
  FT_TRY(ft_tc::make_map(ctx, &m_do, do16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (uint64_t)lddo, T, (uint64_t)lddo, 64, 128));
  FT_TRY(ft_tc::make_map(ctx, &m_o, o16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (uint64_t)ldo, T, (uint64_t)ldo, 64, 128));
  static bool configured[FT_MAX_DEVICES] = {};   // function attributes are per device
  if (!configured[ctx->device]) {
    FT_CUDA(cudaFuncSetAttribute(k_attn_bwd_dq_tc2, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Smem::DYN_BYTES));
    FT_CUDA(cudaFuncSetAttribute(k_attn_bwd_dkv_tc2, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Smem::DYN_BYTES));
    configured[ctx->device] = true;
  }
  const float scale = 1.0f / sqrtf((float)head_dim);
  int* am = ctx->amax_out;   // armed: the gradients' largest magnitude goes to the amax slot
  if (am) ctx->amax_ready = true;
  const int ntile = ft_cdiv(seq, BT);
  {
    const int tiles = ntile * batch * heads;
    const int grid = std::min(tiles, ctx->sm_count);
    FT_LAUNCH_PDL(ctx, k_attn_bwd_dq_tc2, grid, DQ_THREADS, Smem::DYN_BYTES, m_qkv, m_do, m_o, dq, lddq,
                  stats, seq, heads, kv_heads, batch * heads, q_col0, k_col0, v_col0, scale, inv_scale,
                  am, ctx->status_dev, o);
  }
  {
    const int tiles = ntile * batch * kv_heads;
    const int grid = std::min(tiles, ctx->sm_count);
    FT_LAUNCH_PDL(ctx, k_attn_bwd_dkv_tc2, grid, DKV_THREADS, Smem::DYN_BYTES, m_qkv, m_do, dk, dv, ldd,
                  stats, seq, heads, kv_heads, batch * kv_heads, q_col0, k_col0, v_col0, scale,
                  inv_scale, am, ctx->status_dev, o);
  }
  return FT_OK;
}
