// Blackwell tensor-core GEMM:  C[M,N] f32 (+)= alpha * A[M,K] . B[N,K]^T with A and B both
// f16 (or both bf16: tcgen05.mma.kind::f16 wants the two operands in the same format),
// both K-contiguous, f32 accumulation in tensor memory.
//
// One persistent CTA per SM walks the output tiles.  Warp 0 issues TMA loads
// (cp.async.bulk.tensor, 128-byte swizzle) into a ring of shared-memory stages, warp 1
// issues tcgen05.mma (128 x BN x 16 per instruction) into one of two TMEM accumulators,
// warps 2-5 drain the other accumulator with tcgen05.ld and write C.  Producer, MMA and
// epilogue meet only through mbarriers.
//
// Every mbarrier wait is bounded: when a wait runs out the CTA raises a sticky abort flag,
// records a status word the host reads, lets all roles fall through, waits out its
// in-flight copies, frees its tensor memory and returns.  Nothing traps.
#include <map>
#include <string>
#include <stdlib.h>
#include "ft_tc.cuh"

namespace {

using namespace ft_tc;

// MH = number of 128-row halves of the output tile (1: 128 x BN with two accumulators so the
// epilogue overlaps the next tile; 2: 256 x 256 with one accumulator pair - a third less
// operand traffic from L2 per FLOP, which is what bounds the 128-row form).
template <int BN, int STAGES, int MH = 1>
struct SmemLayout {
  static constexpr int A_BYTES = MH * BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;     // 8 epilogue warps x 4 KiB staging
  static constexpr int BAR_OFFSET = EPI_OFFSET + 8 * 4096;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem ptr, abort flag
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack to align the base to 1024 bytes
};

// Progress markers for fault finding, compiled in only with -DFT_DEBUG_MARKERS: when `dbg` is
// set, CTA 0 records how far each role got in pinned host memory (which survives a device
// fault) and lets asynchronous work land before it moves on, so that the last marker names the
// instruction that failed.  Release builds carry none of it.
#ifdef FT_DEBUG_MARKERS
#define FT_MARK(slot, value)                                  \
  do {                                                        \
    if (dbg && blockIdx.x == 0) {                             \
      ((volatile int*)dbg)[slot] = (value);                   \
      __threadfence_system();                                 \
    }                                                         \
  } while (0)
#define FT_SETTLE()                                           \
  do {                                                        \
    if (dbg) for (int _i = 0; _i < 200; ++_i) __nanosleep(1000); \
  } while (0)
#else
#define FT_MARK(slot, value) do { (void)dbg; } while (0)
#define FT_SETTLE() do { } while (0)
#endif

// What the epilogue does with a finished accumulator tile:
//   v = alpha_dev * alpha * acc (+ bias[col]) (+ residual[row, col]);  c = v;  c16 = f16(v)
// (pair kernel, with carry_amax: c16 = f16(S v), S the carried power of two)
struct Epilogue {
  float* c;
  long long ldc;
  __half* c16;
  long long ldc16;
  const float* alpha_ptr;
  float alpha;
  const float* bias;
  const float* residual;
  long long ldr;
  int* amax_slot;   // when set, the largest |v| written is folded into it (atomicMax)
  const int* carry_amax;   // see FtGemmArgs::carry_amax
  int carry_exp;
  float* carry_scales;
  const float2* rope_table;   // see FtGemmArgs::rope_table (pair kernel, f16 result only)
  int rope_seq, rope_cols;
  // SwiGLU in the epilogue (pair kernel; columns are gate|up interleaved in runs of 32):
  __half* swi_f16;            // forward: silu(gate) * up of every 64-column run -> 32 columns here
  long long swi_ldf;
  // backward (the columns are the SwiGLU output's features): the result is the gradient of the
  // SwiGLU output; with the saved gate|up rows it becomes d gate | d up, written interleaved
  const __half* swi_gu16;
  long long swi_ldgu;
  __half* swi_dgu16;
  long long swi_lddgu;
  const int* swi_gu_amax;     // largest |gate| or |up| of the forward pass
  float* swi_scales;          // {S, 1/S, 2^-11/S} of the d gate | d up rows (published)
  int tail_steps;             // 16-column MMA steps of a tail k-block that hold adapter columns (1..4)
};

// sigmoid with the fast exponential and reciprocal (about 2 ulp), as the SwiGLU kernels use
__device__ __forceinline__ float tc_fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// Adapter pre-tiles.  When the K-concatenated tail operand A2 (= alpha/r * A . Bpre^T, 64 columns)
// does not exist yet, the same launch computes it: `tiles` extra tiles of TM rows x 64 columns,
// handed to the CTAs in reverse order (the CTAs with the fewest output tiles take them first),
// each streaming A against Bpre over the whole of K and writing f16 rows to c16.  A finished
// pre-tile raises flags[m tile] by one per epilogue warp; an output tile reads its tail
// k-blocks only after its flag reached 8.  Pre-tiles wait for nothing, so they always finish.
struct PreTile {
  int tiles;          // 0: no pre-tiles in this launch
  __half* c16;        // [M, 64]
  long long ldc16;
  float alpha;
  int* flags;         // one per m tile, zero at launch
  uint32_t idesc;     // instruction descriptor for N = 64
};

__device__ __forceinline__ bool flag_wait(const int* flag, int target, volatile int* abort_flag,
                                          int* status, int where) {
  const uint64_t t0 = global_ns();
  for (;;) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= target) break;
    if (*abort_flag || global_ns() - t0 > WAIT_LIMIT_NS) {
      if (!*abort_flag) {
        *abort_flag = 1;
        volatile int* st = status;
        if (st[0] == 0) {
          st[1] = (int)blockIdx.x;
          st[2] = v;
          st[0] = 100 + where;
        }
      }
      return false;
    }
    __nanosleep(200);
  }
  // what other SMs wrote with ordinary stores is read next by TMA (the async proxy)
  asm volatile("fence.proxy.async.global;" ::: "memory");
  return true;
}

// Token-reduction launches (KOUTER) carry up to two problems that share T and N = 64: problem q
// is P_q[M_q, 64] = sum_t A_q[t, m] B_q[t, n] with A_q = map_a / map_a2 and B_q = map_b / map_b2.
// The tile list is (problem, m tile, K split); every split writes its own f32 slab and a small
// second launch sums the slabs in split order.
struct KoProblem {
  int M, splits, per;   // rows, K splits, k-blocks per split
  float* slabs;         // [splits][M][64]
};
struct KoPair {
  KoProblem p[2];       // p[1].M == 0: one problem only
};
struct KoTile { int q, mt, sp, kb0, kb1; };
__device__ __forceinline__ int ko_tiles(const KoPair& ko) {
  return ((ko.p[0].M + BM - 1) / BM) * ko.p[0].splits + ((ko.p[1].M + BM - 1) / BM) * ko.p[1].splits;
}
__device__ __forceinline__ KoTile ko_decode(const KoPair& ko, int tile, int kb_main) {
  const int tm0 = (ko.p[0].M + BM - 1) / BM, n0 = tm0 * ko.p[0].splits;
  KoTile t;
  t.q = tile >= n0 ? 1 : 0;
  const int r = t.q ? tile - n0 : tile;
  const int tm = t.q ? (ko.p[1].M + BM - 1) / BM : tm0;
  t.mt = r % tm;
  t.sp = r / tm;
  t.kb0 = t.sp * ko.p[t.q].per;
  t.kb1 = min(kb_main, t.kb0 + ko.p[t.q].per);
  return t;
}

// KOUTER = false:  C[M,N] = A[M,K] . B[N,K]^T (+ A2[M,K2] . B2[N,K2]^T), operands K-contiguous.
// KOUTER = true :  C[M,N] = sum_t A[t,m] B[t,n], operands given as [T, M] and [T, N] (the
//                  token-reduction products of the adapter gradients); BN = 64, the tile list
//                  is (m tile, K split) and each split writes its own f32 slab of C.
template <int BN, int STAGES, bool KOUTER, int MH = 1>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_gemm_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
          const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
          const __grid_constant__ CUtensorMap map_b3, Epilogue ep, PreTile pre, KoPair ko, int M,
          int N, int K, int K2, int splits, uint32_t idesc, int* status, int* dbg) {
  using L = SmemLayout<BN, STAGES, MH>;
  static_assert(MH == 1 || (BN == 256 && !KOUTER), "the 256-row tile exists for BN = 256 only");
  constexpr int TM = MH * BM;  // rows of an output tile
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);

  const uint32_t bar_full = base + L::BAR_OFFSET;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_tfull = bar_empty + STAGES * 8;
  const uint32_t bar_tempty = bar_tfull + 2 * 8;
  uint32_t* tmem_slot = (uint32_t*)(gbase + L::BAR_OFFSET + (2 * STAGES + 4) * 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + TM - 1) / TM;
  const int tiles_n = KOUTER ? splits : (N + BN - 1) / BN;
  const int num_tiles = KOUTER ? ko_tiles(ko) : tiles_m * tiles_n;
  const int kb_main = (K + BK - 1) / BK;
  const int kb_total = kb_main + (KOUTER ? 0 : (K2 + BK - 1) / BK);
  // MH = 1: two accumulators of BN columns (epilogue of one overlaps the products of the
  // other); MH = 2: one pair of 256-column accumulators, all of tensor memory
  constexpr uint32_t TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + b * 8, 1);
      mbar_init(bar_tempty + b * 8, 8);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    FT_MARK(4, 1);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    if (lane == 0) FT_MARK(5, 12);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above touched only this CTA's shared and tensor memory: it may run while the
  // previous kernel in the stream drains; global memory is touched from here on
  ft_pdl_wait();
  ft_pdl_launch();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      if constexpr (!KOUTER) {
        for (int p = (int)gridDim.x - 1 - (int)blockIdx.x; p < pre.tiles; p += gridDim.x) {
          for (int kb = 0; kb < kb_main; ++kb) {
            if (!mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, status, 5)) break;
            const uint32_t sa = base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
            const uint32_t bar = bar_full + stage * 8;
            mbar_expect_tx(bar, L::A_BYTES + 64 * BK * 2);
            tma_load_2d(sa, &map_a, bar, kb * BK, p * TM);
            tma_load_2d(sb, &map_b3, bar, kb * BK, 0);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (*abort_flag) break;
        }
      }
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int m0 = (tile % tiles_m) * TM, nt = tile / tiles_m;
        int kb0 = 0, kb1 = kb_total, prob = 0;
        if constexpr (KOUTER) {
          const KoTile kt = ko_decode(ko, tile, kb_main);
          m0 = kt.mt * BM; nt = kt.sp; kb0 = kt.kb0; kb1 = kt.kb1; prob = kt.q;
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          FT_MARK(7, 20);
          if constexpr (!KOUTER) {
            // the tail operand of this row block comes from a pre-tile of this same launch
            if (kb == kb_main && pre.tiles > 0 &&
                !flag_wait(pre.flags + (tile % tiles_m), 8, abort_flag, status, 6))
              break;
          }
          if (!mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, status, 1)) break;
          const uint32_t sa = base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          const uint32_t bar = bar_full + stage * 8;
          mbar_expect_tx(bar, L::STAGE_BYTES);
          if constexpr (KOUTER) {
            // {x = M/N index (64 wide), y = token row}
            const CUtensorMap* pa = prob ? &map_a2 : &map_a;
            tma_load_2d(sa, pa, bar, m0, kb * BK);
            tma_load_2d(sa + 64 * 128, pa, bar, m0 + 64, kb * BK);
            tma_load_2d(sb, prob ? &map_b2 : &map_b, bar, 0, kb * BK);
          } else if (kb < kb_main) {
            tma_load_2d(sa, &map_a, bar, kb * BK, m0);
            tma_load_2d(sb, &map_b, bar, kb * BK, nt * BN);
          } else {
            tma_load_2d(sa, &map_a2, bar, (kb - kb_main) * BK, m0);
            tma_load_2d(sb, &map_b2, bar, (kb - kb_main) * BK, nt * BN);
          }
          FT_SETTLE();
          FT_MARK(7, 24);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (*abort_flag) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      int local = 0;
      if constexpr (!KOUTER) {
        for (int p = (int)gridDim.x - 1 - (int)blockIdx.x; p < pre.tiles; p += gridDim.x, ++local) {
          const uint32_t buf = MH == 1 ? (local & 1) : 0;
          const uint32_t acc_phase = MH == 1 ? ((local >> 1) & 1) : (local & 1);
          if (!mbar_wait(bar_tempty + buf * 8, acc_phase ^ 1, abort_flag, status, 7)) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          for (int kb = 0; kb < kb_main; ++kb) {
            if (!mbar_wait(bar_full + stage * 8, phase, abort_flag, status, 8)) break;
            tc_fence_after();
            const uint32_t sa = base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
            const uint64_t da = make_desc_sw128(sa), db = make_desc_sw128(sb);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              tc_mma_f16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), pre.idesc,
                         (kb > 0 || k > 0) ? 1u : 0u);
              if constexpr (MH == 2)
                tc_mma_f16(d_tmem + BN, da + (uint64_t)(1024 + k * 2), db + (uint64_t)(k * 2),
                           pre.idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit(bar_empty + stage * 8);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (*abort_flag) break;
          tc_commit(bar_tfull + buf * 8);
        }
      }
      for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x, ++local) {
        int kb0 = 0, kb1 = kb_total;
        if constexpr (KOUTER) {
          const KoTile kt = ko_decode(ko, tile, kb_main);
          kb0 = kt.kb0; kb1 = kt.kb1;
        }
        const uint32_t buf = MH == 1 ? (local & 1) : 0;
        const uint32_t acc_phase = MH == 1 ? ((local >> 1) & 1) : (local & 1);
        FT_MARK(8, 30);
        if (!mbar_wait(bar_tempty + buf * 8, acc_phase ^ 1, abort_flag, status, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_full + stage * 8, phase, abort_flag, status, 3)) break;
          FT_MARK(8, 32);
          tc_fence_after();
          const uint32_t sa = base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          if constexpr (KOUTER) {
            const uint64_t da = make_desc_mn_sw128(sa, 64 * 128), db = make_desc_mn_sw128(sb, 64 * 128);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // 16 token rows further = two 1024-byte atoms = +128 in 16-byte units
              tc_mma_f16(d_tmem, da + (uint64_t)(k * 128), db + (uint64_t)(k * 128), idesc,
                         (kb > kb0 || k > 0) ? 1u : 0u);
              FT_SETTLE();
              FT_MARK(8, 33 + k);
            }
          } else {
            const uint64_t da = make_desc_sw128(sa), db = make_desc_sw128(sb);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // advancing K by 16 elements = 32 bytes inside the swizzle row: +2 in the
              // 16-byte units of the start-address field
              tc_mma_f16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc,
                         (kb > kb0 || k > 0) ? 1u : 0u);
              if constexpr (MH == 2)  // rows 128..255 of the tile: 16 KiB further in the A stage
                tc_mma_f16(d_tmem + BN, da + (uint64_t)(1024 + k * 2), db + (uint64_t)(k * 2), idesc,
                           (kb > kb0 || k > 0) ? 1u : 0u);
              FT_SETTLE();
              FT_MARK(8, 33 + k);
            }
          }
          tc_commit(bar_empty + stage * 8);  // frees the stage when these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (*abort_flag) break;
        tc_commit(bar_tfull + buf * 8);      // accumulator complete
        FT_SETTLE();
        FT_MARK(8, 38);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue
    // Eight warps: a warp reaches only the 32 TMEM lanes of its quadrant (warp % 4), so two
    // warps share each quadrant and take alternate 32-column chunks.
    const int quad = warp & 3;               // TMEM lanes [32*quad, 32*quad+32)
    const int grp = (warp - 2) >> 2;
    int local = 0;
    uint8_t* stage_base = gbase + L::EPI_OFFSET + (warp - 2) * 4096;   // 32 x 128 bytes per warp
    const bool vec_c = ep.c && ((ep.ldc & 3) == 0) && ((((uintptr_t)ep.c) & 15) == 0);
    const bool vec_r = !ep.residual || (((ep.ldr & 3) == 0) && ((((uintptr_t)ep.residual) & 15) == 0));
    const bool vec_h = ep.c16 && ((ep.ldc16 & 3) == 0) && ((((uintptr_t)ep.c16) & 7) == 0);
    const float alpha = (ep.alpha_ptr ? *ep.alpha_ptr : 1.0f) * ep.alpha;
    float amax_seen = 0.f;
    constexpr int NCH = MH * (BN / 32);
    if constexpr (!KOUTER) {
      for (int p = (int)gridDim.x - 1 - (int)blockIdx.x; p < pre.tiles; p += gridDim.x, ++local) {
        const uint32_t buf = MH == 1 ? (local & 1) : 0;
        const uint32_t acc_phase = MH == 1 ? ((local >> 1) & 1) : (local & 1);
        if (!mbar_wait(bar_tfull + buf * 8, acc_phase, abort_flag, status, 9)) break;
        tc_fence_after();
        const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
        // 64 columns: the two warps of a lane quadrant take 32 each, per 128-row half
#pragma unroll 1
        for (int half = 0; half < MH; ++half) {
          uint32_t r[32];
          tc_ld32(t_lane + (buf + half) * BN + grp * 32, r);
          tc_wait_ld();
          uint8_t* st = stage_base + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *(float4*)(st + ((j ^ (lane & 7)) << 4)) = make_float4(
                pre.alpha * __uint_as_float(r[4 * j]), pre.alpha * __uint_as_float(r[4 * j + 1]),
                pre.alpha * __uint_as_float(r[4 * j + 2]), pre.alpha * __uint_as_float(r[4 * j + 3]));
          __syncwarp();
          const int row_base = p * TM + half * BM + quad * 32;
          const int j = lane & 7;
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const int rr = 4 * t + (lane >> 3);
            const int grow = row_base + rr;
            const float4 v4 = *(const float4*)(stage_base + rr * 128 + ((j ^ (rr & 7)) << 4));
            if (grow < M) {
              __half2 h0 = __floats2half2_rn(v4.x, v4.y), h1 = __floats2half2_rn(v4.z, v4.w);
              *(uint2*)(pre.c16 + (long long)grow * pre.ldc16 + grp * 32 + 4 * j) =
                  make_uint2(*(uint32_t*)&h0, *(uint32_t*)&h1);
            }
          }
          __syncwarp();
        }
        tc_fence_before();
        // publish: the rows are read by other CTAs' TMA loads once the flag shows all 8 warps
        asm volatile("fence.proxy.async.global;" ::: "memory");
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          atomicAdd(pre.flags + p, 1);
          mbar_arrive(bar_tempty + buf * 8);
        }
      }
    }
    for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x, ++local) {
      int m0 = (tile % tiles_m) * TM, nt = tile / tiles_m;
      const int n0 = KOUTER ? 0 : nt * BN;
      const uint32_t buf = MH == 1 ? (local & 1) : 0;
      const uint32_t acc_phase = MH == 1 ? ((local >> 1) & 1) : (local & 1);
      if (!mbar_wait(bar_tfull + buf * 8, acc_phase, abort_flag, status, 4)) break;
      tc_fence_after();
      if (warp == 2 && lane == 0) FT_MARK(9, 41);
      float* cbase = ep.c;
      KoTile kt = {0, 0, 0, 0, 0};
      if constexpr (KOUTER) {
        // a K split of the token-reduction product writes its own slab
        kt = ko_decode(ko, tile, kb_main);
        m0 = kt.mt * BM;
        M = ko.p[kt.q].M;
        cbase = ko.p[kt.q].slabs + (long long)kt.sp * M * 64;
      }
      const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
      uint32_t r[32];
      // chunk c of the tile: half c / (BN/32) (a 128-row half), 32 columns from (c % (BN/32)) * 32
      tc_ld32(t_lane + (buf + grp / (BN / 32)) * BN + (grp % (BN / 32)) * 32, r);
#pragma unroll 1
      for (int cbh = grp; cbh < NCH; cbh += 2) {
        const int half = cbh / (BN / 32), cb = cbh % (BN / 32);
        tc_wait_ld();
        const int col0 = n0 + cb * 32;
        // Transpose the 32 x 32 chunk through a swizzled staging tile so that global traffic
        // is coalesced: in tensor memory a thread owns a ROW (32 consecutive floats of one
        // output row); after staging, 8 lanes cover one row's 128 bytes and a warp
        // instruction touches 4 rows instead of 32.
        {
          uint8_t* st = stage_base + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *(float4*)(st + ((j ^ (lane & 7)) << 4)) =
                make_float4(alpha * __uint_as_float(r[4 * j]), alpha * __uint_as_float(r[4 * j + 1]),
                            alpha * __uint_as_float(r[4 * j + 2]), alpha * __uint_as_float(r[4 * j + 3]));
        }
        // the next chunk's accumulator read travels while this one is stored
        if (cbh + 2 < NCH) {
          const int nh = (cbh + 2) / (BN / 32), nc = (cbh + 2) % (BN / 32);
          tc_ld32(t_lane + (buf + nh) * BN + nc * 32, r);
        }
        __syncwarp();
        const int row_base = m0 + half * BM + quad * 32;
        const int j = lane & 7, gcol = col0 + 4 * j;
        if (row_base < M && gcol < N) {
          const bool full = gcol + 4 <= N;
          const bool fast_r = ep.residual && full && vec_r;
          float4 resv[8];
          if (fast_r) {   // all residual loads in flight before the first store
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              const int grow = row_base + 4 * t + (lane >> 3);
              resv[t] = grow < M ? *(const float4*)(ep.residual + (long long)grow * ep.ldr + gcol)
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
          float bv[4] = {0.f, 0.f, 0.f, 0.f};
          if (ep.bias) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (gcol + e < N) bv[e] = ep.bias[gcol + e];
          }
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const int rr = 4 * t + (lane >> 3);
            const int grow = row_base + rr;
            float4 v4 = *(const float4*)(stage_base + rr * 128 + ((j ^ (rr & 7)) << 4));
            if (grow >= M) continue;
            float v[4] = {v4.x + bv[0], v4.y + bv[1], v4.z + bv[2], v4.w + bv[3]};
            if (fast_r) {
              v[0] += resv[t].x; v[1] += resv[t].y; v[2] += resv[t].z; v[3] += resv[t].w;
            } else if (ep.residual) {
              const float* rp = ep.residual + (long long)grow * ep.ldr + gcol;
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (gcol + e < N) v[e] += rp[e];
            }
            if (ep.amax_slot) {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (full || gcol + e < N) amax_seen = fmaxf(amax_seen, fabsf(v[e]));
            }
            if (cbase) {
              float* cp = cbase + (long long)grow * ep.ldc + gcol;
              if (full && vec_c) {
                *(float4*)cp = make_float4(v[0], v[1], v[2], v[3]);
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (gcol + e < N) cp[e] = v[e];
              }
            }
            if (ep.c16) {
              __half* hp = ep.c16 + (long long)grow * ep.ldc16 + gcol;
              if (full && vec_h) {
                __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
                *(uint2*)hp = make_uint2(*(uint32_t*)&h0, *(uint32_t*)&h1);
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (gcol + e < N) hp[e] = __float2half_rn(v[e]);
              }
            }
          }
        }
        __syncwarp();   // the staging tile is reused by the next chunk
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + buf * 8);
      if (warp == 2 && lane == 0) FT_MARK(9, 45);
    }
    if (ep.amax_slot) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        amax_seen = fmaxf(amax_seen, __shfl_xor_sync(0xffffffffu, amax_seen, o));
      if (lane == 0 && amax_seen > 0.f && __float_as_int(amax_seen) > *(volatile int*)ep.amax_slot)
        atomicMax(ep.amax_slot, __float_as_int(amax_seen));
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // loads already issued may still be landing in this CTA's shared memory: give them
    // time before the CTA exits and its shared memory is handed to another one
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
    if (lane == 0) FT_MARK(10, 51);
  }
}

// =========================================================================================
// The same product on CTA pairs (tcgen05 cta_group::2): a cluster of two CTAs owns a 256 x 256
// output tile.  Each CTA loads its own 128 rows of A and HALF of the B tile (128 of the 256
// weight rows) - a third less operand traffic per FLOP than the 128 x 256 single-CTA tile - and
// keeps a 128 x 256 accumulator per buffer, so both accumulator buffers fit in tensor memory
// and the epilogue stays hidden behind the next tile's products.  One thread of the even CTA
// (the leader) issues the MMAs for both; barriers:
//   full[s]   in the leader: one arrival (its producer, expecting both CTAs' bytes); both CTAs'
//             TMA loads complete their transaction bytes there
//   empty[s]  in each CTA: one arrival, from the leader's tcgen05.commit multicast
//   tfull[b]  in each CTA: one arrival, commit multicast
//   tempty[b] in the leader: 16 arrivals, the 8 epilogue warps of each CTA (remote for the odd one)
// Pre-tiles (see PreTile) cover 256 rows per pair, 64 columns split 32 + 32.
// =========================================================================================
template <int STAGES>
struct Smem2 {
  static constexpr int A_BYTES = BM * BK * 2;          // this CTA's 128 rows
  static constexpr int B_BYTES = 128 * BK * 2;         // this CTA's half of the 256 weight rows
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = EPI_OFFSET + 8 * 4096;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
k_gemm_tc2(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
           const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
           const __grid_constant__ CUtensorMap map_b3, Epilogue ep, PreTile pre, int M, int N, int K,
           int K2, uint32_t idesc, int* status) {
  using L = Smem2<STAGES>;
  constexpr int BN = 256, TM = 256;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);

  const uint32_t bar_full = base + L::BAR_OFFSET;
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_tfull = bar_empty + STAGES * 8;
  const uint32_t bar_tempty = bar_tfull + 2 * 8;
  uint32_t* tmem_slot = (uint32_t*)(gbase + L::BAR_OFFSET + (2 * STAGES + 4) * 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0: leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int tiles_m = (M + TM - 1) / TM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  // Tiles that run at the same time should share the LARGER operand's rows in L2.  With A the
  // larger one (M >= N) consecutive tiles walk along N, so a wave of pairs covers few row blocks
  // of A for all of B; otherwise they walk along M.  (8192 x 2048 x 8192 read 579 MB from DRAM
  // for 168 MB of operands when it walked along M.)
  const bool n_fast = M >= N;
  auto tile_mn = [&](int tile, int& mt, int& nt) {
    if (n_fast) { nt = tile % tiles_n; mt = tile / tiles_n; }
    else { mt = tile % tiles_m; nt = tile / tiles_m; }
  };
  const int kb_main = (K + BK - 1) / BK;
  const int kb_total = kb_main + (K2 + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + b * 8, 1);
      mbar_init(bar_tempty + b * 8, 16);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  ft_pdl_wait();
  ft_pdl_launch();

  // the leader's copies of the barriers this CTA signals remotely
  const uint32_t lead_full = mapa_shared(bar_full, 0);
  const uint32_t lead_tempty = mapa_shared(bar_tempty, 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      for (int p = npairs - 1 - pair; p < pre.tiles; p += npairs) {
        for (int kb = 0; kb < kb_main; ++kb) {
          if (!mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, status, 5)) break;
          const uint32_t sa = base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          if (rank == 0) mbar_expect_tx(bar_full + stage * 8, 2 * (L::A_BYTES + 32 * BK * 2));
          tma_load_2d_pair(sa, &map_a, lead_full + stage * 8, kb * BK, p * TM + (int)rank * BM);
          tma_load_2d_pair(sb, &map_b3, lead_full + stage * 8, kb * BK, (int)rank * 32);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (*abort_flag) break;
      }
      for (int tile = pair; tile < num_tiles && !*abort_flag; tile += npairs) {
        int mt, nt;
        tile_mn(tile, mt, nt);
        const int m0 = mt * TM + (int)rank * BM;
        const int nrow = nt * BN + (int)rank * 128;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (kb == kb_main && pre.tiles > 0 &&
              !flag_wait(pre.flags + mt, 16, abort_flag, status, 6))
            break;
          if (!mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, status, 1)) break;
          const uint32_t sa = base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          if (rank == 0) mbar_expect_tx(bar_full + stage * 8, 2 * L::STAGE_BYTES);
          if (kb < kb_main) {
            tma_load_2d_pair(sa, &map_a, lead_full + stage * 8, kb * BK, m0);
            tma_load_2d_pair(sb, &map_b, lead_full + stage * 8, kb * BK, nrow);
          } else {
            tma_load_2d_pair(sa, &map_a2, lead_full + stage * 8, (kb - kb_main) * BK, m0);
            tma_load_2d_pair(sb, &map_b2, lead_full + stage * 8, (kb - kb_main) * BK, nrow);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (rank == 0 && elect_one()) {
      uint32_t stage = 0, phase = 0;
      int local = 0;
      for (int p = npairs - 1 - pair; p < pre.tiles; p += npairs, ++local) {
        const uint32_t buf = local & 1, acc_phase = (local >> 1) & 1;
        if (!mbar_wait(bar_tempty + buf * 8, acc_phase ^ 1, abort_flag, status, 7)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < kb_main; ++kb) {
          if (!mbar_wait(bar_full + stage * 8, phase, abort_flag, status, 8)) break;
          tc_fence_after();
          const uint32_t sa = base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          const uint64_t da = make_desc_sw128(sa), db = make_desc_sw128(sb);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_f16_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), pre.idesc,
                            (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit_pair(bar_empty + stage * 8, 3);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (*abort_flag) break;
        tc_commit_pair(bar_tfull + buf * 8, 3);
      }
      for (int tile = pair; tile < num_tiles && !*abort_flag; tile += npairs, ++local) {
        const uint32_t buf = local & 1, acc_phase = (local >> 1) & 1;
        if (!mbar_wait(bar_tempty + buf * 8, acc_phase ^ 1, abort_flag, status, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < kb_main; ++kb) {
          if (!mbar_wait(bar_full + stage * 8, phase, abort_flag, status, 3)) break;
          tc_fence_after();
          const uint32_t sa = base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          const uint64_t da = make_desc_sw128(sa), db = make_desc_sw128(sb);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_f16_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc,
                            (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit_pair(bar_empty + stage * 8, 3);  // frees the stage in both CTAs
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        // adapter tail: the rank-r columns fill only the first tail_steps 16-column steps of
        // the 64-column k-block (the rest is zero padding and is not multiplied)
        for (int kb = kb_main; kb < kb_total; ++kb) {
          if (!mbar_wait(bar_full + stage * 8, phase, abort_flag, status, 3)) break;
          tc_fence_after();
          const uint32_t sa = base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          const uint64_t da = make_desc_sw128(sa), db = make_desc_sw128(sb);
          const int steps = (kb == kb_total - 1) ? ep.tail_steps : BK / UMMA_K;
          for (int k = 0; k < steps; ++k)
            tc_mma_f16_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc,
                            (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit_pair(bar_empty + stage * 8, 3);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (*abort_flag) break;
        tc_commit_pair(bar_tfull + buf * 8, 3);      // accumulator complete, both CTAs
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int quad = warp & 3;               // TMEM lanes [32*quad, 32*quad+32)
    const int grp = (warp - 2) >> 2;
    int local = 0;
    uint8_t* stage_base = gbase + L::EPI_OFFSET + (warp - 2) * 4096;   // 32 x 128 bytes per warp
    const bool vec_c = ep.c && ((ep.ldc & 3) == 0) && ((((uintptr_t)ep.c) & 15) == 0);
    const bool vec_r = !ep.residual || (((ep.ldr & 3) == 0) && ((((uintptr_t)ep.residual) & 15) == 0));
    const bool vec_h = ep.c16 && ((ep.ldc16 & 3) == 0) && ((((uintptr_t)ep.c16) & 7) == 0);
    const float alpha = (ep.alpha_ptr ? *ep.alpha_ptr : 1.0f) * ep.alpha;
    // carried scale of the f16 result (a power of two from an earlier tensor's amax)
    float s16 = 1.0f;
    if (ep.carry_amax && !ep.swi_dgu16) {
      s16 = ft_scale_from_amax_bits(*ep.carry_amax, ep.carry_exp);
      if (blockIdx.x == 0 && warp == 2 && lane == 0) ft_publish_scales(ep.carry_scales, s16);
    }
    // SwiGLU backward in the epilogue: every result is at most 1.1 * max|d f| * max(|gate|, |up|);
    // max|d f| is not known before this launch has finished, so the bound takes the carried one
    // (the block above) and aims it at 2^9: 128-fold growth between neighbours before f16
    // overflows.  One thread publishes {S, 1/S, 2^-11/S}.
    float swi_S = 1.0f;
    if (ep.swi_dgu16) {
      const float bound = 1.1f * __int_as_float(*ep.carry_amax) * __int_as_float(*ep.swi_gu_amax);
      if (bound > 0.f && isfinite(bound)) {
        int e;
        frexpf(bound, &e);
        swi_S = ldexpf(1.0f, 9 - e);
      }
      if (blockIdx.x == 0 && warp == 2 && lane == 0) ft_publish_scales(ep.swi_scales, swi_S);
    }
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    float amax_seen = 0.f;
    constexpr int NCH = BN / 32;
    for (int p = npairs - 1 - pair; p < pre.tiles; p += npairs, ++local) {
      const uint32_t buf = local & 1, acc_phase = (local >> 1) & 1;
      if (!mbar_wait(bar_tfull + buf * 8, acc_phase, abort_flag, status, 9)) break;
      tc_fence_after();
      {
        uint32_t r[32];
        tc_ld32(t_lane + buf * BN + grp * 32, r);
        tc_wait_ld();
        uint8_t* st = stage_base + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *(float4*)(st + ((j ^ (lane & 7)) << 4)) = make_float4(
              pre.alpha * __uint_as_float(r[4 * j]), pre.alpha * __uint_as_float(r[4 * j + 1]),
              pre.alpha * __uint_as_float(r[4 * j + 2]), pre.alpha * __uint_as_float(r[4 * j + 3]));
        __syncwarp();
        const int row_base = p * TM + (int)rank * BM + quad * 32;
        const int j = lane & 7;
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const int rr = 4 * t + (lane >> 3);
          const int grow = row_base + rr;
          const float4 v4 = *(const float4*)(stage_base + rr * 128 + ((j ^ (rr & 7)) << 4));
          if (grow < M) {
            __half2 h0 = __floats2half2_rn(v4.x, v4.y), h1 = __floats2half2_rn(v4.z, v4.w);
            *(uint2*)(pre.c16 + (long long)grow * pre.ldc16 + grp * 32 + 4 * j) =
                make_uint2(*(uint32_t*)&h0, *(uint32_t*)&h1);
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.global;" ::: "memory");
      __threadfence();
      __syncwarp();
      if (lane == 0) {
        atomicAdd(pre.flags + p, 1);
        mbar_arrive_cluster(lead_tempty + buf * 8);
      }
    }
    for (int tile = pair; tile < num_tiles && !*abort_flag; tile += npairs, ++local) {
      int mt, nt;
      tile_mn(tile, mt, nt);
      const int m0 = mt * TM + (int)rank * BM;
      const int n0 = nt * BN;
      const uint32_t buf = local & 1, acc_phase = (local >> 1) & 1;
      if (ep.swi_dgu16) {
        // the saved gate | up rows this thread will want: ask L2 for them while the tile's
        // products are still running
        const int my_row = m0 + quad * 32 + lane;
        if (my_row < M) {
          const __half* gp = ep.swi_gu16 + (long long)my_row * ep.swi_ldgu + 2 * (long long)n0;
#pragma unroll
          for (int cb = 0; cb < NCH / 2; ++cb)
            if (n0 + (grp + 2 * cb) * 32 < N)
              asm volatile("prefetch.global.L2 [%0];" ::"l"(gp + 64 * (grp + 2 * cb)));
        }
      }
      if (!mbar_wait(bar_tfull + buf * 8, acc_phase, abort_flag, status, 4)) break;
      tc_fence_after();
      if (ep.swi_f16) {
        // gate|up projection, forward: a thread holds gate and up of 32 features of one row.
        // gate | up go out as f16 (interleaved as they are), and silu(gate) * up, computed from
        // those rounded values as the backward pass will see them, as the down projection's operand
        uint8_t* st = stage_base + lane * 128;
        uint8_t* sf = stage_base + lane * 64;
#pragma unroll 1
        for (int hd = grp; hd < BN / 64; hd += 2) {
          const int col0 = n0 + hd * 64;
          if (col0 >= N) break;
          uint32_t ra[32], rb[32];
          tc_ld32(t_lane + buf * BN + hd * 64, ra);
          tc_ld32(t_lane + buf * BN + hd * 64 + 32, rb);
          tc_wait_ld();
          uint32_t wf[16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t w1[4], w2[4];
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
              const int i = 8 * j + e;
              const __half2 hg = __floats2half2_rn(alpha * __uint_as_float(ra[i]), alpha * __uint_as_float(ra[i + 1]));
              const __half2 hu = __floats2half2_rn(alpha * __uint_as_float(rb[i]), alpha * __uint_as_float(rb[i + 1]));
              w1[e >> 1] = *(const uint32_t*)&hg;
              w2[e >> 1] = *(const uint32_t*)&hu;
              const float2 g = __half22float2(hg), u = __half22float2(hu);
              amax_seen = fmaxf(amax_seen, fmaxf(fmaxf(fabsf(g.x), fabsf(g.y)), fmaxf(fabsf(u.x), fabsf(u.y))));
              const __half2 hf = __floats2half2_rn(g.x * tc_fast_sigmoid(g.x) * u.x, g.y * tc_fast_sigmoid(g.y) * u.y);
              wf[i >> 1] = *(const uint32_t*)&hf;
            }
            *(uint4*)(st + ((j ^ (lane & 7)) << 4)) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
            *(uint4*)(st + (((4 + j) ^ (lane & 7)) << 4)) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
          }
          __syncwarp();
          {
            const int u = lane & 7;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              const int rr = 4 * t + (lane >> 3);
              const int grow = m0 + quad * 32 + rr;
              const uint4 v = *(const uint4*)(stage_base + rr * 128 + ((u ^ (rr & 7)) << 4));
              if (grow < M) *(uint4*)(ep.c16 + (long long)grow * ep.ldc16 + col0 + u * 8) = v;
            }
          }
          __syncwarp();
          // the 32 products of this row: 64 bytes, staged with a 64-byte pitch
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *(uint4*)(sf + ((j ^ ((lane >> 1) & 3)) << 4)) = make_uint4(wf[4 * j], wf[4 * j + 1], wf[4 * j + 2], wf[4 * j + 3]);
          __syncwarp();
          {
            const int u = lane & 3;
            const int fcol0 = (col0 >> 6) << 5;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const int rr = 8 * t + (lane >> 2);
              const int grow = m0 + quad * 32 + rr;
              const uint4 v = *(const uint4*)(stage_base + rr * 64 + ((u ^ ((rr >> 1) & 3)) << 4));
              if (grow < M) *(uint4*)(ep.swi_f16 + (long long)grow * ep.swi_ldf + fcol0 + u * 8) = v;
            }
          }
          __syncwarp();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_tempty + buf * 8);
        continue;
      }
      if (ep.swi_dgu16) {
        // down projection, input gradient: column c is feature c of the SwiGLU output.  A
        // thread holds 32 adjacent features of one row and needs the row's saved gate | up of
        // those features (128 contiguous bytes); it produces d gate | d up (128 bytes) times S.
        // Both sides pass through the warp's staging tile so that global accesses stay
        // coalesced (eight lanes per 128-byte row) instead of one row per lane.
        const int row_base = m0 + quad * 32;
        const int u8 = lane & 7;
        uint8_t* st = stage_base + lane * 128;
#pragma unroll 1
        for (int cb = grp; cb < NCH; cb += 2) {
          const int col0 = n0 + cb * 32;
          if (col0 >= N) break;
          uint4 v[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const int grow = row_base + 4 * t + (lane >> 3);
            v[t] = grow < M ? *(const uint4*)(ep.swi_gu16 + (long long)grow * ep.swi_ldgu + 2 * (long long)col0 + u8 * 8)
                            : make_uint4(0u, 0u, 0u, 0u);
          }
          uint32_t r[32];
          tc_ld32(t_lane + buf * BN + cb * 32, r);
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const int rr = 4 * t + (lane >> 3);
            *(uint4*)(stage_base + rr * 128 + ((u8 ^ (rr & 7)) << 4)) = v[t];
          }
          __syncwarp();
          uint4 gu[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) gu[q] = *(const uint4*)(st + ((q ^ (lane & 7)) << 4));
          __syncwarp();   // every lane holds its row of gate | up: the tile may be overwritten
          tc_wait_ld();
          const __half2* gh = (const __half2*)gu;        // gate: halves 0..31
          const __half2* uh = gh + 16;                   // up: halves 32..63
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t og[4], ou[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = 8 * q + 2 * e;
              const float2 g = __half22float2(gh[i >> 1]), u = __half22float2(uh[i >> 1]);
              const float d0 = alpha * __uint_as_float(r[i]), d1 = alpha * __uint_as_float(r[i + 1]);
              amax_seen = fmaxf(amax_seen, fmaxf(fabsf(d0), fabsf(d1)));
              const float s0 = tc_fast_sigmoid(g.x), s1 = tc_fast_sigmoid(g.y);
              const float k0 = d0 * swi_S, k1 = d1 * swi_S;
              const __half2 hu = __floats2half2_rn(k0 * (g.x * s0), k1 * (g.y * s1));
              const __half2 hg = __floats2half2_rn(k0 * u.x * (s0 * (1.0f + g.x * (1.0f - s0))),
                                                   k1 * u.y * (s1 * (1.0f + g.y * (1.0f - s1))));
              og[e] = *(const uint32_t*)&hg;
              ou[e] = *(const uint32_t*)&hu;
            }
            *(uint4*)(st + ((q ^ (lane & 7)) << 4)) = make_uint4(og[0], og[1], og[2], og[3]);
            *(uint4*)(st + (((4 + q) ^ (lane & 7)) << 4)) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
          }
          __syncwarp();
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const int rr = 4 * t + (lane >> 3);
            const int grow = row_base + rr;
            const uint4 w = *(const uint4*)(stage_base + rr * 128 + ((u8 ^ (rr & 7)) << 4));
            if (grow < M)
              *(uint4*)(ep.swi_dgu16 + (long long)grow * ep.swi_lddgu + 2 * (long long)col0 + u8 * 8) = w;
          }
          __syncwarp();   // the staging tile is reused by the next chunk
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_tempty + buf * 8);
        continue;
      }
      if (ep.rope_table) {
        // q|k|v projection: the rotary rotation (component i of a 64-wide head pairs with
        // i + 32) and the f16 rounding happen here, on the accumulator; each warp group takes
        // every other head of the tile, a thread one row of it.
        // (the table is transposed, [32][rope_seq]: lanes own consecutive rows, i.e. positions,
        // so each load of the warp covers consecutive addresses)
        const int my_row = m0 + quad * 32 + lane;
        const float2* tcol = ep.rope_table + (my_row % ep.rope_seq);
        const size_t tstep = (size_t)ep.rope_seq;
#pragma unroll 1
        for (int hd = grp; hd < BN / 64; hd += 2) {
          const int col0 = n0 + hd * 64;
          if (col0 >= N) break;
          uint32_t ra[32], rb[32];
          tc_ld32(t_lane + buf * BN + hd * 64, ra);
          tc_ld32(t_lane + buf * BN + hd * 64 + 32, rb);
          tc_wait_ld();
          const bool rot = col0 < ep.rope_cols;
          uint8_t* st = stage_base + lane * 128;
          const float2* tp = tcol;   // walks down the table's rows: one pointer, no index arithmetic
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t w1[4], w2[4];
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
              const int i = 8 * j + e;
              float a0 = alpha * __uint_as_float(ra[i]), a1 = alpha * __uint_as_float(ra[i + 1]);
              float b0 = alpha * __uint_as_float(rb[i]), b1 = alpha * __uint_as_float(rb[i + 1]);
              if (ep.bias) {
                a0 += ep.bias[col0 + i]; a1 += ep.bias[col0 + i + 1];
                b0 += ep.bias[col0 + 32 + i]; b1 += ep.bias[col0 + 32 + i + 1];
              }
              float o10 = a0, o11 = a1, o20 = b0, o21 = b1;
              if (rot) {
                const float2 c0 = tp[0], c1 = tp[tstep];   // {cos, sin} of components i, i + 1
                tp += 2 * tstep;
                o10 = a0 * c0.x - b0 * c0.y; o20 = a0 * c0.y + b0 * c0.x;
                o11 = a1 * c1.x - b1 * c1.y; o21 = a1 * c1.y + b1 * c1.x;
              }
              __half2 h1 = __floats2half2_rn(o10, o11), h2 = __floats2half2_rn(o20, o21);
              w1[e >> 1] = *(uint32_t*)&h1;
              w2[e >> 1] = *(uint32_t*)&h2;
            }
            *(uint4*)(st + ((j ^ (lane & 7)) << 4)) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
            *(uint4*)(st + (((4 + j) ^ (lane & 7)) << 4)) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
          }
          __syncwarp();
          const int u = lane & 7;
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const int rr = 4 * t + (lane >> 3);
            const int grow = m0 + quad * 32 + rr;
            const uint4 v = *(const uint4*)(stage_base + rr * 128 + ((u ^ (rr & 7)) << 4));
            if (grow < M) *(uint4*)(ep.c16 + (long long)grow * ep.ldc16 + col0 + u * 8) = v;
          }
          __syncwarp();   // the staging tile is reused by the next head
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_tempty + buf * 8);
        continue;
      }
      float* cbase = ep.c;
      uint32_t r[32];
      tc_ld32(t_lane + buf * BN + grp * 32, r);
#pragma unroll 1
      for (int cb = grp; cb < NCH; cb += 2) {
        tc_wait_ld();
        const int col0 = n0 + cb * 32;
        {
          uint8_t* st = stage_base + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *(float4*)(st + ((j ^ (lane & 7)) << 4)) =
                make_float4(alpha * __uint_as_float(r[4 * j]), alpha * __uint_as_float(r[4 * j + 1]),
                            alpha * __uint_as_float(r[4 * j + 2]), alpha * __uint_as_float(r[4 * j + 3]));
        }
        if (cb + 2 < NCH) tc_ld32(t_lane + buf * BN + (cb + 2) * 32, r);
        __syncwarp();
        const int row_base = m0 + quad * 32;
        const int j = lane & 7, gcol = col0 + 4 * j;
        if (row_base < M && gcol < N) {
          const bool full = gcol + 4 <= N;
          const bool fast_r = ep.residual && full && vec_r;
          float4 resv[8];
          if (fast_r) {
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              const int grow = row_base + 4 * t + (lane >> 3);
              resv[t] = grow < M ? *(const float4*)(ep.residual + (long long)grow * ep.ldr + gcol)
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
          float bv[4] = {0.f, 0.f, 0.f, 0.f};
          if (ep.bias) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (gcol + e < N) bv[e] = ep.bias[gcol + e];
          }
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const int rr = 4 * t + (lane >> 3);
            const int grow = row_base + rr;
            float4 v4 = *(const float4*)(stage_base + rr * 128 + ((j ^ (rr & 7)) << 4));
            if (grow >= M) continue;
            float v[4] = {v4.x + bv[0], v4.y + bv[1], v4.z + bv[2], v4.w + bv[3]};
            if (fast_r) {
              v[0] += resv[t].x; v[1] += resv[t].y; v[2] += resv[t].z; v[3] += resv[t].w;
            } else if (ep.residual) {
              const float* rp = ep.residual + (long long)grow * ep.ldr + gcol;
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (gcol + e < N) v[e] += rp[e];
            }
            if (ep.amax_slot) {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (full || gcol + e < N) amax_seen = fmaxf(amax_seen, fabsf(v[e]));
            }
            if (cbase) {
              float* cp = cbase + (long long)grow * ep.ldc + gcol;
              if (full && vec_c) {
                *(float4*)cp = make_float4(v[0], v[1], v[2], v[3]);
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (gcol + e < N) cp[e] = v[e];
              }
            }
            if (ep.c16) {
              __half* hp = ep.c16 + (long long)grow * ep.ldc16 + gcol;
              if (full && vec_h) {
                __half2 h0 = __floats2half2_rn(v[0] * s16, v[1] * s16),
                        h1 = __floats2half2_rn(v[2] * s16, v[3] * s16);
                *(uint2*)hp = make_uint2(*(uint32_t*)&h0, *(uint32_t*)&h1);
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (gcol + e < N) hp[e] = __float2half_rn(v[e] * s16);
              }
            }
          }
        }
        __syncwarp();   // the staging tile is reused by the next chunk
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(lead_tempty + buf * 8);
    }
    if (ep.amax_slot) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        amax_seen = fmaxf(amax_seen, __shfl_xor_sync(0xffffffffu, amax_seen, o));
      if (lane == 0 && amax_seen > 0.f && __float_as_int(amax_seen) > *(volatile int*)ep.amax_slot)
        atomicMax(ep.amax_slot, __float_as_int(amax_seen));
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  // neither CTA may leave while the other can still read its shared memory or signal its barriers
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// Up to six sub-blocks in a single launch (the adapters of a q|k|v group, B and A gradients),
// each from its own slab set part[s][M][ldp].
struct SlabSegs {
  int count;
  float* out[6];
  const float* part[6];
  int M[6];
  int m0[6], mcount[6], n0[6], ncount[6];
  long long som[6], son[6];
  int il_off[6];   // FtKoSeg::il_off
};
__global__ void k_slab_reduce_multi(int slabs, int ldp, SlabSegs sg,
                                    const float* __restrict__ alpha_ptr, float alpha,
                                    int accumulate) {
  ft_pdl_wait();
  ft_pdl_launch();
  const float a = (alpha_ptr ? *alpha_ptr : 1.0f) * alpha;
  const int seg = blockIdx.y;
  if (seg >= sg.count) return;
  const int ncount = sg.ncount[seg], M = sg.M[seg];
  const float* __restrict__ part = sg.part[seg];
  size_t total = (size_t)sg.mcount[seg] * ncount;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += st) {
    int m = (int)(i / ncount), n = (int)(i % ncount);
    float acc = 0.f;
    const int il = sg.il_off[seg];
    const int prow = il < 0 ? sg.m0[seg] + m : ((m >> 5) << 6) + il + (m & 31);
    for (int s = 0; s < slabs; ++s)
      acc += part[((size_t)s * M + prow) * ldp + (sg.n0[seg] + n)];
    float* o = sg.out[seg] + (long long)m * sg.som[seg] + (long long)n * sg.son[seg];
    *o = accumulate ? *o + a * acc : a * acc;
  }
}


// ------------------------------------------------------------------------------ f32 -> f16
// Largest magnitude of a strided matrix, as the bit pattern of a non-negative float (which
// orders like an integer), combined with atomicMax: the result does not depend on the order.
__global__ void k_amax(const float* __restrict__ src, long long ld, int rows, int cols,
                       int* __restrict__ amax_bits) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long st = (long long)gridDim.x * blockDim.x;
  float m = 0.f;
  if ((cols & 3) == 0 && (ld & 3) == 0 && (((uintptr_t)src) & 15) == 0) {
    long long per_row = cols / 4, total = (long long)rows * per_row;
    for (; i < total; i += st) {
      long long r = i / per_row, c = (i % per_row) * 4;
      float4 v = *(const float4*)(src + r * ld + c);
      m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
  } else {
    long long total = (long long)rows * cols;
    for (; i < total; i += st) {
      long long r = i / cols, c = i % cols;
      m = fmaxf(m, fabsf(src[r * ld + c]));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(amax_bits, __float_as_int(m));
}


// scales[0] = S (power of two bringing the largest magnitude into [2^(t-1), 2^t), t =
// target_exp), scales[1] = 1/S, scales[2] = 2^-11/S (the factor of the low half in split mode)
__global__ void k_scale_from_amax(const int* __restrict__ amax_bits, float* __restrict__ scales,
                                  int target_exp) {
  ft_pdl_wait();
  ft_pdl_launch();
  float amax = __int_as_float(*amax_bits);
  float S = 1.0f;
  if (amax > 0.f && isfinite(amax)) {
    int e;
    frexpf(amax, &e);           // amax = f * 2^e, f in [0.5, 1)
    S = ldexpf(1.0f, target_exp - e);
  }
  scales[0] = S;
  scales[1] = 1.0f / S;
  scales[2] = ldexpf(1.0f / S, -11);
}

// f32 [rows, cols] (pitch ld) -> f16 [rows, ldo]: hi = f16(x*S); lo (optional) = the rounding
// remainder times 2^11, so that x*S = hi + lo * 2^-11 to about 22 significant bits.
// One thread per 4 output columns; only the group holding the last column is zero-padded
// (TMA zero-fills beyond the tensor map's extent, so the rest of the pitch is never read).
__global__ void k_to_f16(const float* __restrict__ src, long long ld, __half* __restrict__ hi,
                         __half* __restrict__ lo, long long ldo, int rows, int cols,
                         const float* __restrict__ scales, const int* __restrict__ amax_bits,
                         int target_exp, float* __restrict__ scales_out) {
  ft_pdl_wait();
  ft_pdl_launch();
  // the scale is either given, or derived here from the amax a producer left behind (then
  // one thread also publishes {S, 1/S, 2^-11/S} for the products that follow)
  float S = scales ? scales[0] : 1.0f;
  if (amax_bits) {
    S = ft_scale_from_amax_bits(*amax_bits, target_exp);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      scales_out[0] = S;
      scales_out[1] = 1.0f / S;
      scales_out[2] = ldexpf(1.0f / S, -11);
    }
  }
  long long per_row = (cols + 3) / 4;
  long long total = (long long)rows * per_row;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long st = (long long)gridDim.x * blockDim.x;
  for (; i < total; i += st) {
    long long r = i / per_row;
    int c = (int)(i % per_row) * 4;
    const float* s = src + r * ld + c;
    float v[4];
    if (c + 4 <= cols && (((uintptr_t)s) & 15) == 0) {
      float4 t = *(const float4*)s;
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = (c + j < cols) ? s[j] : 0.f;
    }
    unsigned short h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float x = v[j] * S;
      __half hh = __float2half_rn(x);
      __half ll = __float2half_rn((x - __half2float(hh)) * 2048.0f);
      h[j] = __half_as_ushort(hh);
      l[j] = __half_as_ushort(ll);
    }
    uint2 hv = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
    *(uint2*)(hi + r * ldo + c) = hv;
    if (lo) {
      uint2 lv = make_uint2((uint32_t)l[0] | ((uint32_t)l[1] << 16), (uint32_t)l[2] | ((uint32_t)l[3] << 16));
      *(uint2*)(lo + r * ldo + c) = lv;
    }
  }
}

// The common case of k_to_f16 (no low half, widths and pitches multiples of 8, aligned rows):
// eight columns per thread, two 16-byte loads and one 16-byte store, no division in the loop.
__global__ void k_to_f16_v8(const float* __restrict__ src, long long ld, __half* __restrict__ hi,
                            long long ldo, int rows, int cols, const float* __restrict__ scales,
                            const int* __restrict__ amax_bits, int target_exp,
                            float* __restrict__ scales_out) {
  ft_pdl_wait();
  ft_pdl_launch();
  float S = scales ? scales[0] : 1.0f;
  if (amax_bits) {
    S = ft_scale_from_amax_bits(*amax_bits, target_exp);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      scales_out[0] = S;
      scales_out[1] = 1.0f / S;
      scales_out[2] = ldexpf(1.0f / S, -11);
    }
  }
  const size_t per_row = (size_t)cols / 8, total = (size_t)rows * per_row;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t st = (size_t)gridDim.x * blockDim.x;
  RowWalk w(i, st, per_row);
  for (; i < total; i += st, w.next()) {
    const size_t c = (size_t)w.c * 8;
    const float* s = src + w.r * ld + c;
    const float4 x = *(const float4*)s, y = *(const float4*)(s + 4);
    const __half2 h0 = __floats2half2_rn(x.x * S, x.y * S), h1 = __floats2half2_rn(x.z * S, x.w * S);
    const __half2 h2 = __floats2half2_rn(y.x * S, y.y * S), h3 = __floats2half2_rn(y.z * S, y.w * S);
    *(uint4*)(hi + w.r * ldo + c) =
        make_uint4(*(const uint32_t*)&h0, *(const uint32_t*)&h1, *(const uint32_t*)&h2, *(const uint32_t*)&h3);
  }
}

// profile name of a token-reduction launch; FT_PROFILE_SHAPES=1 appends the problem sizes
static const char* ko_name(const KoPair& ko) {
  static const bool shapes = getenv("FT_PROFILE_SHAPES") != nullptr;
  if (!shapes) return "k_gemm_tc<64,token-reduction>";
  static std::map<std::pair<int, int>, std::string> names;
  auto key = std::make_pair(ko.p[0].M, ko.p[1].M);
  auto it = names.find(key);
  if (it == names.end()) {
    char buf[96];
    snprintf(buf, sizeof(buf), "k_gemm_tc<64,token-reduction>[%d+%d,s%d]", ko.p[0].M, ko.p[1].M,
             ko.p[0].splits);
    it = names.emplace(key, buf).first;
  }
  return it->second.c_str();
}

template <int BN, int STAGES, bool KOUTER, int MH = 1>
int launch_tc(FtContext* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& ma2,
              const CUtensorMap& mb2, const Epilogue& ep, int M, int N, int K, int K2, int splits,
              uint32_t idesc, double flops, const CUtensorMap* mb3 = nullptr,
              const PreTile* pre_in = nullptr, const KoPair* ko_in = nullptr, int ko_tiles_host = 0) {
  PreTile pre;
  memset(&pre, 0, sizeof(pre));
  if (pre_in) pre = *pre_in;
  KoPair ko;
  memset(&ko, 0, sizeof(ko));
  if (ko_in) ko = *ko_in;
  const CUtensorMap& map3 = mb3 ? *mb3 : mb;
  using L = SmemLayout<BN, STAGES, MH>;
  // function attributes are per device: set once on each device that launches this kernel
  static bool configured[FT_MAX_DEVICES] = {};
  if (!configured[ctx->device]) {
    FT_CUDA(cudaFuncSetAttribute(k_gemm_tc<BN, STAGES, KOUTER, MH>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
    configured[ctx->device] = true;
  }
  int tiles = KOUTER ? ko_tiles_host : ft_cdiv(M, MH * BM) * ft_cdiv(N, BN);
  int grid = std::min(tiles, ctx->sm_count);
  int* dbg = ctx->debug_markers ? ctx->status_dev : nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (ctx->profile) {
    while (ctx->prof_events.size() < ctx->prof_used + 2) {
      cudaEvent_t e;
      FT_CUDA(cudaEventCreate(&e));
      ctx->prof_events.push_back(e);
    }
    if (ctx->prof_fused.size() < ctx->prof_events.size() / 2) ctx->prof_fused.resize(ctx->prof_events.size() / 2);
    ctx->prof_fused[ctx->prof_used / 2] = ctx->next_launch_fused ? 1 : 0;
    if (ctx->next_launch_fused) ctx->prof_fused_flops += flops;
    e0 = ctx->prof_events[ctx->prof_used++];
    e1 = ctx->prof_events[ctx->prof_used++];
    FT_CUDA(cudaEventRecord(e0, ctx->stream));
  }
  {
    // by-name profiling: one name per instantiation
    const char* nm = KOUTER ? ko_name(ko)
                            : (BN == 256 ? (MH == 2 ? "k_gemm_tc<256x256>" : "k_gemm_tc<128x256>")
                                         : (BN == 128 ? "k_gemm_tc<128x128>" : "k_gemm_tc<128x64>"));
    const bool pa = ctx->profile_all;
    if (pa) ft_prof_begin(ctx, nm);
    ctx->profile_all = false;
    cudaError_t le = ft_launch_ex(ctx, k_gemm_tc<BN, STAGES, KOUTER, MH>, grid, GEMM_THREADS,
                                  L::DYN_BYTES, ma, mb, ma2, mb2, map3, ep, pre, ko, M, N, K, K2, splits,
                                  idesc, ctx->status_dev, dbg);
    ctx->profile_all = pa;
    if (pa) ft_prof_end(ctx);
    ctx->launches++;
    if (le == cudaSuccess) le = cudaPeekAtLastError();
    if (le != cudaSuccess) return ft_cuda_fail(le, "k_gemm_tc", __FILE__, __LINE__);
  }
  if (ctx->profile) {
    FT_CUDA(cudaEventRecord(e1, ctx->stream));
    ctx->prof_flops += flops;
    ctx->prof_bytes += ctx->next_launch_bytes;
    ctx->prof_launches++;
  }
  return FT_OK;
}

// CTA-pair launch: `tiles` 256 x 256 output tiles over as many clusters of two as can be
// resident at once (pre-tiles rely on every cluster making progress).
template <int STAGES>
int launch_tc2(FtContext* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& ma2,
               const CUtensorMap& mb2, const CUtensorMap& mb3, const Epilogue& ep, const PreTile& pre,
               int M, int N, int K, int K2, uint32_t idesc, double flops) {
  using L = Smem2<STAGES>;
  // function attributes and cluster occupancy are per device
  static bool configured_dev[FT_MAX_DEVICES] = {};
  static int max_pairs_dev[FT_MAX_DEVICES] = {};
  bool& configured = configured_dev[ctx->device];
  int& max_pairs = max_pairs_dev[ctx->device];
  if (!configured) {
    FT_CUDA(cudaFuncSetAttribute(k_gemm_tc2<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 L::DYN_BYTES));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(ctx->sm_count & ~1));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = L::DYN_BYTES;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int n = 0;
    FT_CUDA(cudaOccupancyMaxActiveClusters(&n, k_gemm_tc2<STAGES>, &cfg));
    max_pairs = std::min(n, ctx->sm_count / 2);
    configured = true;
  }
  if (max_pairs < 1) return FT_ERR_UNSUPPORTED;
  const int tiles = ft_cdiv(M, 256) * ft_cdiv(N, 256);
  const int pairs = std::max(1, std::min(tiles, max_pairs));
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (ctx->profile) {
    while (ctx->prof_events.size() < ctx->prof_used + 2) {
      cudaEvent_t e;
      FT_CUDA(cudaEventCreate(&e));
      ctx->prof_events.push_back(e);
    }
    if (ctx->prof_fused.size() < ctx->prof_events.size() / 2) ctx->prof_fused.resize(ctx->prof_events.size() / 2);
    ctx->prof_fused[ctx->prof_used / 2] = ctx->next_launch_fused ? 1 : 0;
    if (ctx->next_launch_fused) ctx->prof_fused_flops += flops;
    e0 = ctx->prof_events[ctx->prof_used++];
    e1 = ctx->prof_events[ctx->prof_used++];
    FT_CUDA(cudaEventRecord(e0, ctx->stream));
  }
  {
    const bool pa = ctx->profile_all;
    if (pa) {
      // FT_PROFILE_SHAPES=1 appends the problem sizes (M x N x K + adapter K, p = with pre-tiles)
      static const bool shapes = getenv("FT_PROFILE_SHAPES") != nullptr;
      const char* name = "k_gemm_tc2<pair 256x256>";
      if (shapes) {
        static std::map<std::string, std::string> names;
        char buf[112];
        snprintf(buf, sizeof(buf), "k_gemm_tc2<pair 256x256>[%dx%dx%d+%d%s]", M, N, K, K2,
                 pre.tiles > 0 ? ",p" : "");
        name = names.emplace(buf, buf).first->second.c_str();
      }
      ft_prof_begin(ctx, name);
    }
    ctx->profile_all = false;
    cudaError_t le = ft_launch_ex(ctx, k_gemm_tc2<STAGES>, 2 * pairs, GEMM_THREADS, L::DYN_BYTES, ma, mb,
                                  ma2, mb2, mb3, ep, pre, M, N, K, K2, idesc, ctx->status_dev);
    ctx->profile_all = pa;
    if (pa) ft_prof_end(ctx);
    ctx->launches++;
    if (le == cudaSuccess) le = cudaPeekAtLastError();
    if (le != cudaSuccess) return ft_cuda_fail(le, "k_gemm_tc2", __FILE__, __LINE__);
  }
  if (ctx->profile) {
    FT_CUDA(cudaEventRecord(e1, ctx->stream));
    ctx->prof_flops += flops;
    ctx->prof_bytes += ctx->next_launch_bytes;
    ctx->prof_launches++;
  }
  return FT_OK;
}

}  // namespace

int ft_amax_arm(FtContext* ctx) {
  int* slot = nullptr;
  FT_TRY(ft_take_amax_slot(ctx, &slot));
  ctx->amax_out = slot;
  ctx->amax_ready = false;
  return FT_OK;
}

// {S, 1/S, 2^-11/S} from the amax a producer left in the slot, or from a pass over `src`.
int ft_scales_from_amax_or_pass(FtContext* ctx, const float* src, long long ld, int rows, int cols,
                                int target_exp, const float** scales_out) {
  const bool ready = ctx->amax_ready && ctx->amax_out;
  int* slot = ctx->amax_out;
  ctx->amax_out = nullptr;
  ctx->amax_ready = false;
  if (!ready) {
    FT_TRY(ft_take_amax_slot(ctx, &slot));
    long long n = (long long)rows * cols;
    int g = (int)std::max<long long>(1, std::min<long long>((n + 4095) / 4096,
                                                            (long long)ctx->sm_count * 8));
    FT_LAUNCH(ctx, k_amax, g, 256, 0, src, ld, rows, cols, slot);
  }
  FT_LAUNCH_PDL(ctx, k_scale_from_amax, 1, 1, 0, (const int*)slot, ctx->scale_buf + 4,
            target_exp);
  *scales_out = ctx->scale_buf + 4;
  return FT_OK;
}

int ft_to_f16(FtContext* ctx, const float* src, long long ld, __half* hi, __half* lo,
              long long ldo, int rows, int cols, bool auto_scale, const float** scales_out,
              int target_exp) {
  FT_REQUIRE(ldo % 8 == 0 && ldo >= cols, "to_f16: output pitch %lld must be a multiple of 8", ldo);
  const float* scales = nullptr;
  const int* amax_bits = nullptr;
  if (auto_scale) {
    if (ctx->amax_ready && ctx->amax_out) {
      // a producer already left the amax: the conversion derives the scale itself
      amax_bits = ctx->amax_out;
      ctx->amax_out = nullptr;
      ctx->amax_ready = false;
      if (scales_out) *scales_out = ctx->scale_buf + 4;
    } else {
      FT_TRY(ft_scales_from_amax_or_pass(ctx, src, ld, rows, cols, target_exp, &scales));
      if (scales_out) *scales_out = scales;
    }
  } else if (scales_out) {
    *scales_out = nullptr;
  }
  if (!lo && (cols % 8) == 0 && (ld % 4) == 0 && ((((uintptr_t)src) | ((uintptr_t)hi)) & 15) == 0) {
    const long long total8 = (long long)rows * (cols / 8);
    const int grid8 = (int)std::max<long long>(1, std::min<long long>((total8 + 255) / 256,
                                                                      (long long)ctx->sm_count * 16));
    FT_LAUNCH_PDL(ctx, k_to_f16_v8, grid8, 256, 0, src, ld, hi, ldo, rows, cols, scales, amax_bits,
                  target_exp, ctx->scale_buf + 4);
    return FT_OK;
  }
  long long total = (long long)rows * ((cols + 3) / 4);
  int grid = (int)std::max<long long>(1, std::min<long long>((total + 255) / 256,
                                                             (long long)ctx->sm_count * 16));
  FT_LAUNCH_PDL(ctx, k_to_f16, grid, 256, 0, src, ld, hi, lo, ldo, rows, cols, scales, amax_bits,
            target_exp, ctx->scale_buf + 4);
  return FT_OK;
}

static bool tma_ok(const void* p, long long ld, int k) {
  return p && (((uintptr_t)p) & 15) == 0 && (ld % 8) == 0 && ld >= k;
}

// operands read once, results written once (what a launch must move at least)
static double gemm_algorithmic_bytes(const FtGemmArgs& g) {
  double b = 2.0 * g.M * (double)(g.K + g.K2) + 2.0 * g.N * (double)(g.K + g.K2);
  if (g.c) b += 4.0 * g.M * (double)g.N;
  if (g.c16) b += 2.0 * g.M * (double)g.N;
  if (g.residual) b += 4.0 * g.M * (double)g.N;
  if (g.pre_b) b += 2.0 * 64.0 * g.K + 2.0 * g.M * 64.0;
  return b;
}

// CTA pairs (256 x 256 tile over two SMs) are the default for wide products: measured
// 1340-1480 TFLOP/s against 1150-1280 for the 128-row and 1100-1400 for the 256-row
// single-CTA tiles; FT_GEMM_TILE_M=128|256 selects those, 512 the pairs
bool ft_gemm_tc_pair_eligible(const FtContext* ctx, int M, int N) {
  return N > 128 && M >= 256 && (ctx->tile_m_override == 512 || ctx->tile_m_override == 0);
}

int ft_gemm_tc_ex(FtContext* ctx, const FtGemmArgs& g) {
  ctx->next_launch_bytes = gemm_algorithmic_bytes(g);
  ctx->next_launch_fused = g.rope_table || g.swi_f16 || g.swi_dgu16;
  if (g.ab_type != FT_F16 && g.ab_type != FT_BF16) return FT_ERR_UNSUPPORTED;
  if (!tma_ok(g.a, g.lda, g.K) || !tma_ok(g.b, g.ldb, g.K) || g.K < 8) return FT_ERR_UNSUPPORTED;
  const bool tail = g.K2 > 0;
  if (tail && (!tma_ok(g.a2, g.lda2, g.K2) || !tma_ok(g.b2, g.ldb2, g.K2))) return FT_ERR_UNSUPPORTED;
  CUtensorMap ma, mb, ma2, mb2;
  const int BN = g.N > 128 ? 256 : (g.N > 64 ? 128 : 64);
  // 256-row tiles move a third less operand data per FLOP (the 128-row form is bound by L2
  // bandwidth) but cannot overlap their epilogue and come in coarser waves: take them when
  // the estimated time, waves x relative tile cost, is lower.  FT_GEMM_TILE_M=128|256 forces.
  int MH = 1;
  if (BN == 256 && g.M >= 256) {
    const int sms = ctx->sm_count;
    const long long t1 = (long long)ft_cdiv(g.M, 128) * ft_cdiv(g.N, 256);
    const long long t2 = (long long)ft_cdiv(g.M, 256) * ft_cdiv(g.N, 256);
    const double kk = (double)(g.K + g.K2);
    // measured on B200, in units of one K element of a 128-row tile (about 7 ns): a 128 x 256
    // tile costs K + 200, a 256 x 256 tile 1.6 K + 1680 (its epilogue is not hidden, and every
    // SM stores its 256 KiB at the same moment)
    const double cost1 = (double)((t1 + sms - 1) / sms) * (kk + 200.0);
    const double cost2 = (double)((t2 + sms - 1) / sms) * (1.6 * kk + 1680.0);
    MH = cost2 < cost1 ? 2 : 1;
    if (ctx->tile_m_override == 128) MH = 1;
    if (ctx->tile_m_override == 256) MH = 2;
  }
  const CUtensorMapDataType dt = g.ab_type == FT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const bool pair = ft_gemm_tc_pair_eligible(ctx, g.M, g.N);
  if (g.carry_amax && !g.swi_dgu16) {
    FT_REQUIRE(pair && g.c16 && g.carry_scales,
               "gemm: a carried scale needs a CTA-pair launch with an f16 result");
  }
  if (g.swi_f16) {
    FT_REQUIRE(pair && g.c16 && !g.c && !g.residual && !g.bias && !g.carry_amax && !g.rope_table &&
                   g.amax_slot && (g.N % 64) == 0 && (g.ldc16 % 8) == 0 && (g.swi_ldf % 8) == 0 &&
                   ((((uintptr_t)g.c16) | ((uintptr_t)g.swi_f16)) & 15) == 0,
               "gemm: the SwiGLU epilogue needs a CTA-pair launch, f16 results and 64-column runs");
  }
  if (g.swi_dgu16) {
    FT_REQUIRE(pair && !g.c && !g.c16 && !g.residual && !g.bias && !g.rope_table && !g.swi_f16 &&
                   g.carry_amax && g.swi_gu16 && g.swi_gu_amax && g.swi_scales && g.amax_slot &&
                   (g.N % 32) == 0 && (g.swi_ldgu % 8) == 0 && (g.swi_lddgu % 8) == 0 &&
                   ((((uintptr_t)g.swi_gu16) | ((uintptr_t)g.swi_dgu16)) & 15) == 0,
               "gemm: the SwiGLU backward epilogue needs a CTA-pair launch and interleaved f16 rows");
  }
  if (g.rope_table) {
    FT_REQUIRE(pair && g.c16 && !g.c && !g.residual && !g.carry_amax && !g.want_amax && !g.amax_slot &&
                   (g.N % 64) == 0 && (g.rope_cols % 64) == 0 && g.rope_seq > 0 && (g.ldc16 % 8) == 0 &&
                   ((((uintptr_t)g.c16) | ((uintptr_t)g.rope_table)) & 15) == 0,
               "gemm: the rotary epilogue needs a CTA-pair launch, an f16-only result and 64-wide heads");
  }
  if (pair) {
    const int fmt = g.ab_type == FT_F16 ? 0 : 1;
    FT_TRY(make_map(ctx, &ma, g.a, dt, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, BK, 128));
    FT_TRY(make_map(ctx, &mb, g.b, dt, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, BK, 128));
    if (tail) {
      FT_TRY(make_map(ctx, &ma2, g.a2, dt, (uint64_t)g.K2, (uint64_t)g.M, (uint64_t)g.lda2, BK, 128));
      FT_TRY(make_map(ctx, &mb2, g.b2, dt, (uint64_t)g.K2, (uint64_t)g.N, (uint64_t)g.ldb2, BK, 128));
    } else {
      ma2 = ma;
      mb2 = mb;
    }
    Epilogue ep;
    ep.c = g.c; ep.ldc = g.ldc; ep.c16 = g.c16; ep.ldc16 = g.ldc16;
    ep.alpha_ptr = g.alpha_ptr; ep.alpha = g.alpha; ep.bias = g.bias;
    ep.residual = g.residual; ep.ldr = g.ldr;
    ep.amax_slot = g.amax_slot;
    if (!ep.amax_slot && g.want_amax && ctx->amax_out) {
      ep.amax_slot = ctx->amax_out;
      ctx->amax_ready = true;
    }
    ep.carry_amax = g.carry_amax; ep.carry_exp = g.carry_exp; ep.carry_scales = g.carry_scales;
    ep.rope_table = (const float2*)g.rope_table; ep.rope_seq = g.rope_seq; ep.rope_cols = g.rope_cols;
    ep.swi_f16 = g.swi_f16; ep.swi_ldf = g.swi_ldf;
    ep.swi_gu16 = g.swi_gu16; ep.swi_ldgu = g.swi_ldgu; ep.swi_dgu16 = g.swi_dgu16;
    ep.swi_lddgu = g.swi_lddgu; ep.swi_gu_amax = g.swi_gu_amax; ep.swi_scales = g.swi_scales;
    {
      const int used = g.k2_used > 0 ? std::min(g.k2_used, g.K2) : g.K2;
      const int last = used - (ft_cdiv(std::max(used, 1), BK) - 1) * BK;   // columns in the last tail k-block
      ep.tail_steps = std::max(1, std::min(BK / UMMA_K, ft_cdiv(last, UMMA_K)));
      static const bool full_tail = getenv("FT_TAIL_FULL") != nullptr;   // A/B switch
      if (full_tail || g.k2_used <= 0 || ft_cdiv(used, BK) != ft_cdiv(g.K2, BK)) ep.tail_steps = BK / UMMA_K;
    }
    double flops = 2.0 * g.M * (double)g.N * (double)(g.K + g.K2);
    CUtensorMap mb3 = mb;
    PreTile pre;
    memset(&pre, 0, sizeof(pre));
    if (g.pre_b) {
      const int tiles_m = ft_cdiv(g.M, 256);
      if (!tail || !tma_ok(g.pre_b, g.pre_ldb, g.K) || !g.pre_c16 || (g.pre_ldc16 % 4) ||
          (((uintptr_t)g.pre_c16) & 7) || tiles_m > FT_PRE_FLAGS)
        return FT_ERR_UNSUPPORTED;
      FT_TRY(make_map(ctx, &mb3, g.pre_b, dt, (uint64_t)g.K, 64, (uint64_t)g.pre_ldb, BK, 32));
      FT_TRY(ft_take_pre_flags(ctx, tiles_m, &pre.flags));
      pre.tiles = tiles_m;
      pre.c16 = g.pre_c16; pre.ldc16 = g.pre_ldc16; pre.alpha = g.pre_alpha;
      pre.idesc = make_idesc(256, 64, fmt, fmt);
      flops += 2.0 * g.M * 64.0 * (double)g.K;
    }
    return launch_tc2<6>(ctx, ma, mb, ma2, mb2, mb3, ep, pre, g.M, g.N, g.K, g.K2,
                         make_idesc(256, 256, fmt, fmt), flops);
  }
  const uint32_t a_rows = (uint32_t)(MH * BM);
  FT_TRY(make_map(ctx, &ma, g.a, dt, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, BK, a_rows));
  FT_TRY(make_map(ctx, &mb, g.b, dt, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, BK, (uint32_t)BN));
  if (tail) {
    FT_TRY(make_map(ctx, &ma2, g.a2, dt, (uint64_t)g.K2, (uint64_t)g.M, (uint64_t)g.lda2, BK, a_rows));
    FT_TRY(make_map(ctx, &mb2, g.b2, dt, (uint64_t)g.K2, (uint64_t)g.N, (uint64_t)g.ldb2, BK,
                    (uint32_t)BN));
  } else {
    ma2 = ma;
    mb2 = mb;
  }
  // A and B formats must be equal: a mixed descriptor is rejected by the hardware
  const int fmt = g.ab_type == FT_F16 ? 0 : 1;
  const uint32_t idesc = make_idesc(BM, BN, fmt, fmt);
  Epilogue ep;
  ep.c = g.c; ep.ldc = g.ldc; ep.c16 = g.c16; ep.ldc16 = g.ldc16;
  ep.alpha_ptr = g.alpha_ptr; ep.alpha = g.alpha; ep.bias = g.bias;
  ep.residual = g.residual; ep.ldr = g.ldr;
  ep.amax_slot = g.amax_slot;
  if (!ep.amax_slot && g.want_amax && ctx->amax_out) {
    ep.amax_slot = ctx->amax_out;
    ctx->amax_ready = true;
  }
  ep.carry_amax = nullptr; ep.carry_exp = 0; ep.carry_scales = nullptr;
  ep.rope_table = nullptr; ep.rope_seq = 0; ep.rope_cols = 0;
  ep.swi_f16 = nullptr; ep.swi_ldf = 0; ep.swi_gu16 = nullptr; ep.swi_ldgu = 0; ep.swi_dgu16 = nullptr;
  ep.swi_lddgu = 0; ep.swi_gu_amax = nullptr; ep.swi_scales = nullptr;
  ep.tail_steps = BK / UMMA_K;
  double flops = 2.0 * g.M * (double)g.N * (double)(g.K + g.K2);
  // adapter pre-tiles: the tail operand A2 = pre_alpha * A . pre_b^T is made by this launch
  CUtensorMap mb3;
  PreTile pre;
  memset(&pre, 0, sizeof(pre));
  const bool with_pre = g.pre_b != nullptr;
  if (with_pre) {
    const int tiles_m = ft_cdiv(g.M, MH * BM);
    if (!tail || !tma_ok(g.pre_b, g.pre_ldb, g.K) || !g.pre_c16 || (g.pre_ldc16 % 4) ||
        (((uintptr_t)g.pre_c16) & 7) || tiles_m > FT_PRE_FLAGS)
      return FT_ERR_UNSUPPORTED;
    FT_TRY(make_map(ctx, &mb3, g.pre_b, dt, (uint64_t)g.K, 64, (uint64_t)g.pre_ldb, BK, 64));
    FT_TRY(ft_take_pre_flags(ctx, tiles_m, &pre.flags));
    pre.tiles = tiles_m;
    pre.c16 = g.pre_c16; pre.ldc16 = g.pre_ldc16; pre.alpha = g.pre_alpha;
    pre.idesc = make_idesc(BM, 64, fmt, fmt);
    flops += 2.0 * g.M * 64.0 * (double)g.K;
  }
  const CUtensorMap* p3 = with_pre ? &mb3 : nullptr;
  const PreTile* pp = with_pre ? &pre : nullptr;
  if (MH == 2)
    return launch_tc<256, 3, false, 2>(ctx, ma, mb, ma2, mb2, ep, g.M, g.N, g.K, g.K2, 1, idesc, flops, p3, pp);
  switch (BN) {
    case 256: return launch_tc<256, 4, false>(ctx, ma, mb, ma2, mb2, ep, g.M, g.N, g.K, g.K2, 1, idesc, flops, p3, pp);
    case 128: return launch_tc<128, 6, false>(ctx, ma, mb, ma2, mb2, ep, g.M, g.N, g.K, g.K2, 1, idesc, flops, p3, pp);
    default: return launch_tc<64, 8, false>(ctx, ma, mb, ma2, mb2, ep, g.M, g.N, g.K, g.K2, 1, idesc, flops, p3, pp);
  }
}

int ft_gemm_tc(FtContext* ctx, const void* a, long long lda, const void* b, FtDType ab_type,
               long long ldb, float* c, long long ldc, int M, int N, int K, bool accumulate,
               const float* alpha_ptr) {
  FtGemmArgs g;
  g.a = a; g.lda = lda; g.b = b; g.ldb = ldb; g.ab_type = ab_type;
  g.M = M; g.N = N; g.K = K;
  g.c = c; g.ldc = ldc; g.alpha_ptr = alpha_ptr;
  if (accumulate) { g.residual = c; g.ldr = ldc; }
  return ft_gemm_tc_ex(ctx, g);
}

// Token-reduction products on the tensor cores: P_q[M_q, 64] = sum_t A_q[t, m] B_q[t, n] for one or
// two problems that share T (A_q is [T, M_q], B_q is [T, <=64], both f16), K-split into f32
// slabs prob[q].slabs[nslabs][M_q][64] that the caller reduces (ft_slab_reduce_problems).
static void ko_pick_splits(int sms, int tm0, int tm1, int kb, int* splits_out, int* per_out) {
  // cost of a choice = waves x (k-blocks per split + a fixed per-tile cost of about 6 k-blocks)
  double best = 1e30;
  int bs = 1;
  for (int sp = 1; sp <= std::min(kb, 32); ++sp) {
    const int per = ft_cdiv(kb, sp), real = ft_cdiv(kb, per);
    const int tiles = (tm0 + tm1) * real;
    const double cost = (double)ft_cdiv(tiles, sms) * (per + 6.0);
    if (cost < best - 1e-9) { best = cost; bs = real; }
  }
  *splits_out = bs;
  *per_out = ft_cdiv(kb, bs);
}

int ft_gemm_tc_kouter_pair(FtContext* ctx, int nprob, FtKoProblem* prob, int T) {
  if (nprob < 1 || nprob > 2) return FT_ERR_UNSUPPORTED;
  CUtensorMap ma[2], mb[2];
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const int kb = ft_cdiv(T, BK);
  int tm[2] = {0, 0};
  for (int q = 0; q < nprob; ++q) {
    const FtKoProblem& P = prob[q];
    if (P.N > 64 || !tma_ok(P.a, P.lda, P.M) || !tma_ok(P.b, P.ldb, P.N) || (P.M % 8) || (P.N % 8) ||
        P.nseg > 3)
      return FT_ERR_UNSUPPORTED;
    // inner dimension = M/N index, outer = token row; box = 64 x 64
    FT_TRY(make_map(ctx, &ma[q], P.a, dt, (uint64_t)P.M, (uint64_t)T, (uint64_t)P.lda, 64, BK));
    FT_TRY(make_map(ctx, &mb[q], P.b, dt, (uint64_t)P.N, (uint64_t)T, (uint64_t)P.ldb, 64, BK));
    tm[q] = ft_cdiv(P.M, BM);
  }
  if (nprob == 1) { ma[1] = ma[0]; mb[1] = mb[0]; }
  int splits = 1, per = kb;
  ko_pick_splits(ctx->sm_count, tm[0], tm[1], kb, &splits, &per);
  size_t slab_floats = 0;
  for (int q = 0; q < nprob; ++q) slab_floats += (size_t)splits * prob[q].M * 64;
  void* s = nullptr;
  FT_TRY(ft_scratch(ctx, slab_floats * sizeof(float), &s));
  KoPair ko;
  memset(&ko, 0, sizeof(ko));
  float* slab = (float*)s;
  double flops = 0;
  for (int q = 0; q < nprob; ++q) {
    KoProblem& K = ko.p[q];
    K.M = prob[q].M; K.splits = splits; K.per = per; K.slabs = slab;
    prob[q].slabs = slab;
    prob[q].nslabs = splits;
    slab += (size_t)splits * prob[q].M * 64;
    flops += 2.0 * prob[q].M * 64.0 * T;
  }
  ctx->next_launch_bytes = 0.0;
  for (int q = 0; q < nprob; ++q)
    ctx->next_launch_bytes += 2.0 * T * (double)prob[q].M + 2.0 * T * 64.0 + 4.0 * splits * (double)prob[q].M * 64.0;
  Epilogue ep;
  ep.c = (float*)s; ep.ldc = 64; ep.c16 = nullptr; ep.ldc16 = 0;
  ep.alpha_ptr = nullptr; ep.alpha = 1.f; ep.bias = nullptr; ep.residual = nullptr; ep.ldr = 0;
  ep.amax_slot = nullptr;
  ep.carry_amax = nullptr; ep.carry_exp = 0; ep.carry_scales = nullptr;
  ep.rope_table = nullptr; ep.rope_seq = 0; ep.rope_cols = 0;
  ep.swi_f16 = nullptr; ep.swi_ldf = 0; ep.swi_gu16 = nullptr; ep.swi_ldgu = 0; ep.swi_dgu16 = nullptr;
  ep.swi_lddgu = 0; ep.swi_gu_amax = nullptr; ep.swi_scales = nullptr;
  ep.tail_steps = BK / UMMA_K;
  // both operands M/N-major: bits 15 and 16 of the instruction descriptor
  const uint32_t idesc = make_idesc(BM, 64, 0, 0) | (1u << 15) | (1u << 16);
  return launch_tc<64, 8, true>(ctx, ma[0], mb[0], ma[1], mb[1], ep, prob[0].M, 64, T, 0, splits, idesc,
                                flops, nullptr, nullptr, &ko, (tm[0] + tm[1]) * splits);
}



// The segments of every problem of a token-reduction launch, reduced in one launch.
int ft_slab_reduce_problems(FtContext* ctx, int nprob, const FtKoProblem* prob,
                            const float* alpha_ptr, float alpha, bool accumulate) {
  SlabSegs sg;
  memset(&sg, 0, sizeof(sg));
  size_t most = 0;
  int nslabs = 0;
  for (int q = 0; q < nprob; ++q) {
    nslabs = prob[q].nslabs;
    for (int i = 0; i < prob[q].nseg && sg.count < 6; ++i) {
      const FtKoSeg& S = prob[q].seg[i];
      const int k = sg.count++;
      sg.out[k] = S.out; sg.part[k] = prob[q].slabs; sg.M[k] = prob[q].M;
      sg.m0[k] = S.m0; sg.mcount[k] = S.mcount; sg.n0[k] = S.n0; sg.ncount[k] = S.ncount;
      sg.som[k] = S.som; sg.son[k] = S.son; sg.il_off[k] = S.il_off;
      most = std::max(most, (size_t)S.mcount * S.ncount);
    }
  }
  if (!most) return FT_OK;
  dim3 grid((unsigned)std::min<size_t>((most + 255) / 256, (size_t)ctx->sm_count * 4), sg.count);
  FT_LAUNCH_PDL(ctx, k_slab_reduce_multi, grid, 256, 0, nslabs, 64, sg, alpha_ptr, alpha,
                accumulate ? 1 : 0);
  return FT_OK;
}


// C (=|+=) A(f32, rounded to f16 with optional auto scale) . B(f16)^T, single or split pass.
int ft_gemm_tc_f32a(FtContext* ctx, const float* a, long long lda_f32, __half* stage_hi,
                    __half* stage_lo, const void* b_f16, long long ldb, float* c, long long ldc,
                    int M, int N, int K, bool accumulate, bool auto_scale) {
  const long long kp = (long long)ft_align_up((size_t)K, 8);
  const bool split = ctx->gemm_mode == FT_GEMM_F16X2;
  const float* scales = nullptr;
  FT_TRY(ft_to_f16(ctx, a, lda_f32, stage_hi, split ? stage_lo : nullptr, kp, M, K, auto_scale,
                   &scales));
  // without auto scale: alpha 1 for the high half, 2^-11 (a constant in scale_buf) for the low
  const float* alpha_hi = scales ? scales + 1 : nullptr;
  const float* alpha_lo = scales ? scales + 2 : ctx->scale_buf + 1;
  if (!split)
    return ft_gemm_tc(ctx, stage_hi, kp, b_f16, FT_F16, ldb, c, ldc, M, N, K, accumulate, alpha_hi);
  // The tensor core adds each 16-deep group of products into its f32 accumulator with the
  // low bits cut off, not rounded: a sum over K shrinks by about K/16 * 2^-25 of its size
  // (measured 2.3e-4 at K = 151936, the head's input gradient; 1.1e-4 at K = 49152).  The split
  // mode promises f32 accuracy, so a long K runs in slices that the f32 epilogue adds up.
  const int kSlice = 2048;
  const __half* b = (const __half*)b_f16;
  for (int k0 = 0; k0 < std::max(K, 1); k0 += kSlice) {
    const int kc = std::min(kSlice, K - k0);
    FT_TRY(ft_gemm_tc(ctx, stage_hi + k0, kp, b + k0, FT_F16, ldb, c, ldc, M, N, kc,
                      accumulate || k0 > 0, alpha_hi));
    FT_TRY(ft_gemm_tc(ctx, stage_lo + k0, kp, b + k0, FT_F16, ldb, c, ldc, M, N, kc, true, alpha_lo));
  }
  return FT_OK;
}
