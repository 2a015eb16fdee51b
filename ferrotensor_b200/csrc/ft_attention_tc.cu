// Causal flash attention on the Blackwell tensor cores (head_dim 64, f16 operands, f32
// accumulation and softmax), grouped-query.  Operands are read straight from the fused
// q|k|v buffer [tokens, nq + 2 nkv] (f16, RoPE already applied) with TMA: one 128 x 64 box
// shape serves the query, key and value tiles.
//
// Forward, one CTA per (128 queries, head):
//   S = Q K^T      tcgen05.mma 128 x 128 x 64 into tensor memory
//   softmax        4 warps, thread t owns query row t (= TMEM lane t): tcgen05.ld the row,
//                  online max/sum in the exp2 domain, P written to shared memory as f16 in the
//                  128-byte-swizzled K-major form the next product wants
//   O_j = P V_j    tcgen05.mma 128 x 64 x 128, V used in place as an N-major operand
//   O = sum_j corr * O_j accumulated in registers, normalised at the end.
// One extra warp issues all TMA loads and MMAs; the S product of block j+1 is issued as soon
// as the softmax warps have read block j, so it overlaps with their arithmetic and with P V.
// All waits are bounded (see ft_tc.cuh).
#include <math.h>

#include "ft_tc.cuh"

namespace {

using namespace ft_tc;

constexpr int AT_Q = 128;        // queries per CTA
constexpr int AT_KV = 128;       // keys per block
constexpr int AT_D = 64;         // head_dim
constexpr int AT_THREADS = 160;  // warps 0..3 softmax, warp 4 issuer
constexpr int TILE_BYTES = 128 * 64 * 2;  // one 128 x 64 f16 tile = 16 KiB

struct AttnSmem {
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + TILE_BYTES;          // 1 stage: free as soon as S is done
  static constexpr int V_OFF = K_OFF + TILE_BYTES;          // 2 stages
  static constexpr int P_OFF = V_OFF + 2 * TILE_BYTES;      // 128 x 128 f16 = two K-major tiles
  static constexpr int BAR_OFF = P_OFF + 2 * TILE_BYTES;
  // q_full, k_full, (unused), v_full[2], s_full, s_free, p_full, o_full
  static constexpr int NBAR = 9;
  // 96 KiB of tiles: two CTAs fit in one SM's shared memory
  static constexpr int TOTAL = BAR_OFF + NBAR * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

__device__ __forceinline__ void tc_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) { tc_ld32(taddr, r); }

__global__ void __launch_bounds__(AT_THREADS, 2)
k_attn_fwd_tc(const __grid_constant__ CUtensorMap map_qkv, __half* __restrict__ out16,
              long long ldo16, float* __restrict__ out32, long long ldo32,
              float* __restrict__ stats, int seq, int heads, int kv_heads, int q_col0, int k_col0,
              int v_col0, float scale_log2e, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  const uint32_t bar0 = base + AttnSmem::BAR_OFF;
  const uint32_t bar_q = bar0, bar_k = bar0 + 8, bar_v = bar0 + 24, bar_sfull = bar0 + 40,
                 bar_sfree = bar0 + 48, bar_pfull = bar0 + 56, bar_ofull = bar0 + 64;
  uint32_t* tmem_slot = (uint32_t*)(gbase + AttnSmem::BAR_OFF + AttnSmem::NBAR * 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query blocks first: they have the most key blocks to visit
  const int qblk = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int kvh = h / (heads / kv_heads);
  const int q0 = qblk * AT_Q;
  const int nblk = min(qblk + 1, (seq + AT_KV - 1) / AT_KV);
  const int tok0 = b * seq;  // first token row of this sequence
  constexpr uint32_t TMEM_COLS = 256;  // S: columns [0,128), O_j: [128,192)

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_k, 1);
    mbar_init(bar_k + 8, 1);
    for (int s = 0; s < 2; ++s) mbar_init(bar_v + s * 8, 1);
    mbar_init(bar_sfull, 1);
    mbar_init(bar_sfree, 4);
    mbar_init(bar_pfull, 4);
    mbar_init(bar_ofull, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
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
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA + MMA issuer
    if (lane == 0) {
      const uint32_t sq = base + AttnSmem::Q_OFF, sk = base + AttnSmem::K_OFF,
                     sv = base + AttnSmem::V_OFF, sp = base + AttnSmem::P_OFF;
      const uint32_t idesc_s = make_idesc(128, 128, 0, 0);                 // Q, K both K-major
      const uint32_t idesc_o = make_idesc(128, 64, 0, 0) | (1u << 16);     // V is N-major
      auto load_k = [&](int j) {
        mbar_expect_tx(bar_k, TILE_BYTES);
        tma_load_2d(sk, &map_qkv, bar_k, k_col0 + kvh * AT_D, tok0 + j * AT_KV);
      };
      auto load_v = [&](int j) {
        const int s = j & 1;
        mbar_expect_tx(bar_v + s * 8, TILE_BYTES);
        tma_load_2d(sv + s * TILE_BYTES, &map_qkv, bar_v + s * 8, v_col0 + kvh * AT_D, tok0 + j * AT_KV);
      };
      auto mma_s = [&]() {
        const uint64_t da = make_desc_sw128(sq), db = make_desc_sw128(sk);
#pragma unroll
        for (int k = 0; k < AT_D / 16; ++k)
          tc_mma_f16(tmem_s, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, k > 0 ? 1u : 0u);
        tc_commit(bar_sfull);
      };
      mbar_expect_tx(bar_q, TILE_BYTES);
      tma_load_2d(sq, &map_qkv, bar_q, q_col0 + h * AT_D, tok0 + q0);
      load_k(0);
      load_v(0);
      if (nblk > 1) load_v(1);
      bool ok = mbar_wait(bar_q, 0, abort_flag, status, 11) &&
                mbar_wait(bar_k, 0, abort_flag, status, 12);
      if (ok) {
        tc_fence_after();
        mma_s();
      }
      for (int j = 0; ok && j < nblk; ++j) {
        if (j + 1 < nblk) {
          // the key tile is free once S(j) has been computed: fetch the next one under the
          // softmax of block j, and issue S(j+1) when the softmax warps have read S(j)
          ok = mbar_wait(bar_sfull, j & 1, abort_flag, status, 13);
          if (!ok) break;
          load_k(j + 1);
          ok = mbar_wait(bar_k, (j + 1) & 1, abort_flag, status, 18) &&
               mbar_wait(bar_sfree, j & 1, abort_flag, status, 14);
          if (!ok) break;
          tc_fence_after();
          mma_s();
        }
        ok = mbar_wait(bar_pfull, j & 1, abort_flag, status, 15) &&
             mbar_wait(bar_v + (j & 1) * 8, (j >> 1) & 1, abort_flag, status, 16);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t vt = sv + (j & 1) * TILE_BYTES;
          const uint64_t dv = make_desc_mn_sw128(vt, TILE_BYTES);
#pragma unroll
          for (int k = 0; k < AT_KV / 16; ++k) {
            // P: two K-major 128 x 64 tiles; V: 16 key rows further = +2048 bytes
            const uint64_t dp = make_desc_sw128(sp + (k >> 2) * TILE_BYTES) + (uint64_t)((k & 3) * 2);
            tc_mma_f16(tmem_o, dp, dv + (uint64_t)(k * 128), idesc_o, k > 0 ? 1u : 0u);
          }
          tc_commit(bar_ofull);
        }
        if (j + 2 < nblk) {
          // value stage j&1 is free once P V(j) is done
          ok = mbar_wait(bar_ofull, j & 1, abort_flag, status, 17);
          if (!ok) break;
          load_v(j + 2);
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax warps
    const int row = warp * 32 + lane;          // query row in the tile = TMEM lane
    const int qi = q0 + row;                   // position in the sequence
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    uint8_t* p_smem = gbase + AttnSmem::P_OFF;
    float o_acc[AT_D];
#pragma unroll
    for (int i = 0; i < AT_D; ++i) o_acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; ok && j < nblk; ++j) {
      ok = mbar_wait(bar_sfull, j & 1, abort_flag, status, 21);
      if (!ok) break;
      tc_fence_after();
      // pass 1: the row maximum (scores stay in tensor memory and are read twice)
      float mx = m;
      const bool diag = (j == qblk);
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
        tc_ld32(tmem_s + lane_addr + cb * 32, r);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          float s = __uint_as_float(r[c]) * scale_log2e;
          if (diag && (cb * 32 + c) > row) s = -INFINITY;
          mx = fmaxf(mx, s);
        }
      }
      const float corr = exp2f(m - mx);   // 0 for the first block (m = -inf)
      // fold the previous block's P V into the running output before rescaling it
      if (j > 0) {
        ok = mbar_wait(bar_ofull, (j - 1) & 1, abort_flag, status, 22);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int cb = 0; cb < 2; ++cb) {
          uint32_t r[32];
          tc_ld32(tmem_o + lane_addr + cb * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) o_acc[cb * 32 + c] += __uint_as_float(r[c]);
        }
      }
#pragma unroll
      for (int i = 0; i < AT_D; ++i) o_acc[i] *= corr;
      // pass 2: probabilities -> f16 -> swizzled shared memory
      float sum = 0.f;
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
        tc_ld32(tmem_s + lane_addr + cb * 32, r);
        tc_wait_ld();
        uint32_t packed[16];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float s0 = __uint_as_float(r[c]) * scale_log2e, s1 = __uint_as_float(r[c + 1]) * scale_log2e;
          float p0 = (diag && (cb * 32 + c) > row) ? 0.f : exp2f(s0 - mx);
          float p1 = (diag && (cb * 32 + c + 1) > row) ? 0.f : exp2f(s1 - mx);
          sum += p0 + p1;
          __half2 hp = __floats2half2_rn(p0, p1);
          packed[c >> 1] = *(uint32_t*)&hp;
        }
        // 32 keys = four 16-byte chunks of this row; tile t = keys [64 t, 64 t + 64)
        const int t = cb >> 1;
        uint8_t* rowp = p_smem + t * TILE_BYTES + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = (cb & 1) * 4 + q;
          *(uint4*)(rowp + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
      l = l * corr + sum;
      m = mx;
      // S has been read (next S product may overwrite it); P is visible to the tensor core
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar_sfree);
        mbar_arrive(bar_pfull);
      }
    }
    if (ok) ok = mbar_wait(bar_ofull, (nblk - 1) & 1, abort_flag, status, 23);
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {
        uint32_t r[32];
        tc_ld32(tmem_o + lane_addr + cb * 32, r);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) o_acc[cb * 32 + c] += __uint_as_float(r[c]);
      }
      if (qi < seq) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        const long long tok = (long long)tok0 + qi;
        if (out16) {
          __half* o = out16 + tok * ldo16 + (long long)h * AT_D;
#pragma unroll
          for (int i = 0; i < AT_D; i += 8) {
            __half2 a = __floats2half2_rn(o_acc[i] * inv, o_acc[i + 1] * inv);
            __half2 bb = __floats2half2_rn(o_acc[i + 2] * inv, o_acc[i + 3] * inv);
            __half2 c = __floats2half2_rn(o_acc[i + 4] * inv, o_acc[i + 5] * inv);
            __half2 d = __floats2half2_rn(o_acc[i + 6] * inv, o_acc[i + 7] * inv);
            *(uint4*)(o + i) = make_uint4(*(uint32_t*)&a, *(uint32_t*)&bb, *(uint32_t*)&c, *(uint32_t*)&d);
          }
        }
        if (out32) {
          float* o = out32 + tok * ldo32 + (long long)h * AT_D;
#pragma unroll
          for (int i = 0; i < AT_D; i += 4)
            *(float4*)(o + i) = make_float4(o_acc[i] * inv, o_acc[i + 1] * inv, o_acc[i + 2] * inv,
                                            o_acc[i + 3] * inv);
        }
        if (stats) {
          const size_t srow = ((size_t)b * heads + h) * seq + qi;
          // natural-log LSE of the scaled scores
          stats[2 * srow + 1] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : 3.0e38f;
        }
      }
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
  CUtensorMap map;
  FT_TRY(ft_tc::make_map(ctx, &map, qkv16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (uint64_t)ld,
                         (uint64_t)batch * seq, (uint64_t)ld, 64, 128));
  static bool configured = false;
  if (!configured) {
    FT_CUDA(cudaFuncSetAttribute(k_attn_fwd_tc, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 AttnSmem::DYN_BYTES));
    configured = true;
  }
  dim3 grid(ft_cdiv(seq, AT_Q), batch * heads);
  const float scale_log2e = (1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
  FT_LAUNCH(ctx, k_attn_fwd_tc, grid, AT_THREADS, AttnSmem::DYN_BYTES, map, out16, ldo16, out32,
            ldo32, stats, seq, heads, kv_heads, q_col0, k_col0, v_col0, scale_log2e,
            ctx->status_dev);
  return FT_OK;
}
