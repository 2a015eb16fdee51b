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
#include <cuda.h>
#include <cudaTypedefs.h>

#include "ft_common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;            // 64 x 16-bit = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192; // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr uint32_t SPIN_LIMIT = 1u << 26;  // ~ seconds of polling at most

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises the abort flag) when it gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int where) {
  if (*abort_flag) return false;
  uint32_t spins = 0;
  while (!mbar_test(bar, parity)) {
    if (++spins > SPIN_LIMIT || *abort_flag) {
      if (!*abort_flag) {
        *abort_flag = 1;
        // the status word lives in pinned host memory: plain stores, first writer wins
        // only approximately, which is enough to report "some wait ran out, here"
        volatile int* st = status;
        if (st[0] == 0) {
          st[1] = (int)blockIdx.x;
          st[2] = (int)parity;
          st[0] = 100 + where;
        }
      }
      return false;
    }
    if ((spins & 1023u) == 0) __nanosleep(64);
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];"
      ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, written by TMA
// with 128-byte swizzle: 8-row atoms of 1024 bytes follow each other along M/N (stride byte
// offset 1024); the leading byte offset is not used by swizzled K-major layouts.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address, bits [0,14)
  d |= (uint64_t)0 << 16;                        // leading byte offset, bits [16,30)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                        // descriptor version (Blackwell), bits [46,48)
  d |= (uint64_t)2 << 61;                        // layout type: 128-byte swizzle, bits [61,64)
  return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16: f32 accumulator, A and B K-major.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int a_fmt, int b_fmt) {
  return (1u << 4)                    // D format: f32
         | ((uint32_t)a_fmt << 7)     // A format: 0 f16, 1 bf16
         | ((uint32_t)b_fmt << 10)    // B format
         | (0u << 15) | (0u << 16)    // A, B major: K
         | ((uint32_t)(n >> 3) << 17) // N / 8
         | ((uint32_t)(m >> 4) << 24);// M / 16
}

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem ptr, abort flag
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack to align the base to 1024 bytes
};

// Progress markers for fault finding: when `dbg` is set, CTA 0 records how far each role got
// in pinned host memory (which survives a device fault) and lets asynchronous work land
// before it moves on, so that the last marker names the instruction that failed.
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

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_gemm_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
          float* __restrict__ c, long long ldc, int M, int N, int K, uint32_t idesc,
          int accumulate, const float* __restrict__ alpha_ptr, int* status, int* dbg) {
  using L = SmemLayout<BN, STAGES>;
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
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators; a power of two >= 32

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + b * 8, 1);
      mbar_init(bar_tempty + b * 8, 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    FT_MARK(4, 1);
  }
  if (warp == 1) {
    if (lane == 0) FT_MARK(5, 10);
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    if (lane == 0) FT_MARK(5, 11);
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    if (lane == 0) FT_MARK(5, 12);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) FT_MARK(6, (int)tmem_base);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          FT_MARK(7, 20);
          if (!mbar_wait(bar_empty + stage * 8, phase ^ 1, abort_flag, status, 1)) break;
          const uint32_t sa = base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          FT_MARK(7, 21);
          mbar_expect_tx(bar_full + stage * 8, L::STAGE_BYTES);
          FT_MARK(7, 22);
          tma_load_2d(sa, &map_a, bar_full + stage * 8, kb * BK, m0);
          FT_SETTLE();
          FT_MARK(7, 23);
          tma_load_2d(sb, &map_b, bar_full + stage * 8, kb * BK, n0);
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
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      int local = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
        const uint32_t buf = local & 1, acc_phase = (local >> 1) & 1;
        FT_MARK(8, 30);
        if (!mbar_wait(bar_tempty + buf * 8, acc_phase ^ 1, abort_flag, status, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          FT_MARK(8, 31);
          if (!mbar_wait(bar_full + stage * 8, phase, abort_flag, status, 3)) break;
          FT_MARK(8, 32);
          tc_fence_after();
          const uint32_t sa = base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          const uint64_t da = make_desc_sw128(sa), db = make_desc_sw128(sb);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K by 16 elements = 32 bytes inside the swizzle row: +2 in the
            // 16-byte units of the start-address field
            tc_mma_f16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc,
                       (kb > 0 || k > 0) ? 1u : 0u);
            FT_SETTLE();
            FT_MARK(8, 33 + k);
          }
          tc_commit(bar_empty + stage * 8);  // frees the stage when these MMAs have read it
          FT_SETTLE();
          FT_MARK(8, 37);
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
    const int quad = warp & 3;               // TMEM lanes [32*quad, 32*quad+32)
    int local = 0;
    const bool vec_ok = ((ldc & 3) == 0) && ((((uintptr_t)c) & 15) == 0);
    const float alpha = alpha_ptr ? *alpha_ptr : 1.0f;  // undoes the operand's power-of-two scale
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
      const uint32_t buf = local & 1, acc_phase = (local >> 1) & 1;
      if (warp == 2 && lane == 0) FT_MARK(9, 40);
      if (!mbar_wait(bar_tfull + buf * 8, acc_phase, abort_flag, status, 4)) break;
      tc_fence_after();
      if (warp == 2 && lane == 0) FT_MARK(9, 41);
      const int row = m0 + quad * 32 + lane;
      float* crow = c + (long long)row * ldc;
#pragma unroll 1
      for (int cb = 0; cb < BN / 32; ++cb) {
        uint32_t r[32];
        tc_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN + cb * 32, r);
        tc_wait_ld();
        if (warp == 2 && lane == 0) FT_MARK(9, 42);
        const int col0 = n0 + cb * 32;
        if (row < M && col0 < N) {
          if (vec_ok && col0 + 32 <= N) {
            float4* dst = (float4*)(crow + col0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 v = make_float4(alpha * __uint_as_float(r[4 * j]),
                                     alpha * __uint_as_float(r[4 * j + 1]),
                                     alpha * __uint_as_float(r[4 * j + 2]),
                                     alpha * __uint_as_float(r[4 * j + 3]));
              if (accumulate) {
                float4 o = dst[j];
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
              }
              dst[j] = v;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col0 + j < N) {
                float v = alpha * __uint_as_float(r[j]);
                crow[col0 + j] = accumulate ? crow[col0 + j] + v : v;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + buf * 8);
      if (warp == 2 && lane == 0) FT_MARK(9, 45);
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
    if (lane == 0) FT_MARK(10, 50);
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
    if (lane == 0) FT_MARK(10, 51);
  }
}

// ------------------------------------------------------------------------------ f32 -> f16
// Largest magnitude of a strided matrix, as the bit pattern of a non-negative float (which
// orders like an integer), combined with atomicMax: the result does not depend on the order.
__global__ void k_amax(const float* __restrict__ src, long long ld, int rows, int cols,
                       int* __restrict__ amax_bits) {
  long long total = (long long)rows * cols;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long st = (long long)gridDim.x * blockDim.x;
  float m = 0.f;
  for (; i < total; i += st) {
    long long r = i / cols, c = i % cols;
    m = fmaxf(m, fabsf(src[r * ld + c]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(amax_bits, __float_as_int(m));
}

// scales[0] = S (power of two bringing the largest magnitude into [2^11, 2^12)),
// scales[1] = 1/S, scales[2] = 2^-11/S (the factor of the low half in split mode)
__global__ void k_scale_from_amax(const int* __restrict__ amax_bits, float* __restrict__ scales) {
  float amax = __int_as_float(*amax_bits);
  float S = 1.0f;
  if (amax > 0.f && isfinite(amax)) {
    int e;
    frexpf(amax, &e);           // amax = f * 2^e, f in [0.5, 1)
    S = ldexpf(1.0f, 12 - e);
  }
  scales[0] = S;
  scales[1] = 1.0f / S;
  scales[2] = ldexpf(1.0f / S, -11);
}

// f32 [rows, cols] (pitch ld) -> f16 [rows, ldo]: hi = f16(x*S); lo (optional) = the rounding
// remainder times 2^11, so that x*S = hi + lo * 2^-11 to about 22 significant bits.
// One thread per 4 output columns; ldo is a multiple of 8, padding columns are zeroed.
__global__ void k_to_f16(const float* __restrict__ src, long long ld, __half* __restrict__ hi,
                         __half* __restrict__ lo, long long ldo, int rows, int cols,
                         const float* __restrict__ scales) {
  const float S = scales ? scales[0] : 1.0f;
  long long per_row = ldo / 4;
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

int make_map(FtContext* ctx, CUtensorMap* map, const void* ptr, CUtensorMapDataType dt,
             uint64_t inner, uint64_t outer, uint64_t ld_elems, uint32_t box_inner,
             uint32_t box_outer) {
  auto encode = (PFN_cuTensorMapEncodeTiled_v12000)ctx->encode_tiled;
  if (!encode) {
    ft_set_error("gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
    return FT_ERR_UNSUPPORTED;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    ft_set_error("gemm_tc: cuTensorMapEncodeTiled failed with %d (inner %llu outer %llu ld %llu)",
                 (int)r, (unsigned long long)inner, (unsigned long long)outer,
                 (unsigned long long)ld_elems);
    return FT_ERR_UNSUPPORTED;
  }
  return FT_OK;
}

template <int BN, int STAGES>
int launch_tc(FtContext* ctx, const CUtensorMap& ma, const CUtensorMap& mb, float* c,
              long long ldc, int M, int N, int K, uint32_t idesc, bool accumulate,
              const float* alpha_ptr) {
  using L = SmemLayout<BN, STAGES>;
  static bool configured = false;
  if (!configured) {
    FT_CUDA(cudaFuncSetAttribute(k_gemm_tc<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 L::DYN_BYTES));
    configured = true;
  }
  int tiles = ft_cdiv(M, BM) * ft_cdiv(N, BN);
  int grid = std::min(tiles, ctx->sm_count);
  int* dbg = ctx->debug_markers ? ctx->status_dev : nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (ctx->profile) {
    while (ctx->prof_events.size() < ctx->prof_used + 2) {
      cudaEvent_t e;
      FT_CUDA(cudaEventCreate(&e));
      ctx->prof_events.push_back(e);
    }
    e0 = ctx->prof_events[ctx->prof_used++];
    e1 = ctx->prof_events[ctx->prof_used++];
    FT_CUDA(cudaEventRecord(e0, ctx->stream));
  }
  FT_LAUNCH(ctx, (k_gemm_tc<BN, STAGES>), grid, GEMM_THREADS, L::DYN_BYTES, ma, mb, c, ldc, M, N,
            K, idesc, accumulate ? 1 : 0, alpha_ptr, ctx->status_dev, dbg);
  if (ctx->profile) {
    FT_CUDA(cudaEventRecord(e1, ctx->stream));
    ctx->prof_flops += 2.0 * (double)M * (double)N * (double)K;
    ctx->prof_launches++;
  }
  return FT_OK;
}

}  // namespace

int ft_to_f16(FtContext* ctx, const float* src, long long ld, __half* hi, __half* lo,
              long long ldo, int rows, int cols, bool auto_scale, const float** scales_out) {
  FT_REQUIRE(ldo % 8 == 0 && ldo >= cols, "to_f16: output pitch %lld must be a multiple of 8", ldo);
  const float* scales = nullptr;
  if (auto_scale) {
    FT_CUDA(cudaMemsetAsync(ctx->scale_buf, 0, 4, ctx->stream));
    long long n = (long long)rows * cols;
    int g = (int)std::max<long long>(1, std::min<long long>((n + 1023) / 1024,
                                                            (long long)ctx->sm_count * 8));
    FT_LAUNCH(ctx, k_amax, g, 256, 0, src, ld, rows, cols, (int*)ctx->scale_buf);
    FT_LAUNCH(ctx, k_scale_from_amax, 1, 1, 0, (const int*)ctx->scale_buf, ctx->scale_buf + 4);
    scales = ctx->scale_buf + 4;
  }
  if (scales_out) *scales_out = scales;
  long long total = (long long)rows * (ldo / 4);
  int grid = (int)std::max<long long>(1, std::min<long long>((total + 255) / 256,
                                                             (long long)ctx->sm_count * 16));
  FT_LAUNCH(ctx, k_to_f16, grid, 256, 0, src, ld, hi, lo, ldo, rows, cols, scales);
  return FT_OK;
}

int ft_gemm_tc(FtContext* ctx, const void* a, long long lda, const void* b, FtDType ab_type,
               long long ldb, float* c, long long ldc, int M, int N, int K, bool accumulate,
               const float* alpha_ptr) {
  // TMA rules: 16-byte aligned bases, pitches that are multiples of 16 bytes
  if (ab_type != FT_F16 && ab_type != FT_BF16) return FT_ERR_UNSUPPORTED;
  if ((((uintptr_t)a) & 15) || (((uintptr_t)b) & 15) || (lda % 8) || (ldb % 8) || K < 8 ||
      lda < K || ldb < K)
    return FT_ERR_UNSUPPORTED;
  CUtensorMap ma, mb;
  const int BN = N > 128 ? 256 : (N > 64 ? 128 : 64);
  const CUtensorMapDataType dt = ab_type == FT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                    : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  FT_TRY(make_map(ctx, &ma, a, dt, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM));
  FT_TRY(make_map(ctx, &mb, b, dt, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, (uint32_t)BN));
  // A and B formats must be equal: a mixed descriptor is rejected by the hardware
  const int fmt = ab_type == FT_F16 ? 0 : 1;
  const uint32_t idesc = make_idesc(BM, BN, fmt, fmt);
  switch (BN) {
    case 256: return launch_tc<256, 4>(ctx, ma, mb, c, ldc, M, N, K, idesc, accumulate, alpha_ptr);
    case 128: return launch_tc<128, 6>(ctx, ma, mb, c, ldc, M, N, K, idesc, accumulate, alpha_ptr);
    default: return launch_tc<64, 8>(ctx, ma, mb, c, ldc, M, N, K, idesc, accumulate, alpha_ptr);
  }
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
  int r = ft_gemm_tc(ctx, stage_hi, kp, b_f16, FT_F16, ldb, c, ldc, M, N, K, accumulate, alpha_hi);
  if (r == FT_OK && split)
    r = ft_gemm_tc(ctx, stage_lo, kp, b_f16, FT_F16, ldb, c, ldc, M, N, K, true, alpha_lo);
  return r;
}
