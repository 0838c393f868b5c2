// Wide-tile variant of the tcgen05 GEMM for the single-operand modes (bf16 / f16) at more than 256 tokens:
//   C[M][N] (f32) = X[M][K] (16-bit) * W[N][K]^T,  W in Q4_0 blocks  (the prefill GEMM workload: Q4_0 [14336,4096] and [4096,4096] weights, 128 to 2048 tokens).
// One CTA computes 128 weight rows x 512 tokens: the dequantised A tile (K-major, 128-byte swizzle, in
// SHARED memory) feeds two 256-column accumulators that together fill tensor memory, so each weight
// block is expanded once per 512 tokens.  With all 512 TMEM columns taken by the accumulators the A
// operand cannot live in tensor memory as it does in qgemm_tc.cu; measured on [14336,4096] x 2048 bf16
// this tile shape still wins (267 us against 286 us), and on [4096,4096] x 2048 it runs a single wave
// (66 us against 87 us).  Warp roles, rings and bounded waits are those of qgemm_tc.cu.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int TM = 128;       // weight rows per tile (MMA M)
constexpr int KSTEP = 64;     // elements per stage (128 bytes: one swizzle row)
constexpr int RAW_STEPS = 4;  // 64-element stages per raw weight tile (256 columns = 8 blocks)
constexpr int RAW_NS = 2;     // raw ring depth
constexpr int THREADS = 320;  // TMA warp, MMA warp, eight dequantisation / epilogue warps
constexpr int A_BYTES = TM * KSTEP * 2;

struct Params {
  int n, k;     // weight rows, columns
  int m;        // tokens
  int k_steps;  // 64-element steps per split (blockIdx.z), a multiple of RAW_STEPS
  float *out;   // [splits][m][ldc] when split-K, else [m][ldc]
  int ldc;
  size_t split_stride;
  int *status;
  int accumulate;  // out += result (the residual add of a projection)
};

__device__ __forceinline__ void tma_tile_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row
// groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset: next 8-row group
  d |= (uint64_t)1 << 46;                        // descriptor version
  d |= (uint64_t)2 << 61;                        // layout: 128-byte swizzle
  return d;
}
// Instruction descriptor: f32 accumulate, A and B both f16 (format 0) or both bf16 (format 1),
// both K-major, shape M x N.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, bool f16) {
  return (1u << 4) | ((f16 ? 0u : 1u) << 7) | ((f16 ? 0u : 1u) << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_16bit(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <bool F16>
__device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
  uint32_t d;
  if constexpr (F16) {
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  } else {
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  }
  return d;
}
template <bool F16>
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
  uint32_t d;
  if constexpr (F16) {
    asm("mul.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  } else {
    asm("mul.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  }
  return d;
}
template <bool F16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t d;
  if constexpr (F16) {
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  }
  return d;
}
template <bool F16>
__device__ __forceinline__ uint16_t to16(float v) {
  if constexpr (F16) {
    // finite values beyond the f16 range saturate; infinities and NaN pass through unchanged
    if (fabsf(v) > 65504.0f && fabsf(v) < __int_as_float(0x7f800000)) v = copysignf(65504.0f, v);
    return __half_as_ushort(__float2half_rn(v));
  } else {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  }
}

// One Q4_0 block (scale + 16 quant bytes given as four words) -> 32 values in element order:
// out[0..7] = elements 0..15 (low nibbles), out[8..15] = elements 16..31 (high nibbles).
// Bit patterns: f16 0x6400 | n = 1024 + n, bf16 0x4300 | n = 128 + n; the subtraction gives n - 8 exactly.
template <bool F16>
__device__ __forceinline__ void q4_block_to_16(uint32_t dbits16, const uint32_t (&q)[4], uint32_t (&out)[16]) {
  const uint32_t d2 = F16 ? (dbits16 | (dbits16 << 16)) : pack2<false>(half_bits_to_float(dbits16), half_bits_to_float(dbits16));
  const uint32_t M = 0x000F000Fu, E = F16 ? 0x64006400u : 0x43004300u, OFF = F16 ? 0x64086408u : 0x43084308u;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w = prmt(q[i], 0u, 0x3120u);  // bytes (b0, b2, b1, b3): adjacent elements share a mask
    out[2 * i] = mul2<F16>(sub2<F16>((w & M) | E, OFF), d2);              // elements 4i, 4i+1
    out[2 * i + 1] = mul2<F16>(sub2<F16>(((w >> 8) & M) | E, OFF), d2);   // elements 4i+2, 4i+3
    out[8 + 2 * i] = mul2<F16>(sub2<F16>(((w >> 4) & M) | E, OFF), d2);   // elements 16+4i, 16+4i+1
    out[8 + 2 * i + 1] = mul2<F16>(sub2<F16>(((w >> 12) & M) | E, OFF), d2);
  }
}
// One Q8_0 block (eight words of int8) -> 32 values.
template <bool F16>
__device__ __forceinline__ void q8_block_to_16(uint32_t dbits16, const uint32_t (&q)[8], uint32_t (&out)[16]) {
  const float d = half_bits_to_float(dbits16);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t u = q[i] ^ 0x80808080u;
    const float v0 = __uint_as_float(0x4B000000u | (u & 0xffu)) - 8388736.0f;
    const float v1 = __uint_as_float(0x4B000000u | ((u >> 8) & 0xffu)) - 8388736.0f;
    const float v2 = __uint_as_float(0x4B000000u | ((u >> 16) & 0xffu)) - 8388736.0f;
    const float v3 = __uint_as_float(0x4B000000u | (u >> 24)) - 8388736.0f;
    out[2 * i] = pack2<F16>(v0 * d, v1 * d);
    out[2 * i + 1] = pack2<F16>(v2 * d, v3 * d);
  }
}

__host__ __device__ constexpr int ring_depth(int tn, bool comp) {
  return comp ? (tn >= 128 ? 2 : 3) : (tn > 256 ? 2 : tn > 128 ? 3 : 4);
}

template <int QT, int TN, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
    qgemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap xlo_map,
                    const __grid_constant__ CUtensorMap wmap, const Params P) {
  constexpr bool Q4 = (QT == RG_TYPE_Q4_0);
  constexpr bool F16 = MODE != QGEMM_BF16, COMP = MODE == QGEMM_F16X3;
  constexpr int NPL = COMP ? 2 : 1;  // operand planes per stage: hi (and lo)
  constexpr int BB = Q4 ? 18 : 34;
  constexpr int NS = ring_depth(TN, COMP);  // operand ring depth
  constexpr int B_BYTES = TN * KSTEP * 2;
  constexpr int A_STAGE = NPL * A_BYTES, B_STAGE = NPL * B_BYTES;
  constexpr int RAW_ROW = 8 * BB;  // bytes of one weight row in a raw tile (144 / 272)
  constexpr int RAW_BYTES = TM * RAW_ROW;
  constexpr int TMEM_COLS = TN < 32 ? 32 : TN;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *a_ring = smem;
  uint8_t *b_ring = smem + NS * A_STAGE;
  uint8_t *raw_ring = b_ring + NS * B_STAGE;
  uint64_t *bars = reinterpret_cast<uint64_t *>(raw_ring + RAW_NS * RAW_BYTES);
  uint64_t *b_full = bars, *a_full = bars + NS, *slot_free = bars + 2 * NS;
  uint64_t *raw_full = bars + 3 * NS, *raw_free = raw_full + RAW_NS, *acc_done = raw_free + RAW_NS;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_done + 1);
  volatile int *dead = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TM, tok0 = blockIdx.y * TN;
  const int step0 = blockIdx.z * P.k_steps;
  const int nsteps = min(P.k_steps, P.k / KSTEP - step0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&a_full[s], 256);
      mbar_init(&slot_free[s], 1);
    }
    for (int s = 0; s < RAW_NS; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_free[s], 256);
    }
    mbar_init(acc_done, 1);
    *dead = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA: raw weight tiles and activation tiles
    if (lane == 0) {
      for (int i = 0; i < nsteps; ++i) {
        if (i % RAW_STEPS == 0) {
          const int j = i / RAW_STEPS, rs = j % RAW_NS;
          if (j >= RAW_NS) mbar_wait_bounded(&raw_free[rs], (uint32_t)((j / RAW_NS - 1) & 1), dead, P.status);
          mbar_expect_tx(&raw_full[rs], (uint32_t)RAW_BYTES);
          // x in 8-byte elements; rows beyond the tensor arrive as zeros (zero scale, zero weights)
          tma_tile_2d(raw_ring + rs * RAW_BYTES, &wmap, ((step0 + i) / RAW_STEPS) * (RAW_ROW / 8), n0, &raw_full[rs]);
        }
        const int slot = i % NS;
        if (i >= NS) mbar_wait_bounded(&slot_free[slot], (uint32_t)((i / NS - 1) & 1), dead, P.status);
        mbar_expect_tx(&b_full[slot], (uint32_t)B_STAGE);
        tma_tile_2d(b_ring + slot * B_STAGE, &xmap, (step0 + i) * KSTEP, tok0, &b_full[slot]);
        if constexpr (TN > 256)  // a TMA box holds at most 256 rows: the second half of the token tile
          tma_tile_2d(b_ring + slot * B_STAGE + 256 * 128, &xmap, (step0 + i) * KSTEP, tok0 + 256, &b_full[slot]);
        if constexpr (COMP) tma_tile_2d(b_ring + slot * B_STAGE + B_BYTES, &xlo_map, (step0 + i) * KSTEP, tok0, &b_full[slot]);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      // a 512-token tile is two 256-column accumulators fed by the same dequantised A tile
      constexpr int MMA_N = TN > 256 ? 256 : TN;
      constexpr uint32_t idesc = umma_idesc(TM, MMA_N, F16);
      for (int i = 0; i < nsteps; ++i) {
        const int slot = i % NS;
        const uint32_t ph = (uint32_t)((i / NS) & 1);
        mbar_wait_bounded(&a_full[slot], ph, dead, P.status);
        mbar_wait_bounded(&b_full[slot], ph, dead, P.status);
        tc_fence_after();
        const uint32_t a_addr = smem_u32(a_ring + slot * A_STAGE), b_addr = smem_u32(b_ring + slot * B_STAGE);
#pragma unroll
        for (int kk = 0; kk < KSTEP / 16; ++kk) {
          const uint64_t a_hi = umma_desc(a_addr + kk * 32), b_hi = umma_desc(b_addr + kk * 32);
          if constexpr (COMP) {  // the small terms first, then hi.hi
            umma_16bit(tmem_base, a_hi, umma_desc(b_addr + B_BYTES + kk * 32), idesc, (i > 0 || kk > 0) ? 1u : 0u);
            umma_16bit(tmem_base, umma_desc(a_addr + A_BYTES + kk * 32), b_hi, idesc, 1u);
            umma_16bit(tmem_base, a_hi, b_hi, idesc, 1u);
          } else {
            umma_16bit(tmem_base, a_hi, b_hi, idesc, (i > 0 || kk > 0) ? 1u : 0u);
            if constexpr (TN > 256)
              umma_16bit(tmem_base + 256, a_hi, umma_desc(b_addr + 256 * 128 + kk * 32), idesc, (i > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&slot_free[slot]);  // the slot may be rewritten once these MMAs have read it
      }
      umma_commit(acc_done);
    }
  } else {
    // ---------------------------------------------------------------- dequantisation: one block (half of a
    // stage's 64 columns) of one weight row per thread, two threads per row
    const int tdq = threadIdx.x - 64;          // 0..255
    const int r = tdq & 127, half = tdq >> 7;  // row of the tile, even / odd block of the stage
    constexpr int QW = Q4 ? 4 : 8;             // quant words per block
    for (int i = 0; i < nsteps; ++i) {
      const int slot = i % NS;
      const int j = i / RAW_STEPS, rs = j % RAW_NS, sub = i % RAW_STEPS;
      if (sub == 0) mbar_wait_bounded(&raw_full[rs], (uint32_t)((j / RAW_NS) & 1), dead, P.status);
      // pair layout: [d0 | q0] [d1 | q1] with a 2-byte scale in front of each block: the even block's
      // quants straddle word boundaries (funnel shift), the odd block's are word aligned
      const uint32_t *src = reinterpret_cast<const uint32_t *>(raw_ring + rs * RAW_BYTES + r * RAW_ROW + sub * 2 * BB);
      uint32_t q[QW], dbits, vals[16];  // 32 values of this block, in k order
      if (half == 0) {
        uint32_t raw[QW + 1];
#pragma unroll
        for (int w = 0; w <= QW; ++w) raw[w] = src[w];
#pragma unroll
        for (int w = 0; w < QW; ++w) q[w] = __funnelshift_r(raw[w], raw[w + 1], 16);
        dbits = raw[0] & 0xffffu;
      } else {
        dbits = src[QW] >> 16;
#pragma unroll
        for (int w = 0; w < QW; ++w) q[w] = src[QW + 1 + w];
      }
      uint32_t lows[1];
      static_assert(!COMP, "the compensated mode runs in qgemm_tc.cu");
      if constexpr (Q4) {
        q4_block_to_16<F16>(dbits, q, vals);
      } else {
        q8_block_to_16<F16>(dbits, q, vals);
      }
      if (sub == RAW_STEPS - 1 || i + 1 == nsteps) mbar_arrive(&raw_free[rs]);  // raw bytes are in registers now
      if (i >= NS) mbar_wait_bounded(&slot_free[slot], (uint32_t)((i / NS - 1) & 1), dead, P.status);
      uint8_t *row_dst = a_ring + slot * A_STAGE + r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 chunk = make_uint4(vals[4 * c], vals[4 * c + 1], vals[4 * c + 2], vals[4 * c + 3]);
        *reinterpret_cast<uint4 *>(row_dst + (((4 * half + c) ^ (r & 7)) << 4)) = chunk;
        if constexpr (COMP) {
          chunk = make_uint4(lows[4 * c], lows[4 * c + 1], lows[4 * c + 2], lows[4 * c + 3]);
          *reinterpret_cast<uint4 *>(row_dst + A_BYTES + (((4 * half + c) ^ (r & 7)) << 4)) = chunk;
        }
      }
      proxy_fence_async();  // generic-proxy stores must be visible to the tensor core's async reads
      mbar_arrive(&a_full[slot]);
    }
    // ---------------------------------------------------------------- epilogue: TMEM -> global
    mbar_wait_bounded(acc_done, 0, dead, P.status);
    tc_fence_after();
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 belong to this warp
    const int orow = n0 + quarter * 32 + lane;
    float *out = P.out + (size_t)blockIdx.z * P.split_stride;
    if (nsteps > 0) {
#pragma unroll 1
      for (int c0 = (warp >= 6 ? 16 : 0); c0 < TN; c0 += 32) {  // two warps share a lane quarter
        if (tok0 + c0 >= P.m) break;
        uint32_t v[16];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
              "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int w = 0; w < 16; ++w) {
          const int tok = tok0 + c0 + w;
          if (tok < P.m && orow < P.n) {
            float *dst = out + (size_t)tok * P.ldc + orow;
            *dst = P.accumulate ? __fadd_rn(*dst, __uint_as_float(v[w])) : __uint_as_float(v[w]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
  }
}

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                              const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

template <int QT, int TN, int MODE>
cudaError_t launch_t(const QGemmArgs &a, const LaunchCfg &cfg) {
  EncodeFn fn = encode_fn();
  if (!fn) return cudaErrorNotSupported;
  constexpr bool F16 = MODE != QGEMM_BF16, COMP = MODE == QGEMM_F16X3;
  constexpr int BB = (QT == RG_TYPE_Q4_0) ? 18 : 34;
  constexpr int NS = ring_depth(TN, COMP);
  constexpr int NPL = COMP ? 2 : 1;
  constexpr int RAW_ROW = 8 * BB;
  alignas(64) CUtensorMap xmap, xlo_map, wmap;
  const cuuint32_t elem[2] = {1, 1};
  for (int plane = 0; plane < NPL; ++plane) {
    const cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)a.m};
    const cuuint64_t strides[1] = {(cuuint64_t)a.ldx * 2};
    const cuuint32_t box[2] = {(cuuint32_t)KSTEP, (cuuint32_t)(TN > 256 ? 256 : TN)};
    if (fn(plane ? &xlo_map : &xmap, F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
           const_cast<void *>(plane ? a.x16_lo : a.x16), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  if (!COMP) xlo_map = xmap;
  {
    const size_t row_bytes = (size_t)(a.k / 32) * BB;
    const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 8), (cuuint64_t)a.n};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(RAW_ROW / 8), (cuuint32_t)TM};
    if (fn(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t *>(a.w), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
  Params P{};
  P.n = a.n;
  P.k = a.k;
  P.m = a.m;
  const int total_steps = a.k / KSTEP;
  int splits = a.splits < 1 ? 1 : a.splits;
  P.k_steps = ((total_steps / RAW_STEPS + splits - 1) / splits) * RAW_STEPS;  // whole raw tiles per split
  splits = (total_steps + P.k_steps - 1) / P.k_steps;
  P.out = a.out;
  P.ldc = a.ldc;
  P.split_stride = a.split_stride;
  P.status = cfg.status;
  P.accumulate = a.accumulate ? 1 : 0;
  constexpr size_t smem =
      1024 + NS * NPL * (A_BYTES + TN * KSTEP * 2) + RAW_NS * TM * RAW_ROW + (3 * NS + 2 * RAW_NS + 1) * 8 + 16;
  static_assert(smem <= 227 * 1024, "tile configuration exceeds the shared memory of one SM");
  auto kernel = qgemm_tc_kernel<QT, TN, MODE>;
  static DeviceOnce attr_once;  // per instantiation and device
  bool *attr_flag = attr_once.slot();
  if (!attr_flag || !*attr_flag) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    if (attr_flag) *attr_flag = true;
  }
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3((unsigned)((a.n + TM - 1) / TM), (unsigned)((a.m + TN - 1) / TN), (unsigned)splits);
  lc.blockDim = dim3(THREADS);
  lc.dynamicSmemBytes = smem;
  lc.stream = cfg.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = cfg.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&lc, kernel, xmap, xlo_map, wmap, P);
}

}  // namespace

bool qgemm_tc_wide_applies(const QGemmArgs &a) {
  if (!(a.type == RG_TYPE_Q4_0 && a.mode != QGEMM_F16X3 && a.m > 256 && a.splits <= 1)) return false;
  // with few CTAs the 256-token tiles of qgemm_tc.cu fill more SMs
  const long ctas = (long)((a.n + TM - 1) / TM) * (long)((a.m + 511) / 512);
  return ctas >= 96;
}

cudaError_t launch_qgemm_tc_wide(const QGemmArgs &a, const LaunchCfg &cfg) {
  if (!qgemm_tc_wide_applies(a)) return cudaErrorInvalidValue;
  count_launch(LC_QGEMM_TC_WIDE);
  return a.mode == QGEMM_BF16 ? launch_t<RG_TYPE_Q4_0, 512, QGEMM_BF16>(a, cfg) : launch_t<RG_TYPE_Q4_0, 512, QGEMM_F16>(a, cfg);
}

}  // namespace rg
