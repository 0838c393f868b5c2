// Prefill / wide-batch GEMM on the 5th-generation tensor cores:
//   C[M][N] (f32) = X[M][K] (16-bit) * W[N][K]^T,  W in native Q4_0 / Q8_0 GGML blocks.
// Semantics: the layer linears of the Llama forward for many tokens at once
// (src/models/transformer/layer.rs:445-448, src/backend/cpu.rs:3484-3532 on the dequantised
// weight of src/models/transformer/model.rs:982-995), with 16-bit operands and f32 accumulation.
//
// One CTA computes RT tiles of [128 weight rows] x [TN tokens] (RT * 128 consecutive weight rows) over a K range:
//   * MMA M = 128 weight rows (the dequantised tile is the A operand), MMA N = TN tokens (the
//     activation tile is the B operand), K = 16 per tcgen05.mma, four per 64-element stage;
//     the accumulator lives in TMEM (128 lanes x TN f32 columns).
//   * warp 0: TMA producer.  Activation tiles come as tiled 2-D copies with the 128-byte swizzle;
//     the raw block bytes of the 128 weight rows, 256 columns (8 blocks) at a time, come through
//     a second tiled 2-D map into a small ring, so no thread waits on global memory.
//   * warp 1: allocates TMEM, issues tcgen05.mma from one thread, commits to mbarriers.
//   * warps 2-17 (two groups of eight taking alternate stages): two threads per weight row; each expands one block per stage (nibbles to exact
//     16-bit integers by bit pattern, one packed subtract and one packed multiply by the block
//     scale per two weights) and writes its 32 values with tcgen05.st straight into TENSOR MEMORY:
//     the A operand of the MMA is read from TMEM (lane = weight row, one 32-bit column per two K
//     values), so the dequantised weights never pass through shared memory, whose bandwidth is
//     then left to the activation tiles.  Afterwards the same warps read the accumulator with
//     tcgen05.ld and store it.
//   * Operand rings of 3-4 stages with bounded mbarrier waits; a time-out records a status and
//     the kernel still frees its TMEM and exits.
// Operand modes: bf16 (weights enter as bf16(bf16(d) * (n - 8)) for Q4_0), f16 (weights enter as
// f16(d * (n - 8))), and compensated f16, where every operand is the sum of two halves
// (hi = f16(v), lo = f16(v - hi)) and each K step issues hi.hi + hi.lo + lo.hi into the same
// accumulator: the dropped lo.lo term is 2^-22 of the product, so the result has f32-grade accuracy
// at three times the tensor-core work.  The session uses the compensated mode because logits must
// stay within 1e-3 of the reference's f32 arithmetic.
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
// RT = row tiles of 128 weight rows per CTA.  The compensated mode moves two activation planes per stage and is
// bound by that traffic from L2, so there one activation tile feeds two row tiles (RT = 2, at most 128 tokens);
// the single-operand modes are bound by the dequantisation and prefer one row tile against 256 tokens.
constexpr int MAX_THREADS = 64 + 2 * 256;  // TMA warp, MMA warp, eight dequantisation / epilogue warps per row tile
constexpr int A_COLS = KSTEP / 2;  // TMEM columns of one dequantised A stage (two 16-bit values per column)

struct Params {
  int n, k;     // weight rows, columns
  int m;        // tokens
  int k_steps;  // 64-element steps per split (blockIdx.z), a multiple of RAW_STEPS
  float *out;   // [splits][m][ldc] when split-K, else [m][ldc]
  int ldc;
  size_t split_stride;
  int *status;
  int accumulate;  // out += result (the residual add of a projection); not with split-K
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
// Same with the A operand in tensor memory.
__device__ __forceinline__ void umma_16bit_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_store16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
      "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
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

// Compensated operands: hi = f16(w), lo = f16(w - hi) with w = d * q exact in f32 (Q8_0) or through a
// fused multiply-add (Q4_0: q * d - hi is exact before its single rounding).
__device__ __forceinline__ void q4_block_split(uint32_t dbits16, const uint32_t (&q)[4], uint32_t (&hi)[16], uint32_t (&lo)[16]) {
  const uint32_t d2 = dbits16 | (dbits16 << 16);
  const uint32_t M = 0x000F000Fu, E = 0x64006400u, OFF = 0x64086408u;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w = prmt(q[i], 0u, 0x3120u);
    const uint32_t n[4] = {w & M, (w >> 8) & M, (w >> 4) & M, (w >> 12) & M};
    const int slot[4] = {2 * i, 2 * i + 1, 8 + 2 * i, 8 + 2 * i + 1};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t qf = sub2<true>(n[j] | E, OFF);
      const uint32_t h = mul2<true>(qf, d2);
      uint32_t l;
      asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(l) : "r"(qf), "r"(d2), "r"(h ^ 0x80008000u));
      hi[slot[j]] = h;
      lo[slot[j]] = l;
    }
  }
}
__device__ __forceinline__ void split_pair(float v0, float v1, uint32_t &hi, uint32_t &lo) {
  const __half2 h = __floats2half2_rn(v0, v1);
  const float2 hf = __half22float2(h);
  const __half2 l = __floats2half2_rn(v0 - hf.x, v1 - hf.y);
  hi = *reinterpret_cast<const uint32_t *>(&h);
  lo = *reinterpret_cast<const uint32_t *>(&l);
}
__device__ __forceinline__ void q8_block_split(uint32_t dbits16, const uint32_t (&q)[8], uint32_t (&hi)[16], uint32_t (&lo)[16]) {
  const float d = half_bits_to_float(dbits16);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t u = q[i] ^ 0x80808080u;
    const float v0 = __uint_as_float(0x4B000000u | (u & 0xffu)) - 8388736.0f;
    const float v1 = __uint_as_float(0x4B000000u | ((u >> 8) & 0xffu)) - 8388736.0f;
    const float v2 = __uint_as_float(0x4B000000u | ((u >> 16) & 0xffu)) - 8388736.0f;
    const float v3 = __uint_as_float(0x4B000000u | (u >> 24)) - 8388736.0f;
    split_pair(v0 * d, v1 * d, hi[2 * i], lo[2 * i]);
    split_pair(v2 * d, v3 * d, hi[2 * i + 1], lo[2 * i + 1]);
  }
}

// Ring depth of the activation tiles (shared memory) and of the dequantised A stages (tensor memory).
__host__ __device__ constexpr int ring_depth(int tn, bool comp) { return comp ? (tn >= 64 ? 2 : 3) : 4; }  // tensor-memory budget
__host__ __device__ constexpr int row_tiles(int mode) { return mode == QGEMM_F16X3 ? 2 : 1; }
__host__ __device__ constexpr int pow2_cols(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512; }

template <int QT, int TN, int MODE, int RT>
__global__ void __launch_bounds__(MAX_THREADS, 1)
    qgemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap xlo_map,
                    const __grid_constant__ CUtensorMap wmap, const Params P) {
  constexpr bool Q4 = (QT == RG_TYPE_Q4_0);
  constexpr bool F16 = MODE != QGEMM_BF16, COMP = MODE == QGEMM_F16X3;
  constexpr int NPL = COMP ? 2 : 1;  // operand planes per stage: hi (and lo)
  constexpr int BB = Q4 ? 18 : 34;
  constexpr int NS = ring_depth(TN, COMP);  // operand ring depth
  constexpr int B_BYTES = TN * KSTEP * 2;
  constexpr int B_STAGE = NPL * B_BYTES;
  constexpr int A_TILE_COLS = NPL * A_COLS;       // TMEM columns of one row tile's A stage (hi, lo)
  constexpr int A_STAGE_COLS = RT * A_TILE_COLS;  // both row tiles
  constexpr int RAW_ROW = 8 * BB;  // bytes of one weight row in a raw tile (144 / 272)
  constexpr int RAW_BYTES = TM * RAW_ROW;
  constexpr int ACC_T = TN < 32 ? 32 : TN;  // accumulator columns of one row tile
  constexpr int ACC_COLS = RT * ACC_T;      // accumulators first, then the A ring
  constexpr int TMEM_COLS = pow2_cols(ACC_COLS + NS * A_STAGE_COLS);
  static_assert(ACC_COLS + NS * A_STAGE_COLS <= 512, "tensor memory budget");
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *b_ring = smem;
  uint8_t *raw_ring = b_ring + NS * B_STAGE;
  uint64_t *bars = reinterpret_cast<uint64_t *>(raw_ring + RAW_NS * RT * RAW_BYTES);
  uint64_t *b_full = bars, *a_full = bars + NS, *slot_free = bars + 2 * NS;
  uint64_t *raw_full = bars + 3 * NS, *raw_free = raw_full + RAW_NS, *acc_done = raw_free + RAW_NS;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_done + 1);
  volatile int *dead = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * (TM * RT), tok0 = blockIdx.y * TN;
  const int step0 = blockIdx.z * P.k_steps;
  const int nsteps = min(P.k_steps, P.k / KSTEP - step0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&a_full[s], RT * 256);
      mbar_init(&slot_free[s], 1);
    }
    for (int s = 0; s < RAW_NS; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_free[s], RT * 256);
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
          mbar_expect_tx(&raw_full[rs], (uint32_t)(RT * RAW_BYTES));
          // x in 8-byte elements; rows beyond the tensor arrive as zeros (zero scale, zero weights)
#pragma unroll
          for (int t = 0; t < RT; ++t)
            tma_tile_2d(raw_ring + (rs * RT + t) * RAW_BYTES, &wmap, ((step0 + i) / RAW_STEPS) * (RAW_ROW / 8), n0 + t * TM,
                        &raw_full[rs]);
        }
        const int slot = i % NS;
        if (i >= NS) mbar_wait_bounded(&slot_free[slot], (uint32_t)((i / NS - 1) & 1), dead, P.status);
        mbar_expect_tx(&b_full[slot], (uint32_t)B_STAGE);
        tma_tile_2d(b_ring + slot * B_STAGE, &xmap, (step0 + i) * KSTEP, tok0, &b_full[slot]);
        if constexpr (COMP) tma_tile_2d(b_ring + slot * B_STAGE + B_BYTES, &xlo_map, (step0 + i) * KSTEP, tok0, &b_full[slot]);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(TM, TN, F16);
      // one thread issues every MMA, so the loop is kept lean: a shared-memory descriptor is linear in the
      // address (16-byte units), hence one base descriptor plus small constants per stage, K step and plane
      const uint64_t b_desc0 = umma_desc(smem_u32(b_ring));
      for (int i = 0; i < nsteps; ++i) {
        const int slot = i % NS;
        const uint32_t ph = (uint32_t)((i / NS) & 1);
        mbar_wait_bounded(&a_full[slot], ph, dead, P.status);
        mbar_wait_bounded(&b_full[slot], ph, dead, P.status);
        tc_fence_after();
        const uint64_t b_desc = b_desc0 + (uint64_t)((slot * B_STAGE) >> 4);
        const uint32_t a_tm = tmem_base + (uint32_t)(ACC_COLS + slot * A_STAGE_COLS);  // lane 0, first column of the stage
        const uint32_t first = i > 0 ? 1u : 0u;  // the very first MMA of a tile overwrites the accumulator
#pragma unroll
        for (int kk = 0; kk < KSTEP / 16; ++kk) {
          const uint64_t b_hi = b_desc + (uint64_t)(kk * 2);  // 32 bytes per K step
#pragma unroll
          for (int t = 0; t < RT; ++t) {
            const uint32_t acc = tmem_base + t * ACC_T;
            const uint32_t a_hi = a_tm + t * A_TILE_COLS + kk * 8;  // 16 K values = 8 columns
            if constexpr (COMP) {  // the small terms first, then hi.hi
              umma_16bit_ta(acc, a_hi, b_hi + (uint64_t)(B_BYTES >> 4), idesc, kk > 0 ? 1u : first);
              umma_16bit_ta(acc, a_hi + A_COLS, b_hi, idesc, 1u);
              umma_16bit_ta(acc, a_hi, b_hi, idesc, 1u);
            } else {
              umma_16bit_ta(acc, a_hi, b_hi, idesc, kk > 0 ? 1u : first);
            }
          }
        }
        umma_commit(&slot_free[slot]);  // the slot may be rewritten once these MMAs have read it
      }
      umma_commit(acc_done);
    }
  } else {
    // ---------------------------------------------------------------- dequantisation: one block (half of a
    // stage's 64 columns) of one weight row per thread, two threads per row
    // a warp may touch only the TMEM lanes 32 * (warp % 4) .. +31, so its lanes own exactly those weight rows
    const int r = (warp & 3) * 32 + lane;  // row of the tile
    const int half = ((warp - 2) >> 2) & 1;  // even / odd block of the stage
    const int grp = (warp - 2) >> 3;         // row tile of this warp
    constexpr int QW = Q4 ? 4 : 8;             // quant words per block
    for (int i = 0; i < nsteps; ++i) {
      const int slot = i % NS;
      const int j = i / RAW_STEPS, rs = j % RAW_NS, sub = i % RAW_STEPS;
      if (sub == 0) mbar_wait_bounded(&raw_full[rs], (uint32_t)((j / RAW_NS) & 1), dead, P.status);
      // pair layout: [d0 | q0] [d1 | q1] with a 2-byte scale in front of each block: the even block's
      // quants straddle word boundaries (funnel shift), the odd block's are word aligned
      const uint32_t *src =
          reinterpret_cast<const uint32_t *>(raw_ring + (rs * RT + grp) * RAW_BYTES + r * RAW_ROW + sub * 2 * BB);
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
      uint32_t lows[16];
      if constexpr (COMP) {
        if constexpr (Q4) {
          q4_block_split(dbits, q, vals, lows);
        } else {
          q8_block_split(dbits, q, vals, lows);
        }
      } else if constexpr (Q4) {
        q4_block_to_16<F16>(dbits, q, vals);
      } else {
        q8_block_to_16<F16>(dbits, q, vals);
      }
      if (sub == RAW_STEPS - 1) mbar_arrive(&raw_free[rs]);  // the raw tile's last stage is in registers
      if (i >= NS) mbar_wait_bounded(&slot_free[slot], (uint32_t)((i / NS - 1) & 1), dead, P.status);
      tc_fence_after();
      // this thread's block = 16 columns of its row's lane: [stage][plane][even block | odd block]
      const uint32_t a_tm = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) +
                            (uint32_t)(ACC_COLS + slot * A_STAGE_COLS + grp * A_TILE_COLS + half * 16);
      tmem_store16(a_tm, vals);
      if constexpr (COMP) tmem_store16(a_tm + A_COLS, lows);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      mbar_arrive(&a_full[slot]);
    }
    // ---------------------------------------------------------------- epilogue: TMEM -> global
    mbar_wait_bounded(acc_done, 0, dead, P.status);
    tc_fence_after();
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 belong to this warp
    const int orow = n0 + grp * TM + quarter * 32 + lane;  // this warp's row tile
    float *out = P.out + (size_t)blockIdx.z * P.split_stride;
    if (nsteps > 0) {
#pragma unroll 1
      for (int c0 = half * 16; c0 < TN; c0 += 32) {  // two warps share a lane quarter of a row tile
        if (tok0 + c0 >= P.m) break;
        uint32_t v[16];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(grp * ACC_T + c0);
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

template <int QT, int TN, int MODE, int RT>
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
    const cuuint32_t box[2] = {(cuuint32_t)KSTEP, (cuuint32_t)TN};
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
  if (a.accumulate && splits > 1) return cudaErrorInvalidValue;
  constexpr size_t smem = 1024 + NS * NPL * (TN * KSTEP * 2) + RAW_NS * RT * TM * RAW_ROW + (3 * NS + 2 * RAW_NS + 1) * 8 + 16;
  static_assert(smem <= 227 * 1024, "tile configuration exceeds the shared memory of one SM");
  auto kernel = qgemm_tc_kernel<QT, TN, MODE, RT>;
  static DeviceOnce attr_once;  // per instantiation and device
  bool *attr_flag = attr_once.slot();
  if (!attr_flag || !*attr_flag) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    if (attr_flag) *attr_flag = true;
  }
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3((unsigned)((a.n + TM * RT - 1) / (TM * RT)), (unsigned)((a.m + TN - 1) / TN), (unsigned)splits);
  lc.blockDim = dim3(64 + RT * 256);
  lc.dynamicSmemBytes = smem;
  lc.stream = cfg.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = cfg.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&lc, kernel, xmap, xlo_map, wmap, P);
}

template <int QT, int MODE>
cudaError_t launch_n(const QGemmArgs &a, const LaunchCfg &cfg) {
  constexpr int RT = row_tiles(MODE);
  // accumulators (RT tiles of TN columns) and the A ring share the 512 columns of tensor memory
  if constexpr (RT == 1) {
    if (a.m > 128) return launch_t<QT, 256, MODE, RT>(a, cfg);
  }
  if (a.m > 64) return launch_t<QT, 128, MODE, RT>(a, cfg);
  if (a.m > 32) return launch_t<QT, 64, MODE, RT>(a, cfg);
  if (a.m > 16) return launch_t<QT, 32, MODE, RT>(a, cfg);
  return launch_t<QT, 16, MODE, RT>(a, cfg);
}
template <int QT>
cudaError_t launch_m(const QGemmArgs &a, const LaunchCfg &cfg) {
  if (a.mode == QGEMM_BF16) return launch_n<QT, QGEMM_BF16>(a, cfg);
  if (a.mode == QGEMM_F16) return launch_n<QT, QGEMM_F16>(a, cfg);
  return launch_n<QT, QGEMM_F16X3>(a, cfg);
}

// One value to its operand: hi (and, when lo is given, the f16 of what hi left over).
template <bool F16>
__device__ __forceinline__ void put16(float v, uint16_t *hi, uint16_t *lo, size_t at) {
  const uint16_t h = to16<F16>(v);
  hi[at] = h;
  if constexpr (F16) {
    if (lo) lo[at] = to16<true>(v - __half2float(__ushort_as_half(h)));
  }
}

template <bool F16>
__global__ void to16_kernel(const float *x, int ldx, int k, uint16_t *y, uint16_t *ylo, int ldy) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
  if (i < k) put16<F16>(x[(size_t)row * ldx + i], y, ylo, (size_t)row * ldy + i);
}

// RMSNorm of one token row straight to the 16-bit GEMM operand; f32 steps rounded like the
// reference (src/models/transformer/layer.rs:423-443), then one rounding to the operand type.
template <bool F16>
__global__ void rmsnorm16_kernel(const float *x, int ldx, const float *w, int d, float eps, uint16_t *y, uint16_t *ylo, int ldy) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float partial[32];
  __shared__ float inv_s;
  const float *xr = x + (size_t)blockIdx.x * ldx;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = (threadIdx.x < (blockDim.x >> 5)) ? partial[threadIdx.x] : 0.0f;
    v = warp_sum(v);
    if (threadIdx.x == 0) inv_s = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(v, (float)d), eps)));
  }
  __syncthreads();
  const float inv = inv_s;
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    put16<F16>(__fmul_rn(__fmul_rn(xr[i], inv), w[i]), y, ylo, (size_t)blockIdx.x * ldy + i);
}

// h = silu(gate) * up (src/ir/elementwise.rs:6772-6830,7046-7050) to the operand of the down projection.
template <bool F16>
__global__ void swiglu16_kernel(const float *g, const float *u, int n, int ld, uint16_t *y, uint16_t *ylo, int ldy) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
  if (i < n) put16<F16>(swiglu(g[(size_t)row * ld + i], u[(size_t)row * ld + i]), y, ylo, (size_t)row * ldy + i);
}

// out[r][i] = sum over splits of part[s][r][i]: the K-split partial tiles of a small-M GEMM
__global__ void reduce_splits_kernel(const float *part, int splits, size_t stride, int n, float *out, int ldo) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
  if (i >= n) return;
  const float *p = part + (size_t)row * n + i;
  float acc = 0.0f;
  for (int s0 = 0; s0 < splits; s0 += 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = (s0 + j < splits) ? p[(size_t)(s0 + j) * stride] : 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += v[j];
  }
  out[(size_t)row * ldo + i] = acc;
}

template <typename K, typename... Args>
cudaError_t launch_simple(K kernel, dim3 grid, dim3 block, const LaunchCfg &cfg, Args... args) {
  cudaLaunchConfig_t lc{};
  lc.gridDim = grid;
  lc.blockDim = block;
  lc.stream = cfg.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = cfg.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&lc, kernel, args...);
}

}  // namespace

cudaError_t launch_rmsnorm16(const float *x, int ldx, const float *w, int d, float eps, int rows, const Operand16 &y,
                             const LaunchCfg &cfg) {
  uint16_t *hi = static_cast<uint16_t *>(y.hi), *lo = static_cast<uint16_t *>(y.lo);
  if (y.f16) return launch_simple(rmsnorm16_kernel<true>, dim3((unsigned)rows), dim3(512), cfg, x, ldx, w, d, eps, hi, lo, y.ld);
  return launch_simple(rmsnorm16_kernel<false>, dim3((unsigned)rows), dim3(512), cfg, x, ldx, w, d, eps, hi, lo, y.ld);
}
cudaError_t launch_swiglu16(const float *g, const float *u, int n, int ld, int rows, const Operand16 &y, const LaunchCfg &cfg) {
  uint16_t *hi = static_cast<uint16_t *>(y.hi), *lo = static_cast<uint16_t *>(y.lo);
  const dim3 grid((unsigned)((n + 255) / 256), (unsigned)rows);
  if (y.f16) return launch_simple(swiglu16_kernel<true>, grid, dim3(256), cfg, g, u, n, ld, hi, lo, y.ld);
  return launch_simple(swiglu16_kernel<false>, grid, dim3(256), cfg, g, u, n, ld, hi, lo, y.ld);
}
cudaError_t launch_to16(const float *x, int ldx, int k, int rows, const Operand16 &y, const LaunchCfg &cfg) {
  uint16_t *hi = static_cast<uint16_t *>(y.hi), *lo = static_cast<uint16_t *>(y.lo);
  const dim3 grid((unsigned)((k + 255) / 256), (unsigned)rows);
  if (y.f16) return launch_simple(to16_kernel<true>, grid, dim3(256), cfg, x, ldx, k, hi, lo, y.ld);
  return launch_simple(to16_kernel<false>, grid, dim3(256), cfg, x, ldx, k, hi, lo, y.ld);
}

cudaError_t launch_reduce_splits(const float *part, int splits, size_t stride, int n, int rows, float *out, int ldo,
                                 const LaunchCfg &cfg) {
  return launch_simple(reduce_splits_kernel, dim3((unsigned)((n + 255) / 256), (unsigned)rows), dim3(256), cfg, part, splits,
                       stride, n, out, ldo);
}

// Weight rows one CTA covers in this operand mode.
int qgemm_rows_per_cta(int mode) { return TM * row_tiles(mode); }

// Number of K splits a launch with these arguments will actually use (whole 256-column raw tiles each).
int qgemm_effective_splits(int k, int splits) {
  const int total_steps = k / KSTEP;
  if (splits < 1) splits = 1;
  const int k_steps = ((total_steps / RAW_STEPS + splits - 1) / splits) * RAW_STEPS;
  return (total_steps + k_steps - 1) / k_steps;
}

cudaError_t launch_qgemm_tc(const QGemmArgs &a, const LaunchCfg &cfg) {
  if (!a.w || !a.x16 || !a.out || a.m < 1 || a.n < 1 || a.k < KSTEP || a.k % 256) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a.x16) & 15) || (a.ldx * 2) % 16 || (reinterpret_cast<uintptr_t>(a.w) & 15))
    return cudaErrorInvalidValue;
  if (a.mode == QGEMM_F16X3 && (!a.x16_lo || (reinterpret_cast<uintptr_t>(a.x16_lo) & 15))) return cudaErrorInvalidValue;
  if (a.mode < QGEMM_BF16 || a.mode > QGEMM_F16X3) return cudaErrorInvalidValue;
  if (qgemm_tc_wide_applies(a)) return launch_qgemm_tc_wide(a, cfg);  // more than 256 tokens, one operand plane
  count_launch(LC_QGEMM_TC);
  if (a.type == RG_TYPE_Q4_0) return launch_m<RG_TYPE_Q4_0>(a, cfg);
  if (a.type == RG_TYPE_Q8_0) return launch_m<RG_TYPE_Q8_0>(a, cfg);
  return cudaErrorInvalidValue;
}

}  // namespace rg
