// Prefill / wide-batch GEMM on the 5th-generation tensor cores:
//   C[M][N] (f32) = X[M][K] (bf16) * W[N][K]^T,  W in native Q4_0 / Q8_0 GGML blocks.
// Semantics: the layer linears of the Llama forward for many tokens at once
// (src/models/transformer/layer.rs:445-448, src/backend/cpu.rs:3484-3532 on the dequantised
// weight of src/models/transformer/model.rs:982-995), with bf16 operands and f32 accumulation.
//
// One CTA computes a [128 weight rows] x [TN tokens] tile over a K range:
//   * MMA M = 128 weight rows (the dequantised tile is the A operand), MMA N = TN tokens (the
//     activation tile is the B operand), K = 16 per tcgen05.mma, four per 64-element stage;
//     the accumulator lives in TMEM (128 lanes x TN f32 columns).
//   * warp 0: TMA producer of the activation tiles (tiled 2-D copy, 128-byte swizzle).
//   * warp 1: allocates TMEM, issues tcgen05.mma from one thread, commits to mbarriers.
//   * warp 0 also streams the raw block bytes of the 128 weight rows, 256 columns (8 blocks) at a
//     time, into a small ring with a second tiled 2-D TMA map, so no thread waits on global memory.
//   * warps 2-9: two threads per weight row, each reads the row's two raw blocks of the stage from that
//     ring, expands nibbles to exact bf16 integers with
//     the 128+n bit pattern and applies the block scale with one bf16x2 FMA per two weights, and
//     writes the 128-byte row into the K-major / 128-byte-swizzled A tile; afterwards the same
//     warps read the accumulator with tcgen05.ld and store it.
//   * Four-stage ring with bounded mbarrier waits; a time-out records a status and the kernel
//     still frees its TMEM and exits.
// The weight scale enters as bf16(d): the A operand is bf16(bf16(d) * (n - 8)).
#include <cuda.h>
#include <cuda_bf16.h>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int TM = 128;     // weight rows per tile (MMA M)
constexpr int KSTEP = 64;   // elements per stage (128 bytes of bf16: one swizzle row)
constexpr int RAW_STEPS = 4;  // 64-element stages per raw weight tile (256 columns = 8 blocks)
constexpr int RAW_NS = 2;     // raw ring depth
constexpr int THREADS = 320;  // TMA warp, MMA warp, eight dequantisation / epilogue warps
constexpr int A_BYTES = TM * KSTEP * 2;

struct Params {
  const uint8_t *w;
  int n, k;       // weight rows, columns
  int m;          // tokens
  int k_begin_steps, k_steps;  // this launch covers steps [blockIdx.z * k_steps, ...) of k / 64
  float *out;     // [splits][m][ldc] when split-K, else [m][ldc]
  int ldc;
  size_t split_stride;
  int *status;
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
// Instruction descriptor: f32 accumulate, bf16 A and B, both K-major, shape M x N.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
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

__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

// One Q4_0 block (scale + 16 quant bytes given as four words) -> 32 bf16 in element order:
// out[0..7] = elements 0..15 (low nibbles), out[8..15] = elements 16..31 (high nibbles).
__device__ __forceinline__ void q4_block_to_bf16(uint32_t dbits16, const uint32_t (&q)[4], uint32_t (&out)[16]) {
  const float d = half_bits_to_float(dbits16);
  const uint32_t d2 = pack_bf16x2(d, d);
  const uint32_t M = 0x000F000Fu, E = 0x43004300u, OFF = 0x43084308u;  // bf16 128 + n, minus 136: exact n - 8
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w = prmt(q[i], 0u, 0x3120u);  // bytes (b0, b2, b1, b3): adjacent elements share a mask
    out[2 * i] = bf16x2_mul(bf16x2_sub((w & M) | E, OFF), d2);              // elements 4i, 4i+1
    out[2 * i + 1] = bf16x2_mul(bf16x2_sub(((w >> 8) & M) | E, OFF), d2);   // elements 4i+2, 4i+3
    out[8 + 2 * i] = bf16x2_mul(bf16x2_sub(((w >> 4) & M) | E, OFF), d2);   // elements 16+4i, 16+4i+1
    out[8 + 2 * i + 1] = bf16x2_mul(bf16x2_sub(((w >> 12) & M) | E, OFF), d2);
  }
}
// One Q8_0 block (eight words of int8) -> 32 bf16.
__device__ __forceinline__ void q8_block_to_bf16(uint32_t dbits16, const uint32_t (&q)[8], uint32_t (&out)[16]) {
  const float d = half_bits_to_float(dbits16);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t u = q[i] ^ 0x80808080u;
    const float v0 = __uint_as_float(0x4B000000u | (u & 0xffu)) - 8388736.0f;
    const float v1 = __uint_as_float(0x4B000000u | ((u >> 8) & 0xffu)) - 8388736.0f;
    const float v2 = __uint_as_float(0x4B000000u | ((u >> 16) & 0xffu)) - 8388736.0f;
    const float v3 = __uint_as_float(0x4B000000u | (u >> 24)) - 8388736.0f;
    out[2 * i] = pack_bf16x2(v0 * d, v1 * d);
    out[2 * i + 1] = pack_bf16x2(v2 * d, v3 * d);
  }
}

template <int QT, int TN>
__global__ void __launch_bounds__(THREADS, 1)
    qgemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const Params P) {
  constexpr bool Q4 = (QT == RG_TYPE_Q4_0);
  constexpr int BB = Q4 ? 18 : 34;
  constexpr int NS = TN > 128 ? 3 : 4;  // operand ring depth
  constexpr int B_BYTES = TN * KSTEP * 2;
  constexpr int RAW_ROW = 8 * BB;  // bytes of one weight row in a raw tile (144 / 272)
  constexpr int RAW_BYTES = TM * RAW_ROW;
  constexpr int TMEM_COLS = TN < 32 ? 32 : TN;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *a_ring = smem;
  uint8_t *b_ring = smem + NS * A_BYTES;
  uint8_t *raw_ring = b_ring + NS * B_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(raw_ring + RAW_NS * RAW_BYTES);
  uint64_t *b_full = bars, *a_full = bars + NS, *slot_free = bars + 2 * NS;
  uint64_t *raw_full = bars + 3 * NS, *raw_free = raw_full + RAW_NS, *acc_done = raw_free + RAW_NS;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_done + 1);
  volatile int *dead = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TM, tok0 = blockIdx.y * TN;
  const int step0 = blockIdx.z * P.k_steps;  // k_steps is a multiple of RAW_STEPS
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
        mbar_expect_tx(&b_full[slot], (uint32_t)B_BYTES);
        tma_tile_2d(b_ring + slot * B_BYTES, &xmap, (step0 + i) * KSTEP, tok0, &b_full[slot]);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(TM, TN);
      for (int i = 0; i < nsteps; ++i) {
        const int slot = i % NS;
        const uint32_t ph = (uint32_t)((i / NS) & 1);
        mbar_wait_bounded(&a_full[slot], ph, dead, P.status);
        mbar_wait_bounded(&b_full[slot], ph, dead, P.status);
        tc_fence_after();
        const uint32_t a_addr = smem_u32(a_ring + slot * A_BYTES), b_addr = smem_u32(b_ring + slot * B_BYTES);
#pragma unroll
        for (int kk = 0; kk < KSTEP / 16; ++kk)
          umma_bf16(tmem_base, umma_desc(a_addr + kk * 32), umma_desc(b_addr + kk * 32), idesc, (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&slot_free[slot]);  // the slot may be rewritten once these MMAs have read it
      }
      umma_commit(acc_done);
    }
  } else {
    // ---------------------------------------------------------------- dequantisation: one block (half of a
    // stage's 64 columns) of one weight row per thread, two threads per row
    const int tdq = threadIdx.x - 64;            // 0..255
    const int r = tdq & 127, half = tdq >> 7;    // row of the tile, even / odd block of the stage
    constexpr int QW = Q4 ? 4 : 8;               // quant words per block
    for (int i = 0; i < nsteps; ++i) {
      const int slot = i % NS;
      const int j = i / RAW_STEPS, rs = j % RAW_NS, sub = i % RAW_STEPS;
      if (sub == 0) mbar_wait_bounded(&raw_full[rs], (uint32_t)((j / RAW_NS) & 1), dead, P.status);
      // pair layout: [d0 | q0] [d1 | q1] with a 2-byte scale in front of each block: the even block's
      // quants straddle word boundaries (funnel shift), the odd block's are word aligned
      const uint32_t *src = reinterpret_cast<const uint32_t *>(raw_ring + rs * RAW_BYTES + r * RAW_ROW + sub * 2 * BB);
      uint32_t q[QW], dbits, vals[16];  // 32 bf16 of this block, in k order
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
      if constexpr (Q4) {
        q4_block_to_bf16(dbits, q, vals);
      } else {
        q8_block_to_bf16(dbits, q, vals);
      }
      if (sub == RAW_STEPS - 1 || i + 1 == nsteps) mbar_arrive(&raw_free[rs]);  // raw bytes are in registers now
      if (i >= NS) mbar_wait_bounded(&slot_free[slot], (uint32_t)((i / NS - 1) & 1), dead, P.status);
      uint8_t *row_dst = a_ring + slot * A_BYTES + r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 chunk = make_uint4(vals[4 * c], vals[4 * c + 1], vals[4 * c + 2], vals[4 * c + 3]);
        *reinterpret_cast<uint4 *>(row_dst + (((4 * half + c) ^ (r & 7)) << 4)) = chunk;
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
          if (tok < P.m && orow < P.n) out[(size_t)tok * P.ldc + orow] = __uint_as_float(v[w]);
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

template <int QT, int TN>
cudaError_t launch_t(const QGemmArgs &a, const LaunchCfg &cfg) {
  EncodeFn fn = encode_fn();
  if (!fn) return cudaErrorNotSupported;
  constexpr int BB = (QT == RG_TYPE_Q4_0) ? 18 : 34;
  constexpr int NS = TN > 128 ? 3 : 4;
  constexpr int RAW_ROW = 8 * BB;
  alignas(64) CUtensorMap xmap, wmap;
  const cuuint32_t elem[2] = {1, 1};
  {
    const cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)a.m};
    const cuuint64_t strides[1] = {(cuuint64_t)a.ldx * 2};
    const cuuint32_t box[2] = {(cuuint32_t)KSTEP, (cuuint32_t)TN};
    if (fn(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(a.x_bf16), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorInvalidValue;
  }
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
  P.w = a.w;
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
  constexpr size_t smem = 1024 + NS * (A_BYTES + TN * KSTEP * 2) + RAW_NS * TM * RAW_ROW + (3 * NS + 2 * RAW_NS + 1) * 8 + 16;
  auto kernel = qgemm_tc_kernel<QT, TN>;
  static bool attr_done = false;  // per instantiation
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_done = true;
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
  return cudaLaunchKernelEx(&lc, kernel, xmap, wmap, P);
}

template <int QT>
cudaError_t launch_n(const QGemmArgs &a, const LaunchCfg &cfg) {
  if (a.m > 128) return launch_t<QT, 256>(a, cfg);
  if (a.m > 64) return launch_t<QT, 128>(a, cfg);
  if (a.m > 32) return launch_t<QT, 64>(a, cfg);
  if (a.m > 16) return launch_t<QT, 32>(a, cfg);
  return launch_t<QT, 16>(a, cfg);
}

__global__ void to_bf16_kernel(const float *x, int ldx, int k, __nv_bfloat16 *y, int ldy) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
  if (i < k) y[(size_t)row * ldy + i] = __float2bfloat16_rn(x[(size_t)row * ldx + i]);
}

// RMSNorm of one token row straight to the bf16 GEMM operand; f32 steps rounded like the
// reference (src/models/transformer/layer.rs:423-443), then one rounding to bf16.
__global__ void rmsnorm_bf16_kernel(const float *x, int ldx, const float *w, int d, float eps, __nv_bfloat16 *y, int ldy) {
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
    y[(size_t)blockIdx.x * ldy + i] = __float2bfloat16_rn(__fmul_rn(__fmul_rn(xr[i], inv), w[i]));
}

// h = silu(gate) * up (src/ir/elementwise.rs:6772-6830,7046-7050) to the bf16 operand of the down projection.
__global__ void swiglu_bf16_kernel(const float *g, const float *u, int n, int ld, __nv_bfloat16 *y, int ldy) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
  if (i < n) y[(size_t)row * ldy + i] = __float2bfloat16_rn(swiglu(g[(size_t)row * ld + i], u[(size_t)row * ld + i]));
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

cudaError_t launch_rmsnorm_bf16(const float *x, int ldx, const float *w, int d, float eps, int rows, void *y, int ldy,
                                const LaunchCfg &cfg) {
  return launch_simple(rmsnorm_bf16_kernel, dim3((unsigned)rows), dim3(512), cfg, x, ldx, w, d, eps, static_cast<__nv_bfloat16 *>(y),
                       ldy);
}
cudaError_t launch_swiglu_bf16(const float *g, const float *u, int n, int ld, int rows, void *y, int ldy, const LaunchCfg &cfg) {
  return launch_simple(swiglu_bf16_kernel, dim3((unsigned)((n + 255) / 256), (unsigned)rows), dim3(256), cfg, g, u, n, ld,
                       static_cast<__nv_bfloat16 *>(y), ldy);
}

cudaError_t launch_qgemm_tc(const QGemmArgs &a, const LaunchCfg &cfg) {
  if (!a.w || !a.x_bf16 || !a.out || a.m < 1 || a.n < 1 || a.k < KSTEP || a.k % 256) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a.x_bf16) & 15) || (a.ldx * 2) % 16 || (reinterpret_cast<uintptr_t>(a.w) & 15))
    return cudaErrorInvalidValue;
  if (a.type == RG_TYPE_Q4_0) return launch_n<RG_TYPE_Q4_0>(a, cfg);
  if (a.type == RG_TYPE_Q8_0) return launch_n<RG_TYPE_Q8_0>(a, cfg);
  return cudaErrorInvalidValue;
}

cudaError_t launch_to_bf16(const float *x, int ldx, int k, int rows, void *y, int ldy, const LaunchCfg &cfg) {
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3((unsigned)((k + 255) / 256), (unsigned)rows);
  lc.blockDim = dim3(256);
  lc.stream = cfg.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = cfg.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&lc, to_bf16_kernel, x, ldx, k, static_cast<__nv_bfloat16 *>(y), ldy);
}

}  // namespace rg
