// Decode GEMV (batch 1..2) for Q4_0 / Q8_0 weights in their native GGML block bytes, integer
// tensor-core variant.  Semantics: the per-layer linear of the Llama forward
// (src/models/transformer/layer.rs:445-448) with the dequantised weight of
// src/gguf/quantization/blocks.rs:1244-1257,1493-1505; RMSNorm of layer.rs:423-443 fused in front.
//
// Why a second GEMV kernel: the f16-MMA kernel (qgemv.cu) is bound by the instructions that expand
// nibbles to f16, not by HBM.  Here the weights never leave the integer domain:
//  * Q8_0 quants are already the s8 A operand of mma.sync.m16n8k32.  A Q4_0 word is used as it
//    lies in memory: byte i of word t is n[4t+i] + 16 n[16+4t+i] (low nibble = element 4t+i, high
//    nibble = element 16+4t+i), an unsigned A operand (u8 x s8 MMA).  For k < 16 the A bytes are the
//    raw word and the activation operand holds 16 X[k]; for k >= 16 they are the word with the low
//    nibbles masked off (16 n[k], one logic op per 8 weights) against X[k] - 16 X[k-16].  The cross
//    terms cancel exactly: the integer sum is 16 * sum(n X).  The offset of the format,
//    -8 * sum(X) per block, does not depend on the row: the prologue stores 128 * sum(X) split in
//    two words and the main loop subtracts it from the folded digit sums.
//  * The activation block (32 values) is converted once per CTA to 32-bit block fixed point,
//    x = s_b * X with s_b a power of two and |X| < 2^30 (Q8_0) or 2^26 (Q4_0, which leaves room
//    for the factor 16 and the difference above), and X is split into four signed base-256
//    digits that sit in four B columns.  One MMA per (16 rows x 32 k) block gives four exact int32
//    digit sums; (c0 + 256 c1) and (c2 + 256 c3) are converted to f32 and accumulated with the
//    factor d * s_b.  Everything up to that conversion is exact, so the result carries the f32
//    activation to 2^-30 (Q4_0: 2^-26) of the block maximum and f32 accumulation over blocks.
//  * The packed activations stay resident in shared memory for the whole kernel, produced by the
//    CTA itself in the prologue from the previous kernel's f32 output, optionally through RMSNorm:
//    no separate normalisation / packing kernel, no activation traffic per stage.
//  * Weight streaming is the same as in qgemv.cu: persistent CTA per SM, tiled 2-D TMA boxes of
//    8 rows into a 3-6 stage mbarrier pipeline with bounded waits, bank-conflict-free pitch, weight
//    prefetch issued before the grid dependency wait.
//  * Warp roles: 16 consumer warps (MMA), four per scheduler, one producer warp (TMA), one epilogue warp.  At the end
//    of a row group the consumers fold their accumulators into one value per row, drop them into one
//    of two shared buffers and arrive on an mbarrier; the epilogue warp sums the 16 partials in warp
//    order and applies the epilogue while the consumers are already in the next row group.
//  * Batch 1 can take its activations already packed (`xq`): the kernel that produced the vector
//    wrote the digit planes, the per-block side words and a per-block sum of squares, and this
//    kernel's prologue is one bulk copy into shared memory.  RMSNorm then runs in deferred form:
//    the producer folds the norm weight into the packed values, and 1 / sqrt(mean(x^2) + eps), a
//    scalar, multiplies the finished dot products (x.w is packed instead of (x.inv).w: one rounding
//    moves, far inside the 1e-3 bar).  The residual epilogue is such a producer (`pack_out`).
#include <cuda.h>

#include <stdlib.h>

#include <type_traits>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int R = 32;     // weight rows per stage: two m16 tiles
constexpr int BOXR = 8;   // rows per TMA box
constexpr int CW = 16;    // consumer warps: four per scheduler
constexpr int MAX_STAGES = 6;
constexpr int THREADS = (CW + 2) * 32;  // consumers, producer warp, epilogue warp
constexpr int HDR_BYTES = 256;          // mbarriers and flags at the start of shared memory
constexpr int RED_BYTES = 2 * CW * R * 2 * 4;  // [2 buffers][CW][R][batch <= 2] partial sums
// One CTA per SM.  (Letting two CTAs share an SM so that the next kernel could move in early under
// programmatic dependent launch was measured slower: freed slots fill unevenly and some SMs end up
// with two CTAs of the same kernel.)
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int SMEM_FULL = 227 * 1024;

template <int QT>
struct Geo {
  static constexpr bool Q4 = (QT == RG_TYPE_Q4_0);
  static constexpr int BB = Q4 ? 18 : 34;
  // Blocks per stage: 32 pairs (Q4_0) or 16 pairs (Q8_0), a whole number of rounds of the 16 consumer
  // warps, and a divisor of every K that is a multiple of 2048 / 1024 elements.  A row of a stage
  // is the chunk's bytes plus 16 bytes of padding (the TMA box simply reaches 16 bytes into the
  // next chunk): pitch 1168 / 1104 bytes = 4 / 20 words mod 32, so the eight rows of a fragment
  // load fall into distinct banks.
  static constexpr int KC = Q4 ? 64 : 32;
  static constexpr int CHUNK_BYTES = KC * BB;
  static constexpr int RS = CHUNK_BYTES + 16;
  static_assert(CHUNK_BYTES % 16 == 0 && RS % 16 == 0 && (BOXR * RS) % 128 == 0 && RS / 8 <= 256, "TMA box geometry");
  static_assert((RS / 4) % 8 == 4, "bank-conflict-free pitch");
};

struct Params {
  int seg_rows[3];
  int nseg;
  int n_rows;  // virtual rows (EPI_SWIGLU: rows of the gate matrix)
  int kb;      // K / 32
  const float *x;  // [cols][ldx] f32 input of the previous kernel
  int ldx;
  const int32_t *col_map;  // nullable: source row of each batch column
  const float *norm_w;     // nullable: RMSNorm weight (prologue normalises when set)
  float eps;
  int batch;  // 1..2
  int epi;    // GemvEpilogue
  float *y;
  int ldy;
  int rows_per_cta;
  int stages;
  int *status;
  const uint8_t *xq;    // batch 1: activations already packed (see xq_* below); x / norm_w unused
  int xq_norm;          // the packed values carry the norm weight: scale the results by inv_rms from the block sums
  unsigned long long *trace;
  const int32_t *xq_fix;  // blocks of xq its producer could not pack (they straddle two of its CTAs): packed here from x
  int xq_nfix;
  uint8_t *pack_out;    // EPI_RESIDUAL / EPI_SWIGLU, batch 1: also write the new rows packed for the next GEMV
  const float *pack_w;  // norm weight folded into the packed output (nullable)
  int pack_q4;          // block type of the GEMV that will read pack_out: 1 Q4_0, 0 Q8_0
  const uint8_t *pf[3];   // weights of the next kernel, asked into L2 once this CTA's own loads are issued
  uint32_t pf_bytes[3];
};

constexpr uint32_t PF_CHUNK = 8192;  // bytes per L2 prefetch request

// (layout of a packed activation vector in global memory: xq_side_offset / xq_ssq_offset in rg_device.cuh)

template <int OFF>
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(addr), "n"(OFF));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ void tma_box_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// D(16x8,s32) = A(16x32,s8,row) * B(32x8,s8,col)
// UA: the A bytes are unsigned (Q4_0 words), else signed (Q8_0 quants); B is always signed digits
template <bool UA>
__device__ __forceinline__ void mma_i8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  const int z = 0;
  if constexpr (UA)
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
  else
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}
template <bool UA>
__device__ __forceinline__ void mma_i8_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  if constexpr (UA)
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Row slot rs of a stage is shared row (rs >> 1) * 16 + (rs & 1) * 8 + g; `a` points at
// (row g, word t) of the block pair, `s` at the pair's first scale of row g.
template <int QT, int RSLOT>
__device__ __forceinline__ void load_slot(uint32_t a, uint32_t s, uint32_t (&w)[6], uint32_t (&sc)[2]) {
  using G = Geo<QT>;
  constexpr int R0 = ((RSLOT >> 1) * 16 + (RSLOT & 1) * 8) * G::RS;
  if constexpr (G::Q4) {
    w[0] = lds32<R0>(a);
    w[1] = lds32<R0 + 4>(a);
    w[2] = lds32<R0 + 20>(a);
  } else {
    w[0] = lds32<R0>(a);
    w[1] = lds32<R0 + 4>(a);
    w[2] = lds32<R0 + 16>(a);
    w[3] = lds32<R0 + 20>(a);
    w[4] = lds32<R0 + 36>(a);
    w[5] = lds32<R0 + 52>(a);
  }
  sc[0] = lds16<R0>(s);
  sc[1] = lds16<R0 + G::BB>(s);
}

// Batch-1 variant: `s` already points at the scale of the block this lane scales; one scale per row.
template <int QT, int RSLOT>
__device__ __forceinline__ void load_slot_b1(uint32_t a, uint32_t s, uint32_t (&w)[6], uint32_t (&sc)[2]) {
  using G = Geo<QT>;
  constexpr int R0 = ((RSLOT >> 1) * 16 + (RSLOT & 1) * 8) * G::RS;
  if constexpr (G::Q4) {
    w[0] = lds32<R0>(a);
    w[1] = lds32<R0 + 4>(a);
    w[2] = lds32<R0 + 20>(a);
  } else {
    w[0] = lds32<R0>(a);
    w[1] = lds32<R0 + 4>(a);
    w[2] = lds32<R0 + 16>(a);
    w[3] = lds32<R0 + 20>(a);
    w[4] = lds32<R0 + 36>(a);
    w[5] = lds32<R0 + 52>(a);
  }
  sc[0] = lds16<R0>(s);
}

// A operands of the even and the odd block of a pair for one row slot: {k 0..15, k 16..31}
template <int QT>
__device__ __forceinline__ void expand(const uint32_t (&w)[6], uint32_t (&ae)[2], uint32_t (&ao)[2]) {
  if constexpr (Geo<QT>::Q4) {
    ae[0] = __funnelshift_r(w[0], w[1], 16);  // n[k] + 16 n[k+16], against 16 X[k]
    ae[1] = ae[0] & 0xF0F0F0F0u;              // 16 n[k+16], against X[k+16] - 16 X[k]
    ao[0] = w[2];
    ao[1] = w[2] & 0xF0F0F0F0u;
  } else {
    ae[0] = __funnelshift_r(w[0], w[1], 16);
    ae[1] = __funnelshift_r(w[2], w[3], 16);
    ao[0] = w[4];
    ao[1] = w[5];
  }
}

// Shared layout of the resident activations: digits then block scales.
//   digit byte of element e of block kb, column c (= 4*batch + digit):
//     ((kb * S + c) * 4 + t) * 8 + r * 4 + i,  e < 16: t = e/4, r = 0;  e >= 16: t = (e-16)/4, r = 1;  i = e%4
//   side words of (block kb, batch b), four 32-bit words at (kb * B + b) * 4:
//     {scale, T_lo, scale, T_hi}; T = 128 * sum(X) = T_lo + 65536 T_hi is the Q4_0 offset term (0 for Q8_0)
__device__ __forceinline__ uint32_t digit_offset(int S, int kb, int c, int e) {
  const int t = (e & 15) >> 2, r = e >> 4, i = e & 3;
  return (uint32_t)((((kb * S + c) * 4 + t) * 8) + r * 4 + i);
}

// B1 (batch 1): the four digit columns leave half of the MMA's eight columns idle, so the even and
// the odd block of a pair share one accumulator tile: columns 0-3 take the even block's digits
// (B rows k < 16 only), columns 4-7 the odd block's (B rows k >= 16 only), and the A operand carries
// the even block in k < 16 and the odd block in k >= 16.  Two MMAs (low / high halves of both blocks)
// accumulate in place; afterwards lanes t < 2 scale the even block and lanes t >= 2 the odd one, so
// the per-lane scale / convert / accumulate work is half of the general layout's.
// XQ: the activations arrive packed (batch 1).  Those instantiations carry no self-packing code at
// all: the kernels of a decode step alternate, and a step runs faster the less code they hold (the
// unrolled register-resident prologues alone are 50 KB per instantiation; with them in, every launch
// of a step started on cold instruction caches and the step took 9 % longer).
template <int QT, bool B1, bool XQ>
__global__ void __launch_bounds__(THREADS, 1)
    qgemv_i8_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                    const __grid_constant__ CUtensorMap map2, const Params P) {
  using G = Geo<QT>;
  // The epilogue is a run-time switch: every projection of a decode step then runs the same kernel
  // (per block type), which stays in the instruction caches from launch to launch.
  const int EPI = P.epi;
  const bool PAIR = (EPI == EPI_SWIGLU);
  const int GROUP_ROWS = PAIR ? 16 : 32;
  constexpr int NB = B1 ? 1 : 2;  // batch columns a partial-sum slot holds
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + MAX_STAGES;
  uint64_t *red_full = empty + MAX_STAGES;  // [2]: the consumers' partial sums of a row group are in place
  uint64_t *red_free = red_full + 2;        // [2]: the epilogue warp has read them
  uint64_t *xbar = red_free + 2;            // bulk copy of pre-packed activations
  volatile int *dead = reinterpret_cast<volatile int *>(xbar + 1);
  static_assert((2 * MAX_STAGES + 5) * 8 + 4 <= HDR_BYTES, "header");
  float *red = reinterpret_cast<float *>(smem + HDR_BYTES);  // [2][CW][R][NB]; also scratch of the prologue
  static_assert(RED_BYTES % 128 == 0 && HDR_BYTES % 128 == 0, "alignment");
  const int S = 4 * P.batch;
  const int xs_bytes = (P.kb * S * 32 + 127) & ~127;
  const int sb_bytes = (P.kb * P.batch * 16 + 127) & ~127;
  uint8_t *xs = smem + HDR_BYTES + RED_BYTES;
  float *sb = reinterpret_cast<float *>(xs + xs_bytes);
  uint8_t *stage0 = xs + xs_bytes + sb_bytes;
  constexpr int STAGE_BYTES = R * G::RS;
  static_assert(STAGE_BYTES % 128 == 0, "alignment");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r_begin = blockIdx.x * P.rows_per_cta;
  const int r_end = min(P.n_rows, r_begin + P.rows_per_cta);
  // Row groups of GROUP_ROWS rows.  A SwiGLU launch hands out rows in units of 8, so a CTA may start
  // in the middle of a 16-row unit of its output: its first group is then 8 rows, and every later
  // group is one aligned half of a 32-element block of the next GEMV's input (see the packing below).
  const int first_rows = (PAIR && (r_begin & 8)) ? 8 : GROUP_ROWS;
  const int cta_rows = r_end - r_begin;
  const int n_groups = cta_rows <= 0 ? 0 : cta_rows <= first_rows ? 1 : 1 + (cta_rows - first_rows + GROUP_ROWS - 1) / GROUP_ROWS;
  auto group_start = [&](int grp) { return grp == 0 ? r_begin : r_begin + first_rows + (grp - 1) * GROUP_ROWS; };
  auto group_rows = [&](int grp, int vr0) { return min(grp == 0 ? first_rows : GROUP_ROWS, r_end - vr0); };
  const int n_chunks = (P.kb + G::KC - 1) / G::KC;
  const int units = n_groups * n_chunks;
  const int stages = P.stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CW);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&red_full[b], CW);
      mbar_init(&red_free[b], 1);
    }
    mbar_init(xbar, 1);
    *dead = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();
  const bool tr_first = blockIdx.x == 0, tr_last = blockIdx.x == gridDim.x - 1;
  if (threadIdx.x == 0) trace_stamp(P.trace, 0, tr_first, tr_last);  // CTA started

  // 1 / sqrt(mean(x^2) + eps) from the per-block sums of squares of a pre-packed vector; every warp
  // that needs it computes it alone, in the same order
  auto inv_from_blocks = [&]() {
    const float *ssq = reinterpret_cast<const float *>(P.xq + xq_ssq_offset(P.kb));
    float ss = 0.0f;
    for (int i = lane; i < P.kb; i += 32) ss += __ldcg(ssq + i);
    ss = warp_sum(ss);
    const float mean = __fdiv_rn(ss, (float)(P.kb * 32));
    return __frcp_rn(__fsqrt_rn(__fadd_rn(mean, P.eps)));
  };

  // One row group's epilogue, run by a whole warp (lane = row of the group): sum the consumer warps'
  // partials in warp order, scale, apply the epilogue, optionally pack the new rows.
  constexpr float A_SCALE = G::Q4 ? 0.0625f : 1.0f;  // the Q4_0 digit sums carry a factor 16
  [[maybe_unused]] float half0 = 0.0f;   // SwiGLU packing: first 16 rows of the block in progress
  [[maybe_unused]] int half0_blk = -1;
  auto group_epilogue = [&](int grp, float out_scale, auto wait_for_partials) {
      const int buf = grp & 1;
      const int vr0 = group_start(grp);
      const int vrow = vr0 + lane;
      const int vend = vr0 + group_rows(grp, vr0);  // rows of this group are [vr0, vend)
      float resid[NB];
#pragma unroll
      for (int b = 0; b < NB; ++b) resid[b] = 0.0f;
      if (EPI == EPI_RESIDUAL && vrow < vend) {  // requested before the wait: off the critical path
#pragma unroll
        for (int b = 0; b < NB; ++b)
          if (b < P.batch) resid[b] = P.y[(size_t)b * P.ldy + vrow];
      }
      float pw = 1.0f;
      if (EPI == EPI_RESIDUAL && B1 && P.pack_out && P.pack_w && vrow < vend) pw = __ldg(P.pack_w + vrow);
      wait_for_partials();
      float tot[NB];
#pragma unroll
      for (int b = 0; b < NB; ++b) tot[b] = 0.0f;
      const float *rb = red + (size_t)buf * CW * R * NB + lane * NB;
#pragma unroll
      for (int w = 0; w < CW; ++w)
#pragma unroll
        for (int b = 0; b < NB; ++b) tot[b] += rb[w * R * NB + b];
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_free[buf]);
#pragma unroll
      for (int b = 0; b < NB; ++b) tot[b] *= out_scale;
      float xn[NB];
      if (EPI == EPI_SWIGLU) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const float up = __shfl_down_sync(0xffffffffu, tot[b], 16);
          xn[b] = swiglu(tot[b], up);
          if (lane < 16 && vrow < vend && b < P.batch) P.y[(size_t)b * P.ldy + vrow] = xn[b];
        }
        if constexpr (B1) {
          // The 16 new rows are half a block of the next GEMV's input.  When both halves of a block
          // belong to this CTA the block is packed here (first half kept from the previous group);
          // blocks that straddle two CTAs are left to the consumer (its xq_fix list).
          if (P.pack_out) {
            if ((vr0 & 31) == 0) {
              half0 = xn[0];
              half0_blk = vr0 + 32 <= r_end ? (vr0 >> 5) : -1;
            } else if ((vr0 & 31) == 16 && vend - vr0 == 16 && half0_blk == (vr0 >> 5)) {
              const float second = __shfl_sync(0xffffffffu, xn[0], lane & 15);
              pack_block_warp(lane < 16 ? half0 : second, P.pack_q4 != 0, P.pack_out, vr0 >> 5, P.n_rows >> 5, lane, false, 0.0f);
              half0_blk = -1;
            }
          }
        }
      } else {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          xn[b] = EPI == EPI_RESIDUAL ? __fadd_rn(resid[b], tot[b]) : tot[b];
          if (vrow < vend && b < P.batch) P.y[(size_t)b * P.ldy + vrow] = xn[b];
        }
      }
      if constexpr (B1) {
        if (EPI == EPI_RESIDUAL && P.pack_out) {
          // the 32 new rows are block vr0 / 32 of the next GEMV's input: pack them here (the launcher
          // gives every CTA whole blocks), with that GEMV's norm weight folded in
          const float ssq = warp_sum(__fmul_rn(xn[0], xn[0]));
          pack_block_warp(__fmul_rn(xn[0], pw), P.pack_q4 != 0, P.pack_out, vr0 >> 5, P.n_rows >> 5, lane, true, ssq);
        }
      }
  };

  if (warp == CW) {
    // ------------------------------------------------------------------ producer (weights only:
    // constant data, so it never waits for the previous kernel)
    int grp = 0, c = 0, stage = 0, round = 0;
    for (int u = 0; u < units; ++u) {
      if (round > 0) mbar_wait_bounded(&empty[stage], (uint32_t)((round - 1) & 1), dead, P.status);
      const int vr0 = group_start(grp);
      uint8_t *sw = stage0 + (size_t)stage * STAGE_BYTES;
      // a partial group fetches only the boxes that hold its rows
      const int nbx = (group_rows(grp, vr0) + BOXR - 1) / BOXR;
      const bool box_live = PAIR ? (lane & 1) < nbx : lane < nbx;
      if (lane == 0) mbar_expect_tx(&full[stage], (uint32_t)((PAIR ? 2 * nbx : nbx) * BOXR * G::RS));
      __syncwarp();
      if (lane < R / BOXR && box_live) {
        const CUtensorMap *map = &map0;
        int row;
        if (PAIR) {
          map = (lane < 2) ? &map0 : &map1;
          row = vr0 + (lane & 1) * BOXR;
        } else {
          row = vr0 + lane * BOXR;
          if (P.nseg > 1 && row >= P.seg_rows[0]) {
            row -= P.seg_rows[0];
            map = &map1;
            if (P.nseg > 2 && row >= P.seg_rows[1]) {
              row -= P.seg_rows[1];
              map = &map2;
            }
          }
        }
        tma_box_2d(sw + lane * BOXR * G::RS, map, c * (G::CHUNK_BYTES / 8), row, &full[stage]);
      }
      if (++c == n_chunks) {
        c = 0;
        ++grp;
      }
      if (++stage == stages) {
        stage = 0;
        ++round;
      }
    }
    if (lane == 0) trace_stamp(P.trace, 7, tr_first, tr_last);  // every load of this CTA issued
    // every load of this CTA is issued: spend the rest of the kernel asking L2 for the next kernel's
    // weights (constant data; a hint that nothing waits for), one slice per CTA
#pragma unroll 1
    for (int i = 0; i < 3; ++i) {
      const uint32_t total = P.pf_bytes[i];
      for (uint32_t off = (blockIdx.x * 32u + (uint32_t)lane) * PF_CHUNK; off < total; off += gridDim.x * 32u * PF_CHUNK)
        l2_prefetch_bulk(P.pf[i] + off, min(PF_CHUNK, total - off));
    }
    return;
  }

  if (warp == CW + 1) {
    // ------------------------------------------------------------------ epilogue warp
    if (n_groups == 0) return;
    pdl_wait();  // the residual rows, the block sums and every store below touch the step's buffers
    if (lane == 0) trace_stamp(P.trace, 1, tr_first, tr_last);  // grid dependency resolved
    float out_scale = A_SCALE;
    if (XQ && P.xq_norm) out_scale *= inv_from_blocks();
    for (int grp = 0; grp < n_groups; ++grp) {
      const int buf = grp & 1;
      group_epilogue(grp, out_scale, [&]() {
        // a row group takes microseconds: poll with a pause so this warp leaves the issue slots to the consumers
        {
          bool ok = *dead != 0;
          for (uint32_t i = 0; !ok && i < (1u << 22); ++i) {
            ok = mbar_try_wait(&red_full[buf], (uint32_t)((grp >> 1) & 1));
            if (!ok) {
              __nanosleep(100);
              if ((i & 1023u) == 1023u && *dead) break;
            }
          }
          if (!ok && !*dead) {
            *dead = 1;
            if (P.status) atomicExch(P.status, DEV_TIMEOUT);
          }
        }
      });
      if (lane == 0 && grp == 0) trace_stamp(P.trace, 4, tr_first, tr_last);  // first row group stored
    }
    if (lane == 0) trace_stamp(P.trace, 5, tr_first, tr_last);  // last row group stored
    return;
  }

  // -------------------------------------------------------------------- consumers
  const int ctid = threadIdx.x;  // 0 .. CW*32-1
  // ---- prologue: (RMSNorm and) block fixed-point packing of the activations into shared memory.
  // Four lanes per block: lane q of a block holds elements 4q..4q+3 and 16+4q..16+4q+3 (the two
  // 32-bit words of each digit plane that one consumer lane fetches together); a warp converts
  // eight blocks per pass, the CTA PASS_BLOCKS.  All lanes run every shuffle; `live` only guards
  // the stores, so independent passes can be interleaved by the compiler.
  constexpr int PASS_BLOCKS = CW * 8;
  const int q4 = lane & 3;
  const int kbw = warp * 8 + (lane >> 2);
  auto pack_block = [&](float (&v)[8], int kb, int b, bool live) {
    float m = 0.0f, tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      m = fmaxf(m, fabsf(v[i]));
      tot += v[i];
    }
    if (!(fabsf(tot) <= 3.0e38f)) m = __uint_as_float(0x7f800000u);  // fmaxf drops NaN: keep it visible
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    const uint32_t E = __float_as_uint(m) >> 23;  // biased exponent of the block maximum (m >= 0)
    constexpr uint32_t XBITS = G::Q4 ? 25u : 29u;  // |X| < 2^(XBITS + 1)
    float s = 0.0f;
    int X[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (E >= 40u && E < 255u) {
      s = __uint_as_float((E - XBITS) << 23);  // 2^(floor(log2 m) - XBITS)
      const float up = __uint_as_float((254u + XBITS - E) << 23);
#pragma unroll
      for (int i = 0; i < 8; ++i) X[i] = __float2int_rn(v[i] * up);
    } else if (E == 255u) {  // inf / NaN input must stay visible in the result
      s = __uint_as_float(0x7fc00000u);
      X[0] = 1;
    }
    int t_lo = 0, t_hi = 0;
    if constexpr (G::Q4) {
      int sum = ((X[0] + X[1]) + (X[2] + X[3])) + ((X[4] + X[5]) + (X[6] + X[7]));  // |sum over the block| < 2^31
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      t_lo = (sum & 0x1FF) << 7;  // 128 * sum = t_lo + 65536 * t_hi
      t_hi = sum >> 9;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        X[4 + i] -= X[i] << 4;  // X[k] - 16 X[k-16]
        X[i] <<= 4;             // 16 X[k]
      }
    }
    // X + 0x80808080 turns the four signed base-256 digits of X into unsigned bytes (digit + 128);
    // 4x4 byte transposes: word d = digit d of four elements, then back to signed
    uint32_t Y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) Y[i] = (uint32_t)X[i] + 0x80808080u;
    uint32_t D[2][4];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const uint32_t t0 = prmt(Y[4 * r], Y[4 * r + 1], 0x5140u), t1 = prmt(Y[4 * r + 2], Y[4 * r + 3], 0x5140u);
      const uint32_t t2 = prmt(Y[4 * r], Y[4 * r + 1], 0x7362u), t3 = prmt(Y[4 * r + 2], Y[4 * r + 3], 0x7362u);
      D[r][0] = prmt(t0, t1, 0x5410u) ^ 0x80808080u;
      D[r][1] = prmt(t0, t1, 0x7632u) ^ 0x80808080u;
      D[r][2] = prmt(t2, t3, 0x5410u) ^ 0x80808080u;
      D[r][3] = prmt(t2, t3, 0x7632u) ^ 0x80808080u;
    }
    if (live) {
      uint2 *dst = reinterpret_cast<uint2 *>(xs + digit_offset(S, kb, 4 * b, q4 * 4));
      const int plane = 32 / 8;  // 64-bit words between consecutive columns of a block
#pragma unroll
      for (int d = 0; d < 4; ++d) dst[d * plane] = make_uint2(D[0][d], D[1][d]);
      if (q4 == 0)
        *reinterpret_cast<float4 *>(sb + (kb * P.batch + b) * 4) =
            make_float4(s, __int_as_float(t_lo), s, __int_as_float(t_hi));
    }
  };
  // y = (x * (1 / sqrt(mean(x^2) + eps))) * w, every step rounded to f32 (layer.rs:423-443)
  auto inv_rms = [&](float ss) {
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < CW; ++w) tot += red[w];
    const float mean = __fdiv_rn(tot, (float)(P.kb * 32));
    const float inv = __frcp_rn(__fsqrt_rn(__fadd_rn(mean, P.eps)));
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    return inv;
  };
  auto load8 = [&](const float *base, int kb, float4 &lo, float4 &hi) {
    lo = __ldg(reinterpret_cast<const float4 *>(base + (size_t)kb * 32) + q4);
    hi = __ldg(reinterpret_cast<const float4 *>(base + (size_t)kb * 32) + 4 + q4);
  };
  auto sumsq = [](float ss, const float4 &f) {
    ss = fmaf(f.x, f.x, ss);
    ss = fmaf(f.y, f.y, ss);
    ss = fmaf(f.z, f.z, ss);
    return fmaf(f.w, f.w, ss);
  };
  auto normed = [](float (&v)[8], float inv, const float4 &wl, const float4 &wh) {
    const float w[8] = {wl.x, wl.y, wl.z, wl.w, wh.x, wh.y, wh.z, wh.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(v[i], inv), w[i]);
  };

  // Register-resident form (batch 1, up to four passes, three with a norm): the norm weights are
  // constant data and are fetched before the grid dependency resolves, the activation is read
  // once, and both uses (sum of squares, packing) run from registers as straight-line code.
  auto fast = [&](auto np_c, auto norm_c) {
    constexpr int NP = decltype(np_c)::value;
    constexpr bool NORM = decltype(norm_c)::value;
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 wl[NORM ? NP : 1], wh[NORM ? NP : 1], xl[NP], xh[NP];
    if constexpr (NORM) {
#pragma unroll
      for (int it = 0; it < NP; ++it) {
        wl[it] = wh[it] = zero;
        if (it * PASS_BLOCKS + kbw < P.kb) load8(P.norm_w, it * PASS_BLOCKS + kbw, wl[it], wh[it]);
      }
    }
    pdl_wait();
    const float *xr = P.x + (size_t)(P.col_map ? P.col_map[0] : 0) * P.ldx;
#pragma unroll
    for (int it = 0; it < NP; ++it) {
      xl[it] = xh[it] = zero;
      if (it * PASS_BLOCKS + kbw < P.kb) load8(xr, it * PASS_BLOCKS + kbw, xl[it], xh[it]);
    }
    float inv = 1.0f;
    if constexpr (NORM) {
      float ss = 0.0f;
#pragma unroll
      for (int it = 0; it < NP; ++it) ss = sumsq(sumsq(ss, xl[it]), xh[it]);
      inv = inv_rms(ss);
    }
#pragma unroll
    for (int it = 0; it < NP; ++it) {
      float v[8] = {xl[it].x, xl[it].y, xl[it].z, xl[it].w, xh[it].x, xh[it].y, xh[it].z, xh[it].w};
      if constexpr (NORM) normed(v, inv, wl[it], wh[it]);
      const int kb = it * PASS_BLOCKS + kbw;
      pack_block(v, kb, 0, kb < P.kb);
    }
  };
  using std::integral_constant;
  if constexpr (XQ) {
    // the producer of the vector packed it: one bulk copy of digits and side words
    // blocks the producer could not pack come from the plain f32 copy of the vector; the list is
    // constant data, so the first pass's block index is fetched before the grid dependency resolves
    const bool fix0 = kbw < P.xq_nfix;
    const int kb0 = fix0 ? __ldg(P.xq_fix + kbw) : 0;
    pdl_wait();
    if (ctid == 0) {
      const uint32_t db = (uint32_t)P.kb * 128u, sbb = (uint32_t)P.kb * 16u;
      mbar_expect_tx(xbar, db + sbb);
      bulk_g2s(xs, P.xq, db, xbar);
      bulk_g2s(sb, P.xq + xq_side_offset(P.kb), sbb, xbar);
    }
    const float *xr = P.xq_nfix > 0 ? P.x + (size_t)(P.col_map ? P.col_map[0] : 0) * P.ldx : nullptr;
    float4 xl0 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), xh0 = xl0;
    if (fix0) load8(xr, kb0, xl0, xh0);  // in flight together with the bulk copy
    mbar_wait_bounded(xbar, 0, dead, P.status);
    if (P.xq_nfix > 0) {
      float v0[8] = {xl0.x, xl0.y, xl0.z, xl0.w, xh0.x, xh0.y, xh0.z, xh0.w};
      pack_block(v0, kb0, 0, fix0);
      for (int s0 = PASS_BLOCKS; s0 < P.xq_nfix; s0 += PASS_BLOCKS) {  // uniform trip count
        const int slot = s0 + kbw;
        const bool live = slot < P.xq_nfix;
        const int kb = live ? __ldg(P.xq_fix + slot) : 0;
        float4 xl = make_float4(0.0f, 0.0f, 0.0f, 0.0f), xh = xl;
        if (live) load8(xr, kb, xl, xh);
        float v[8] = {xl.x, xl.y, xl.z, xl.w, xh.x, xh.y, xh.z, xh.w};
        pack_block(v, kb, 0, live);
      }
    }
  } else {
  const int npass = (P.kb + PASS_BLOCKS - 1) / PASS_BLOCKS;
  if (B1 && npass <= (P.norm_w ? 3 : 4)) {
    if (P.norm_w) {
      if (npass == 1) fast(integral_constant<int, 1>{}, integral_constant<bool, true>{});
      else if (npass == 2) fast(integral_constant<int, 2>{}, integral_constant<bool, true>{});
      else fast(integral_constant<int, 3>{}, integral_constant<bool, true>{});
    } else {
      if (npass == 1) fast(integral_constant<int, 1>{}, integral_constant<bool, false>{});
      else if (npass == 2) fast(integral_constant<int, 2>{}, integral_constant<bool, false>{});
      else if (npass == 3) fast(integral_constant<int, 3>{}, integral_constant<bool, false>{});
      else fast(integral_constant<int, 4>{}, integral_constant<bool, false>{});
    }
  } else {
    pdl_wait();
    for (int b = 0; b < P.batch; ++b) {
      const float *xr = P.x + (size_t)(P.col_map ? P.col_map[b] : b) * P.ldx;
      float inv = 1.0f;
      if (P.norm_w) {
        float ss = 0.0f;
        for (int i = ctid; i < P.kb * 8; i += CW * 32) ss = sumsq(ss, __ldg(reinterpret_cast<const float4 *>(xr) + i));
        inv = inv_rms(ss);
      }
      for (int kbb = warp * 8; kbb < P.kb; kbb += PASS_BLOCKS) {  // warp-uniform trip count
        const int kb = kbb + (lane >> 2);
        const bool live = kb < P.kb;
        float4 xl = make_float4(0.0f, 0.0f, 0.0f, 0.0f), xh = xl;
        if (live) load8(xr, kb, xl, xh);
        float v[8] = {xl.x, xl.y, xl.z, xl.w, xh.x, xh.y, xh.z, xh.w};
        if (P.norm_w && live) {
          float4 wl, wh;
          load8(P.norm_w, kb, wl, wh);
          normed(v, inv, wl, wh);
        }
        pack_block(v, kb, b, live);
      }
    }
  }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
  if (ctid == 0) trace_stamp(P.trace, 2, tr_first, tr_last);  // activations in shared memory

  const int g = lane >> 2, t = lane & 3;
  const bool col_live = B1 ? true : g < S;  // this lane's B column carries a digit
  const int my_batch = B1 ? 0 : t >> 1;     // batch of this lane's accumulator columns
  const bool acc_live = B1 ? true : my_batch < P.batch;
  const int blk_sel = t >> 1;               // B1: block of the pair this lane scales (0 even, 1 odd)
  float acc[2][2];  // [m-tile][row g / row g+8]
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) acc[mt][0] = acc[mt][1] = 0.0f;

  int stage = 0, c = 0, grp = 0;
  uint32_t phase = 0;
  const uint32_t smem_stage0 = smem_u32(stage0);
  // B1: lanes g >= 4 feed the odd block's digits (column g - 4 of the next block)
  const uint32_t xs_lane = B1 ? smem_u32(xs) + (uint32_t)(((g & 3) * 4 + t) * 8 + (g >> 2) * 128)
                              : smem_u32(xs) + (uint32_t)((g * 4 + t) * 8);
  // this lane's accumulator columns are digits 0,1 (t even) or 2,3 (t odd): {scale, T_lo} or {scale, T_hi}
  const uint32_t sb_lane = smem_u32(sb) + (uint32_t)((B1 ? blk_sel : my_batch) * 16 + (t & 1) * 8);
  const uint32_t lane_w_off = (uint32_t)(g * G::RS + t * 4);
  const uint32_t lane_s_off = B1 ? (uint32_t)(g * G::RS + blk_sel * G::BB) : (uint32_t)(g * G::RS);
  const float fold = (t & 1) ? 65536.0f : 1.0f;  // this lane's accumulators hold the low or the high digit pair
  constexpr uint32_t PAIRB = 2 * G::BB;
  for (int u = 0; u < units; ++u) {
    const int nb = min(G::KC, P.kb - c * G::KC);
    mbar_wait_bounded(&full[stage], phase, dead, P.status);
    if (u == 0 && ctid == 0) trace_stamp(P.trace, 6, tr_first, tr_last);  // first weight stage landed
    const uint32_t sw = smem_stage0 + (uint32_t)stage * (uint32_t)STAGE_BYTES;
    uint32_t aw = sw + lane_w_off + (uint32_t)warp * PAIRB;
    uint32_t as = sw + lane_s_off + (uint32_t)warp * PAIRB;
    int gb = c * G::KC + 2 * warp;  // global block index of the pair's even block
    // rows 16..31 of a partial last group are not this CTA's: their boxes were not fetched
    const bool two_tiles = PAIR || r_end - group_start(grp) > 16;
    if constexpr (B1) {
      // one block pair of all 32 rows: loads, then two accumulating MMAs per m-tile, then scales;
      // no branch inside, so the two m-tiles are scheduled as interleaved chains
      auto fetch = [&](auto tt, uint32_t a, uint32_t s, int gbp, uint32_t (&wq)[4][6], uint32_t (&sc)[4][2], uint2 &xv, uint2 &side) {
        constexpr bool TT = decltype(tt)::value;
        load_slot_b1<QT, 0>(a, s, wq[0], sc[0]);
        load_slot_b1<QT, 1>(a, s, wq[1], sc[1]);
        if constexpr (TT) {
          load_slot_b1<QT, 2>(a, s, wq[2], sc[2]);
          load_slot_b1<QT, 3>(a, s, wq[3], sc[3]);
        }
        xv = lds64(xs_lane + (uint32_t)(gbp * 128));
        side = lds64(sb_lane + (uint32_t)(gbp * 16));
      };
      auto math = [&](auto tt, const uint32_t (&wq)[4][6], const uint32_t (&sc)[4][2], const uint2 &xv, const uint2 &side) {
        constexpr bool TT = decltype(tt)::value;
        const float sv = __uint_as_float(side.x);
        const int off = G::Q4 ? (int)side.y : 0;
        const bool ev = g < 4;
        const uint32_t b_lo0 = ev ? xv.x : 0u, b_lo1 = ev ? 0u : xv.x;  // MMA 1: low halves of both blocks
        const uint32_t b_hi0 = ev ? xv.y : 0u, b_hi1 = ev ? 0u : xv.y;  // MMA 2: high halves
#pragma unroll
        for (int mt = 0; mt < (TT ? 2 : 1); ++mt) {
          uint32_t ae[2][2], ao[2][2];
          expand<QT>(wq[mt * 2], ae[0], ao[0]);
          expand<QT>(wq[mt * 2 + 1], ae[1], ao[1]);
          int cc[4];
          mma_i8<G::Q4>(cc, ae[0][0], ae[1][0], ao[0][0], ao[1][0], b_lo0, b_lo1);
          mma_i8_acc<G::Q4>(cc, ae[0][1], ae[1][1], ao[0][1], ao[1][1], b_hi0, b_hi1);
          const float f0 = (float)(cc[0] + (cc[1] << 8) - off), f1 = (float)(cc[2] + (cc[3] << 8) - off);
          acc[mt][0] = fmaf(half_bits_to_float(sc[mt * 2][0]) * sv, f0, acc[mt][0]);
          acc[mt][1] = fmaf(half_bits_to_float(sc[mt * 2 + 1][0]) * sv, f1, acc[mt][1]);
        }
      };
      // both m-tiles always: rows of a tile that is not this CTA's are computed on whatever the stage
      // holds and never stored
      for (int p = warp; 2 * p < nb; p += CW, aw += CW * PAIRB, as += CW * PAIRB, gb += 2 * CW) {
        uint32_t wa[4][6], sa[4][2];
        uint2 xa, sda;
        fetch(std::true_type{}, aw, as, gb, wa, sa, xa, sda);
        math(std::true_type{}, wa, sa, xa, sda);
      }
    } else {
      for (int p = warp; 2 * p < nb; p += CW, aw += CW * PAIRB, as += CW * PAIRB, gb += 2 * CW) {
        uint32_t wq[4][6], sc[4][2];
        load_slot<QT, 0>(aw, as, wq[0], sc[0]);
        load_slot<QT, 1>(aw, as, wq[1], sc[1]);
        load_slot<QT, 2>(aw, as, wq[2], sc[2]);
        load_slot<QT, 3>(aw, as, wq[3], sc[3]);
        uint2 xe = make_uint2(0, 0), xo = make_uint2(0, 0);
        if (col_live) {
          xe = lds64(xs_lane + (uint32_t)(gb * S * 32));
          xo = lds64(xs_lane + (uint32_t)((gb + 1) * S * 32));
        }
        float se = 0.0f, so = 0.0f;
        int offe = 0, offo = 0;
        if (acc_live) {
          const uint2 sde = lds64(sb_lane + (uint32_t)(gb * P.batch * 16));
          const uint2 sdo = lds64(sb_lane + (uint32_t)((gb + 1) * P.batch * 16));
          se = __uint_as_float(sde.x);
          so = __uint_as_float(sdo.x);
          if constexpr (G::Q4) {
            offe = (int)sde.y;
            offo = (int)sdo.y;
          }
        }
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          if (mt == 1 && !two_tiles) break;
          uint32_t ae[2][2], ao[2][2];
          expand<QT>(wq[mt * 2], ae[0], ao[0]);
          expand<QT>(wq[mt * 2 + 1], ae[1], ao[1]);
          int ce[4], co[4];
          mma_i8<G::Q4>(ce, ae[0][0], ae[1][0], ae[0][1], ae[1][1], xe.x, xe.y);
          mma_i8<G::Q4>(co, ao[0][0], ao[1][0], ao[0][1], ao[1][1], xo.x, xo.y);
          // this lane's two columns are digit 2j and 2j+1 of one batch: fold them exactly
          const float fe0 = (float)(ce[0] + (ce[1] << 8) - offe), fe1 = (float)(ce[2] + (ce[3] << 8) - offe);
          const float fo0 = (float)(co[0] + (co[1] << 8) - offo), fo1 = (float)(co[2] + (co[3] << 8) - offo);
          acc[mt][0] = fmaf(half_bits_to_float(sc[mt * 2][0]) * se, fe0, acc[mt][0]);
          acc[mt][1] = fmaf(half_bits_to_float(sc[mt * 2 + 1][0]) * se, fe1, acc[mt][1]);
          acc[mt][0] = fmaf(half_bits_to_float(sc[mt * 2][1]) * so, fo0, acc[mt][0]);
          acc[mt][1] = fmaf(half_bits_to_float(sc[mt * 2 + 1][1]) * so, fo1, acc[mt][1]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[stage]);

    if (c == n_chunks - 1) {
      // ---- end of a row group: one value per row (and batch column) from this warp into the
      // group's buffer, then on to the next group; the epilogue warp does the rest
      const int buf = grp & 1;
      if (grp >= 2) mbar_wait_bounded(&red_free[buf], (uint32_t)(((grp >> 1) - 1) & 1), dead, P.status);
      float *rb = red + ((size_t)buf * CW + warp) * R * NB;
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int hs = 0; hs < 2; ++hs) {
          float v = acc[mt][hs] * fold;  // low digits + 65536 * high digits
          acc[mt][hs] = 0.0f;
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          if constexpr (B1) {
            v += __shfl_xor_sync(0xffffffffu, v, 2);  // even block + odd block
            if (t == 0) rb[mt * 16 + hs * 8 + g] = v;
          } else {
            if ((t & 1) == 0) rb[(mt * 16 + hs * 8 + g) * NB + (t >> 1)] = v;
          }
        }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_full[buf]);
    }
    if (++c == n_chunks) {
      c = 0;
      ++grp;
    }
    if (++stage == stages) {
      stage = 0;
      phase ^= 1u;
    }
  }
  if (ctid == 0) trace_stamp(P.trace, 3, tr_first, tr_last);  // last weight stage consumed
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
cudaError_t make_map(CUtensorMap *map, const uint8_t *w, int rows, size_t row_bytes, int pitch) {
  EncodeFn fn = encode_fn();
  if (!fn) return cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 8), (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(pitch / 8), (cuuint32_t)BOXR};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t *>(w), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <int QT, bool B1, bool XQ>
cudaError_t launch_t(const GemvI8Args &a, const LaunchCfg &cfg) {
  using G = Geo<QT>;
  Params P{};
  for (int i = 0; i < 3; ++i) P.seg_rows[i] = a.seg_rows[i];
  P.nseg = a.nseg;
  const int EPI = a.epi;
  P.epi = a.epi;
  if (EPI == EPI_SWIGLU) {
    P.n_rows = a.seg_rows[0];
  } else {
    P.n_rows = 0;
    for (int i = 0; i < a.nseg; ++i) P.n_rows += a.seg_rows[i];
  }
  P.kb = a.k / 32;
  P.x = a.x;
  P.ldx = a.ldx;
  P.col_map = a.col_map;
  P.norm_w = a.norm_w;
  P.eps = a.eps;
  P.batch = a.batch;
  P.y = a.y;
  P.ldy = a.ldy;
  P.status = cfg.status;
  P.trace = cfg.trace;
  P.xq = a.xq;
  P.xq_norm = a.xq_norm ? 1 : 0;
  P.pack_out = a.pack_out;
  P.pack_w = a.pack_w;
  P.pack_q4 = a.pack_type == RG_TYPE_Q4_0 ? 1 : 0;
  P.xq_fix = a.xq_fix;
  P.xq_nfix = a.xq_fix ? a.xq_nfix : 0;
  for (int i = 0; i < 3; ++i) {
    const bool ok = a.next_w[i] && (reinterpret_cast<uintptr_t>(a.next_w[i]) & 15) == 0;
    P.pf[i] = ok ? a.next_w[i] : nullptr;
    P.pf_bytes[i] = ok ? (uint32_t)(a.next_bytes[i] > 0xFFFFFFF0u ? 0xFFFFFFF0u : a.next_bytes[i]) & ~15u : 0u;
  }
  P.rows_per_cta = qgemv_i8_rows_per_cta(P.n_rows, cfg.sm_count, EPI == EPI_RESIDUAL && a.pack_out != nullptr);
  const int grid = (P.n_rows + P.rows_per_cta - 1) / P.rows_per_cta;
  const int S = 4 * a.batch;
  const int fixed = HDR_BYTES + RED_BYTES + ((P.kb * S * 32 + 127) & ~127) + ((P.kb * a.batch * 16 + 127) & ~127);
  const int stage_bytes = R * G::RS;
  int stages = (SMEM_LIMIT - fixed) / stage_bytes;
  if (stages < 3) stages = (SMEM_FULL - fixed) / stage_bytes;  // too large to share an SM: take it whole
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) return cudaErrorInvalidConfiguration;
  P.stages = stages;
  const size_t smem = (size_t)fixed + (size_t)stages * stage_bytes;

  alignas(64) CUtensorMap maps[3];
  const size_t row_bytes = (size_t)P.kb * G::BB;
  for (int i = 0; i < 3; ++i) {
    const int src = i < a.nseg ? i : 0;
    cudaError_t e = make_map(&maps[i], a.w[src], a.seg_rows[src], row_bytes, G::RS);
    if (e != cudaSuccess) return e;
  }
  auto kernel = qgemv_i8_kernel<QT, B1, XQ>;
  static DeviceOnce attr_once;  // per instantiation and device
  bool *attr_flag = attr_once.slot();
  if (!attr_flag || !*attr_flag) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_FULL);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    if (attr_flag) *attr_flag = true;
  }
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3((unsigned)grid);
  lc.blockDim = dim3(THREADS);
  lc.dynamicSmemBytes = smem;
  lc.stream = cfg.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = cfg.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&lc, kernel, maps[0], maps[1], maps[2], P);
}

template <int QT>
cudaError_t launch_e(const GemvI8Args &a, const LaunchCfg &cfg) {
  if (a.epi != EPI_STORE && a.epi != EPI_RESIDUAL && a.epi != EPI_SWIGLU) return cudaErrorInvalidValue;
  if (a.batch != 1) return launch_t<QT, false, false>(a, cfg);
  return a.xq ? launch_t<QT, true, true>(a, cfg) : launch_t<QT, true, false>(a, cfg);
}

}  // namespace

bool qgemv_i8_supported(int k, int batch) {
  // resident activations: digits (4 bytes per element and batch row) + block scales must leave
  // room for at least three weight stages
  return k > 0 && k % 256 == 0 && batch >= 1 && batch <= 2 && (size_t)k * 4 * batch <= 120 * 1024;
}

int qgemv_i8_rows_per_cta(int n_rows, int sm_count, bool whole_blocks) {
  const int sms = sm_count > 0 ? sm_count : 148;
  const int boxes = (n_rows + BOXR - 1) / BOXR;
  int rows = ((boxes + sms - 1) / sms) * BOXR;
  if (whole_blocks) rows = (rows + 31) & ~31;  // a residual epilogue that packs owns whole 32-element blocks
  return rows;
}

size_t qgemv_i8_xq_bytes(int k) {
  const int kb = k / 32;
  return xq_ssq_offset(kb) + (((size_t)kb * 4 + 127) & ~(size_t)127);
}

cudaError_t launch_qgemv_i8(const GemvI8Args &a, const LaunchCfg &cfg) {
  if (!qgemv_i8_supported(a.k, a.batch) || a.nseg < 1 || a.nseg > 3 || (!a.x && !a.xq) || !a.y) return cudaErrorInvalidValue;
  if (a.xq && (a.batch != 1 || (reinterpret_cast<uintptr_t>(a.xq) & 127) || (a.xq_fix && a.xq_nfix > 0 && !a.x)))
    return cudaErrorInvalidValue;
  if (a.pack_out) {  // only the residual epilogue of a batch-1 step packs, and only whole blocks
    int rows = 0;
    for (int i = 0; i < a.nseg; ++i) rows += a.seg_rows[i];
    if (a.epi == EPI_SWIGLU) rows = a.seg_rows[0];
    if ((a.epi != EPI_RESIDUAL && a.epi != EPI_SWIGLU) || a.batch != 1 || rows % 32 || (reinterpret_cast<uintptr_t>(a.pack_out) & 127) ||
        (a.pack_type != RG_TYPE_Q4_0 && a.pack_type != RG_TYPE_Q8_0))
      return cudaErrorInvalidValue;
  }
  count_launch(LC_QGEMV_I8);
  if (a.epi == EPI_SWIGLU && (a.nseg != 2 || a.seg_rows[0] != a.seg_rows[1])) return cudaErrorInvalidValue;
  for (int i = 0; i + 1 < a.nseg; ++i)
    if (a.epi != EPI_SWIGLU && a.seg_rows[i] % BOXR) return cudaErrorInvalidValue;
  for (int i = 0; i < a.nseg; ++i)
    if ((reinterpret_cast<uintptr_t>(a.w[i]) & 15) != 0) return cudaErrorInvalidValue;
  if (a.type == RG_TYPE_Q4_0) return launch_e<RG_TYPE_Q4_0>(a, cfg);
  if (a.type == RG_TYPE_Q8_0) return launch_e<RG_TYPE_Q8_0>(a, cfg);
  return cudaErrorInvalidValue;
}

}  // namespace rg
