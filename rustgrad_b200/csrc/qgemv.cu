// Dequant-fused GEMV / small-batch GEMM for Q4_0 and Q8_0 weights kept in their native GGML block
// bytes (18 / 34 bytes per 32 elements), batch 1..8.  Semantics: QuantizedMatmulPlan::execute
// (src/matmul/quantized.rs:126-182) and the per-layer linear of the Llama forward
// (src/models/transformer/layer.rs:445-448).
//
// Design (HBM-bound; nothing here is reshaped to chase tensor-core flops):
//  * One persistent CTA per SM owns a contiguous slice of output rows (dealt out in 8-row units
//    so the last wave is not short).
//  * A producer warp streams [32 rows x KC blocks] of raw block bytes per stage into shared
//    memory with tiled 2-D TMA (`cp.async.bulk.tensor.2d`, one request per 8 rows; the weight
//    matrix is described as [rows][row bytes / 8] 64-bit elements), 3-6 stages deep.  KC is chosen
//    so that the dense box pitch is 12, 20 or 28 banks (mod 32): the eight rows a warp reads at
//    the same K offset fall in distinct banks without padding.  The matching slice of the packed
//    activations rides in the same stage as one untiled bulk copy.
//  * Consumer warps each take block pairs of the stage for all 32 rows.  A lane reads 4-byte
//    words of quant bytes (the 2-byte scale in front of every block makes half of them
//    unaligned: two aligned words + funnel shift), expands nibbles / int8 to exact f16 integers
//    with one logic op + one half2 subtract per two weights, and feeds them as the A operand of
//    m16n8k16 MMAs.  The B operand is the activation split in two f16 parts (hi, lo*2048) in
//    adjacent columns, so products are exact and accumulation is f32: the result carries ~22
//    bits of the f32 activation at the cost of no extra weight traffic, for any batch <= 4
//    (<= 8 with two column tiles).
//  * The f16 block scale multiplies the per-block accumulator (4 FMAs per 16 rows x 32 k).
//  * Cross-warp K reduction in shared memory in fixed order (deterministic), then the epilogue:
//    plain store, residual add, or SwiGLU of a (gate,up) row pair written directly as the next
//    GEMV's packed activations.
//  * Programmatic dependent launch: weight prefetch of the first stages is issued before the
//    grid dependency wait, so it overlaps the tail of the previous kernel.
//  * Every mbarrier wait is bounded; on expiry the kernel records a status and finishes.
#include <cuda.h>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int R = 32;     // weight rows per stage: two m16 tiles
constexpr int BOXR = 8;   // rows per TMA box: BOXR * pitch is a multiple of 128 bytes (TMA destination alignment)
constexpr int CW = 14;    // consumer warps
constexpr int MAX_STAGES = 6;
constexpr int THREADS = (CW + 1) * 32;
constexpr int SMEM_LIMIT = 227 * 1024;

template <int QT, int NT>
struct Geo {
  static constexpr bool Q4 = (QT == RG_TYPE_Q4_0);
  static constexpr int BB = Q4 ? 18 : 34;         // bytes per block
  static constexpr int PAIR_WORDS = Q4 ? 9 : 17;  // 32-bit words per two blocks
  // blocks per stage; pitch = KC * BB bytes: 1008 (28 banks), 432 (12), 1360 (20), 816 (12)
  static constexpr int KC = NT == 1 ? (Q4 ? 56 : 40) : 24;
  static constexpr int RS = KC * BB;  // dense box pitch in shared memory
  static_assert(RS % 16 == 0 && (BOXR * RS) % 128 == 0 && RS / 8 <= 256, "box inner extent must be 16-byte granular and <= 256 elements");
  static_assert(((RS / 4) % 32) % 4 == 0 && ((RS / 4) % 32) % 8 != 0, "pitch must spread eight rows over distinct banks");
};

struct KParams {
  const uint8_t *w[3];
  int seg_rows[3];
  int nseg;
  int n_rows;  // virtual rows (EPI_SWIGLU: rows of the gate matrix)
  int kb;      // K / 32
  const uint8_t *xpack;
  int S;  // 2 * batch
  int batch;
  float *y;
  int ldy;
  __half *ypack;
  int rows_per_cta;
  int stages;
  int *status;
  // deferred RMSNorm (see GemvArgs)
  __half *pack_next;
  const float *pack_w;
  float *ssq_out;
  const float *ssq_in;
  int ssq_n;
  float norm_eps;
};
constexpr int STATIC_SMEM = 2304;  // sq_s, inv_s, inv_bar below (rounded up)

// Eight nibbles of one 32-bit word -> four half2 registers of exact integers (n - 8).
// Low nibbles: (1024 | n) - 1032.  High nibbles stay in place: (1024 | 16 n) * (1/16) - 72, one
// half2 FMA, so only the odd bytes need a shift.  5 logic ops + 4 half2 ops per 8 weights.
__device__ __forceinline__ void unpack_q4(uint32_t q, uint32_t (&p)[4]) {
  const uint32_t MLO = 0x000F000Fu, MHI = 0x00F000F0u, E = 0x64006400u;
  const uint32_t SUB = 0x64086408u, SIXTEENTH = 0x2C002C00u, NEG72 = 0xD480D480u;
  const uint32_t qs = q >> 8;
  p[0] = hsub2_u32((q & MLO) | E, SUB);
  p[1] = hsub2_u32((qs & MLO) | E, SUB);
  p[2] = hfma2_u32((q & MHI) | E, SIXTEENTH, NEG72);
  p[3] = hfma2_u32((qs & MHI) | E, SIXTEENTH, NEG72);
}
__device__ __forceinline__ void unpack_q8(uint32_t q, uint32_t &p0, uint32_t &p1) {
  const uint32_t OFF = 0x64806480u;  // 1024 + 128
  uint32_t u = q ^ 0x80808080u;
  p0 = hsub2_u32(prmt(u, 0x64646464u, 0x4240u), OFF);
  p1 = hsub2_u32(prmt(u, 0x64646464u, 0x4341u), OFF);
}

// Explicit shared-memory loads with immediate offsets: one address register per block pair.
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
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// Row slot rs of a stage is shared row (rs >> 1) * 16 + (rs & 1) * 8 + g; `a` already points at
// (row g, word t) of the block pair.
template <int RS, int RSLOT>
__device__ __forceinline__ void lds_q4_slot(uint32_t a, uint32_t (&w)[6]) {
  constexpr int R0 = ((RSLOT >> 1) * 16 + (RSLOT & 1) * 8) * RS;
  w[0] = lds32<R0>(a);
  w[1] = lds32<R0 + 4>(a);
  w[2] = lds32<R0 + 20>(a);
}
template <int RS, int RSLOT>
__device__ __forceinline__ void lds_q8_slot(uint32_t a, uint32_t (&w)[6]) {
  constexpr int R0 = ((RSLOT >> 1) * 16 + (RSLOT & 1) * 8) * RS;
  w[0] = lds32<R0>(a);
  w[1] = lds32<R0 + 4>(a);
  w[2] = lds32<R0 + 16>(a);
  w[3] = lds32<R0 + 20>(a);
  w[4] = lds32<R0 + 36>(a);
  w[5] = lds32<R0 + 52>(a);
}
template <int RS, int BB, int RSLOT>
__device__ __forceinline__ void lds_scale_slot(uint32_t a, uint32_t (&sc)[2]) {
  constexpr int R0 = ((RSLOT >> 1) * 16 + (RSLOT & 1) * 8) * RS;
  sc[0] = lds16<R0>(a);
  sc[1] = lds16<R0 + BB>(a);
}

__device__ __forceinline__ void tma_box_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

template <int QT, int NT, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
    qgemv_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                 const __grid_constant__ CUtensorMap map2, const KParams P) {
  using G = Geo<QT, NT>;
  constexpr bool PAIR = (EPI == EPI_SWIGLU);
  constexpr int GROUP_ROWS = PAIR ? 16 : 32;  // virtual rows per stage
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + MAX_STAGES;
  volatile int *dead = reinterpret_cast<volatile int *>(empty + MAX_STAGES);
  float *red = reinterpret_cast<float *>(smem + 128);
  constexpr int RED_BYTES = CW * R * 4 * NT * 4;
  static_assert(RED_BYTES % 128 == 0, "stage buffers must stay 128-byte aligned");
  uint8_t *stage0 = smem + 128 + RED_BYTES;
  constexpr int W_STAGE_BYTES = R * G::RS;
  const int x_stage_bytes = G::KC * P.S * 64;
  const int stage_bytes = (W_STAGE_BYTES + x_stage_bytes + 127) & ~127;

  __shared__ float sq_s[R][16];  // squares of the new residual rows of a group, per batch column
  __shared__ float inv_s[16];    // 1 / rms of this launch's input, per batch column
  __shared__ __align__(8) uint64_t inv_bar;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r_begin = blockIdx.x * P.rows_per_cta;
  const int r_end = min(P.n_rows, r_begin + P.rows_per_cta);
  const int n_groups = (r_end > r_begin) ? (r_end - r_begin + GROUP_ROWS - 1) / GROUP_ROWS : 0;
  const int n_chunks = (P.kb + G::KC - 1) / G::KC;
  const int units = n_groups * n_chunks;
  const int stages = P.stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CW);
    }
    mbar_init(&inv_bar, 1);
    *dead = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == CW) {
    // ------------------------------------------------------------------ producer
    // lane i < 4 moves box i: shared rows [8i, 8i+8) of the stage
    auto issue = [&](int stage, int grp, int c, bool do_w, bool do_x) {
      const int nb = min(G::KC, P.kb - c * G::KC);
      const int vr0 = r_begin + grp * GROUP_ROWS;
      const uint32_t xbytes = (uint32_t)(nb * P.S * 64);
      uint8_t *sw = stage0 + (size_t)stage * stage_bytes;
      if (do_w) {
        if (lane == 0) mbar_expect_tx(&full[stage], (uint32_t)W_STAGE_BYTES + xbytes);
        __syncwarp();
        if (lane < R / BOXR) {
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
          // x coordinate in 8-byte elements; rows or bytes outside the tensor arrive as zeros
          tma_box_2d(sw + lane * BOXR * G::RS, map, c * (G::RS / 8), row, &full[stage]);
        }
      }
      if (do_x && lane == 0)
        bulk_g2s(sw + W_STAGE_BYTES, P.xpack + (size_t)c * G::KC * P.S * 64, xbytes, &full[stage]);
    };
    const int pro = min(units, stages);
    int grp = 0, c = 0;
    auto next = [&]() {
      if (++c == n_chunks) {
        c = 0;
        ++grp;
      }
    };
    for (int u = 0; u < pro; ++u, next()) issue(u, grp, c, true, false);  // weights do not depend on earlier kernels
    pdl_wait();
    grp = 0, c = 0;
    for (int u = 0; u < pro; ++u, next()) issue(u, grp, c, false, true);
    if (P.ssq_in) {
      // 1 / rms of the input rows from the producers' per-CTA sums of squares: lane b + 16 h adds the CTAs
      // h, h + 2, ...; even and odd halves meet in a fixed order.  The consumers need it at their first epilogue.
      const int b = lane & 15;
      float sum = 0.0f;
#pragma unroll 8
      for (int i = lane >> 4; i < P.ssq_n; i += 2) sum += __ldcg(P.ssq_in + i * 16 + b);
      sum += __shfl_down_sync(0xffffffffu, sum, 16);
      if (lane < 16) inv_s[lane] = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)(P.kb * 32)), P.norm_eps)));
      __syncwarp();
      if (lane == 0) mbar_arrive(&inv_bar);
    }
    int stage = 0;
    uint32_t phase = 0;  // parity of the consumers' release being waited for
    for (int u = pro; u < units; ++u, next()) {
      mbar_wait_bounded(&empty[stage], phase, dead, P.status);
      issue(stage, grp, c, true, true);
      if (++stage == stages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  pdl_wait();
  const int g = lane >> 2, t = lane & 3;
  float acc[2][NT][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][j][i] = 0.0f;

  bool inv_ready = false;
  float run_ssq = 0.0f;  // threads 0..15: sum of squares of this CTA's new residual rows, batch column tid
  // loop state kept incrementally: no integer division in the steady state
  int stage = 0, c = 0, grp = 0;
  uint32_t phase = 0;
  const uint32_t smem_stage0 = smem_u32(stage0);
  const uint32_t lane_w_off = (uint32_t)(g * G::RS + t * 4);  // (row g, word t) of pair 0
  const uint32_t lane_s_off = (uint32_t)(g * G::RS);          // scale of (row g, pair 0)
  for (int u = 0; u < units; ++u) {
    const int nb = min(G::KC, P.kb - c * G::KC);
    mbar_wait_bounded(&full[stage], phase, dead, P.status);
    const uint32_t sw = smem_stage0 + (uint32_t)stage * (uint32_t)stage_bytes;
    const uint32_t sx = sw + W_STAGE_BYTES;

    uint32_t aw = sw + lane_w_off + (uint32_t)warp * (2 * G::BB);
    uint32_t as = sw + lane_s_off + (uint32_t)warp * (2 * G::BB);
    for (int p = warp; 2 * p < nb; p += CW, aw += CW * 2 * G::BB, as += CW * 2 * G::BB) {
      // ---- all shared loads of this block pair first (explicit ld.shared, immediate offsets)
      uint32_t wq[4][6];
      uint32_t sc[4][2];
      if constexpr (G::Q4) {
        lds_q4_slot<G::RS, 0>(aw, wq[0]);
        lds_q4_slot<G::RS, 1>(aw, wq[1]);
        lds_q4_slot<G::RS, 2>(aw, wq[2]);
        lds_q4_slot<G::RS, 3>(aw, wq[3]);
      } else {
        lds_q8_slot<G::RS, 0>(aw, wq[0]);
        lds_q8_slot<G::RS, 1>(aw, wq[1]);
        lds_q8_slot<G::RS, 2>(aw, wq[2]);
        lds_q8_slot<G::RS, 3>(aw, wq[3]);
      }
      lds_scale_slot<G::RS, G::BB, 0>(as, sc[0]);
      lds_scale_slot<G::RS, G::BB, 1>(as, sc[1]);
      lds_scale_slot<G::RS, G::BB, 2>(as, sc[2]);
      lds_scale_slot<G::RS, G::BB, 3>(as, sc[3]);
      uint4 xe[NT], xo[NT];
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int slot = 8 * j + g;
        if (slot < P.S) {
          const uint32_t ax = sx + (uint32_t)((((2 * p) * P.S + slot) * 4 + t) * 16);
          xe[j] = lds128(ax);
          xo[j] = lds128(ax + (uint32_t)(P.S * 64));
        } else {
          xe[j] = make_uint4(0, 0, 0, 0);
          xo[j] = make_uint4(0, 0, 0, 0);
        }
      }
      // ---- expand and multiply
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        uint32_t ae[2][4], ao[2][4];
        float de[2], dd[2];
#pragma unroll
        for (int hs = 0; hs < 2; ++hs) {
          const int rs = mt * 2 + hs;
          de[hs] = half_bits_to_float(sc[rs][0]);
          dd[hs] = half_bits_to_float(sc[rs][1]);
          if (G::Q4) {
            unpack_q4(__funnelshift_r(wq[rs][0], wq[rs][1], 16), ae[hs]);
            unpack_q4(wq[rs][2], ao[hs]);
          } else {
            unpack_q8(__funnelshift_r(wq[rs][0], wq[rs][1], 16), ae[hs][0], ae[hs][1]);
            unpack_q8(__funnelshift_r(wq[rs][2], wq[rs][3], 16), ae[hs][2], ae[hs][3]);
            unpack_q8(wq[rs][4], ao[hs][0], ao[hs][1]);
            unpack_q8(wq[rs][5], ao[hs][2], ao[hs][3]);
          }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          float ce[4], co[4];
          mma_16816_zero(ce, ae[0][0], ae[1][0], ae[0][1], ae[1][1], xe[j].x, xe[j].y);
          mma_16816(ce, ae[0][2], ae[1][2], ae[0][3], ae[1][3], xe[j].z, xe[j].w);
          mma_16816_zero(co, ao[0][0], ao[1][0], ao[0][1], ao[1][1], xo[j].x, xo[j].y);
          mma_16816(co, ao[0][2], ao[1][2], ao[0][3], ao[1][3], xo[j].z, xo[j].w);
          // the block scales multiply two accumulator lanes at a time (packed f32x2 FMA)
          ffma2_scale(acc[mt][j][0], acc[mt][j][1], de[0], ce[0], ce[1]);
          ffma2_scale(acc[mt][j][2], acc[mt][j][3], de[1], ce[2], ce[3]);
          ffma2_scale(acc[mt][j][0], acc[mt][j][1], dd[0], co[0], co[1]);
          ffma2_scale(acc[mt][j][2], acc[mt][j][3], dd[1], co[2], co[3]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[stage]);

    if (c == n_chunks - 1) {
      // ---- cross-warp K reduction (fixed order) and epilogue for this row group
      constexpr int NB = 4 * NT;  // batch columns per row in the reduction buffer
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
          for (int hs = 0; hs < 2; ++hs) {
            const int row = mt * 16 + hs * 8 + g;
            red[(warp * R + row) * NB + 4 * j + t] = acc[mt][j][hs * 2] + acc[mt][j][hs * 2 + 1] * XPACK_LO_INV;
            acc[mt][j][hs * 2] = 0.0f;
            acc[mt][j][hs * 2 + 1] = 0.0f;
          }
      asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
      if (P.ssq_in && !inv_ready) {
        mbar_wait_bounded(&inv_bar, 0, dead, P.status);
        inv_ready = true;
      }
      const int vr0 = r_begin + grp * GROUP_ROWS;
      const int tid = threadIdx.x;
      const bool fuse_norm = EPI == EPI_RESIDUAL && P.pack_next != nullptr;
      for (int idx = tid; idx < GROUP_ROWS * NB; idx += CW * 32) {
        const int row = idx / NB, b = idx - row * NB;
        const int vrow = vr0 + row;
        if (vrow >= r_end || b >= P.batch) {
          if (fuse_norm) sq_s[row][b] = 0.0f;
          continue;
        }
        float v = 0.0f;
#pragma unroll
        for (int w8 = 0; w8 < CW; ++w8) v += red[(w8 * R + row) * NB + b];
        const float inv = P.ssq_in ? inv_s[b] : 1.0f;  // the input rows were packed without their 1 / rms
        if (P.ssq_in) v = __fmul_rn(v, inv);
        if (EPI == EPI_STORE) {
          P.y[(size_t)b * P.ldy + vrow] = v;
        } else if (EPI == EPI_RESIDUAL) {
          float *dst = P.y + (size_t)b * P.ldy + vrow;
          const float nv = __fadd_rn(*dst, v);
          *dst = nv;
          if (fuse_norm) {  // the next norm's input: weight now, 1 / rms behind the next GEMV
            xpack_store(P.pack_next, P.S, b, vrow, __fmul_rn(nv, P.pack_w[vrow]));
            sq_s[row][b] = __fmul_rn(nv, nv);
          }
        } else {
          float up = 0.0f;
#pragma unroll
          for (int w8 = 0; w8 < CW; ++w8) up += red[(w8 * R + row + 16) * NB + b];
          if (P.ssq_in) up = __fmul_rn(up, inv);
          xpack_store(P.ypack, P.S, b, vrow, swiglu(v, up));
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
      if (fuse_norm && tid < 16) {  // rows in order; the next write of sq_s comes after this thread's next barrier
        float sum = 0.0f;
        for (int row = 0; row < GROUP_ROWS; ++row) sum += sq_s[row][tid];
        run_ssq += sum;
      }
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
  if (EPI == EPI_RESIDUAL && P.ssq_out && threadIdx.x < 16)
    P.ssq_out[blockIdx.x * 16 + threadIdx.x] = (int)threadIdx.x < P.batch ? run_ssq : 0.0f;
}

// cuTensorMapEncodeTiled resolved through the runtime, so the library needs no link to libcuda.
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

// Describes packed weights [rows][row_bytes] as a 2-D tensor of 8-byte elements with a
// [BOXR rows][pitch bytes] box.
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

template <int QT, int NT, int EPI>
cudaError_t launch_t(const GemvArgs &a, const LaunchCfg &cfg) {
  using G = Geo<QT, NT>;
  KParams P{};
  for (int i = 0; i < 3; ++i) {
    P.w[i] = a.w[i];
    P.seg_rows[i] = a.seg_rows[i];
  }
  P.nseg = a.nseg;
  if (EPI == EPI_SWIGLU) {
    P.n_rows = a.seg_rows[0];
  } else {
    P.n_rows = 0;
    for (int i = 0; i < a.nseg; ++i) P.n_rows += a.seg_rows[i];
  }
  P.kb = a.k / 32;
  P.xpack = static_cast<const uint8_t *>(a.xpack);
  P.batch = a.batch;
  P.S = 2 * a.batch;
  P.y = a.y;
  P.ldy = a.ldy;
  P.ypack = static_cast<__half *>(a.ypack);
  P.status = cfg.status;
  P.pack_next = EPI == EPI_RESIDUAL ? static_cast<__half *>(a.pack_next) : nullptr;
  P.pack_w = a.pack_w;
  P.ssq_out = a.ssq_out;
  P.ssq_in = a.ssq_in;
  P.ssq_n = a.ssq_n;
  P.norm_eps = a.norm_eps;
  const int sms = cfg.sm_count > 0 ? cfg.sm_count : 148;
  // rows are dealt out in box-height units so that no TMA box straddles two CTAs or two segments
  const int units = (P.n_rows + BOXR - 1) / BOXR;
  P.rows_per_cta = ((units + sms - 1) / sms) * BOXR;
  const int grid = (P.n_rows + P.rows_per_cta - 1) / P.rows_per_cta;
  const int stage_bytes = (R * G::RS + G::KC * P.S * 64 + 127) & ~127;
  const int fixed = 128 + CW * R * 4 * NT * 4;
  int stages = (SMEM_LIMIT - STATIC_SMEM - fixed) / stage_bytes;
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

  auto kernel = qgemv_kernel<QT, NT, EPI>;
  static DeviceOnce attr_once;  // per instantiation and device
  bool *attr_flag = attr_once.slot();
  if (!attr_flag || !*attr_flag) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT - STATIC_SMEM);
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

template <int QT, int NT>
cudaError_t launch_e(const GemvArgs &a, const LaunchCfg &cfg) {
  switch (a.epi) {
    case EPI_STORE: return launch_t<QT, NT, EPI_STORE>(a, cfg);
    case EPI_RESIDUAL: return launch_t<QT, NT, EPI_RESIDUAL>(a, cfg);
    case EPI_SWIGLU: return launch_t<QT, NT, EPI_SWIGLU>(a, cfg);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

int qgemv_grid(int n_rows, int sm_count) {
  const int sms = sm_count > 0 ? sm_count : 148;
  const int units = (n_rows + BOXR - 1) / BOXR;
  const int rows_per_cta = ((units + sms - 1) / sms) * BOXR;
  return (n_rows + rows_per_cta - 1) / rows_per_cta;
}

size_t xpack_bytes(int k, int batch) { return (size_t)((k + 31) / 32 * 32) * (size_t)batch * 4; }

cudaError_t launch_qgemv(const GemvArgs &a, const LaunchCfg &cfg) {
  if (a.k <= 0 || a.k % 256 || a.batch < 1 || a.batch > 16 || a.nseg < 1 || a.nseg > 3) return cudaErrorInvalidValue;
  if (a.epi == EPI_SWIGLU && (a.nseg != 2 || a.seg_rows[0] != a.seg_rows[1])) return cudaErrorInvalidValue;
  for (int i = 0; i + 1 < a.nseg; ++i)
    if (a.epi != EPI_SWIGLU && a.seg_rows[i] % BOXR) return cudaErrorInvalidValue;  // boxes may not straddle segments
  for (int i = 0; i < a.nseg; ++i)
    if ((reinterpret_cast<uintptr_t>(a.w[i]) & 15) != 0) return cudaErrorInvalidValue;
  if (a.pack_next && (a.epi != EPI_RESIDUAL || !a.pack_w || !a.ssq_out)) return cudaErrorInvalidValue;
  if (a.ssq_in && a.ssq_n < 1) return cudaErrorInvalidValue;
  if (qgemv_rows_applies(a)) {
    if (a.pack_next || a.ssq_in) return cudaErrorInvalidValue;  // the deferred norm lives in this file's kernel only
    return launch_qgemv_rows(a, cfg);
  }
  count_launch(LC_QGEMV);
  // column tiles of four batch rows (hi and lo column each): 1, 2 or 4 tiles
  const int nt = a.batch > 8 ? 4 : a.batch > 4 ? 2 : 1;
  if (a.type == RG_TYPE_Q4_0)
    return nt == 4 ? launch_e<RG_TYPE_Q4_0, 4>(a, cfg) : nt == 2 ? launch_e<RG_TYPE_Q4_0, 2>(a, cfg) : launch_e<RG_TYPE_Q4_0, 1>(a, cfg);
  if (a.type == RG_TYPE_Q8_0)
    return nt == 4 ? launch_e<RG_TYPE_Q8_0, 4>(a, cfg) : nt == 2 ? launch_e<RG_TYPE_Q8_0, 2>(a, cfg) : launch_e<RG_TYPE_Q8_0, 1>(a, cfg);
  return cudaErrorInvalidValue;
}

}  // namespace rg
