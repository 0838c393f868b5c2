// Dequant-fused GEMV / small-batch GEMM for Q4_0 and Q8_0 weights kept in their native GGML block
// bytes (18 / 34 bytes per 32 elements), batch 1..8.  Semantics: QuantizedMatmulPlan::execute
// (src/matmul/quantized.rs:126-182) and the per-layer linear of the Llama forward
// (src/models/transformer/layer.rs:445-448).
//
// Design (HBM-bound; nothing here is reshaped to chase tensor-core flops):
//  * One persistent CTA per SM owns a contiguous slice of output rows; rows are dealt out evenly
//    so the last wave is not short.
//  * A producer warp streams [32 rows x KC blocks] of raw block bytes per stage into shared
//    memory with the TMA engine's untiled bulk copy (row pieces are contiguous, 16-byte aligned
//    because KC is a multiple of 8 blocks), 3-4 stages deep, >= 140 KB in flight per SM.  The
//    matching slice of the packed activations rides in the same stage.
//  * Eight consumer warps each take a K slice of the stage for all 32 rows.  A lane reads 4-byte
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
#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int R = 32;   // weight rows per stage: two m16 tiles
constexpr int CW = 8;   // consumer warps
constexpr int MAX_STAGES = 4;
constexpr int THREADS = (CW + 1) * 32;
constexpr int SMEM_LIMIT = 227 * 1024;

template <int QT, int NT>
struct Geo {
  static constexpr bool Q4 = (QT == RG_TYPE_Q4_0);
  static constexpr int BB = Q4 ? 18 : 34;          // bytes per block
  static constexpr int PAIR_WORDS = Q4 ? 9 : 17;   // 32-bit words per two blocks
  static constexpr int KC = (Q4 ? 64 : 32) / NT;   // blocks per stage
  static constexpr int RS = KC * BB + 16;          // padded row stride: bank = 4*row + word
  static constexpr int PPW = KC / 2 / CW;          // block pairs per consumer warp per stage
  static_assert(PPW >= 1, "stage too small for eight consumer warps");
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
};

__device__ __forceinline__ void unpack_q4(uint32_t q, uint32_t (&p)[4]) {
  const uint32_t M = 0x000F000Fu, E = 0x64006400u, OFF = 0x64086408u;  // 1024 | n, minus 1032
  p[0] = hsub2_u32((q & M) | E, OFF);
  p[1] = hsub2_u32(((q >> 8) & M) | E, OFF);
  p[2] = hsub2_u32(((q >> 4) & M) | E, OFF);
  p[3] = hsub2_u32(((q >> 12) & M) | E, OFF);
}
__device__ __forceinline__ void unpack_q8(uint32_t q, uint32_t &p0, uint32_t &p1) {
  const uint32_t OFF = 0x64806480u;  // 1024 + 128
  uint32_t u = q ^ 0x80808080u;
  p0 = hsub2_u32(prmt(u, 0x64646464u, 0x4240u), OFF);
  p1 = hsub2_u32(prmt(u, 0x64646464u, 0x4341u), OFF);
}

template <int QT, int NT, int EPI>
__global__ void __launch_bounds__(THREADS, 1) qgemv_kernel(const KParams P) {
  using G = Geo<QT, NT>;
  constexpr bool PAIR = (EPI == EPI_SWIGLU);
  constexpr int GROUP_ROWS = PAIR ? 16 : 32;  // virtual rows per stage
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + MAX_STAGES;
  volatile int *dead = reinterpret_cast<volatile int *>(empty + MAX_STAGES);
  float *red = reinterpret_cast<float *>(smem + 128);
  constexpr int RED_BYTES = CW * R * 4 * NT * 4;
  uint8_t *stage0 = smem + 128 + RED_BYTES;
  const int x_stage_bytes = G::KC * P.S * 64;
  const int stage_bytes = R * G::RS + x_stage_bytes;

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
    *dead = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == CW) {
    // ------------------------------------------------------------------ producer
    const size_t row_bytes = (size_t)P.kb * G::BB;
    auto issue = [&](int u, bool do_w, bool do_x) {
      const int stage = u % stages;
      const int grp = u / n_chunks, c = u - grp * n_chunks;
      const int nb = min(G::KC, P.kb - c * G::KC);
      const int vr0 = r_begin + grp * GROUP_ROWS;
      const uint32_t wbytes = (uint32_t)(nb * G::BB), xbytes = (uint32_t)(nb * P.S * 64);
      // shared row `lane` <- which weight row?
      const uint8_t *src = nullptr;
      int vrow = PAIR ? vr0 + (lane & 15) : vr0 + lane;
      if (vrow < r_end) {
        if (PAIR) {
          src = P.w[lane >> 4] + (size_t)vrow * row_bytes;
        } else {
          int local = vrow, seg = 0;
          while (seg + 1 < P.nseg && local >= P.seg_rows[seg]) {
            local -= P.seg_rows[seg];
            ++seg;
          }
          src = P.w[seg] + (size_t)local * row_bytes;
        }
        src += (size_t)c * G::KC * G::BB;
      }
      uint8_t *sw = stage0 + (size_t)stage * stage_bytes;
      if (do_w) {
        const int nvalid = __popc(__ballot_sync(0xffffffffu, src != nullptr));
        if (lane == 0) mbar_expect_tx(&full[stage], (uint32_t)nvalid * wbytes + xbytes);
        __syncwarp();
        if (src) bulk_g2s(sw + lane * G::RS, src, wbytes, &full[stage]);
      }
      if (do_x && lane == 0)
        bulk_g2s(sw + R * G::RS, P.xpack + (size_t)c * G::KC * P.S * 64, xbytes, &full[stage]);
    };
    const int pro = min(units, stages);
    for (int u = 0; u < pro; ++u) issue(u, true, false);  // weights do not depend on earlier kernels
    pdl_wait();
    for (int u = 0; u < pro; ++u) issue(u, false, true);
    for (int u = pro; u < units; ++u) {
      const int stage = u % stages, round = u / stages;
      mbar_wait_bounded(&empty[stage], (uint32_t)((round - 1) & 1), dead, P.status);
      issue(u, true, true);
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

  for (int u = 0; u < units; ++u) {
    const int stage = u % stages;
    const int grp = u / n_chunks, c = u - grp * n_chunks;
    const int nb = min(G::KC, P.kb - c * G::KC);
    mbar_wait_bounded(&full[stage], (uint32_t)((u / stages) & 1), dead, P.status);
    const uint8_t *sw = stage0 + (size_t)stage * stage_bytes;
    const uint4 *sx = reinterpret_cast<const uint4 *>(sw + R * G::RS);

#pragma unroll
    for (int i = 0; i < G::PPW; ++i) {
      const int p = warp * G::PPW + i;
      if (2 * p >= nb) break;
      uint4 xe[NT], xo[NT];
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int slot = 8 * j + g;
        if (slot < P.S) {
          xe[j] = sx[((2 * p) * P.S + slot) * 4 + t];
          xo[j] = sx[((2 * p + 1) * P.S + slot) * 4 + t];
        } else {
          xe[j] = make_uint4(0, 0, 0, 0);
          xo[j] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        uint32_t ae[2][4], ao[2][4];
        float de[2], dd[2];
#pragma unroll
        for (int hs = 0; hs < 2; ++hs) {
          const int row = mt * 16 + hs * 8 + g;
          const uint32_t *wr = reinterpret_cast<const uint32_t *>(sw + row * G::RS) + p * G::PAIR_WORDS;
          if (G::Q4) {
            const uint32_t w0 = wr[t], w1 = wr[t + 1], w2 = wr[5 + t];
            de[hs] = half_bits_to_float(__shfl_sync(0xffffffffu, w0, lane & ~3) & 0xffffu);
            dd[hs] = half_bits_to_float(__shfl_sync(0xffffffffu, w1, lane | 3) >> 16);
            unpack_q4(__funnelshift_r(w0, w1, 16), ae[hs]);
            unpack_q4(w2, ao[hs]);
          } else {
            const uint32_t w0 = wr[t], w1 = wr[t + 1], w2 = wr[4 + t], w3 = wr[5 + t];
            const uint32_t w4 = wr[9 + t], w5 = wr[13 + t];
            de[hs] = half_bits_to_float(__shfl_sync(0xffffffffu, w0, lane & ~3) & 0xffffu);
            dd[hs] = half_bits_to_float(__shfl_sync(0xffffffffu, w3, lane | 3) >> 16);
            unpack_q8(__funnelshift_r(w0, w1, 16), ae[hs][0], ae[hs][1]);
            unpack_q8(__funnelshift_r(w2, w3, 16), ae[hs][2], ae[hs][3]);
            unpack_q8(w4, ao[hs][0], ao[hs][1]);
            unpack_q8(w5, ao[hs][2], ao[hs][3]);
          }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          float ce[4] = {0.f, 0.f, 0.f, 0.f}, co[4] = {0.f, 0.f, 0.f, 0.f};
          mma_16816(ce, ae[0][0], ae[1][0], ae[0][1], ae[1][1], xe[j].x, xe[j].y);
          mma_16816(ce, ae[0][2], ae[1][2], ae[0][3], ae[1][3], xe[j].z, xe[j].w);
          mma_16816(co, ao[0][0], ao[1][0], ao[0][1], ao[1][1], xo[j].x, xo[j].y);
          mma_16816(co, ao[0][2], ao[1][2], ao[0][3], ao[1][3], xo[j].z, xo[j].w);
          acc[mt][j][0] = fmaf(de[0], ce[0], acc[mt][j][0]);
          acc[mt][j][1] = fmaf(de[0], ce[1], acc[mt][j][1]);
          acc[mt][j][2] = fmaf(de[1], ce[2], acc[mt][j][2]);
          acc[mt][j][3] = fmaf(de[1], ce[3], acc[mt][j][3]);
          acc[mt][j][0] = fmaf(dd[0], co[0], acc[mt][j][0]);
          acc[mt][j][1] = fmaf(dd[0], co[1], acc[mt][j][1]);
          acc[mt][j][2] = fmaf(dd[1], co[2], acc[mt][j][2]);
          acc[mt][j][3] = fmaf(dd[1], co[3], acc[mt][j][3]);
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
      const int vr0 = r_begin + grp * GROUP_ROWS;
      const int tid = threadIdx.x;
      for (int idx = tid; idx < GROUP_ROWS * NB; idx += CW * 32) {
        const int row = idx / NB, b = idx - row * NB;
        const int vrow = vr0 + row;
        if (vrow >= r_end || b >= P.batch) continue;
        float v = 0.0f;
#pragma unroll
        for (int w8 = 0; w8 < CW; ++w8) v += red[(w8 * R + row) * NB + b];
        if (EPI == EPI_STORE) {
          P.y[(size_t)b * P.ldy + vrow] = v;
        } else if (EPI == EPI_RESIDUAL) {
          float *dst = P.y + (size_t)b * P.ldy + vrow;
          *dst = __fadd_rn(*dst, v);
        } else {
          float up = 0.0f;
#pragma unroll
          for (int w8 = 0; w8 < CW; ++w8) up += red[(w8 * R + row + 16) * NB + b];
          xpack_store(P.ypack, P.S, b, vrow, swiglu(v, up));
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    }
  }
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
  const int sms = cfg.sm_count > 0 ? cfg.sm_count : 148;
  P.rows_per_cta = (P.n_rows + sms - 1) / sms;
  if (P.rows_per_cta < 1) P.rows_per_cta = 1;
  const int grid = (P.n_rows + P.rows_per_cta - 1) / P.rows_per_cta;
  const int stage_bytes = R * G::RS + G::KC * P.S * 64;
  const int fixed = 128 + CW * R * 4 * NT * 4;
  int stages = (SMEM_LIMIT - fixed) / stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) return cudaErrorInvalidConfiguration;
  P.stages = stages;
  const size_t smem = (size_t)fixed + (size_t)stages * stage_bytes;

  auto kernel = qgemv_kernel<QT, NT, EPI>;
  static bool attr_done = false;  // per instantiation
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    if (e != cudaSuccess) return e;
    attr_done = true;
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
  return cudaLaunchKernelEx(&lc, kernel, P);
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

size_t xpack_bytes(int k, int batch) { return (size_t)((k + 31) / 32 * 32) * (size_t)batch * 4; }

cudaError_t launch_qgemv(const GemvArgs &a, const LaunchCfg &cfg) {
  if (a.k <= 0 || a.k % 256 || a.batch < 1 || a.batch > 8 || a.nseg < 1 || a.nseg > 3) return cudaErrorInvalidValue;
  if (a.epi == EPI_SWIGLU && (a.nseg != 2 || a.seg_rows[0] != a.seg_rows[1])) return cudaErrorInvalidValue;
  const bool two = a.batch > 4;
  if (a.type == RG_TYPE_Q4_0) return two ? launch_e<RG_TYPE_Q4_0, 2>(a, cfg) : launch_e<RG_TYPE_Q4_0, 1>(a, cfg);
  if (a.type == RG_TYPE_Q8_0) return two ? launch_e<RG_TYPE_Q8_0, 2>(a, cfg) : launch_e<RG_TYPE_Q8_0, 1>(a, cfg);
  return cudaErrorInvalidValue;
}

}  // namespace rg
