// Weight-streaming GEMV for 3..16 batch rows on Q4_0 weights kept in their native GGML block bytes.
// Semantics as launch_qgemv: QuantizedMatmulPlan::execute (src/matmul/quantized.rs:126-182) and the
// per-layer linears of a batched decode step (src/models/transformer/batch.rs:177-325,
// src/models/transformer/layer.rs:445-448).
//
// The packed activations of B rows take 128 * B bytes per 32-element block against 18 bytes of one
// weight row, so what a kernel of this shape moves out of L2 is decided by how many weight rows
// share one copy of the activations.  Here a CTA owns a tile of up to 256 weight rows and a
// contiguous range of K:
//   * a producer warp streams [16 * nw rows] x [8 blocks] of raw block bytes per stage with tiled
//     2-D TMA boxes of 8 rows (row pitch 144 bytes: the eight rows a warp reads at one K offset sit
//     in distinct banks) together with the matching 8-block slice of the packed activations, which
//     every warp of the CTA then shares; 4-6 stages deep, weights of the first stages are requested
//     before the grid dependency wait;
//   * consumer warp w owns rows [16 w, 16 w + 16) of the tile for the CTA's whole K range: nibbles
//     become exact f16 integers (one logic op + one half2 op per two weights), m16n8k16 MMAs
//     against the activation columns (hi and lo f16 part of each batch row side by side), and the
//     f16 block scale multiplies the per-block result into f32 accumulators that stay in registers.
//     No partial sum crosses warps inside the CTA;
//   * EPI_SWIGLU tiles interleave 8 gate rows and 8 up rows per warp, so gate and up of one output
//     meet in one thread;
//   * matrices with few rows split K over CTAs: every CTA writes its partial tile to scratch in the
//     threads' own layout, and the CTA that arrives last at the tile's counter adds the slices in
//     slice order (a fixed order: the result does not depend on which CTA does it) and runs the
//     epilogue.  Nothing waits for another CTA.
//   * Every mbarrier wait is bounded; on expiry the kernel records a status and finishes.
#include <cuda.h>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int CW = 16;    // consumer warps: one m16 row tile each
constexpr int BOXR = 8;   // rows per TMA box
constexpr int KC = 8;     // blocks per stage
constexpr int BB = 18;    // bytes per Q4_0 block
constexpr int RS = KC * BB;  // 144: row pitch of a stage; 36 words, so rows g = 0..7 start 4 banks apart
constexpr int MAX_STAGES = 6;
constexpr int THREADS = (CW + 1) * 32;
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int HDR = 128;
static_assert(RS % 16 == 0 && (BOXR * RS) % 128 == 0, "TMA box geometry");

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
  int stages;
  int *status;
  int nw;       // warps that own rows: the tile has 16 * nw stage rows
  int tiles;    // row tiles
  int slices;   // K slices per tile
  int cps;      // stage chunks per slice
  float *scratch;      // [tiles * slices][CW * 32][2 * NT * 2] partial sums when slices > 1
  unsigned *counters;  // [tiles], zero between launches
};

__device__ __forceinline__ void unpack_q4(uint32_t q, uint32_t (&p)[4]) {
  // low nibbles: (1024 | n) - 1032; high nibbles in place: (1024 | 16 n) / 16 - 72
  const uint32_t MLO = 0x000F000Fu, MHI = 0x00F000F0u, E = 0x64006400u;
  const uint32_t SUB = 0x64086408u, SIXTEENTH = 0x2C002C00u, NEG72 = 0xD480D480u;
  const uint32_t qs = q >> 8;
  p[0] = hsub2_u32((q & MLO) | E, SUB);
  p[1] = hsub2_u32((qs & MLO) | E, SUB);
  p[2] = hfma2_u32((q & MHI) | E, SIXTEENTH, NEG72);
  p[3] = hfma2_u32((qs & MHI) | E, SIXTEENTH, NEG72);
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void tma_box_2d(uint32_t smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_dst),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

template <int NT, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
    qgemv_rows_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                      const __grid_constant__ CUtensorMap map2, const KParams P) {
  constexpr bool PAIR = (EPI == EPI_SWIGLU);
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + MAX_STAGES;
  volatile int *dead = reinterpret_cast<volatile int *>(empty + MAX_STAGES);
  volatile int *last_flag = dead + 1;
  const int w_stage_bytes = 16 * P.nw * RS;
  const int stage_bytes = (w_stage_bytes + KC * P.S * 64 + 127) & ~127;
  const uint32_t stage0 = smem_u32(smem + HDR);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_rows = (PAIR ? 8 : 16) * P.nw;  // virtual rows per tile
  const int n_chunks = (P.kb + KC - 1) / KC;
  const int units = P.tiles * P.slices;
  const int stages = P.stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CW);
    }
    *dead = 0;
    *last_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == CW) {
    // ------------------------------------------------------------------ producer
    // lane i < 2 nw moves box i: stage rows [8 i, 8 i + 8)
    auto issue = [&](int stage, int tile, int c, bool do_w, bool do_x) {
      const int nb = min(KC, P.kb - c * KC);
      const uint32_t xbytes = (uint32_t)(nb * P.S * 64);
      const uint32_t sw = stage0 + (uint32_t)stage * (uint32_t)stage_bytes;
      if (do_w) {
        if (lane == 0) mbar_expect_tx(&full[stage], (uint32_t)w_stage_bytes + xbytes);
        __syncwarp();
        if (lane < 2 * P.nw) {
          const CUtensorMap *map = &map0;
          int row;
          if (PAIR) {
            map = (lane & 1) ? &map1 : &map0;
            row = tile * tile_rows + (lane >> 1) * BOXR;
          } else {
            row = tile * tile_rows + lane * BOXR;
            if (P.nseg > 1 && row >= P.seg_rows[0]) {
              row -= P.seg_rows[0];
              map = &map1;
              if (P.nseg > 2 && row >= P.seg_rows[1]) {
                row -= P.seg_rows[1];
                map = &map2;
              }
            }
          }
          // x in 8-byte elements; rows or bytes outside the tensor arrive as zeros
          tma_box_2d(sw + (uint32_t)(lane * BOXR * RS), map, c * (RS / 8), row, &full[stage]);
        }
      }
      if (do_x && lane == 0)
        bulk_g2s(smem + HDR + (size_t)stage * stage_bytes + w_stage_bytes, P.xpack + (size_t)c * KC * P.S * 64, xbytes,
                 &full[stage]);
    };
    // the CTA's (unit, chunk) sequence
    int u = blockIdx.x, c = 0, c_end = 0;
    auto open_unit = [&]() {
      if (u < units) {
        const int slice = u % P.slices;
        c = slice * P.cps;
        c_end = min(n_chunks, c + P.cps);
      }
    };
    auto next = [&]() {
      if (++c >= c_end) {
        u += gridDim.x;
        open_unit();
      }
    };
    open_unit();
    int issued = 0;
    for (; issued < stages && u < units; ++issued, next()) issue(issued, u / P.slices, c, true, false);  // weights do not depend on earlier kernels
    pdl_wait();
    u = blockIdx.x;
    open_unit();
    for (int i = 0; i < issued; ++i, next()) issue(i, u / P.slices, c, false, true);
    int stage = 0;
    uint32_t phase = 0;  // parity of the consumers' release being waited for
    for (; u < units; next()) {
      mbar_wait_bounded(&empty[stage], phase, dead, P.status);
      issue(stage, u / P.slices, c, true, true);
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
  const bool active = warp < P.nw;
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;

  int stage = 0;
  uint32_t phase = 0;
  const uint32_t row_off = (uint32_t)((16 * warp + g) * RS);  // row g of this warp's tile
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int tile = u / P.slices, slice = u - tile * P.slices;
    const int c_begin = slice * P.cps, c_end = min(n_chunks, c_begin + P.cps);
    for (int c = c_begin; c < c_end; ++c) {
      const int nb = min(KC, P.kb - c * KC);
      mbar_wait_bounded(&full[stage], phase, dead, P.status);
      const uint32_t sw = stage0 + (uint32_t)stage * (uint32_t)stage_bytes;
      const uint32_t sx = sw + (uint32_t)w_stage_bytes;
      if (active) {
#pragma unroll
        for (int p = 0; p < KC / 2; ++p) {
          if (2 * p < nb) {
            const uint32_t a0 = sw + row_off + (uint32_t)(p * 2 * BB), a1 = a0 + 8 * RS;
            // ---- shared loads of this block pair: quant words of rows g and g + 8, the four scales, the activations
            uint32_t wq[2][3], sc[2][2];
            wq[0][0] = lds32(a0 + 4 * t);
            wq[0][1] = lds32(a0 + 4 * t + 4);
            wq[0][2] = lds32(a0 + 4 * t + 20);
            wq[1][0] = lds32(a1 + 4 * t);
            wq[1][1] = lds32(a1 + 4 * t + 4);
            wq[1][2] = lds32(a1 + 4 * t + 20);
            sc[0][0] = lds16(a0);
            sc[0][1] = lds16(a0 + BB);
            sc[1][0] = lds16(a1);
            sc[1][1] = lds16(a1 + BB);
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
            uint32_t ae[2][4], ao[2][4];
            float de[2], dd[2];
#pragma unroll
            for (int hs = 0; hs < 2; ++hs) {
              de[hs] = half_bits_to_float(sc[hs][0]);
              dd[hs] = half_bits_to_float(sc[hs][1]);
              unpack_q4(__funnelshift_r(wq[hs][0], wq[hs][1], 16), ae[hs]);
              unpack_q4(wq[hs][2], ao[hs]);
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
              float ce[4], co[4];
              mma_16816_zero(ce, ae[0][0], ae[1][0], ae[0][1], ae[1][1], xe[j].x, xe[j].y);
              mma_16816(ce, ae[0][2], ae[1][2], ae[0][3], ae[1][3], xe[j].z, xe[j].w);
              mma_16816_zero(co, ao[0][0], ao[1][0], ao[0][1], ao[1][1], xo[j].x, xo[j].y);
              mma_16816(co, ao[0][2], ao[1][2], ao[0][3], ao[1][3], xo[j].z, xo[j].w);
              ffma2_scale(acc[j][0], acc[j][1], de[0], ce[0], ce[1]);
              ffma2_scale(acc[j][2], acc[j][3], de[1], ce[2], ce[3]);
              ffma2_scale(acc[j][0], acc[j][1], dd[0], co[0], co[1]);
              ffma2_scale(acc[j][2], acc[j][3], dd[1], co[2], co[3]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
      if (++stage == stages) {
        stage = 0;
        phase ^= 1u;
      }
    }

    // ---- this unit's sums: v[j][hs] = output of row (g + 8 hs) for batch row 4 j + t
    float v[NT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int hs = 0; hs < 2; ++hs) {
        v[j][hs] = acc[j][hs * 2] + acc[j][hs * 2 + 1] * XPACK_LO_INV;
        acc[j][hs * 2] = 0.0f;
        acc[j][hs * 2 + 1] = 0.0f;
      }
    if (P.slices > 1) {
      // partial tile to scratch in the threads' own layout; the last CTA to arrive adds the slices in order
      const int tid = threadIdx.x;  // consumers: 0 .. CW * 32 - 1
      float *mine = P.scratch + ((size_t)u * (CW * 32) + tid) * (2 * NT);
#pragma unroll
      for (int j = 0; j < NT; ++j) *reinterpret_cast<float2 *>(mine + 2 * j) = make_float2(v[j][0], v[j][1]);
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
      if (tid == 0) {
        const unsigned old = atomicAdd(P.counters + tile, 1u);
        const bool last = old == (unsigned)(P.slices - 1);
        if (last) P.counters[tile] = 0;  // ready for the next launch
        *last_flag = last ? 1 : 0;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
      const bool last = *last_flag != 0;
      asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");  // the flag may be rewritten for the next unit
      if (!last) continue;
      __threadfence();
#pragma unroll
      for (int j = 0; j < NT; ++j) v[j][0] = v[j][1] = 0.0f;
      for (int sl = 0; sl < P.slices; ++sl) {
        const float *part = P.scratch + ((size_t)(tile * P.slices + sl) * (CW * 32) + tid) * (2 * NT);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const float2 q = __ldcg(reinterpret_cast<const float2 *>(part + 2 * j));
          v[j][0] += q.x;
          v[j][1] += q.y;
        }
      }
    }
    if (!active) continue;
    // ---- epilogue
    if (PAIR) {
      const int vrow = tile * tile_rows + 8 * warp + g;
      if (vrow < P.n_rows) {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const int b = 4 * j + t;
          if (b < P.batch) xpack_store(P.ypack, P.S, b, vrow, swiglu(v[j][0], v[j][1]));
        }
      }
    } else {
#pragma unroll
      for (int hs = 0; hs < 2; ++hs) {
        const int vrow = tile * tile_rows + 16 * warp + 8 * hs + g;
        if (vrow >= P.n_rows) continue;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const int b = 4 * j + t;
          if (b >= P.batch) continue;
          float *dst = P.y + (size_t)b * P.ldy + vrow;
          if (EPI == EPI_STORE) {
            *dst = v[j][hs];
          } else {
            *dst = __fadd_rn(*dst, v[j][hs]);
          }
        }
      }
    }
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

// Packed weights [rows][row_bytes] as a 2-D tensor of 8-byte elements with a [BOXR rows][RS bytes] box.
cudaError_t make_map(CUtensorMap *map, const uint8_t *w, int rows, size_t row_bytes) {
  EncodeFn fn = encode_fn();
  if (!fn) return cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 8), (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(RS / 8), (cuuint32_t)BOXR};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t *>(w), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Tile height (16 * nw stage rows) and K slices: the plan that moves the fewest bytes per CTA, counted per stage
// chunk in units of 256 bytes (weights 9 nw, activations 2 S at half weight since they come out of L2), taller
// tiles on ties.
void plan(int n_rows, bool pair, int n_chunks, int S, int sms, bool can_split, KParams *P) {
  long best = -1;
  for (int nw = CW; nw >= 4; --nw) {
    const int tile_rows = (pair ? 8 : 16) * nw;
    const int tiles = (n_rows + tile_rows - 1) / tile_rows;
    int slices = 1, cps = n_chunks;
    if (can_split && tiles * 2 <= sms) {
      slices = sms / tiles;
      if (slices > n_chunks) slices = n_chunks;
      cps = (n_chunks + slices - 1) / slices;
      slices = (n_chunks + cps - 1) / cps;
    }
    const long units = (long)tiles * slices;
    const long waves = (units + sms - 1) / sms;
    const long cost = waves * cps * (9 * nw + S);
    if (best < 0 || cost < best) {
      best = cost;
      P->nw = nw;
      P->tiles = tiles;
      P->slices = slices;
      P->cps = cps;
    }
  }
}

template <int NT, int EPI>
cudaError_t launch_t(const GemvArgs &a, const LaunchCfg &cfg) {
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
  P.scratch = a.split_scratch;
  P.counters = a.split_counters;
  const int sms = cfg.sm_count > 0 ? cfg.sm_count : 148;
  const int n_chunks = (P.kb + KC - 1) / KC;
  const bool can_split = a.split_scratch && a.split_counters && sms <= 2 * QGEMV_ROWS_MAX_TILES;  // split tiles <= sms / 2
  plan(P.n_rows, EPI == EPI_SWIGLU, n_chunks, P.S, sms, can_split, &P);
  if (P.slices > 1 && (size_t)P.tiles * P.slices * (CW * 32) * (2 * NT) > a.split_scratch_floats) {
    P.slices = 1;
    P.cps = n_chunks;
  }
  const int units = P.tiles * P.slices;
  const int grid = units < sms ? units : sms;
  const int stage_bytes = (16 * P.nw * RS + KC * P.S * 64 + 127) & ~127;
  int stages = (SMEM_LIMIT - HDR) / stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) return cudaErrorInvalidConfiguration;
  P.stages = stages;
  const size_t smem = (size_t)HDR + (size_t)stages * stage_bytes;

  alignas(64) CUtensorMap maps[3];
  const size_t row_bytes = (size_t)P.kb * BB;
  for (int i = 0; i < 3; ++i) {
    const int src = i < a.nseg ? i : 0;
    cudaError_t e = make_map(&maps[i], a.w[src], a.seg_rows[src], row_bytes);
    if (e != cudaSuccess) return e;
  }

  auto kernel = qgemv_rows_kernel<NT, EPI>;
  static DeviceOnce attr_once;  // per instantiation and device
  bool *attr_flag = attr_once.slot();
  if (!attr_flag || !*attr_flag) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
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

template <int NT>
cudaError_t launch_e(const GemvArgs &a, const LaunchCfg &cfg) {
  switch (a.epi) {
    case EPI_STORE: return launch_t<NT, EPI_STORE>(a, cfg);
    case EPI_RESIDUAL: return launch_t<NT, EPI_RESIDUAL>(a, cfg);
    case EPI_SWIGLU: return launch_t<NT, EPI_SWIGLU>(a, cfg);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

// Opt-in (RG_B200_ROWS_GEMV=1): measured level with the older f16-MMA kernel at 16 rows and behind it at 4 and 8.
bool qgemv_rows_enabled() {
  static const bool on = [] {
    const char *v = getenv("RG_B200_ROWS_GEMV");
    return v && *v && *v != '0';
  }();
  return on;
}

bool qgemv_rows_applies(const GemvArgs &a) {
  return qgemv_rows_enabled() && a.type == RG_TYPE_Q4_0 && a.batch >= 3 && a.batch <= 16 && a.k % 256 == 0;
}

// Arguments are checked by launch_qgemv, which dispatches here.
cudaError_t launch_qgemv_rows(const GemvArgs &a, const LaunchCfg &cfg) {
  count_launch(LC_QGEMV_ROWS);
  const int nt = a.batch > 8 ? 4 : a.batch > 4 ? 2 : 1;
  return nt == 4 ? launch_e<4>(a, cfg) : nt == 2 ? launch_e<2>(a, cfg) : launch_e<1>(a, cfg);
}

}  // namespace rg
