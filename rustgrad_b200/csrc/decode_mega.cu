// One persistent kernel for a whole batch-1 decode step of the Llama forward
// (src/models/transformer/model.rs:555-760 driving layer.rs:291-470): embedding row, then per layer
// RMSNorm + QKV, RoPE + KV append + GQA attention, output projection + residual, RMSNorm + gate/up +
// SwiGLU, down projection + residual, and finally norm + head + greedy selection.
//
// Why one kernel: at batch 1 every projection is a GEMV whose HBM time is 1.4 - 10 us; launched one
// by one, each pays its own activation-packing prologue, pipeline fill and drain with the memory
// system idle in between.  Here one CTA per SM stays resident for the whole step:
//   * warp 14 is the weight producer.  It walks the step's list of projections and streams this
//     CTA's rows of each one through a ring of shared-memory slots with tiled 2-D TMA boxes.  Weights
//     are constants, so the producer never waits for a phase boundary: while the consumers sit in a
//     grid barrier or run attention, the ring fills with the next projection's tiles.
//   * warps 0-13 are consumers.  Per projection they pack the input vector to int8 digit planes
//     (RMSNorm fused), run the integer tensor-core GEMV of qgemv_i8.cu on the ring, reduce over K
//     and apply the epilogue (store / residual add / SwiGLU / logits + arg-max candidates).
//   * phases that depend on other CTAs' results are separated by a grid barrier: one global counter,
//     one arrival per CTA, bounded polling.  The kernel is launched cooperatively so that all CTAs
//     are co-resident.
//   * attention for the new token runs between the QKV and the output projection: one work item per
//     (kv head, context span); K and V spans are staged by bulk copies into the region that otherwise
//     holds the packed activations; the last item of a kv head to finish combines the spans.
// Every wait is bounded; a time-out raises a global flag that every other wait observes, the CTA
// drains its outstanding copies and the host reads the status word.
#include <cuda.h>
#include <cuda_fp16.h>
#include <math.h>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int R = 32;    // weight rows per ring slot: two m16 tiles
constexpr int BOXR = 8;  // rows per TMA box
constexpr int CW = 14;   // consumer warps
constexpr int NCONS = CW * 32;
constexpr int THREADS = NCONS + 32;
constexpr int SLOT_BYTES = 32256;  // 32 rows x 1008 bytes (56 Q4_0 blocks); Q8_0 uses 32 x 816 (24 blocks)
constexpr int MAX_SLOTS = 6;
constexpr int HD = 128;      // head dimension this kernel is written for
constexpr int MAX_G = 8;     // query heads per kv head
constexpr int SMEM_BARS = 256;
constexpr int RED_BYTES = CW * R * 4 * 4;
constexpr int QS_BYTES = MAX_G * HD * 4;
constexpr int SC_BYTES = 128 * MAX_G * 4;
constexpr uint32_t SPIN_LIMIT = 1u << 21;

template <int QT>
struct Geo {
  static constexpr bool Q4 = (QT == RG_TYPE_Q4_0);
  static constexpr int BB = Q4 ? 18 : 34;
  static constexpr int KC = Q4 ? 56 : 24;  // blocks per slot; pitch 1008 / 816 bytes (28 / 12 banks mod 32)
  static constexpr int RS = KC * BB;
  static_assert(RS % 16 == 0 && (BOXR * RS) % 128 == 0 && RS / 8 <= 256 && R * RS <= SLOT_BYTES, "TMA box geometry");
};

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
__device__ __forceinline__ float ldsf(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void tma_box_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  const int z = 0;
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}
__device__ __forceinline__ void mma_s8_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void q4_to_s8(uint32_t q, uint32_t &lo, uint32_t &hi) {
  lo = ((q << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
  hi = (q & 0xF0F0F0F0u) ^ 0x80808080u;
}
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
  sc[0] = lds16<R0>(s);  // `s` points at the scale of the block this lane scales
}
template <int QT>
__device__ __forceinline__ void expand(const uint32_t (&w)[6], uint32_t (&ae)[2], uint32_t (&ao)[2]) {
  if constexpr (Geo<QT>::Q4) {
    q4_to_s8(__funnelshift_r(w[0], w[1], 16), ae[0], ae[1]);
    q4_to_s8(w[2], ao[0], ao[1]);
  } else {
    ae[0] = __funnelshift_r(w[0], w[1], 16);
    ae[1] = __funnelshift_r(w[2], w[3], 16);
    ao[0] = w[4];
    ao[1] = w[5];
  }
}
// digit byte of element e of block kb, digit column c (batch 1: four columns)
__device__ __forceinline__ uint32_t digit_offset(int kb, int c, int e) {
  const int t = (e & 15) >> 2, r = e >> 4, i = e & 3;
  return (uint32_t)((((kb * 4 + c) * 4 + t) * 8) + r * 4 + i);
}

__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NCONS) : "memory"); }
__device__ __forceinline__ unsigned ld_relaxed(const unsigned *p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Per-CTA state of the consumer side that persists across phases.
struct Cons {
  uint64_t *full, *empty;
  volatile int *dead;  // shared: this CTA gave up
  int *gdead;          // global: some CTA gave up
  int *status;
  unsigned *bar_counter;
  unsigned bar_base;
  unsigned bar_index;  // barriers passed so far
  int stage;
  uint32_t phase;
  int slots;
  uint32_t ring;  // shared address of slot 0
  unsigned consumed;
  unsigned long long wait_ns;
  bool timed;                                 // thread 0 of CTA 0 in a profiling launch
  unsigned long long t_pack, t_main, t_epi, t_stage;  // inside projections / attention staging wait
};

// Grid barrier for the consumer warps of every CTA.  Returns false once the step is dead.
template <bool PROF>
__device__ __forceinline__ bool grid_sync(Cons &cs, int ctid) {
  cons_sync();
  cs.bar_index++;
  if (ctid == 0) {
    const unsigned long long t0 = PROF ? global_ns() : 0ull;
    // release: the CTA's writes (ordered before this thread by the barrier above) become visible
    // to whoever observes the increment; no return value, so no round trip before polling starts
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(cs.bar_counter) : "memory");
    const unsigned target = cs.bar_base + cs.bar_index * gridDim.x;
    bool ok = false;
    if (!*cs.dead) {
      for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if ((int)(ld_relaxed(cs.bar_counter) - target) >= 0) {
          ok = true;
          break;
        }
        if ((i & 255u) == 255u && *reinterpret_cast<volatile int *>(cs.gdead)) break;
        if (i > 256) __nanosleep(64);  // a late CTA: stop hammering the counter
      }
    }
    if (!ok) {
      *cs.dead = 1;
      if (!*reinterpret_cast<volatile int *>(cs.gdead)) {
        atomicExch(cs.gdead, 1);
        atomicExch(cs.status, DEV_TIMEOUT);
      }
    }
    __threadfence();
    if (PROF) cs.wait_ns += global_ns() - t0;
  }
  cons_sync();
  return *cs.dead == 0;
}

// Balanced split of a projection's 8-row boxes (pairs of boxes for gate/up) over the grid.
__device__ __forceinline__ void box_range(int n_boxes, int *b0, int *b1) {
  const long long g = gridDim.x, i = blockIdx.x;
  *b0 = (int)((i * n_boxes) / g);
  *b1 = (int)(((i + 1) * n_boxes) / g);
}

// ---------------------------------------------------------------------------------------------- producer
template <int QT>
__device__ __forceinline__ bool produce_op(const MegaOp &op, const CUtensorMap *maps, uint64_t *full, uint64_t *empty,
                                           volatile int *dead, int *status, uint8_t *ring, int slots, int &stage, int &round,
                                           unsigned &issued, int lane) {
  using G = Geo<QT>;
  const bool pair = op.epi == EPI_SWIGLU;
  const int n_boxes = (op.n_rows + BOXR - 1) / BOXR;
  int b0, b1;
  box_range(n_boxes, &b0, &b1);
  const int per_group = pair ? 2 : 4;  // virtual boxes per ring slot
  const int n_chunks = (op.kb + G::KC - 1) / G::KC;
  const CUtensorMap *m0 = maps + op.map0;
  for (int gb = b0; gb < b1; gb += per_group) {
    const int nv = min(per_group, b1 - gb);
    for (int c = 0; c < n_chunks; ++c) {
      if (round > 0 && !mbar_wait_bounded(&empty[stage], (uint32_t)((round - 1) & 1), dead, status)) return false;
      uint8_t *sw = ring + (size_t)stage * SLOT_BYTES;
      const int phys = pair ? 2 * nv : nv;
      if (lane == 0) mbar_expect_tx(&full[stage], (uint32_t)(phys * BOXR * G::RS));
      __syncwarp();
      if (lane < 4) {
        const CUtensorMap *map = m0;
        int row;
        bool live;
        if (pair) {  // shared rows 0-15: gate boxes gb, gb+1; rows 16-31: the same rows of up
          live = (lane & 1) < nv;
          row = (gb + (lane & 1)) * BOXR;
          map = m0 + (lane >> 1);
        } else {
          live = lane < nv;
          row = (gb + lane) * BOXR;
          if (op.nseg > 1 && row >= op.seg_rows[0]) {
            row -= op.seg_rows[0];
            map = m0 + 1;
            if (op.nseg > 2 && row >= op.seg_rows[1]) {
              row -= op.seg_rows[1];
              map = m0 + 2;
            }
          }
        }
        if (live) tma_box_2d(sw + lane * BOXR * G::RS, map, c * (G::RS / 8), row, &full[stage]);
      }
      ++issued;
      if (++stage == slots) {
        stage = 0;
        ++round;
      }
    }
  }
  return true;
}

// ---------------------------------------------------------------------------------------------- GEMV phase
// RMSNorm (optional) and block fixed-point packing of the input vector into shared memory:
// digits at xs, block scales at sb.  The arithmetic is that of qgemv_i8.cu.
// One lane's four consecutive elements of block kb (eight lanes per block) to digit planes + scale.
__device__ __forceinline__ void pack_block(const float (&v)[4], int kb, int quad, uint8_t *xs, float *sb) {
  float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  if (!(fabsf(v[0] + v[1] + v[2] + v[3]) <= 3.0e38f)) m = __uint_as_float(0x7f800000u);  // fmaxf drops NaN: keep it visible
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const uint32_t E = __float_as_uint(m) >> 23;  // biased exponent of the block maximum
  float s = 0.0f;
  uint32_t Y[4] = {0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u};
  if (E >= 40u && E < 255u) {
    s = __uint_as_float((E - 29u) << 23);  // 2^(floor(log2 m) - 29), so |X| < 2^30
    const float up = __uint_as_float((283u - E) << 23);
#pragma unroll
    for (int i = 0; i < 4; ++i) Y[i] = (uint32_t)__float2int_rn(v[i] * up) + 0x80808080u;
  } else if (E == 255u) {  // inf / NaN input must stay visible in the result
    s = __uint_as_float(0x7fc00000u);
    Y[0] = 0x80808081u;
  }
  const uint32_t t0 = prmt(Y[0], Y[1], 0x5140u), t1 = prmt(Y[2], Y[3], 0x5140u);
  const uint32_t t2 = prmt(Y[0], Y[1], 0x7362u), t3 = prmt(Y[2], Y[3], 0x7362u);
  uint32_t *dst = reinterpret_cast<uint32_t *>(xs + digit_offset(kb, 0, quad * 4));
  const int plane = 32 / 4;
  dst[0 * plane] = prmt(t0, t1, 0x5410u) ^ 0x80808080u;
  dst[1 * plane] = prmt(t0, t1, 0x7632u) ^ 0x80808080u;
  dst[2 * plane] = prmt(t2, t3, 0x5410u) ^ 0x80808080u;
  dst[3 * plane] = prmt(t2, t3, 0x7632u) ^ 0x80808080u;
  if (quad == 0) sb[kb] = s;
}

__device__ __forceinline__ void pack_input(const MegaOp &op, float eps, uint8_t *xs, float *sb, float *red, int ctid) {
  const int warp = ctid >> 5, lane = ctid & 31;
  const float *xr = op.x;
  const int quad = lane & 7;
  const int kb0 = warp * 4 + (lane >> 3);
  constexpr int KEEP = 4;  // blocks per thread held in registers across the norm reduction
  if (op.norm_w && op.kb <= CW * 4 * KEEP) {
    // one read of x: the values wait in registers while the sum of squares is reduced
    float4 f[KEEP], w[KEEP];
    float ss = 0.0f;
#pragma unroll
    for (int it = 0; it < KEEP; ++it) {
      const int kb = kb0 + it * CW * 4;
      if (kb < op.kb) {
        f[it] = __ldcg(reinterpret_cast<const float4 *>(xr + kb * 32) + quad);
        w[it] = __ldg(reinterpret_cast<const float4 *>(op.norm_w + kb * 32) + quad);
        ss = fmaf(f[it].x, f[it].x, ss);
        ss = fmaf(f[it].y, f[it].y, ss);
        ss = fmaf(f[it].z, f[it].z, ss);
        ss = fmaf(f[it].w, f[it].w, ss);
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    cons_sync();
    float tot = 0.0f;
#pragma unroll
    for (int wi = 0; wi < CW; ++wi) tot += red[wi];
    // y = (x * (1 / sqrt(mean(x^2) + eps))) * w, every step rounded to f32 (layer.rs:423-443)
    const float inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)(op.kb * 32)), eps)));
#pragma unroll
    for (int it = 0; it < KEEP; ++it) {
      const int kb = kb0 + it * CW * 4;
      if (kb < op.kb) {
        const float v[4] = {__fmul_rn(__fmul_rn(f[it].x, inv), w[it].x), __fmul_rn(__fmul_rn(f[it].y, inv), w[it].y),
                            __fmul_rn(__fmul_rn(f[it].z, inv), w[it].z), __fmul_rn(__fmul_rn(f[it].w, inv), w[it].w)};
        pack_block(v, kb, quad, xs, sb);
      }
    }
    cons_sync();
    return;
  }
  float inv = 1.0f;
  if (op.norm_w) {
    float ss = 0.0f;
    for (int i = ctid; i < op.kb * 8; i += NCONS) {
      const float4 f = __ldcg(reinterpret_cast<const float4 *>(xr) + i);
      ss = fmaf(f.x, f.x, ss);
      ss = fmaf(f.y, f.y, ss);
      ss = fmaf(f.z, f.z, ss);
      ss = fmaf(f.w, f.w, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    cons_sync();
    float tot = 0.0f;
#pragma unroll
    for (int wi = 0; wi < CW; ++wi) tot += red[wi];
    inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)(op.kb * 32)), eps)));
    cons_sync();
  }
#pragma unroll 4
  for (int kb = kb0; kb < op.kb; kb += CW * 4) {
    const float4 f = __ldcg(reinterpret_cast<const float4 *>(xr + kb * 32) + quad);
    float v[4] = {f.x, f.y, f.z, f.w};
    if (op.norm_w) {
      const float4 w = __ldg(reinterpret_cast<const float4 *>(op.norm_w + kb * 32) + quad);
      v[0] = __fmul_rn(__fmul_rn(v[0], inv), w.x);
      v[1] = __fmul_rn(__fmul_rn(v[1], inv), w.y);
      v[2] = __fmul_rn(__fmul_rn(v[2], inv), w.z);
      v[3] = __fmul_rn(__fmul_rn(v[3], inv), w.w);
    }
    pack_block(v, kb, quad, xs, sb);
  }
  cons_sync();
}

struct Best {
  float v;
  int idx;
  int bad;
};

template <int QT, bool PROF>
__device__ __forceinline__ void gemv_op(const MegaOp &op, float eps, Cons &cs, uint8_t *xs, float *red, int ctid, Best &best) {
  using G = Geo<QT>;
  const int warp = ctid >> 5, lane = ctid & 31;
  const bool pair = op.epi == EPI_SWIGLU;
  const int n_boxes = (op.n_rows + BOXR - 1) / BOXR;
  int b0, b1;
  box_range(n_boxes, &b0, &b1);
  if (b1 <= b0) return;
  const int per_group = pair ? 2 : 4;
  const int n_chunks = (op.kb + G::KC - 1) / G::KC;
  float *sb = reinterpret_cast<float *>(xs + op.kb * 128);
  unsigned long long tq = (PROF && cs.timed) ? global_ns() : 0ull;
  pack_input(op, eps, xs, sb, red, ctid);
  if (PROF && cs.timed) {
    const unsigned long long now = global_ns();
    cs.t_pack += now - tq;
    tq = now;
  }

  // Batch 1 leaves four of the MMA's eight columns free, so the two blocks of a pair share one
  // accumulator tile: columns 0-3 = digits of the even block (B rows k < 16), columns 4-7 = digits of
  // the odd block (k >= 16); A carries the even block in k < 16 and the odd one in k >= 16.  Lanes
  // t < 2 then scale the even block's sums, lanes t >= 2 the odd block's.
  const int g = lane >> 2, t = lane & 3;
  const int blk_sel = t >> 1;
  const bool ev = g < 4;
  float acc[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
  const uint32_t xs_lane = smem_u32(xs) + (uint32_t)(((g & 3) * 4 + t) * 8 + (g >> 2) * 128);
  const uint32_t sb_base = smem_u32(sb) + (uint32_t)(blk_sel * 4);
  const uint32_t lane_w_off = (uint32_t)(g * G::RS + t * 4);
  const uint32_t lane_s_off = (uint32_t)(g * G::RS + blk_sel * G::BB);
  const int r_end = min(op.n_rows, b1 * BOXR);
  for (int gb = b0; gb < b1; gb += per_group) {
    for (int c = 0; c < n_chunks; ++c) {
      const int nb = min(G::KC, op.kb - c * G::KC);
      mbar_wait_bounded(&cs.full[cs.stage], cs.phase, cs.dead, cs.status);
      const uint32_t sw = cs.ring + (uint32_t)cs.stage * (uint32_t)SLOT_BYTES;
      uint32_t aw = sw + lane_w_off + (uint32_t)warp * (2 * G::BB);
      uint32_t as = sw + lane_s_off + (uint32_t)warp * (2 * G::BB);
      int kb = c * G::KC + 2 * warp;
      for (int p = warp; 2 * p < nb; p += CW, aw += CW * 2 * G::BB, as += CW * 2 * G::BB, kb += 2 * CW) {
        uint32_t wq[4][6], sc[4][2];
        load_slot<QT, 0>(aw, as, wq[0], sc[0]);
        load_slot<QT, 1>(aw, as, wq[1], sc[1]);
        load_slot<QT, 2>(aw, as, wq[2], sc[2]);
        load_slot<QT, 3>(aw, as, wq[3], sc[3]);
        const uint2 xv = lds64(xs_lane + (uint32_t)(kb * 128));
        const float sv = ldsf(sb_base + (uint32_t)(kb * 4));
        const uint32_t b_lo0 = ev ? xv.x : 0u, b_lo1 = ev ? 0u : xv.x;  // low halves of both blocks
        const uint32_t b_hi0 = ev ? xv.y : 0u, b_hi1 = ev ? 0u : xv.y;  // high halves
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          uint32_t ae[2][2], ao[2][2];
          expand<QT>(wq[mt * 2], ae[0], ao[0]);
          expand<QT>(wq[mt * 2 + 1], ae[1], ao[1]);
          int c[4];
          mma_s8(c, ae[0][0], ae[1][0], ao[0][0], ao[1][0], b_lo0, b_lo1);
          mma_s8_acc(c, ae[0][1], ae[1][1], ao[0][1], ao[1][1], b_hi0, b_hi1);
          const float f0 = (float)(c[0] + (c[1] << 8)), f1 = (float)(c[2] + (c[3] << 8));
          acc[mt][0] = fmaf(half_bits_to_float(sc[mt * 2][0]) * sv, f0, acc[mt][0]);
          acc[mt][1] = fmaf(half_bits_to_float(sc[mt * 2 + 1][0]) * sv, f1, acc[mt][1]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&cs.empty[cs.stage]);
      ++cs.consumed;
      if (++cs.stage == cs.slots) {
        cs.stage = 0;
        cs.phase ^= 1u;
      }
    }
    if (PROF && cs.timed) {
      const unsigned long long now = global_ns();
      cs.t_main += now - tq;
      tq = now;
    }
    // ---- cross-warp K reduction (fixed order) and epilogue of this row group
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int hs = 0; hs < 2; ++hs) {
        red[(warp * R + mt * 16 + hs * 8 + g) * 4 + t] = acc[mt][hs];
        acc[mt][hs] = 0.0f;
      }
    cons_sync();
    constexpr float A_SCALE = G::Q4 ? 0.0625f : 1.0f;
    const int group_rows = pair ? 16 : 32;
    if (ctid < group_rows) {
      const int vrow = gb * BOXR + ctid;
      if (vrow < r_end) {
        auto total = [&](int rr) {
          float lo = 0.0f, hi = 0.0f;
#pragma unroll
          for (int w = 0; w < CW; ++w) {  // slots: even block low / high digits, odd block low / high digits
            lo += red[(w * R + rr) * 4] + red[(w * R + rr) * 4 + 2];
            hi += red[(w * R + rr) * 4 + 1] + red[(w * R + rr) * 4 + 3];
          }
          return fmaf(hi, 65536.0f, lo) * A_SCALE;
        };
        const float v = total(ctid);
        if (op.epi == EPI_STORE) {
          op.y[vrow] = v;
          if (op.flags & MEGA_OP_LOGITS) {
            if (!finite_f32(v)) best.bad = 1;
            if (v > best.v || best.idx == 0x7fffffff) {
              best.v = v;
              best.idx = vrow;
            }
          }
        } else if (op.epi == EPI_RESIDUAL) {
          op.y[vrow] = __fadd_rn(__ldcg(op.y + vrow), v);
        } else {
          op.y[vrow] = swiglu(v, total(ctid + 16));
        }
      }
    }
    cons_sync();
    if (PROF && cs.timed) {
      const unsigned long long now = global_ns();
      cs.t_epi += now - tq;
      tq = now;
    }
  }
}

// ---------------------------------------------------------------------------------------------- attention
template <typename KV>
__device__ __forceinline__ KV to_kv(float v);
template <>
__device__ __forceinline__ float to_kv<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __half to_kv<__half>(float v) {
  return __float2half_rn(v);
}
// eight / two consecutive cache elements from shared memory as f32
__device__ __forceinline__ void load8(const float *p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4 *>(p)[0], b = reinterpret_cast<const float4 *>(p)[1];
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void load8(const __half *p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4 *>(p);
  const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x, v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ float2 load2(const float *p) { return *reinterpret_cast<const float2 *>(p); }
__device__ __forceinline__ float2 load2(const __half *p) { return __half22float2(*reinterpret_cast<const __half2 *>(p)); }

// One new token of one sequence attends to positions 0..pos (src/ir/attention.rs:946-981,1157-1240
// with the mask of layer.rs:374-380).  Work item = (kv head, span of the context).
template <typename KV, bool PROF>
__device__ __forceinline__ void attention_op(const MegaOp &op, const MegaParams &P, Cons &cs, uint8_t *U, float *qs, float *sc,
                                             float *red, uint64_t *abar, uint32_t &aphase, int *flag, int pos, int seq,
                                             int ctid) {
  constexpr int SPAN_MAX = 65536 / (2 * HD * (int)sizeof(KV));  // 128 positions of f16, 64 of f32
  const int warp = ctid >> 5, lane = ctid & 31;
  const int G = P.heads / P.kv_heads;
  const int total = pos + 1;
  const int ipk = max(1, (int)gridDim.x / P.kv_heads);
  int span = (((total + ipk - 1) / ipk) + 15) & ~15;
  span = min(SPAN_MAX, max(16, span));
  const int nspl = (total + span - 1) / span;
  const int items = P.kv_heads * nspl;
  KV *kc = static_cast<KV *>(P.k_cache[op.layer]);
  KV *vc = static_cast<KV *>(P.v_cache[op.layer]);
  KV *ks = reinterpret_cast<KV *>(U);
  KV *vs = ks + (size_t)SPAN_MAX * HD;
  const int qw = P.heads * HD, kw = P.kv_heads * HD;
  const float *ct = P.cos_t + (size_t)pos * (HD / 2), *st = P.sin_t + (size_t)pos * (HD / 2);
  const float inv_scale = (float)(1.0 / (1.0 / sqrt((double)HD)));
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int kvh = item / nspl, sp = item - kvh * nspl;
    const int p0 = sp * span;
    const int np = min(span, total - p0);
    const bool has_new = (p0 + np == total);  // the span that ends with the new token
    const int ncopy = has_new ? np - 1 : np;  // the new token's row is produced here, not read
    const size_t row0 = ((size_t)seq * P.kv_heads + kvh) * P.ctx + p0;
    if (ctid == 0 && ncopy > 0) {
      // the staging region was last touched by ordinary loads and stores (packed activations)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      const uint32_t bytes = (uint32_t)((size_t)ncopy * HD * sizeof(KV));
      mbar_expect_tx(abar, 2 * bytes);
      bulk_g2s(ks, kc + row0 * HD, bytes, abar);
      bulk_g2s(vs, vc + row0 * HD, bytes, abar);
    }
    // rotate the G query heads of this kv head into shared memory (pairs (2i, 2i+1) -> (i, 64+i))
    for (int it = ctid; it < G * (HD / 2); it += NCONS) {
      const int gq = it / (HD / 2), i = it - gq * (HD / 2);
      const float2 xv = __ldcg(reinterpret_cast<const float2 *>(P.qkv + (size_t)(kvh * G + gq) * HD) + i);
      const float cs_ = __ldg(ct + i), sn = __ldg(st + i);
      qs[gq * HD + i] = __fsub_rn(__fmul_rn(xv.x, cs_), __fmul_rn(xv.y, sn));
      qs[gq * HD + HD / 2 + i] = __fadd_rn(__fmul_rn(xv.y, cs_), __fmul_rn(xv.x, sn));
    }
    if (has_new) {  // rotate and append k, append v: cache row `pos` and the last staged row
      if (ctid < HD / 2) {
        const int i = ctid;
        const float2 xv = __ldcg(reinterpret_cast<const float2 *>(P.qkv + qw + (size_t)kvh * HD) + i);
        const float cs_ = __ldg(ct + i), sn = __ldg(st + i);
        const KV y1 = to_kv<KV>(__fsub_rn(__fmul_rn(xv.x, cs_), __fmul_rn(xv.y, sn)));
        const KV y2 = to_kv<KV>(__fadd_rn(__fmul_rn(xv.y, cs_), __fmul_rn(xv.x, sn)));
        KV *g = kc + (row0 + (np - 1)) * HD, *s = ks + (size_t)(np - 1) * HD;
        g[i] = y1, g[HD / 2 + i] = y2;
        s[i] = y1, s[HD / 2 + i] = y2;
      } else if (ctid >= 64 && ctid < 64 + HD) {
        const int j = ctid - 64;
        const KV v = to_kv<KV>(__ldcg(P.qkv + qw + kw + (size_t)kvh * HD + j));
        vc[(row0 + (np - 1)) * HD + j] = v;
        vs[(size_t)(np - 1) * HD + j] = v;
      }
    }
    cons_sync();
    if (ncopy > 0) {
      const unsigned long long tq = (PROF && cs.timed) ? global_ns() : 0ull;
      mbar_wait_bounded(abar, aphase, cs.dead, cs.status);
      aphase ^= 1u;
      if (PROF && cs.timed) cs.t_stage += global_ns() - tq;
    }
    // ---- scores: 16 lanes per position, 8 dims per lane
    {
      const int sub = lane & 15, hi = lane >> 4;
      for (int gq = 0; gq < G; ++gq) {
        float qr[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) qr[i] = qs[gq * HD + sub * 8 + i];
        for (int base = 0; base < np; base += 2 * CW) {
          const int p = base + warp * 2 + hi;
          float dot = 0.0f;
          if (p < np) {
            float kr[8];
            load8(ks + (size_t)p * HD + sub * 8, kr);
#pragma unroll
            for (int i = 0; i < 8; ++i) dot = fmaf(qr[i], kr[i], dot);
          }
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
          if (sub == 0 && p < np) sc[p * MAX_G + gq] = __fdiv_rn(dot, inv_scale);
        }
      }
    }
    cons_sync();
    // ---- softmax pieces per head (attention.rs:495-558): e = exp2((s - m) * log2(e))
    float *ml = red;  // [G][2]
    if (warp < G) {
      const int gq = warp;
      float m = -INFINITY;
      for (int p = lane; p < np; p += 32) m = fmaxf(m, sc[p * MAX_G + gq]);
      m = warp_max(m);
      float l = 0.0f;
      for (int p = lane; p < np; p += 32) {
        const float e = exp2f(__fmul_rn(__fsub_rn(sc[p * MAX_G + gq], m), 1.44269504088896340736f));
        sc[p * MAX_G + gq] = e;
        l += e;
      }
      l = warp_sum(l);
      if (lane == 0) {
        ml[gq * 2] = m;
        ml[gq * 2 + 1] = l;
      }
    }
    cons_sync();
    // ---- P.V: one thread per (head, pair of dims); partial result to the scratch
    for (int o = ctid; o < G * (HD / 2); o += NCONS) {
      const int gq = o / (HD / 2), dp = o - gq * (HD / 2);
      float a0 = 0.0f, a1 = 0.0f;
      for (int p = 0; p < np; ++p) {
        const float pr = sc[p * MAX_G + gq];
        const float2 vv = load2(vs + (size_t)p * HD + 2 * dp);
        a0 = fmaf(pr, vv.x, a0);
        a1 = fmaf(pr, vv.y, a1);
      }
      float *dst = P.attn_scratch + ((size_t)(kvh * G + gq) * P.max_splits + sp) * (HD + 2);
      dst[2 + 2 * dp] = a0;
      dst[2 + 2 * dp + 1] = a1;
      if (dp == 0) {
        dst[0] = ml[gq * 2];
        dst[1] = ml[gq * 2 + 1];
      }
    }
    cons_sync();
    // ---- the last span of this kv head to finish combines all spans
    if (ctid == 0) {
      __threadfence();  // this CTA's partial results before its arrival
      const unsigned old = atomicAdd(P.attn_counters + kvh, 1u);
      const int last = (old == (unsigned)(nspl - 1));
      if (last) {
        P.attn_counters[kvh] = 0u;  // every arrival of this phase has happened
        __threadfence();            // the other spans' results before the combine reads them
      }
      *flag = last;
    }
    cons_sync();
    if (*flag) {
      for (int o = ctid; o < G * HD; o += NCONS) {
        const int gq = o / HD, d = o - gq * HD;
        const float *base = P.attn_scratch + (size_t)(kvh * G + gq) * P.max_splits * (HD + 2);
        float M = -INFINITY;
        for (int s = 0; s < nspl; ++s) M = fmaxf(M, __ldcg(base + (size_t)s * (HD + 2)));
        float L = 0.0f, acc = 0.0f;
        for (int s = 0; s < nspl; ++s) {
          const float *ps = base + (size_t)s * (HD + 2);
          const float wgt = exp2f(__fmul_rn(__fsub_rn(__ldcg(ps), M), 1.44269504088896340736f));
          L = fmaf(__ldcg(ps + 1), wgt, L);
          acc = fmaf(__ldcg(ps + 2 + d), wgt, acc);
        }
        P.attn_out[(size_t)(kvh * G + gq) * HD + d] = __fmul_rn(acc, __frcp_rn(L));
      }
    }
    cons_sync();
  }
}

// ---------------------------------------------------------------------------------------------- small phases
__device__ __forceinline__ float decode_element(int type, const uint8_t *bytes, size_t e) {
  if (type == RG_TYPE_F32) return reinterpret_cast<const float *>(bytes)[e];
  if (type == RG_TYPE_F16) return half_bits_to_float(reinterpret_cast<const uint16_t *>(bytes)[e]);
  const size_t blk = e >> 5;
  const int lane = (int)(e & 31);
  if (type == RG_TYPE_Q4_0) {
    const uint8_t *b = bytes + blk * 18;
    const float d = half_bits_to_float((uint32_t)b[0] | ((uint32_t)b[1] << 8));
    const uint8_t packed = b[2 + (lane & 15)];
    const int nib = (lane < 16) ? (packed & 0x0f) : (packed >> 4);
    return __fmul_rn(__fsub_rn((float)nib, 8.0f), d);
  }
  const uint8_t *b = bytes + blk * 34;
  const float d = half_bits_to_float((uint32_t)b[0] | ((uint32_t)b[1] << 8));
  return __fmul_rn((float)(int8_t)b[2 + lane], d);
}

template <typename KV, bool PROF>
__global__ void __launch_bounds__(THREADS, 1) decode_mega_kernel(const MegaParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + MAX_SLOTS;
  uint64_t *abar = empty + MAX_SLOTS;
  uint64_t *prod_done = abar + 1;
  volatile int *dead = reinterpret_cast<volatile int *>(prod_done + 1);
  int *flag = const_cast<int *>(dead) + 1;
  int *boot = flag + 1;                 // [0] token, [1] pos, [2] seq, [3] barrier base
  unsigned *issued_total = reinterpret_cast<unsigned *>(boot + 4);
  float *red = reinterpret_cast<float *>(smem + SMEM_BARS);
  float *qs = reinterpret_cast<float *>(smem + SMEM_BARS + RED_BYTES);
  float *sc = reinterpret_cast<float *>(smem + SMEM_BARS + RED_BYTES + QS_BYTES);
  uint8_t *U = smem + SMEM_BARS + RED_BYTES + QS_BYTES + SC_BYTES;
  uint8_t *ring = U + P.u_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P.slots; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CW);
    }
    mbar_init(abar, 1);
    mbar_init(prod_done, 1);
    *dead = 0;
    *flag = 0;
    *issued_total = 0;
    boot[0] = P.tokens[0];
    boot[1] = P.pos[0];
    boot[2] = P.seq[0];
    boot[3] = (int)__ldcg(P.bar_base);
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == CW) {
    // ------------------------------------------------------------------ producer: weights of every projection
    int stage = 0, round = 0;
    unsigned issued = 0;
    const CUtensorMap *maps = static_cast<const CUtensorMap *>(P.maps);
    for (int oi = 0; oi < P.n_ops; ++oi) {
      const MegaOp &op = P.ops[oi];
      if (op.kind != MEGA_GEMV) continue;
      const bool ok = (op.type == RG_TYPE_Q4_0)
                          ? produce_op<RG_TYPE_Q4_0>(op, maps, full, empty, dead, P.status, ring, P.slots, stage, round, issued, lane)
                          : produce_op<RG_TYPE_Q8_0>(op, maps, full, empty, dead, P.status, ring, P.slots, stage, round, issued, lane);
      if (!ok) break;
    }
    if (lane == 0) {
      *issued_total = issued;
      mbar_arrive(prod_done);
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  const int ctid = threadIdx.x;
  Cons cs;
  cs.full = full;
  cs.empty = empty;
  cs.dead = dead;
  cs.gdead = P.gdead;
  cs.status = P.status;
  cs.bar_counter = P.bar_counter;
  cs.bar_base = (unsigned)boot[3];
  cs.bar_index = 0;
  cs.stage = 0;
  cs.phase = 0;
  cs.slots = P.slots;
  cs.ring = smem_u32(ring);
  cs.consumed = 0;
  cs.wait_ns = 0;
  cs.timed = PROF && blockIdx.x == 0 && ctid == 0;
  cs.t_pack = cs.t_main = cs.t_epi = cs.t_stage = 0;
  const int token = boot[0], pos = boot[1], seq = boot[2];
  uint32_t aphase = 0;
  Best best{-INFINITY, 0x7fffffff, 0};
  unsigned long long t_kind[4] = {0, 0, 0, 0};
  bool alive = true;
  for (int oi = 0; oi < P.n_ops && alive; ++oi) {
    const MegaOp &op = P.ops[oi];
    const unsigned long long t0 = (PROF && ctid == 0) ? global_ns() : 0ull;
    if (op.kind == MEGA_EMBED) {
      // embedding row of the token (src/gguf/quantization/row_gather.rs:149-226)
      const size_t base = (size_t)token * (size_t)P.d_model;
      for (int i = blockIdx.x * NCONS + ctid; i < P.d_model; i += gridDim.x * NCONS)
        P.x[i] = decode_element(P.embed_type, P.embed, base + i);
    } else if (op.kind == MEGA_GEMV) {
      if (op.type == RG_TYPE_Q4_0) {
        gemv_op<RG_TYPE_Q4_0, PROF>(op, P.eps, cs, U, red, ctid, best);
      } else {
        gemv_op<RG_TYPE_Q8_0, PROF>(op, P.eps, cs, U, red, ctid, best);
      }
      if (op.flags & MEGA_OP_LOGITS) {
        // this CTA's arg-max candidate: lowest id wins ties (generation.rs:260-287)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, best.v, o);
          const int oi2 = __shfl_xor_sync(0xffffffffu, best.idx, o);
          best.bad |= __shfl_xor_sync(0xffffffffu, best.bad, o);
          if (ov > best.v || (ov == best.v && oi2 < best.idx)) {
            best.v = ov;
            best.idx = oi2;
          }
        }
        if (ctid == 0) {  // only warp 0 runs epilogues, so its reduction is the CTA's
          P.cand_val[blockIdx.x] = best.v;
          P.cand_idx[blockIdx.x] = best.idx;
          P.cand_bad[blockIdx.x] = best.bad;
        }
      }
    } else if (op.kind == MEGA_ATTN) {
      attention_op<KV, PROF>(op, P, cs, U, qs, sc, red, abar, aphase, flag, pos, seq, ctid);
    } else if (op.kind == MEGA_FINISH) {
      if (blockIdx.x == 0 && warp == 0) {
        float bv = -INFINITY;
        int bi = 0x7fffffff, bad = 0;
        for (int i = lane; i < (int)gridDim.x; i += 32) {
          const float v = __ldcg(P.cand_val + i);
          const int id = __ldcg(P.cand_idx + i);
          bad |= __ldcg(P.cand_bad + i);
          if (id != 0x7fffffff && (v > bv || (v == bv && id < bi) || bi == 0x7fffffff)) {
            bv = v;
            bi = id;
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
          const int oi2 = __shfl_xor_sync(0xffffffffu, bi, o);
          bad |= __shfl_xor_sync(0xffffffffu, bad, o);
          if (oi2 != 0x7fffffff && (ov > bv || (ov == bv && oi2 < bi) || bi == 0x7fffffff)) {
            bv = ov;
            bi = oi2;
          }
        }
        if (lane == 0) {
          const int id = (bad || bi == 0x7fffffff) ? -1 : bi;
          P.d_ids[0] = id;
          if (P.advance) {
            const int step = *P.step;
            P.tokens[0] = id < 0 ? 0 : id;
            P.pos[0] = pos + 1;
            if (P.history) P.history[step] = id;
            *P.step = step + 1;
          }
          // the next launch counts its barriers from where this one stopped
          *P.bar_base = cs.bar_base + cs.bar_index * gridDim.x;
        }
      }
    }
    if (PROF && ctid == 0) t_kind[op.kind & 3] += global_ns() - t0;
    if (oi + 1 < P.n_ops) alive = grid_sync<PROF>(cs, ctid);
  }
  if (!alive) {
    // a wait gave up somewhere: let this CTA's outstanding weight copies land before it exits
    if (ctid == 0) {
      for (uint32_t i = 0; i < (1u << 22); ++i)
        if (mbar_try_wait(prod_done, 0)) break;
      unsigned issued = *issued_total;
      int stage = cs.stage;
      uint32_t phase = cs.phase;
      for (unsigned u = cs.consumed; u < issued; ++u) {
        for (uint32_t i = 0; i < (1u << 20); ++i)
          if (mbar_try_wait(&full[stage], phase)) break;
        if (++stage == cs.slots) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    cons_sync();
  }
  if (PROF && ctid == 0 && blockIdx.x == 0 && P.prof) {
    P.prof[0] += t_kind[MEGA_GEMV];
    P.prof[1] += t_kind[MEGA_ATTN];
    P.prof[2] += t_kind[MEGA_EMBED] + t_kind[MEGA_FINISH];
    P.prof[3] += cs.wait_ns;
    P.prof[4] += cs.t_pack;
    P.prof[5] += cs.t_main;
    P.prof[6] += cs.t_epi;
    P.prof[7] += cs.t_stage;
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

}  // namespace

size_t mega_tensor_map_bytes() { return sizeof(CUtensorMap); }

cudaError_t mega_make_map(void *map_out, int type, const uint8_t *w, int rows, int k) {
  EncodeFn fn = encode_fn();
  if (!fn) return cudaErrorNotSupported;
  const int bb = type == RG_TYPE_Q4_0 ? 18 : 34;
  const int pitch = type == RG_TYPE_Q4_0 ? Geo<RG_TYPE_Q4_0>::RS : Geo<RG_TYPE_Q8_0>::RS;
  const size_t row_bytes = (size_t)(k / 32) * bb;
  const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 8), (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(pitch / 8), (cuuint32_t)BOXR};
  const cuuint32_t elem[2] = {1, 1};
  alignas(64) CUtensorMap m;
  const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t *>(w), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  memcpy(map_out, &m, sizeof(m));
  return cudaSuccess;
}

// Shared memory plan: barriers, reduction scratch, rotated queries, scores, the activation / KV
// staging region and as many ring slots as fit.  Returns false when fewer than three slots fit.
bool mega_plan_smem(int max_k, int *u_bytes, int *slots, size_t *smem) {
  const int need = max_k * 4 + (max_k / 32) * 4;  // digit planes + block scales of the widest input
  int u = 65536;                                  // the KV staging size
  if (need > u) u = (need + 127) & ~127;
  const int fixed = SMEM_BARS + RED_BYTES + QS_BYTES + SC_BYTES + u;
  int n = (227 * 1024 - fixed) / SLOT_BYTES;
  if (n > MAX_SLOTS) n = MAX_SLOTS;
  if (n < 3) return false;
  *u_bytes = u;
  *slots = n;
  *smem = (size_t)fixed + (size_t)n * SLOT_BYTES;
  return true;
}

int mega_max_splits(int ctx, int grid, int kv_heads, bool kv_f32) {
  const int span_max = 65536 / (2 * HD * (kv_f32 ? 4 : 2));
  const int ipk = grid / kv_heads > 1 ? grid / kv_heads : 1;
  const int by_ctx = (ctx + span_max - 1) / span_max;
  return (ipk > by_ctx ? ipk : by_ctx) + 1;
}

cudaError_t launch_decode_mega(const MegaParams &P, bool kv_f32, size_t smem, int grid, cudaStream_t stream) {
  const bool prof = P.prof != nullptr;  // the timed variant clocks its phases; the plain one carries no timers
  auto kernel = kv_f32 ? (prof ? decode_mega_kernel<float, true> : decode_mega_kernel<float, false>)
                       : (prof ? decode_mega_kernel<__half, true> : decode_mega_kernel<__half, false>);
  static bool attr_done[4] = {false, false, false, false};
  const int which = (kv_f32 ? 2 : 0) + (prof ? 1 : 0);
  if (!attr_done[which]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    attr_done[which] = true;
  }
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3((unsigned)grid);
  lc.blockDim = dim3(THREADS);
  lc.dynamicSmemBytes = smem;
  lc.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;  // all CTAs co-resident: they wait on one another
  at[0].val.cooperative = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  return cudaLaunchKernelEx(&lc, kernel, P);
}

}  // namespace rg
