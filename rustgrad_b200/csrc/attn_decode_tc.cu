// Decode attention for a batch of rows (one new token each, every row with its own cache) on the
// tensor cores, for f16 K / V caches and head dimension 128 (src/ir/attention.rs:495-558,1157-1240;
// rows of distinct sequences as in src/models/transformer/batch.rs:177-325).
//
// With several rows the work is the stream of K and V rows, so the kernel is built around keeping
// that stream going: a CTA owns one span of one (row, kv head) and each of its four warps walks its
// own 16-key tiles of the span through a private three-stage cp.async ring (no CTA-wide barrier in
// the loop; 2 CTAs per SM keep 16-24 tiles in flight).  The G query heads that share the kv head
// are rows 0 .. G-1 of one m16 tile (the rest is padding), so a K / V row is read once for all of
// them:
//  * S = Q K^T with the f32 query split into two f16 planes (hi, lo) against the exact f16 K rows;
//  * online softmax per warp (exp2 form, running max / sum);
//  * O += P V with P as hi + lo planes straight from the score accumulators, V read transposed by
//    ldmatrix.
// The four warps' (max, sum, O) merge in shared memory into one partial result of the span, and a
// second small kernel merges the spans of a head in span order.  Every f16 x f16 product is exact in
// the f32 accumulator; what differs from the f32 kernels is the order of the sums and the 2^-22 tail
// of q and p.
#include <cuda_fp16.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int HD = 128;
constexpr int THREADS = 128;  // four warps, each with its own key tiles
constexpr int WARPS = 4;
constexpr int TK = 16;        // keys per tile
constexpr int NSTG = 3;       // cp.async stages per warp
constexpr int LD = HD + 8;    // shared row pitch in halves: 272 bytes, eight rows of an 8 x 8 matrix in distinct banks
constexpr int SPAN_UNIT = WARPS * TK;
constexpr int MAX_G = 8;
constexpr int Q_BYTES = 2 * 16 * LD * 2;                    // hi and lo plane of the 16-row query tile
constexpr int STAGE_BYTES = 2 * TK * LD * 2;                // K tile + V tile
constexpr int RING_BYTES = WARPS * NSTG * STAGE_BYTES;
constexpr int SMEM_BYTES = Q_BYTES + RING_BYTES;
static_assert(WARPS * MAX_G * (HD + 2) * 4 <= RING_BYTES, "the merge buffer reuses the ring");

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (x0, x1) as two f16 planes: hi = f16(x), lo = f16(x - hi), packed as half2 words
__device__ __forceinline__ void split2(float x0, float x1, uint32_t &hi, uint32_t &lo) {
  const __half2 h = __floats2half2_rn(x0, x1);
  const float2 hf = __half22float2(h);
  const __half2 l = __floats2half2_rn(x0 - hf.x, x1 - hf.y);
  hi = *reinterpret_cast<const uint32_t *>(&h);
  lo = *reinterpret_cast<const uint32_t *>(&l);
}
// 16 bytes global -> shared without a register stop; src_bytes = 0 writes zeros
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Span length for `total` positions spread over at most `per_head` CTAs: whole groups of 64 keys
// (one 16-key tile per warp).  Both kernels derive the span count from it.
__host__ __device__ inline int span_len(int total, int per_head) {
  const int span = (((total + per_head - 1) / per_head) + SPAN_UNIT - 1) / SPAN_UNIT * SPAN_UNIT;
  return span < SPAN_UNIT ? SPAN_UNIT : span;
}

template <int G>
__global__ void __launch_bounds__(THREADS, 2) attn_decode_tc_kernel(const AttnArgs A, int per_head) {
  pdl_wait();
  pdl_launch_dependents();
  const int sp = blockIdx.x, kvh = blockIdx.y, c = blockIdx.z;
  const int pos = A.col_pos[c], seq = A.col_seq[c];
  const int total = pos + 1;
  const int span = span_len(total, per_head);
  const int nspl = (total + span - 1) / span;
  if (sp >= nspl) return;
  const int p0 = sp * span, p1 = min(total, p0 + span);

  extern __shared__ __align__(16) uint8_t smem[];
  __half *q_hi = reinterpret_cast<__half *>(smem);  // [16][LD]
  __half *q_lo = q_hi + 16 * LD;
  uint8_t *ring = smem + Q_BYTES;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;

  // rows 0 .. G-1: the query heads of this kv head; the other rows of the tile are zero
  for (int i = tid; i < 16 * (HD / 4); i += THREADS) {
    const int r = i / (HD / 4), c4 = i - r * (HD / 4);
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (r < G) v = reinterpret_cast<const float4 *>(A.q + ((size_t)c * A.heads + (size_t)(kvh * G + r)) * HD)[c4];
    uint2 hi, lo;
    split2(v.x, v.y, hi.x, lo.x);
    split2(v.z, v.w, hi.y, lo.y);
    *reinterpret_cast<uint2 *>(q_hi + r * LD + 4 * c4) = hi;
    *reinterpret_cast<uint2 *>(q_lo + r * LD + 4 * c4) = lo;
  }
  const __half *kc = static_cast<const __half *>(A.k_cache) + ((size_t)seq * A.kv_heads + kvh) * (size_t)A.ctx * HD;
  const __half *vc = static_cast<const __half *>(A.v_cache) + ((size_t)seq * A.kv_heads + kvh) * (size_t)A.ctx * HD;
  const float inv_scale = (float)(1.0 / (1.0 / sqrt((double)HD)));

  // this warp's tiles: keys p0 + 16 (warp + 4 j) ..
  const int n_tiles_cta = (p1 - p0 + TK - 1) / TK;
  const int n_my = n_tiles_cta > warp ? (n_tiles_cta - warp + WARPS - 1) / WARPS : 0;
  const uint32_t ring_s = smem_u32(ring) + (uint32_t)(warp * NSTG * STAGE_BYTES);
  // a lane copies 16-byte piece (lane & 15) of keys (lane >> 4) + 2 r, r = 0..7, of K and of V
  auto issue = [&](int j) {
    if (j < n_my) {
      const int k0 = p0 + TK * (warp + WARPS * j);
      const int piece = lane & 15, key0 = lane >> 4;
      const uint32_t dst0 = ring_s + (uint32_t)((j % NSTG) * STAGE_BYTES) + (uint32_t)((key0 * LD + 8 * piece) * 2);
      if (k0 + TK <= p1) {  // a whole tile: fixed offsets from one address per cache
        const __half *ksrc = kc + (size_t)(k0 + key0) * HD + 8 * piece, *vsrc = vc + (size_t)(k0 + key0) * HD + 8 * piece;
#pragma unroll
        for (int r = 0; r < TK / 2; ++r) {
          cp_async16(dst0 + (uint32_t)(r * 2 * LD * 2), ksrc + r * 2 * HD, 16u);
          cp_async16(dst0 + (uint32_t)(r * 2 * LD * 2 + TK * LD * 2), vsrc + r * 2 * HD, 16u);
        }
      } else {  // the span's last tile: keys past the end arrive as zeros
#pragma unroll
        for (int r = 0; r < TK / 2; ++r) {
          const int key = key0 + 2 * r;
          const bool live = k0 + key < p1;
          const size_t src = (size_t)(live ? k0 + key : p1 - 1) * HD + 8 * piece;  // a valid address either way
          cp_async16(dst0 + (uint32_t)(r * 2 * LD * 2), kc + src, live ? 16u : 0u);
          cp_async16(dst0 + (uint32_t)(r * 2 * LD * 2 + TK * LD * 2), vc + src, live ? 16u : 0u);
        }
      }
    }
    cp_async_commit();  // an empty group keeps the count of groups in flight uniform
  };
  issue(0);
  issue(1);
  __syncthreads();  // the query planes are in place

  float m_run = -INFINITY, l_run = 0.0f;  // of row g (a query head when g < G)
  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  const uint32_t a_off = (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * LD + (lane >> 4) * 8) * 2);   // A: query rows
  const uint32_t kb_off = (uint32_t)((((lane & 7) + (lane >> 4) * 8) * LD + ((lane >> 3) & 1) * 8) * 2);  // B: two 8-key tiles
  const uint32_t vb_off = (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * LD + (lane >> 4) * 8) * 2);  // B^T: two hd tiles
  const uint32_t qh_s = smem_u32(q_hi), ql_s = smem_u32(q_lo);

  for (int j = 0; j < n_my; ++j) {
    issue(j + 2);
    cp_async_wait<2>();  // tile j has landed (for this lane's copies)
    __syncwarp();        // ... and for every lane's
    const int k0 = p0 + TK * (warp + WARPS * j);
    const uint32_t ks_s = ring_s + (uint32_t)((j % NSTG) * STAGE_BYTES), vs_s = ks_s + TK * LD * 2;
    // ---- scores of 16 rows x 16 keys
    // (the two query planes accumulate separately: four independent chains of eight products)
    float s[2][4], sl[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
      sl[n][0] = sl[n][1] = sl[n][2] = sl[n][3] = 0.0f;
    }
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
      uint32_t ah[4], al[4], b[4];
      ldsm4(ah, qh_s + a_off + kk * 32);
      ldsm4(al, ql_s + a_off + kk * 32);
      ldsm4(b, ks_s + kb_off + kk * 32);
      mma_f16(sl[0], al, b[0], b[1]);
      mma_f16(s[0], ah, b[0], b[1]);
      mma_f16(sl[1], al, b[2], b[3]);
      mma_f16(s[1], ah, b[2], b[3]);
    }
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      s[n][0] += sl[n][0];
      s[n][1] += sl[n][1];
    }
    // ---- scale, mask, online softmax of row g (rows 8.. are padding: their probabilities stay zero)
    float mx = -INFINITY;
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int kp = k0 + 8 * n + 2 * t + i;
        float &v = s[n][i];
        v = kp < p1 ? __fdiv_rn(v, inv_scale) : -INFINITY;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    float sum = 0.0f, corr = 1.0f;
    if (m_new > -INFINITY) {
      corr = exp2f(__fmul_rn(__fsub_rn(m_run, m_new), 1.44269504088896340736f));  // 0 when m_run is -inf
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float e = exp2f(__fmul_rn(__fsub_rn(s[n][i], m_new), 1.44269504088896340736f));
          s[n][i] = e;
          sum += e;
        }
    } else {
      s[0][0] = s[0][1] = s[1][0] = s[1][1] = 0.0f;
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    l_run = fmaf(l_run, corr, sum);
    m_run = m_new;
    if (__any_sync(0xffffffffu, corr != 1.0f)) {  // the running maximum of some row moved
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        o[n][0] *= corr;
        o[n][1] *= corr;
      }
    }
    // ---- O += P V: the two 8-key score tiles are one 16-key A fragment
    uint32_t ph[4], pl[4];
    split2(s[0][0], s[0][1], ph[0], pl[0]);  // row g, keys 2t, 2t + 1
    split2(s[1][0], s[1][1], ph[2], pl[2]);  // row g, keys 8 + 2t, 9 + 2t
    ph[1] = pl[1] = ph[3] = pl[3] = 0u;      // rows g + 8
#pragma unroll
    for (int n2 = 0; n2 < HD / 16; ++n2) {
      uint32_t b[4];
      ldsm4_t(b, vs_s + vb_off + n2 * 32);
      mma_f16(o[2 * n2], pl, b[0], b[1]);
      mma_f16(o[2 * n2], ph, b[0], b[1]);
      mma_f16(o[2 * n2 + 1], pl, b[2], b[3]);
      mma_f16(o[2 * n2 + 1], ph, b[2], b[3]);
    }
    __syncwarp();  // the stage may be refilled by the next iteration's copies
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its ring: the merge buffer takes its place

  // ---- merge the four warps: [warp][head][m, l, o[HD]]
  float *mb = reinterpret_cast<float *>(ring);
  if (g < G) {
    float *dst = mb + ((size_t)warp * G + g) * (HD + 2);
    if (t == 0) {
      dst[0] = m_run;
      dst[1] = l_run;
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) *reinterpret_cast<float2 *>(dst + 2 + 8 * n + 2 * t) = make_float2(o[n][0], o[n][1]);
  }
  __syncthreads();
  for (int head = 0; head < G; ++head) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, mb[((size_t)w * G + head) * (HD + 2)]);
    float L = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float *ps = mb + ((size_t)w * G + head) * (HD + 2);
      const float wgt = ps[0] > -INFINITY ? exp2f(__fmul_rn(__fsub_rn(ps[0], M), 1.44269504088896340736f)) : 0.0f;
      L = fmaf(ps[1], wgt, L);
      acc = fmaf(ps[2 + tid], wgt, acc);
    }
    float *dst = A.scratch + (((size_t)c * A.heads + (size_t)(kvh * G + head)) * per_head + sp) * (HD + 2);
    dst[2 + tid] = acc;
    if (tid == 0) {
      dst[0] = M;
      dst[1] = L;
    }
  }
}

// Spans of one head in span order: softmax weights of the span maxima, then the normalised sum.
__global__ void __launch_bounds__(HD) attn_decode_tc_combine_kernel(const float *scratch, int heads, const int32_t *col_pos,
                                                                    int per_head, int cols, __half *out_pack, float *out_f32) {
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, c = blockIdx.y, tid = threadIdx.x;
  const int total = col_pos[c] + 1;
  const int span = span_len(total, per_head);
  const int ns = (total + span - 1) / span;
  const float *base = scratch + ((size_t)c * heads + h) * per_head * (HD + 2);
  float M = -INFINITY;
  for (int s = 0; s < ns; ++s) M = fmaxf(M, base[(size_t)s * (HD + 2)]);
  float L = 0.0f, acc = 0.0f;
  for (int s = 0; s < ns; ++s) {
    const float *ps = base + (size_t)s * (HD + 2);
    const float wgt = exp2f(__fmul_rn(__fsub_rn(ps[0], M), 1.44269504088896340736f));
    L = fmaf(ps[1], wgt, L);
    acc = fmaf(ps[2 + tid], wgt, acc);
  }
  const float v = __fmul_rn(acc, __frcp_rn(L));
  const int k = h * HD + tid;
  if (out_pack) xpack_store(out_pack, 2 * cols, c, k, v);
  if (out_f32) out_f32[(size_t)c * heads * HD + k] = v;
}

template <int G>
cudaError_t launch_g(const AttnArgs &a, const LaunchCfg &cfg, int per_head) {
  auto kernel = attn_decode_tc_kernel<G>;
  static DeviceOnce attr_once;  // per instantiation and device
  bool *attr_flag = attr_once.slot();
  if (!attr_flag || !*attr_flag) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (attr_flag) *attr_flag = true;
  }
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3((unsigned)per_head, (unsigned)a.kv_heads, (unsigned)a.cols);
  lc.blockDim = dim3(THREADS);
  lc.dynamicSmemBytes = SMEM_BYTES;
  lc.stream = cfg.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = cfg.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&lc, kernel, a, per_head);
}

// Spans per (row, kv head): about `waves` CTAs per SM over the whole grid (two are resident), never shorter
// than 64 keys.
int spans_per_head(int sm_count, int kv_heads, int cols, int ctx) {
  static const int waves = [] {
    const char *v = getenv("RG_B200_ATTN_TC_WAVES");
    const int w = v ? atoi(v) : 2;
    return w >= 1 && w <= 16 ? w : 2;
  }();
  int n = waves * sm_count / (kv_heads * cols);
  const int by_ctx = (ctx + SPAN_UNIT - 1) / SPAN_UNIT;
  if (n > by_ctx) n = by_ctx;
  return n < 1 ? 1 : n;
}

}  // namespace

bool attention_decode_tc_supported(const AttnArgs &a) {
  if (a.kv_f32 || a.hd != HD || a.kv_heads < 1 || a.heads % a.kv_heads) return false;
  const int g = a.heads / a.kv_heads;
  return g == 1 || g == 2 || g == 4 || g == 8;
}

size_t attention_decode_tc_scratch_floats(int sm_count, int heads, int kv_heads, int cols, int ctx) {
  return (size_t)cols * heads * spans_per_head(sm_count, kv_heads, cols, ctx) * (HD + 2);
}

cudaError_t launch_attention_decode_tc(const AttnArgs &a, const LaunchCfg &cfg) {
  count_launch(LC_ATTN_DECODE_TC);
  if (!attention_decode_tc_supported(a) || !a.q || !a.k_cache || !a.v_cache || !a.scratch || a.cols < 1 ||
      (!a.out_pack && !a.out_f32))
    return cudaErrorInvalidValue;
  const int sms = cfg.sm_count > 0 ? cfg.sm_count : 148;
  const int per_head = spans_per_head(sms, a.kv_heads, a.cols, a.ctx);
  cudaError_t e;
  switch (a.heads / a.kv_heads) {
    case 1: e = launch_g<1>(a, cfg, per_head); break;
    case 2: e = launch_g<2>(a, cfg, per_head); break;
    case 4: e = launch_g<4>(a, cfg, per_head); break;
    default: e = launch_g<8>(a, cfg, per_head); break;
  }
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3((unsigned)a.heads, (unsigned)a.cols);
  lc.blockDim = dim3(HD);
  lc.stream = cfg.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = cfg.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&lc, attn_decode_tc_combine_kernel, (const float *)a.scratch, a.heads, a.col_pos, per_head, a.cols,
                            static_cast<__half *>(a.out_pack), a.out_f32);
}

}  // namespace rg
