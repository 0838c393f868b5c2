// Causal GQA attention for a chunk of consecutive prompt tokens of one sequence
// (src/ir/attention.rs:946-981,1157-1240 with the mask `col <= past + row` of
// src/models/transformer/layer.rs:374-380): tiled, f32 arithmetic, online softmax.
//
// One CTA owns 64 score rows = (64 / G) query tokens x the G query heads that share one kv head,
// and walks the keys 0 .. last query position in tiles of 64.  Per tile: K is staged transposed
// ([d][key], f32) so that the 4 x 4 register tile of q.k products reads conflict-free vectors; the
// scores get the reference's scale (division by f32(sqrt(hd))) and mask; running max / sum per row
// are kept across tiles (exp2 form of attention.rs:495-558; the rescaling of earlier tiles differs
// from the two-pass form only in rounding); P goes through shared memory into the 4 x 8 register
// tile of P.V.  Every K / V element is read from the cache once per CTA instead of once per query
// token, which is what makes a 2048-token prompt cheap.
#include <cuda_fp16.h>
#include <math.h>
#include <stdlib.h>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int HD = 128;
constexpr int ROWS = 64;  // score rows per CTA
constexpr int TK = 64;    // keys per tile
constexpr int THREADS = 256;
constexpr int QS_LD = HD + 4;  // padded: rows 4 apart must not share a bank group
constexpr int PS_LD = TK + 4;

// eight consecutive cache elements (16-byte aligned for f16, 32-byte for f32) as f32; zeros when !live
__device__ __forceinline__ void load8(const float *p, bool live, float (&v)[8]) {
  float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f), b = a;
  if (live) a = reinterpret_cast<const float4 *>(p)[0], b = reinterpret_cast<const float4 *>(p)[1];
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void load8(const __half *p, bool live, float (&v)[8]) {
  uint4 u = make_uint4(0u, 0u, 0u, 0u);
  if (live) u = *reinterpret_cast<const uint4 *>(p);
  const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x, v[2 * i + 1] = f.y;
  }
}
// raw copy of eight elements (the V tile keeps the cache's element type)
__device__ __forceinline__ void copy8(const float *src, bool live, float *dst) {
  float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f), b = a;
  if (live) a = reinterpret_cast<const float4 *>(src)[0], b = reinterpret_cast<const float4 *>(src)[1];
  reinterpret_cast<float4 *>(dst)[0] = a;
  reinterpret_cast<float4 *>(dst)[1] = b;
}
__device__ __forceinline__ void copy8(const __half *src, bool live, __half *dst) {
  uint4 u = make_uint4(0u, 0u, 0u, 0u);
  if (live) u = *reinterpret_cast<const uint4 *>(src);
  *reinterpret_cast<uint4 *>(dst) = u;
}

template <typename KV, int G>
__global__ void __launch_bounds__(THREADS, 2) attn_prefill_kernel(const PrefillAttnArgs A) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int TQ = ROWS / G;  // query tokens per CTA
  extern __shared__ __align__(16) uint8_t smem[];
  float *qs = reinterpret_cast<float *>(smem);         // [ROWS][QS_LD]
  float *kt = qs + ROWS * QS_LD;                        // [HD][TK] keys transposed
  float *ps = kt + HD * TK;                             // [ROWS][PS_LD]
  KV *vs = reinterpret_cast<KV *>(ps + ROWS * PS_LD);   // [TK][HD]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int kvh = blockIdx.y;
  const int t0 = blockIdx.x * TQ;  // first query token of this CTA within the chunk
  if (t0 >= A.cols) return;
  const int nq = min(TQ, A.cols - t0);
  // row r = g * TQ + t  <->  query head kvh * G + g, token t0 + t
  for (int i = tid; i < ROWS * (HD / 4); i += THREADS) {
    const int r = i / (HD / 4), c4 = i - r * (HD / 4);
    const int g = r / TQ, t = r - g * TQ;
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (t < nq) v = reinterpret_cast<const float4 *>(A.q + ((size_t)(t0 + t) * A.heads + (size_t)(kvh * G + g)) * HD)[c4];
    *reinterpret_cast<float4 *>(qs + r * QS_LD + 4 * c4) = v;
  }
  const KV *kc = static_cast<const KV *>(A.k_cache) + ((size_t)A.seq * A.kv_heads + kvh) * (size_t)A.ctx * HD;
  const KV *vc = static_cast<const KV *>(A.v_cache) + ((size_t)A.seq * A.kv_heads + kvh) * (size_t)A.ctx * HD;
  const int last_q = A.pos0 + t0 + nq - 1;  // last position any row of this CTA may see
  const float inv_scale = (float)(1.0 / (1.0 / sqrt((double)HD)));
  float m_run[4], l_run[4], acc[4][8];
  int qpos[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = 4 * ty + i, t = r % TQ;
    m_run[i] = -INFINITY;
    l_run[i] = 0.0f;
    qpos[i] = (t < nq) ? A.pos0 + t0 + t : -1;  // -1: padding row, sees nothing
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
  }
  for (int k0 = 0; k0 <= last_q; k0 += TK) {
    __syncthreads();  // the previous tile's kt / vs / ps are no longer read
    {  // K tile transposed to f32 [d][key]; keys beyond the last visible position read as zero
      const int key = tid & 63, dq = (tid >> 6) * 32;
      const bool live = k0 + key <= last_q;
      const KV *src = kc + (size_t)(k0 + key) * HD + dq;
#pragma unroll
      for (int d8 = 0; d8 < 32; d8 += 8) {
        float v[8];
        load8(src + d8, live, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) kt[(dq + d8 + j) * TK + key] = v[j];
      }
    }
    for (int i = tid; i < TK * HD / 8; i += THREADS) {  // V tile, 8 elements per thread-iteration
      const int key = i / (HD / 8), c = i - key * (HD / 8);
      copy8(vc + (size_t)(k0 + key) * HD + 8 * c, k0 + key <= last_q, vs + key * HD + 8 * c);
    }
    __syncthreads();
    // ---- scores: rows 4ty..4ty+3 x keys 4tx..4tx+3
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
#pragma unroll 2
    for (int d = 0; d < HD; d += 4) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4 *>(qs + (4 * ty + i) * QS_LD + d);
#pragma unroll
      for (int e = 0; e < 4; ++e) kv[e] = *reinterpret_cast<const float4 *>(kt + (d + e) * TK + 4 * tx);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float qe[4] = {qv[i].x, qv[i].y, qv[i].z, qv[i].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[i][0] = fmaf(qe[e], kv[e].x, s[i][0]);
          s[i][1] = fmaf(qe[e], kv[e].y, s[i][1]);
          s[i][2] = fmaf(qe[e], kv[e].z, s[i][2]);
          s[i][3] = fmaf(qe[e], kv[e].w, s[i][3]);
        }
      }
    }
    // ---- scale, mask, online softmax per row (16 lanes share a row)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kp = k0 + 4 * tx + j;
        s[i][j] = (kp <= qpos[i]) ? __fdiv_rn(s[i][j], inv_scale) : -INFINITY;
        mx = fmaxf(mx, s[i][j]);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m_run[i], mx);
      float corr = 1.0f, sum = 0.0f;
      if (m_new > -INFINITY) {
        corr = exp2f(__fmul_rn(__fsub_rn(m_run[i], m_new), 1.44269504088896340736f));  // 0 when m_run is -inf
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float e = exp2f(__fmul_rn(__fsub_rn(s[i][j], m_new), 1.44269504088896340736f));
          s[i][j] = e;
          sum += e;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      l_run[i] = fmaf(l_run[i], corr, sum);
      m_run[i] = m_new;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] *= corr;
      *reinterpret_cast<float4 *>(ps + (4 * ty + i) * PS_LD + 4 * tx) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
    }
    __syncthreads();
    // ---- P.V: rows 4ty..4ty+3 x dims 8tx..8tx+7
#pragma unroll 2
    for (int key = 0; key < TK; key += 4) {
      float4 pv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = *reinterpret_cast<const float4 *>(ps + (4 * ty + i) * PS_LD + key);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float vv[8];
        load8(vs + (key + e) * HD + 8 * tx, true, vv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float p = e == 0 ? pv[i].x : e == 1 ? pv[i].y : e == 2 ? pv[i].z : pv[i].w;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(p, vv[j], acc[i][j]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = 4 * ty + i, g = r / TQ, t = r - g * TQ;
    if (t >= nq) continue;
    const float inv = __frcp_rn(l_run[i]);
    float *dst = A.out + (size_t)(t0 + t) * A.heads * HD + (size_t)(kvh * G + g) * HD + 8 * tx;
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = __fmul_rn(acc[i][j], inv);
  }
}

template <typename KV, int G>
cudaError_t launch_t(const PrefillAttnArgs &a, const LaunchCfg &cfg) {
  auto kernel = attn_prefill_kernel<KV, G>;
  constexpr size_t smem = (size_t)(ROWS * QS_LD + HD * TK + ROWS * PS_LD) * sizeof(float) + (size_t)TK * HD * sizeof(KV);
  static DeviceOnce attr_once;  // per instantiation and device
  bool *attr_flag = attr_once.slot();
  if (!attr_flag || !*attr_flag) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    if (attr_flag) *attr_flag = true;
  }
  constexpr int TQ = ROWS / G;
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3((unsigned)((a.cols + TQ - 1) / TQ), (unsigned)a.kv_heads);
  lc.blockDim = dim3(THREADS);
  lc.dynamicSmemBytes = smem;
  lc.stream = cfg.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = cfg.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&lc, kernel, a);
}

template <typename KV>
cudaError_t launch_g(const PrefillAttnArgs &a, const LaunchCfg &cfg) {
  switch (a.heads / a.kv_heads) {
    case 1: return launch_t<KV, 1>(a, cfg);
    case 2: return launch_t<KV, 2>(a, cfg);
    case 4: return launch_t<KV, 4>(a, cfg);
    case 8: return launch_t<KV, 8>(a, cfg);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

bool prefill_attention_supported(int heads, int kv_heads, int hd) {
  if (hd != HD || kv_heads < 1 || heads % kv_heads) return false;
  const int g = heads / kv_heads;
  return g == 1 || g == 2 || g == 4 || g == 8;
}

static bool prefill_simt_forced() {
  static const bool simt = [] {
    const char *v = getenv("RG_B200_PREFILL_ATTN_F32");
    return v && *v && *v != '0';
  }();
  return simt;
}

// f16 caches: K and V rows are exact tensor-core operands (attn_prefill_tc.cu)
bool prefill_attention_uses_tc(const PrefillAttnArgs &a) { return !a.kv_f32 && !prefill_simt_forced(); }

cudaError_t launch_attention_prefill(const PrefillAttnArgs &a, const LaunchCfg &cfg) {
  count_launch(LC_ATTN_PREFILL);
  const bool tc = prefill_attention_uses_tc(a);
  if (!prefill_attention_supported(a.heads, a.kv_heads, HD) || !a.q || !a.k_cache || !a.v_cache || a.cols < 1 || a.pos0 < 0 ||
      a.pos0 + a.cols > a.ctx)
    return cudaErrorInvalidValue;
  if (a.out16_hi ? (!tc || a.out16_ld < a.heads * HD || (a.out16_ld & 1)) : !a.out) return cudaErrorInvalidValue;
  if (a.kv_f32) return launch_g<float>(a, cfg);
  return tc ? launch_attention_prefill_tc(a, cfg) : launch_g<__half>(a, cfg);
}

}  // namespace rg
