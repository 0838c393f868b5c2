// The non-GEMV kernels of the decode step: block decode, embedding gather, RMSNorm (+ pack),
// RoPE + KV append, split-context GQA attention + combine, greedy selection, dense-weight GEMV,
// and the synthetic-tensor generator.  All are HBM/latency-bound SIMT kernels; each calls
// pdl_wait() before touching step data so programmatic dependent launch stays transitive.
#include <math.h>

#include <mutex>
#include <string>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

template <typename K, typename... Args>
cudaError_t launch(K kernel, dim3 grid, dim3 block, size_t smem, const LaunchCfg &cfg, Args... args) {
  cudaLaunchConfig_t lc{};
  lc.gridDim = grid;
  lc.blockDim = block;
  lc.dynamicSmemBytes = smem;
  lc.stream = cfg.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = cfg.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&lc, kernel, args...);
}

// ------------------------------------------------------------------------------ block decode
// One element of a tensor in its GGML bytes; the f32 operation order is the reference's
// (src/gguf/quantization/blocks.rs:1251-1254,1501-1503): (f32(nibble) - 8) * d, f32(int8) * d.
__device__ __forceinline__ float decode_element(int type, const uint8_t *bytes, size_t e, bool *bad) {
  if (type == RG_TYPE_F32) return reinterpret_cast<const float *>(bytes)[e];
  if (type == RG_TYPE_F16) return half_bits_to_float(reinterpret_cast<const uint16_t *>(bytes)[e]);
  const size_t blk = e >> 5;
  const int lane = (int)(e & 31);
  if (type == RG_TYPE_Q4_0) {
    const uint8_t *b = bytes + blk * 18;
    const float d = half_bits_to_float((uint32_t)b[0] | ((uint32_t)b[1] << 8));
    const uint8_t packed = b[2 + (lane & 15)];
    const int nib = (lane < 16) ? (packed & 0x0f) : (packed >> 4);
    if (bad && !finite_f32(d)) *bad = true;
    return __fmul_rn(__fsub_rn((float)nib, 8.0f), d);
  }
  if (type == RG_TYPE_Q4_K) {
    // blocks.rs:1164-1187: value = d * f32(scale) * f32(q) - dmin * f32(min), each step rounded to f32;
    // the 6-bit scales and mins of the eight 32-element groups are packed as in blocks.rs:1511-1522
    const uint8_t *b = bytes + (e >> 8) * 144;
    const int idx = (int)(e & 255), group = idx >> 5, gl = idx & 31;
    const float d = half_bits_to_float((uint32_t)b[0] | ((uint32_t)b[1] << 8));
    const float dmin = half_bits_to_float((uint32_t)b[2] | ((uint32_t)b[3] << 8));
    if (bad && (!finite_f32(d) || !finite_f32(dmin))) *bad = true;
    const uint8_t *p = b + 4;
    int sc, mn;
    if (group < 4) {
      sc = p[group] & 0x3f;
      mn = p[4 + group] & 0x3f;
    } else {
      sc = (p[4 + group] & 0x0f) | ((p[group - 4] >> 6) << 4);
      mn = (p[4 + group] >> 4) | ((p[group] >> 6) << 4);
    }
    const int q = (b[16 + (group >> 1) * 32 + gl] >> ((group & 1) * 4)) & 0x0f;
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
  }
  if (type == RG_TYPE_Q6_K) {
    // blocks.rs:1219-1240: value = d * f32((q - 32) * scale)
    const uint8_t *b = bytes + (e >> 8) * 210;
    const int idx = (int)(e & 255), half_index = idx >> 7, within = idx & 127;
    const float d = half_bits_to_float((uint32_t)b[208] | ((uint32_t)b[209] << 8));
    if (bad && !finite_f32(d)) *bad = true;
    const int low = (b[half_index * 64 + (within & 63)] >> ((within >> 6) * 4)) & 0x0f;
    const int high = ((b[128 + half_index * 32 + (within & 31)] >> ((within >> 5) * 2)) & 0x03) << 4;
    const int quant = (low | high) - 32;
    const int scale = (int)(int8_t)b[192 + (idx >> 4)];
    return __fmul_rn(d, (float)(quant * scale));
  }
  const uint8_t *b = bytes + blk * 34;
  const float d = half_bits_to_float((uint32_t)b[0] | ((uint32_t)b[1] << 8));
  if (bad && !finite_f32(d)) *bad = true;
  return __fmul_rn((float)(int8_t)b[2 + lane], d);
}

__global__ void dequantize_kernel(int type, const uint8_t *bytes, size_t n, float *out, int *status) {
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  bool bad = false;
  const float v = decode_element(type, bytes, i, &bad);
  out[i] = v;
  if ((bad || !finite_f32(v)) && status) atomicExch(status, DEV_NON_FINITE);
}

__global__ void row_gather_kernel(int type, const uint8_t *bytes, int cols, const int32_t *ids, float *out, int ldo) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = blockIdx.x;
  const size_t base = (size_t)ids[c] * (size_t)cols;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) out[(size_t)c * ldo + i] = decode_element(type, bytes, base + i, nullptr);
}

// ------------------------------------------------------------------------------ pack / unpack
__global__ void pack_kernel(const float *x, int ldx, int k, int batch, __half *xpack) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (i < k) xpack_store(xpack, 2 * batch, b, i, x[(size_t)b * ldx + i]);
}
__global__ void unpack_kernel(const __half *xpack, int k, int batch, float *x, int ldx) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (i >= k) return;
  const float hi = __half2float(xpack[xpack_half_index(2 * batch, i, 2 * b)]);
  const float lo = __half2float(xpack[xpack_half_index(2 * batch, i, 2 * b + 1)]);
  x[(size_t)b * ldx + i] = hi + lo * XPACK_LO_INV;
}

// ------------------------------------------------------------------------------ RMSNorm
// y = (x * (1 / sqrt(mean(x^2) + eps))) * w with each step rounded to f32 like the reference
// (src/models/transformer/layer.rs:423-443); only the order of the sum of squares differs.
__global__ void rmsnorm_pack_kernel(const float *x, int ldx, const float *w, int d, float eps, int cols, const int32_t *col_map,
                                    __half *xpack, float *y, int ldy) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float partial[32];
  __shared__ float inv_s;
  const int c = blockIdx.x;
  const int src = col_map ? col_map[c] : c;
  const float *xr = x + (size_t)src * ldx;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = (threadIdx.x < (blockDim.x >> 5)) ? partial[threadIdx.x] : 0.0f;
    v = warp_sum(v);
    if (threadIdx.x == 0) {
      const float mean = __fdiv_rn(v, (float)d);
      inv_s = __frcp_rn(__fsqrt_rn(__fadd_rn(mean, eps)));
    }
  }
  __syncthreads();
  const float inv = inv_s;
  // gridDim.y CTAs share a column: each sums the whole row (in the same order, so they agree bit for bit)
  // and writes its own slice
  const int per = (d + (int)gridDim.y - 1) / (int)gridDim.y;
  const int i0 = (int)blockIdx.y * per, i1 = min(d, i0 + per);
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
    const float v = __fmul_rn(__fmul_rn(xr[i], inv), w[i]);
    if (xpack) xpack_store(xpack, 2 * cols, c, i, v);
    if (y) y[(size_t)c * ldy + i] = v;
  }
}

// ------------------------------------------------------------------------------ RoPE + KV append
// De-interleave (src/models/transformer/layer.rs:481-525: out[j] = in[2j], out[half+j] = in[2j+1])
// then split-half rotation (layer.rs:528-571) with every product and sum rounded separately.
template <typename KV>
__device__ __forceinline__ KV to_kv(float v);
template <>
__device__ __forceinline__ float to_kv<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half to_kv<__half>(float v) { return __float2half_rn(v); }

template <typename KV>
__global__ void rope_append_kernel(const float *qkv, int heads, int kv_heads, int hd, int ctx, const int32_t *col_seq,
                                   const int32_t *col_pos, const float *cos_t, const float *sin_t, float *q_out, KV *k_cache,
                                   KV *v_cache) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = blockIdx.x;
  const int half = hd >> 1;
  const int qw = heads * hd, kw = kv_heads * hd;
  const int pos = col_pos[c], seq = col_seq[c];
  const float *row = qkv + (size_t)c * (qw + 2 * kw);
  const float *ct = cos_t + (size_t)pos * half, *st = sin_t + (size_t)pos * half;
  const int rot_items = (heads + kv_heads) * half;
  const int first = blockIdx.y * blockDim.x + threadIdx.x, step = blockDim.x * gridDim.y;  // gridDim.y CTAs share a column
  for (int it = first; it < rot_items; it += step) {
    const int h = it / half, i = it - h * half;
    const float *src = row + (size_t)h * hd;  // q heads then k heads are contiguous in the row
    const float x1 = src[2 * i], x2 = src[2 * i + 1];
    const float cs = ct[i], sn = st[i];
    const float y1 = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
    const float y2 = __fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn));
    if (h < heads) {
      float *dst = q_out + ((size_t)c * heads + h) * hd;
      dst[i] = y1;
      dst[half + i] = y2;
    } else {
      KV *dst = k_cache + (((size_t)seq * kv_heads + (h - heads)) * ctx + pos) * hd;
      dst[i] = to_kv<KV>(y1);
      dst[half + i] = to_kv<KV>(y2);
    }
  }
  for (int it = first; it < kw; it += step) {
    const int h = it / hd, j = it - h * hd;
    v_cache[(((size_t)seq * kv_heads + h) * ctx + pos) * hd + j] = to_kv<KV>(row[qw + kw + it]);
  }
}

// The same step for the model variants (layer.rs:274-346,481-571): one CTA per column keeps the
// column's q, k and v in shared memory and applies, in the reference's order, the lane permutation
// (query: its last rope_dim lanes; key: the whole head), the biases, the RMS norm of q and k over the
// projection or inside every head, and the rotation of lanes [0, rope_dim).  Every step rounds to
// f32 like the reference; only the order of the sums of squares differs.
template <typename KV>
__global__ void qkv_variant_kernel(const RopeArgs A, KV *k_cache, KV *v_cache) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float vs[];
  __shared__ float red[33];
  const int c = blockIdx.x, tid = threadIdx.x, hd = A.hd;
  const int qw = A.heads * hd, kw = A.kv_heads * hd, rope = A.rope_dim ? A.rope_dim : hd, half = rope / 2;
  const int pos = A.col_pos[c], seq = A.col_seq[c];
  const float *row = A.qkv + (size_t)c * (qw + 2 * kw);
  float *q = vs, *k = vs + qw;  // permuted (+ bias); v needs no staging
  for (int i = tid; i < qw + kw; i += blockDim.x) {
    const bool is_q = i < qw;
    const int e = is_q ? i : i - qw, h = e / hd, j = e - h * hd;
    const int permuted = is_q ? rope : hd, prefix = hd - permuted;
    int src = j;
    if (j >= prefix) {
      const int r = j - prefix;
      src = prefix + (r < permuted / 2 ? 2 * r : 2 * (r - permuted / 2) + 1);
    }
    float v = row[(is_q ? 0 : qw) + h * hd + src];
    const float *bias = is_q ? A.q_bias : A.k_bias;
    if (bias) v = __fadd_rn(v, bias[e]);
    vs[i] = v;
  }
  __syncthreads();
  // y = (x * (1 / sqrt(mean(x^2) + eps))) * w over `n` elements starting at `base`
  auto block_sumsq = [&](const float *base, int n) {
    float ss = 0.0f;
    for (int i = tid; i < n; i += blockDim.x) ss = fmaf(base[i], base[i], ss);
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
      float tot = 0.0f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
      red[32] = tot;
    }
    __syncthreads();
    const float tot = red[32];
    __syncthreads();
    return tot;
  };
  auto inv_of = [&](float ss, int n) { return __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)n), A.eps))); };
  if (A.qk_norm == 2) {
    for (int which = 0; which < 2; ++which) {
      float *base = which ? k : q;
      const int n = which ? kw : qw;
      const float *w = which ? A.k_norm : A.q_norm;
      const float inv = inv_of(block_sumsq(base, n), n);
      for (int i = tid; i < n; i += blockDim.x) base[i] = __fmul_rn(__fmul_rn(base[i], inv), w[i]);
      __syncthreads();
    }
  } else if (A.qk_norm == 1) {
    const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
    for (int h = warp; h < A.heads + A.kv_heads; h += nwarps) {  // one warp per head
      float *base = vs + (size_t)h * hd;  // q heads then k heads are contiguous
      const float *w = h < A.heads ? A.q_norm : A.k_norm;
      float ss = 0.0f;
      for (int j = lane; j < hd; j += 32) ss = fmaf(base[j], base[j], ss);
      const float inv = inv_of(warp_sum(ss), hd);
      for (int j = lane; j < hd; j += 32) base[j] = __fmul_rn(__fmul_rn(base[j], inv), w[j]);
    }
    __syncthreads();
  }
  const float *ct = A.cos_t + (size_t)pos * half, *st = A.sin_t + (size_t)pos * half;
  for (int it = tid; it < (A.heads + A.kv_heads) * hd; it += blockDim.x) {
    const int h = it / hd, j = it - h * hd;
    const float *base = vs + (size_t)h * hd;
    float y = base[j];
    if (j < rope) {  // lanes [0, half) and [half, rope) rotate as pairs (i, half + i)
      const int i = j < half ? j : j - half;
      const float x1 = base[i], x2 = base[half + i], cs = ct[i], sn = st[i];
      y = j < half ? __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn)) : __fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn));
    }
    if (h < A.heads)
      A.q_out[((size_t)c * A.heads + h) * hd + j] = y;
    else
      k_cache[(((size_t)seq * A.kv_heads + (h - A.heads)) * A.ctx + pos) * hd + j] = to_kv<KV>(y);
  }
  for (int it = tid; it < kw; it += blockDim.x) {
    const int h = it / hd, j = it - h * hd;
    float v = row[qw + kw + it];
    if (A.v_bias) v = __fadd_rn(v, A.v_bias[it]);
    v_cache[(((size_t)seq * A.kv_heads + h) * A.ctx + pos) * hd + j] = to_kv<KV>(v);
  }
}

// ------------------------------------------------------------------------------ attention
// Split-context decode attention.  One CTA per (context span, kv head, column) handles the G query
// heads that share the kv head.  Scratch per (column, head, split): [m, l, out[hd]].
//  phase 0: the span's K rows and V rows (each one contiguous range of the cache) are staged in
//           shared memory by two bulk copies of the TMA engine, so no lane waits on DRAM in a loop.
//  phase 1: scores.  16 lanes per position, each lane owns HD/16 dims of K (one 128-bit load for
//           f16, hd 128) and the matching slice of every q head in registers; 4 shuffles per head.
//  phase 2: per-head max / exp2 / sum over the span (one warp per head).
//  phase 3: P.V.  A warp takes every 8th position, a lane owns HD/32 dims of V (coalesced row
//           reads), G accumulators per dim; cross-warp sum in shared memory.
// Softmax pieces follow src/ir/attention.rs:495-558: e = exp2((s - m) * log2(e)); the scores are
// q.k / f32(sqrt(hd)) (attention.rs:1183-1188).  Query head h reads kv head h / (H/KV) (:1226-1240).
constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int MAX_HD = 128;

template <int N>
__device__ __forceinline__ void kv_load_vec(const float *p, float (&v)[N]) {
  if constexpr (N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const float4 f = reinterpret_cast<const float4 *>(p)[i];
      v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
      const float2 f = reinterpret_cast<const float2 *>(p)[i];
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
  }
}
template <int N>
__device__ __forceinline__ void kv_load_vec(const __half *p, float (&v)[N]) {
  if constexpr (N == 8) {
    const uint4 u = *reinterpret_cast<const uint4 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
  } else if constexpr (N == 4) {
    const uint2 u = *reinterpret_cast<const uint2 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
  } else {
    static_assert(N == 2, "unsupported vector width");
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(p));
    v[0] = f.x, v[1] = f.y;
  }
}

template <typename KV, int G, int HD>
__global__ void __launch_bounds__(ATT_THREADS) attn_split_kernel(const float *q, const KV *k_cache, const KV *v_cache, int heads,
                                                                 int kv_heads, int ctx, const int32_t *col_seq,
                                                                 const int32_t *col_pos, float *scratch, int max_splits,
                                                                 int *status) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int DPL = HD / 16;  // dims per lane, phase 1
  constexpr int DV = HD / 32;   // dims per lane, phase 3
  const int split = blockIdx.x, kvh = blockIdx.y, c = blockIdx.z;
  const int pos = col_pos[c];
  const int p0 = split * ATTN_SPAN;
  if (p0 > pos) return;
  const int np = min(ATTN_SPAN, pos + 1 - p0);
  const int seq = col_seq[c];
  __shared__ __align__(16) float sc[ATTN_SPAN][G];
  __shared__ float ml[G][2];
  __shared__ __align__(16) float red[ATT_WARPS][G][HD];
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int dead_flag;
  extern __shared__ __align__(128) uint8_t att_smem[];
  KV *ks = reinterpret_cast<KV *>(att_smem);
  KV *vs = ks + (size_t)ATTN_SPAN * HD;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    dead_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (tid == 0) {
    const uint32_t bytes = (uint32_t)((size_t)np * HD * sizeof(KV));
    mbar_expect_tx(&bars[0], bytes);
    bulk_g2s(ks, k_cache + (((size_t)seq * kv_heads + kvh) * ctx + p0) * HD, bytes, &bars[0]);
    mbar_expect_tx(&bars[1], bytes);
    bulk_g2s(vs, v_cache + (((size_t)seq * kv_heads + kvh) * ctx + p0) * HD, bytes, &bars[1]);
  }
  const KV *kbase = ks, *vbase = vs;
  const float inv_scale = (float)(1.0 / (1.0 / sqrt((double)HD)));
  {
    const int sub = lane & 15, hi = lane >> 4;
    float qr[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int i = 0; i < DPL; ++i) qr[g][i] = q[((size_t)c * heads + (size_t)kvh * G + g) * HD + sub * DPL + i];
    mbar_wait_bounded(&bars[0], 0, &dead_flag, status);
    for (int base = 0; base < np; base += 2 * ATT_WARPS) {
      const int p = base + warp * 2 + hi;
      float kv[DPL];
      if (p < np) {
        kv_load_vec<DPL>(kbase + (size_t)p * HD + sub * DPL, kv);
      } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i) kv[i] = 0.0f;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) dot = fmaf(qr[g][i], kv[i], dot);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (sub == 0 && p < np) sc[p][g] = __fdiv_rn(dot, inv_scale);
      }
    }
  }
  __syncthreads();
  if (warp < G) {
    const int g = warp;
    float m = -INFINITY;
    for (int p = lane; p < np; p += 32) m = fmaxf(m, sc[p][g]);
    m = warp_max(m);
    float l = 0.0f;
    for (int p = lane; p < np; p += 32) {
      const float e = exp2f(__fmul_rn(__fsub_rn(sc[p][g], m), 1.44269504088896340736f));
      sc[p][g] = e;
      l += e;
    }
    l = warp_sum(l);
    if (lane == 0) {
      ml[g][0] = m;
      ml[g][1] = l;
    }
  }
  __syncthreads();
  mbar_wait_bounded(&bars[1], 0, &dead_flag, status);
  {
    float acc[G][DV];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int i = 0; i < DV; ++i) acc[g][i] = 0.0f;
    for (int p = warp; p < np; p += ATT_WARPS) {
      float v[DV];
      kv_load_vec<DV>(vbase + (size_t)p * HD + lane * DV, v);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pr = sc[p][g];
#pragma unroll
        for (int i = 0; i < DV; ++i) acc[g][i] = fmaf(pr, v[i], acc[g][i]);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int i = 0; i < DV; ++i) red[warp][g][lane * DV + i] = acc[g][i];
  }
  __syncthreads();
  for (int idx = tid; idx < G * HD; idx += ATT_THREADS) {
    const int g = idx / HD, d = idx - g * HD;
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) v += red[w][g][d];
    float *dst = scratch + (((size_t)c * heads + (size_t)kvh * G + g) * max_splits + split) * (HD + 2);
    dst[2 + d] = v;
    if (d == 0) {
      dst[0] = ml[g][0];
      dst[1] = ml[g][1];
    }
  }
}

__global__ void attn_combine_kernel(const float *scratch, int heads, int hd, const int32_t *col_pos, int max_splits, int cols,
                                    __half *out_pack, float *out_f32) {
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.x, c = blockIdx.y, tid = threadIdx.x;
  const int ns = col_pos[c] / ATTN_SPAN + 1;
  const float *base = scratch + ((size_t)c * heads + h) * max_splits * (hd + 2);
  float M = -INFINITY;
  for (int s = 0; s < ns; ++s) M = fmaxf(M, base[(size_t)s * (hd + 2)]);
  float L = 0.0f, acc = 0.0f;
  for (int s = 0; s < ns; ++s) {
    const float *ps = base + (size_t)s * (hd + 2);
    const float wgt = exp2f(__fmul_rn(__fsub_rn(ps[0], M), 1.44269504088896340736f));
    L = fmaf(ps[1], wgt, L);
    if (tid < hd) acc = fmaf(ps[2 + tid], wgt, acc);
  }
  if (tid < hd) {
    const float v = __fmul_rn(acc, __frcp_rn(L));
    const int k = h * hd + tid;
    if (out_pack) xpack_store(out_pack, 2 * cols, c, k, v);
    if (out_f32) out_f32[(size_t)c * heads * hd + k] = v;
  }
}

// ------------------------------------------------------------------------------ greedy selection
// src/models/transformer/generation.rs:260-287: strict '>' so the lowest id wins ties; any
// non-finite logit is an error, reported as id -1 (the sentinel of metal_step.rs:964-987).
// With a uniform tape the score is the Gumbel-max transform of generation.rs:10-19,273-278:
// logit / max(T, 1e-12) - ln(-ln(max(u, 1e-12))), one row of `vocab` uniforms per column.
// `temps` (nullable) holds one temperature per column; a column whose temperature is not
// positive is selected greedily whatever the tape holds (mixed batches of a serving step).
__global__ void argmax_kernel(const float *logits, int ld, int vocab, const float *uniforms, float temperature,
                              const float *temps, int32_t *out_ids) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = blockIdx.x;
  const float *row = logits + (size_t)c * ld;
  const float tc = temps ? temps[c] : temperature;
  const float *urow = uniforms && (!temps || tc > 0.0f) ? uniforms + (size_t)c * vocab : nullptr;
  const float t = fmaxf(tc, 1e-12f);
  float best = -INFINITY;
  int idx = 0x7fffffff;
  int bad = 0;
  auto consider = [&](float v, float u, int i) {
    if (!finite_f32(v)) bad = 1;
    if (urow) v = __fsub_rn(__fdiv_rn(v, t), logf(-logf(fmaxf(u, 1e-12f))));
    if (v > best || idx == 0x7fffffff) {
      best = v;
      idx = i;
    }
  };
  const bool vec = ((vocab | ld) & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0 &&
                   (!urow || (reinterpret_cast<uintptr_t>(urow) & 15) == 0);
  if (vec) {  // four logits per load, several loads in flight per thread; ids still ascend within a thread
    const float4 *row4 = reinterpret_cast<const float4 *>(row);
    const float4 *u4 = reinterpret_cast<const float4 *>(urow);
    for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) {
      const float4 v = row4[i];
      const float4 u = urow ? u4[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      consider(v.x, u.x, 4 * i);
      consider(v.y, u.y, 4 * i + 1);
      consider(v.z, u.z, 4 * i + 2);
      consider(v.w, u.w, 4 * i + 3);
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) consider(row[i], urow ? urow[i] : 0.0f, i);
  }
  __shared__ float sv[32];
  __shared__ int si[32], sb[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    bad |= __shfl_xor_sync(0xffffffffu, bad, o);
    if (ov > best || (ov == best && oi < idx)) {
      best = ov;
      idx = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = idx;
    sb[warp] = bad;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = (lane < nw) ? sv[lane] : -INFINITY;
    idx = (lane < nw) ? si[lane] : 0x7fffffff;
    bad = (lane < nw) ? sb[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      bad |= __shfl_xor_sync(0xffffffffu, bad, o);
      if (ov > best || (ov == best && oi < idx)) {
        best = ov;
        idx = oi;
      }
    }
    if (lane == 0) out_ids[c] = bad ? -1 : idx;
  }
}

__global__ void advance_kernel(const int32_t *ids, int32_t *tokens, int32_t *pos, int32_t *history, int32_t *step_counter,
                               int cols) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = threadIdx.x;
  const int step = *step_counter;
  if (c < cols) {
    const int id = ids[c];
    tokens[c] = id < 0 ? 0 : id;
    pos[c] += 1;
    if (history) history[(size_t)step * cols + c] = id;
  }
  __syncthreads();
  if (c == 0) *step_counter = step + 1;
}

// ------------------------------------------------------------------------------ dense GEMV
template <typename W>
__device__ __forceinline__ float w_load(const W *p);
template <>
__device__ __forceinline__ float w_load<float>(const float *p) { return *p; }
template <>
__device__ __forceinline__ float w_load<__half>(const __half *p) { return __half2float(*p); }

template <typename W>
__global__ void dense_gemv_kernel(const W *w, int rows, int k, const float *x, int ldx, int batch, int epi, float *y, int ldy) {
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  const W *wr = w + (size_t)row * k;
  float acc[8];
#pragma unroll
  for (int b = 0; b < 8; ++b) acc[b] = 0.0f;
  for (int i = lane; i < k; i += 32) {
    const float wv = w_load<W>(wr + i);
#pragma unroll
    for (int b = 0; b < 8; ++b)
      if (b < batch) acc[b] = fmaf(x[(size_t)b * ldx + i], wv, acc[b]);
  }
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    if (b >= batch) break;
    const float v = warp_sum(acc[b]);
    if (lane == 0) {
      float *dst = y + (size_t)b * ldy + row;
      *dst = (epi == EPI_RESIDUAL) ? __fadd_rn(*dst, v) : v;
    }
  }
}

// K-quant GEMV: one warp per weight row, one 256-element super-block per warp iteration, eight
// consecutive elements per lane (so a lane decodes its group's 6-bit scale / min or its int8 scale once and
// reads its quants as whole bytes).  The scale (and, for Q4_K, the minimum) of a lane's group is applied
// once per super-block to the sum of quant * x (and of x), not per element.
// STAGED: the CTA's eight rows (contiguous bytes) arrive in shared memory by one TMA bulk copy issued
// before the grid dependency wait; with one super-block load in flight per warp the direct form
// keeps under 5 KB per SM in flight and stays near 0.7 TB/s whatever its inner loop does.
template <int TYPE, bool STAGED>
__global__ void kquant_gemv_kernel(const uint8_t *w, int rows, int k, const float *x, int ldx, int batch, int epi, float *y,
                                   int ldy, int *status) {
  constexpr int BB = TYPE == RG_TYPE_Q4_K ? 144 : 210;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  const int nsb = k >> 8;
  const uint8_t *wr = w + (size_t)row * (size_t)nsb * BB;
  if constexpr (STAGED) {
    extern __shared__ __align__(128) uint8_t wsm[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ int dead_flag;
    const int row0 = blockIdx.x * (blockDim.x >> 5);
    const int nrows = min((int)(blockDim.x >> 5), rows - row0);
    const uint32_t row_bytes = (uint32_t)nsb * BB;  // a multiple of 16 (checked by the launcher)
    if (threadIdx.x == 0) {
      mbar_init(&bar, 1);
      dead_flag = 0;
      mbar_fence_init();
      mbar_expect_tx(&bar, (uint32_t)nrows * row_bytes);
      bulk_g2s(wsm, w + (size_t)row0 * row_bytes, (uint32_t)nrows * row_bytes, &bar);
    }
    __syncthreads();
    pdl_wait();
    pdl_launch_dependents();
    const bool ok = mbar_wait_bounded(&bar, 0, &dead_flag, status);
    if (!ok || row >= rows) return;
    wr = wsm + (size_t)warp * row_bytes;
  } else {
    pdl_wait();
    pdl_launch_dependents();
    if (row >= rows) return;
  }
  float acc[8];
#pragma unroll
  for (int b = 0; b < 8; ++b) acc[b] = 0.0f;
  for (int sb = 0; sb < nsb; ++sb) {  // (unrolling by four was measured slower: register pressure)
    const uint8_t *blk = wr + (size_t)sb * BB;
    float wv[8];          // the lane's eight quants as floats
    float mul, sub = 0.0f;  // weight = mul * quant - sub, applied to the lane's sums once per super-block
    if constexpr (TYPE == RG_TYPE_Q4_K) {
      const int group = lane >> 2;
      // d, dmin and the twelve packed scale bytes as one 16-byte load (blocks are 16-byte aligned)
      const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
      const float d = half_bits_to_float(hdr.x & 0xffffu);
      const float dmin = half_bits_to_float(hdr.x >> 16);
      auto pbyte = [&](int i) -> int {
        const uint32_t word = i < 4 ? hdr.y : (i < 8 ? hdr.z : hdr.w);
        return (int)((word >> ((i & 3) * 8)) & 0xffu);
      };
      int sc, mn;
      if (group < 4) {
        sc = pbyte(group) & 0x3f;
        mn = pbyte(4 + group) & 0x3f;
      } else {
        sc = (pbyte(4 + group) & 0x0f) | ((pbyte(group - 4) >> 6) << 4);
        mn = (pbyte(4 + group) >> 4) | ((pbyte(group) >> 6) << 4);
      }
      mul = __fmul_rn(d, (float)sc);
      sub = __fmul_rn(dmin, (float)mn);
      const uint2 q8 = *reinterpret_cast<const uint2 *>(blk + 16 + (group >> 1) * 32 + (lane & 3) * 8);  // 8-byte aligned
      const int shift = (group & 1) * 4;
      // one shift + mask per word leaves each nibble alone in its byte: the conversions then read bytes
      const uint32_t m0 = (q8.x >> shift) & 0x0F0F0F0Fu, m1 = (q8.y >> shift) & 0x0F0F0F0Fu;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t word = j < 4 ? m0 : m1;
        const uint32_t q = (word >> ((j & 3) * 8)) & 0xffu;
        wv[j] = (float)q;
      }
    } else {
      const int half_index = lane >> 4, l16 = lane & 15;
      const float d = half_bits_to_float((uint32_t)blk[208] | ((uint32_t)blk[209] << 8));
      const uint8_t *lo = blk + half_index * 64 + (l16 & 7) * 8;
      const uint8_t *hi = blk + 128 + half_index * 32 + (l16 & 3) * 8;
      const int low_shift = (l16 >> 3) * 4, high_shift = (l16 >> 2) * 2;
      mul = __fmul_rn(d, (float)(int)(int8_t)blk[192 + (lane >> 1)]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int quant = (((lo[j] >> low_shift) & 0x0f) | (((hi[j] >> high_shift) & 0x03) << 4)) - 32;
        wv[j] = (float)quant;
      }
    }
    const int e0 = sb * 256 + lane * 8;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      if (b >= batch) break;
      const float4 x0 = *reinterpret_cast<const float4 *>(x + (size_t)b * ldx + e0);
      const float4 x1 = *reinterpret_cast<const float4 *>(x + (size_t)b * ldx + e0 + 4);
      float a = x0.x * wv[0];
      a = fmaf(x0.y, wv[1], a);
      a = fmaf(x0.z, wv[2], a);
      a = fmaf(x0.w, wv[3], a);
      a = fmaf(x1.x, wv[4], a);
      a = fmaf(x1.y, wv[5], a);
      a = fmaf(x1.z, wv[6], a);
      a = fmaf(x1.w, wv[7], a);
      float r = fmaf(mul, a, acc[b]);
      if constexpr (TYPE == RG_TYPE_Q4_K) r = fmaf(-sub, ((x0.x + x0.y) + (x0.z + x0.w)) + ((x1.x + x1.y) + (x1.z + x1.w)), r);
      acc[b] = r;
    }
  }
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    if (b >= batch) break;
    const float v = warp_sum(acc[b]);
    if (lane == 0) {
      float *dst = y + (size_t)b * ldy + row;
      *dst = (epi == EPI_RESIDUAL) ? __fadd_rn(*dst, v) : v;
    }
  }
}

// Decode-and-multiply GEMV for any block type, element by element (used when the activation rows are not
// 16-byte aligned): one warp per weight row, every lane decodes its elements with decode_element.
__global__ void block_gemv_kernel(int type, const uint8_t *w, int rows, int k, const float *x, int ldx, int batch, int epi,
                                  float *y, int ldy) {
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  const size_t base = (size_t)row * (size_t)k;
  float acc[8];
#pragma unroll
  for (int b = 0; b < 8; ++b) acc[b] = 0.0f;
  for (int i = lane; i < k; i += 32) {
    const float wv = decode_element(type, w, base + (size_t)i, nullptr);
#pragma unroll
    for (int b = 0; b < 8; ++b)
      if (b < batch) acc[b] = fmaf(x[(size_t)b * ldx + i], wv, acc[b]);
  }
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    if (b >= batch) break;
    const float v = warp_sum(acc[b]);
    if (lane == 0) {
      float *dst = y + (size_t)b * ldy + row;
      *dst = (epi == EPI_RESIDUAL) ? __fadd_rn(*dst, v) : v;
    }
  }
}

// ------------------------------------------------------------------------------ synthetic tensors
__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
// Sum of sixteen 16-bit uniforms (Irwin-Hall, n = 16) centred and scaled to unit variance:
// integer arithmetic up to one float multiply, so any host can reproduce it bit for bit.
__device__ __forceinline__ float synth_normal(uint64_t seed, uint64_t element) {
  uint32_t sum = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint64_t r = splitmix64(seed * 0xD1342543DE82EF95ull + element * 4 + i);
    sum += (uint32_t)(r & 0xffff) + (uint32_t)((r >> 16) & 0xffff) + (uint32_t)((r >> 32) & 0xffff) + (uint32_t)(r >> 48);
  }
  return (float)((int)sum - 524280) * (1.0f / 75674.5234375f);
}

__global__ void synth_kernel(int type, uint8_t *out, uint64_t seed, float std, uint64_t full_cols, uint64_t row0, uint64_t rows,
                             uint64_t col0, uint64_t cols) {
  const uint64_t bpr = cols / 32;  // 32-element groups per local row (dense types use the same tiling)
  const uint64_t gidx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gidx >= rows * bpr) return;
  const uint64_t r = gidx / bpr, cb = gidx - r * bpr;
  const uint64_t e0 = (row0 + r) * full_cols + col0 + cb * 32;
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __fmul_rn(synth_normal(seed, e0 + i), std);
  if (type == RG_TYPE_F32) {
    float *o = reinterpret_cast<float *>(out) + gidx * 32;
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = v[i];
  } else if (type == RG_TYPE_F16) {
    __half *o = reinterpret_cast<__half *>(out) + gidx * 32;
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = __float2half_rn(v[i]);
  } else if (type == RG_TYPE_Q8_0) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
    uint16_t *o = reinterpret_cast<uint16_t *>(out + gidx * 34);
    o[0] = __half_as_ushort(__float2half_rn(d));
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int q0 = (int)roundf(__fmul_rn(v[2 * i], id)), q1 = (int)roundf(__fmul_rn(v[2 * i + 1], id));
      o[1 + i] = (uint16_t)((q0 & 0xff) | ((q1 & 0xff) << 8));
    }
  } else {  // Q4_0
    float amax = 0.0f, mx = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (amax < fabsf(v[i])) {
        amax = fabsf(v[i]);
        mx = v[i];
      }
    const float d = __fdiv_rn(mx, -8.0f);
    const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
    uint16_t *o = reinterpret_cast<uint16_t *>(out + gidx * 18);
    o[0] = __half_as_ushort(__float2half_rn(d));
    uint8_t q[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int qi = (int)__fadd_rn(__fmul_rn(v[i], id), 8.5f);
      q[i] = (uint8_t)min(15, qi);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t b0 = q[2 * i] | (q[2 * i + 16] << 4), b1 = q[2 * i + 1] | (q[2 * i + 17] << 4);
      o[1 + i] = (uint16_t)(b0 | (b1 << 8));
    }
  }
}

// Dense (F32/F16) synthetic tensor: one element per thread, any column count.
__global__ void synth_dense_kernel(int type, uint8_t *out, uint64_t seed, float std, uint64_t full_cols, uint64_t row0,
                                   uint64_t rows, uint64_t col0, uint64_t cols) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * cols) return;
  const uint64_t r = i / cols, c = i - r * cols;
  const float v = __fmul_rn(synth_normal(seed, (row0 + r) * full_cols + col0 + c), std);
  if (type == RG_TYPE_F32)
    reinterpret_cast<float *>(out)[i] = v;
  else
    reinterpret_cast<__half *>(out)[i] = __float2half_rn(v);
}

// h = silu(g) * u for dense-weight gate/up projections; written packed and/or plain.
__global__ void swiglu_kernel(const float *g, const float *u, int n, int ld, int batch, __half *pack, float *out, int ldo) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (i >= n) return;
  const float h = swiglu(g[(size_t)b * ld + i], u[(size_t)b * ld + i]);
  if (pack) xpack_store(pack, 2 * batch, b, i, h);
  if (out) out[(size_t)b * ldo + i] = h;
}

// x[b, :] += partial[b, :] (residual add after a tensor-parallel all-reduce).
__global__ void add_rows_kernel(float *x, int ldx, const float *p, int ldp, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (i < n) x[(size_t)b * ldx + i] = __fadd_rn(x[(size_t)b * ldx + i], p[(size_t)b * ldp + i]);
}

__global__ void fill_kernel(float *out, size_t n, float v) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = v;
}

}  // namespace

// ============================================================================== launchers
cudaError_t launch_dequantize(int type, const uint8_t *bytes, size_t n, float *out, const LaunchCfg &cfg) {
  if (n == 0) return cudaSuccess;
  return launch(dequantize_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, cfg, type, bytes, n, out, cfg.status);
}
cudaError_t launch_row_gather(int type, const uint8_t *bytes, int cols, const int32_t *ids, int count, float *out, int ldo,
                              const LaunchCfg &cfg) {
  if (count == 0) return cudaSuccess;
  return launch(row_gather_kernel, dim3(count), dim3(256), 0, cfg, type, bytes, cols, ids, out, ldo);
}
cudaError_t launch_pack(const float *x, int ldx, int k, int batch, void *xpack, const LaunchCfg &cfg) {
  return launch(pack_kernel, dim3((k + 255) / 256, batch), dim3(256), 0, cfg, x, ldx, k, batch, static_cast<__half *>(xpack));
}
cudaError_t launch_unpack(const void *xpack, int k, int batch, float *x, int ldx, const LaunchCfg &cfg) {
  return launch(unpack_kernel, dim3((k + 255) / 256, batch), dim3(256), 0, cfg, static_cast<const __half *>(xpack), k, batch, x,
                ldx);
}
cudaError_t launch_rmsnorm_pack(const float *x, int ldx, const float *w, int d, float eps, int cols, const int32_t *col_map,
                                void *xpack, float *y, int ldy, const LaunchCfg &cfg) {
  // few columns: four CTAs per column, so the slices are packed side by side instead of by one CTA
  const unsigned parts = cols <= 64 && d >= 2048 ? 4u : 1u;
  return launch(rmsnorm_pack_kernel, dim3((unsigned)cols, parts), dim3(512), 0, cfg, x, ldx, w, d, eps, cols, col_map,
                static_cast<__half *>(xpack), y, ldy);
}
cudaError_t launch_rope_append(const RopeArgs &a, const LaunchCfg &cfg) {
  const int rope = a.rope_dim ? a.rope_dim : a.hd;
  if (rope != a.hd || a.qk_norm || a.q_bias || a.k_bias || a.v_bias) {
    if (rope < 2 || rope > a.hd || (rope & 1) || (a.qk_norm && (!a.q_norm || !a.k_norm)) || a.qk_norm > 2) return cudaErrorInvalidValue;
    const size_t smem = (size_t)(a.heads + a.kv_heads) * a.hd * sizeof(float);
    auto set = [&](auto kernel) {
      static DeviceOnce once;
      bool *flag = once.slot();
      if (flag && *flag) return cudaSuccess;
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      if (e == cudaSuccess && flag) *flag = true;
      return e;
    };
    if (smem > 160 * 1024) return cudaErrorInvalidValue;
    cudaError_t e = a.kv_f32 ? set(qkv_variant_kernel<float>) : set(qkv_variant_kernel<__half>);
    if (e != cudaSuccess) return e;
    if (a.kv_f32)
      return launch(qkv_variant_kernel<float>, dim3(a.cols), dim3(256), smem, cfg, a, static_cast<float *>(a.k_cache),
                    static_cast<float *>(a.v_cache));
    return launch(qkv_variant_kernel<__half>, dim3(a.cols), dim3(256), smem, cfg, a, static_cast<__half *>(a.k_cache),
                  static_cast<__half *>(a.v_cache));
  }
  const dim3 grid((unsigned)a.cols, a.cols <= 64 ? 4u : 1u);  // few columns: four CTAs share one
  if (a.kv_f32)
    return launch(rope_append_kernel<float>, grid, dim3(256), 0, cfg, a.qkv, a.heads, a.kv_heads, a.hd, a.ctx, a.col_seq,
                  a.col_pos, a.cos_t, a.sin_t, a.q_out, static_cast<float *>(a.k_cache), static_cast<float *>(a.v_cache));
  return launch(rope_append_kernel<__half>, grid, dim3(256), 0, cfg, a.qkv, a.heads, a.kv_heads, a.hd, a.ctx, a.col_seq,
                a.col_pos, a.cos_t, a.sin_t, a.q_out, static_cast<__half *>(a.k_cache), static_cast<__half *>(a.v_cache));
}
size_t attn_scratch_floats(int cols, int heads, int hd, int ctx) {
  const int splits = (ctx + ATTN_SPAN - 1) / ATTN_SPAN;
  return (size_t)cols * heads * splits * (hd + 2);
}
template <typename KV, int G, int HD>
static cudaError_t launch_attn_t(const AttnArgs &a, const LaunchCfg &cfg, int splits) {
  constexpr size_t smem = 2 * (size_t)ATTN_SPAN * HD * sizeof(KV);
  auto kernel = attn_split_kernel<KV, G, HD>;
  static DeviceOnce attr_once;  // per instantiation and device
  bool *attr_flag = attr_once.slot();
  if (!attr_flag || !*attr_flag) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    if (attr_flag) *attr_flag = true;
  }
  return launch(kernel, dim3(splits, a.kv_heads, a.cols), dim3(ATT_THREADS), smem, cfg, a.q, static_cast<const KV *>(a.k_cache),
                static_cast<const KV *>(a.v_cache), a.heads, a.kv_heads, a.ctx, a.col_seq, a.col_pos, a.scratch, splits,
                cfg.status);
}
template <typename KV, int HD>
static cudaError_t launch_attn_g(const AttnArgs &a, const LaunchCfg &cfg, int splits) {
  switch (a.heads / a.kv_heads) {
    case 1: return launch_attn_t<KV, 1, HD>(a, cfg, splits);
    case 2: return launch_attn_t<KV, 2, HD>(a, cfg, splits);
    case 4: return launch_attn_t<KV, 4, HD>(a, cfg, splits);
    case 8: return launch_attn_t<KV, 8, HD>(a, cfg, splits);
    default: return cudaErrorInvalidValue;
  }
}
bool attention_supported(int heads, int kv_heads, int hd) {
  if (kv_heads <= 0 || heads % kv_heads) return false;
  const int g = heads / kv_heads;
  return (hd == 64 || hd == 128) && (g == 1 || g == 2 || g == 4 || g == 8);
}
cudaError_t launch_attention(const AttnArgs &a, const LaunchCfg &cfg) {
  count_launch(LC_ATTN_SPLIT);
  if (!attention_supported(a.heads, a.kv_heads, a.hd)) return cudaErrorInvalidValue;
  const int splits = (a.ctx + ATTN_SPAN - 1) / ATTN_SPAN;
  cudaError_t e;
  if (a.kv_f32)
    e = a.hd == 128 ? launch_attn_g<float, 128>(a, cfg, splits) : launch_attn_g<float, 64>(a, cfg, splits);
  else
    e = a.hd == 128 ? launch_attn_g<__half, 128>(a, cfg, splits) : launch_attn_g<__half, 64>(a, cfg, splits);
  if (e != cudaSuccess) return e;
  return launch(attn_combine_kernel, dim3(a.heads, a.cols), dim3(MAX_HD), 0, cfg, (const float *)a.scratch, a.heads, a.hd,
                a.col_pos, splits, a.cols, static_cast<__half *>(a.out_pack), a.out_f32);
}
cudaError_t launch_select(const float *logits, int ld, int vocab, int cols, const float *uniforms, float temperature,
                          int32_t *out_ids, const LaunchCfg &cfg, const float *temps) {
  return launch(argmax_kernel, dim3((unsigned)cols), dim3(1024), 0, cfg, logits, ld, vocab, uniforms, temperature, temps, out_ids);
}
cudaError_t launch_argmax(const float *logits, int ld, int vocab, int cols, int32_t *out_ids, const LaunchCfg &cfg) {
  return launch_select(logits, ld, vocab, cols, nullptr, 1.0f, out_ids, cfg);
}
cudaError_t launch_advance(const int32_t *ids, int32_t *tokens, int32_t *pos, int32_t *history, int32_t *step_counter, int cols,
                           const LaunchCfg &cfg) {
  return launch(advance_kernel, dim3(1), dim3(32), 0, cfg, ids, tokens, pos, history, step_counter, cols);
}
cudaError_t launch_dense_gemv(const DenseGemvArgs &a, const LaunchCfg &cfg) {
  if (a.batch < 1 || a.batch > 8 || a.epi == EPI_SWIGLU) return cudaErrorInvalidValue;
  const dim3 grid((a.rows + 7) / 8), block(256);
  if (a.type == RG_TYPE_F32 || a.type == RG_TYPE_F16) count_launch(LC_DENSE_GEMV);
  if (a.type == RG_TYPE_F32)
    return launch(dense_gemv_kernel<float>, grid, block, 0, cfg, reinterpret_cast<const float *>(a.w), a.rows, a.k, a.x, a.ldx,
                  a.batch, a.epi, a.y, a.ldy);
  if (a.type == RG_TYPE_F16)
    return launch(dense_gemv_kernel<__half>, grid, block, 0, cfg, reinterpret_cast<const __half *>(a.w), a.rows, a.k, a.x, a.ldx,
                  a.batch, a.epi, a.y, a.ldy);
  if (a.type == RG_TYPE_Q4_0 || a.type == RG_TYPE_Q8_0) {  // rows whose K is not a multiple of 256
    if (a.k % 32) return cudaErrorInvalidValue;
    count_launch(LC_DENSE_GEMV);
    return launch(block_gemv_kernel, grid, block, 0, cfg, a.type, a.w, a.rows, a.k, a.x, a.ldx, a.batch, a.epi, a.y, a.ldy);
  }
  if (a.type == RG_TYPE_Q4_K || a.type == RG_TYPE_Q6_K) {
    count_launch(LC_KQUANT_GEMV);
    const bool aligned = (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (a.ldx & 3) == 0 && (a.k & 255) == 0 &&
                         (a.type == RG_TYPE_Q6_K || (reinterpret_cast<uintptr_t>(a.w) & 15) == 0);
    if (!aligned)
      return launch(block_gemv_kernel, grid, block, 0, cfg, a.type, a.w, a.rows, a.k, a.x, a.ldx, a.batch, a.epi, a.y, a.ldy);
    const size_t row_bytes = (size_t)(a.k >> 8) * (a.type == RG_TYPE_Q4_K ? 144 : 210);
    const size_t stage = 8 * row_bytes;
    if (row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(a.w) & 15) == 0 && stage <= 72 * 1024) {
      auto k4 = kquant_gemv_kernel<RG_TYPE_Q4_K, true>;
      auto k6 = kquant_gemv_kernel<RG_TYPE_Q6_K, true>;
      static DeviceOnce attr_once;  // per instantiation and device
      bool *attr_flag = attr_once.slot();
      if (!attr_flag || !*attr_flag) {
        cudaError_t e = cudaFuncSetAttribute(k4, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(k6, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
        if (e != cudaSuccess) return e;
        if (attr_flag) *attr_flag = true;
      }
      if (a.type == RG_TYPE_Q4_K)
        return launch(k4, grid, block, stage, cfg, a.w, a.rows, a.k, a.x, a.ldx, a.batch, a.epi, a.y, a.ldy, cfg.status);
      return launch(k6, grid, block, stage, cfg, a.w, a.rows, a.k, a.x, a.ldx, a.batch, a.epi, a.y, a.ldy, cfg.status);
    }
    if (a.type == RG_TYPE_Q4_K)
      return launch(kquant_gemv_kernel<RG_TYPE_Q4_K, false>, grid, block, 0, cfg, a.w, a.rows, a.k, a.x, a.ldx, a.batch, a.epi,
                    a.y, a.ldy, cfg.status);
    return launch(kquant_gemv_kernel<RG_TYPE_Q6_K, false>, grid, block, 0, cfg, a.w, a.rows, a.k, a.x, a.ldx, a.batch, a.epi,
                  a.y, a.ldy, cfg.status);
  }
  return cudaErrorInvalidValue;
}
cudaError_t launch_synth(int type, uint8_t *out, uint64_t seed, float std, uint64_t full_cols, uint64_t row0, uint64_t rows,
                         uint64_t col0, uint64_t cols, const LaunchCfg &cfg) {
  LaunchCfg plain = cfg;
  plain.pdl = false;
  if (type == RG_TYPE_F32 || type == RG_TYPE_F16) {
    const uint64_t n = rows * cols;
    if (n == 0) return cudaSuccess;
    return launch(synth_dense_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, plain, type, out, seed, std, full_cols,
                  row0, rows, col0, cols);
  }
  if (cols % 32 || col0 % 32) return cudaErrorInvalidValue;
  const uint64_t groups = rows * (cols / 32);
  if (groups == 0) return cudaSuccess;
  return launch(synth_kernel, dim3((unsigned)((groups + 127) / 128)), dim3(128), 0, plain, type, out, seed, std, full_cols, row0,
                rows, col0, cols);
}
cudaError_t launch_swiglu(const float *g, const float *u, int n, int ld, int batch, void *pack, float *out, int ldo,
                          const LaunchCfg &cfg) {
  return launch(swiglu_kernel, dim3((n + 255) / 256, batch), dim3(256), 0, cfg, g, u, n, ld, batch, static_cast<__half *>(pack),
                out, ldo);
}
cudaError_t launch_add_rows(float *x, int ldx, const float *p, int ldp, int n, int batch, const LaunchCfg &cfg) {
  return launch(add_rows_kernel, dim3((n + 255) / 256, batch), dim3(256), 0, cfg, x, ldx, p, ldp, n);
}
cudaError_t launch_fill_f32(float *out, size_t n, float v, const LaunchCfg &cfg) {
  if (n == 0) return cudaSuccess;
  LaunchCfg plain = cfg;
  plain.pdl = false;
  return launch(fill_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, plain, out, n, v);
}

// ------------------------------------------------------------------------------ no-allocation attention
// Decode attention for callers that must not allocate device memory while they run: a host
// runtime that hands out all of its HBM from its own arena at start-up (rustgrad's pooled CUDA
// allocator is one), a latency-critical serving loop in which a cudaMalloc would stall the
// device, or code running between the begin and end of a stream capture, where allocation calls
// are not permitted.  The split-context partial results that the ordinary entry point keeps in a
// cudaMalloc'ed buffer live here in a fixed array inside the library image instead.
//
// Limits and rules for users:
//  * heads * ceil(ctx / 128) * (head_dim + 2) must not exceed RG_NOALLOC_SCRATCH_FLOATS
//    (1 Mi floats = 4 MiB; e.g. 64 heads of 128 dims up to a context of 15 872 positions).
//    Larger problems are refused with RG_UNSUPPORTED_GEOMETRY before anything is launched.
//  * Every GPU that loads the library holds these 4 MiB until the process exits.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
//    prepares the kernels; make that first call outside any stream capture.
//  * All calls on a device share the one array.  Two calls whose kernels may overlap on the GPU
//    (different streams without an ordering between them) race on it; order them.  Nothing in
//    the array has to start at zero: each call overwrites every partial it later reads, and the
//    three control words in front of the partials are rewritten by a kernel at the start of each call.
namespace {
constexpr size_t NOALLOC_SCRATCH_FLOATS = size_t(1) << 20;
constexpr size_t NOALLOC_HEADER_FLOATS = 64;  // control words: sequence, position, status
static __device__ __align__(256) float g_noalloc_attn[NOALLOC_HEADER_FLOATS + NOALLOC_SCRATCH_FLOATS];

__global__ void noalloc_header_kernel(int32_t *header, int32_t pos) {
  header[0] = 0;    // the single sequence
  header[1] = pos;  // position of the new token
  header[2] = DEV_OK;
}

// The array's name is only a host-side handle; kernels need the device address, looked up once
// per device with that device current.
cudaError_t noalloc_base(float **out) {
  static std::mutex mu;
  static float *base[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (!base[dev]) {
    float *p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_noalloc_attn);
    if (e != cudaSuccess) return e;
    base[dev] = p;
  }
  *out = base[dev];
  return cudaSuccess;
}
}  // namespace

extern thread_local std::string g_last_error;

}  // namespace rg

extern "C" int32_t rg_b200_attention_decode_noalloc(const float *q_dev, const void *keys_dev, const void *values_dev, int32_t heads,
                                                    int32_t kv_heads, int32_t head_dim, int32_t ctx, int32_t n_pos, int32_t kv_f32,
                                                    float *out_dev, void *stream, int32_t wait) {
  using namespace rg;
  auto fail = [](int32_t status, const std::string &why) {
    g_last_error = why;
    return status;
  };
  if (!q_dev || !keys_dev || !values_dev || !out_dev) return fail(RG_INVALID_ARGUMENT, "null device pointer");
  // the K / V spans travel by bulk copies, which need 16-byte aligned global addresses (every row is a
  // multiple of 16 bytes); q and out are read and written as f32 words.  A pointer cut from the middle
  // of an arena is refused here rather than left to fault on the device.
  if ((reinterpret_cast<uintptr_t>(keys_dev) & 15) || (reinterpret_cast<uintptr_t>(values_dev) & 15))
    return fail(RG_INVALID_ARGUMENT, "keys_dev and values_dev must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(q_dev) & 3) || (reinterpret_cast<uintptr_t>(out_dev) & 3))
    return fail(RG_INVALID_ARGUMENT, "q_dev and out_dev must be 4-byte aligned");
  if (n_pos < 1 || ctx < n_pos) return fail(RG_INVALID_ARGUMENT, "need 1 <= n_pos <= ctx");
  if (heads < 1 || kv_heads < 1 || !attention_supported(heads, kv_heads, head_dim))
    return fail(RG_UNSUPPORTED_GEOMETRY, "head_dim must be 64 or 128 and query heads per kv head 1, 2, 4 or 8");
  const size_t need = attn_scratch_floats(1, heads, head_dim, ctx);
  if (need > NOALLOC_SCRATCH_FLOATS)
    return fail(RG_UNSUPPORTED_GEOMETRY, "the allocation-free attention holds " + std::to_string(NOALLOC_SCRATCH_FLOATS) +
                                             " scratch floats; heads * ceil(ctx / 128) * (head_dim + 2) = " +
                                             std::to_string(need) + " is beyond that");
  float *base = nullptr;
  cudaError_t e = noalloc_base(&base);
  if (e != cudaSuccess) return fail(RG_CUDA_ERROR, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
  int32_t *header = reinterpret_cast<int32_t *>(base);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  noalloc_header_kernel<<<1, 1, 0, st>>>(header, n_pos - 1);
  if ((e = cudaGetLastError()) != cudaSuccess) return fail(RG_CUDA_ERROR, std::string("header launch: ") + cudaGetErrorString(e));
  LaunchCfg cfg;
  cfg.stream = st;
  cfg.pdl = false;
  cfg.status = header + 2;
  AttnArgs a;
  a.q = q_dev;
  a.k_cache = keys_dev;
  a.v_cache = values_dev;
  a.kv_f32 = kv_f32 != 0;
  a.cols = 1;
  a.heads = heads;
  a.kv_heads = kv_heads;
  a.hd = head_dim;
  a.ctx = ctx;
  a.col_seq = header;
  a.col_pos = header + 1;
  a.scratch = base + NOALLOC_HEADER_FLOATS;
  a.out_f32 = out_dev;
  if ((e = launch_attention(a, cfg)) != cudaSuccess) return fail(RG_CUDA_ERROR, std::string("attention launch: ") + cudaGetErrorString(e));
  if (wait) {
    int status = 0;
    if ((e = cudaMemcpyAsync(&status, header + 2, sizeof(int), cudaMemcpyDeviceToHost, st)) != cudaSuccess ||
        (e = cudaStreamSynchronize(st)) != cudaSuccess)
      return fail(RG_CUDA_ERROR, std::string("synchronize: ") + cudaGetErrorString(e));
    if (status == DEV_TIMEOUT) return fail(RG_TIMEOUT, "a bounded device-side wait gave up");
    if (status) return fail(RG_CUDA_ERROR, "device status " + std::to_string(status));
  }
  return RG_OK;
}
