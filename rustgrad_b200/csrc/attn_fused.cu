// Decode attention for one or two new tokens in ONE launch: RoPE of q and k, KV-cache append,
// split-context GQA attention and the combine of the spans
// (src/models/transformer/layer.rs:349-421 with src/ir/attention.rs:946-981,1157-1240; mask of
// layer.rs:374-380 for a single new row; softmax pieces of attention.rs:495-558).
//
// One CTA per (context span, kv head, column).  The CTA rotates the query heads that share its kv
// head into shared memory; the CTA whose span ends with the new token also rotates k, writes the k
// and v rows into the cache and into its own staging buffer (that row is produced here, so it is
// not part of the bulk copy).  K and V spans are staged by two bulk copies of the TMA engine.  Each
// CTA leaves [max, sum, out[hd]] per head in a scratch; the last CTA of a (column, kv head) to
// arrive (one atomic counter) combines the spans and writes the attention output, so no second
// launch is needed.  The span length adapts to the position so that short contexts still spread
// over the SMs.  Waits are bounded (status word).
#include <cuda_fp16.h>
#include <math.h>
#include <stdlib.h>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;
constexpr int MAX_G = 8;
constexpr int STAGE_BYTES = 65536;  // K span + V span
constexpr int SC_POS = 256;         // most positions a span can hold (head_dim 64, f16)

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
template <int N>
__device__ __forceinline__ void load_n(const float *p, float (&v)[N]) {
#pragma unroll
  for (int i = 0; i < N / 4; ++i) {
    const float4 f = reinterpret_cast<const float4 *>(p)[i];
    v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
  }
}
template <int N>
__device__ __forceinline__ void load_n(const __half *p, float (&v)[N]) {
  if constexpr (N == 8) {
    const uint4 u = *reinterpret_cast<const uint4 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
  } else {
    const uint2 u = *reinterpret_cast<const uint2 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
  }
}
__device__ __forceinline__ float2 load2(const float *p) { return *reinterpret_cast<const float2 *>(p); }
__device__ __forceinline__ float2 load2(const __half *p) { return __half22float2(*reinterpret_cast<const __half2 *>(p)); }

__host__ __device__ constexpr int span_max(int hd, int kv_bytes) { return STAGE_BYTES / (2 * hd * kv_bytes); }

// Span length for a context of `total` positions: spread over `per_head` CTAs, multiples of 16.
__host__ __device__ inline int span_for(int total, int per_head, int smax) {
  int span = (((total + per_head - 1) / per_head) + 15) & ~15;
  if (span < 16) span = 16;
  if (span < 64 && total > 64) span = 64;  // shorter spans only add partial results for the combine to gather
  return span > smax ? smax : span;
}

// Sum over the 16 lanes of a half-warp of NV values per lane (NV = 16, 8 or 4): while more than
// one value is left, each level halves them (a lane keeps the half its lane bit selects and adds
// the partner's copy of it), then plain butterfly adds.  Returns the total of value index
// sub >> log2(16 / NV); 15 shuffles for 16 values instead of 64.
template <int NV>
__device__ __forceinline__ float reduce_scatter16(float (&val)[NV], int sub) {
  int n = NV;
#pragma unroll
  for (int off = 8; off >= 1; off >>= 1) {
    if (n > 1) {
      n >>= 1;
      const bool up = (sub & off) != 0;
#pragma unroll
      for (int j = 0; j < NV / 2; ++j)
        if (j < n) {
          const float a = val[j], b = val[j + n];
          const float send = up ? a : b, keep = up ? b : a;
          val[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    } else {
      val[0] += __shfl_xor_sync(0xffffffffu, val[0], off);
    }
  }
  return val[0];
}

template <typename KV, int HD, int G>
__global__ void __launch_bounds__(THREADS, 2) attn_fused_kernel(const FusedAttnArgs A, int per_head, int *status,
                                                                 unsigned long long *trace) {
  // A.early: the positions and the cached rows of earlier positions were written at least one
  // attention launch ago, and every attention launch lets its dependents start only after its own
  // dependency wait, so they are complete whenever this CTA runs: the position, the rotation
  // factors and the bulk copies of the cached spans need not wait for the projection kernel.
  if (!A.early) pdl_wait();
  constexpr int SMAX = span_max(HD, (int)sizeof(KV));
  constexpr int DPL = HD / 16;  // dims per lane in the score phase
  const int c = blockIdx.z, kvh = blockIdx.y, sp = blockIdx.x;
  const int pos = A.col_pos[c], seq = A.col_seq[c];
  const int total = pos + 1;
  const int span = span_for(total, per_head, SMAX);
  const int nspl = (total + span - 1) / span;
  if (sp >= nspl) {
    pdl_launch_dependents();
    return;
  }
  const int p0 = sp * span;
  const int np = min(span, total - p0);
  const bool has_new = (p0 + np == total);
  const int ncopy = has_new ? np - 1 : np;

  extern __shared__ __align__(128) uint8_t smem[];
  KV *ks = reinterpret_cast<KV *>(smem);
  KV *vs = ks + (size_t)SMAX * HD;
  float *qs = reinterpret_cast<float *>(smem + STAGE_BYTES);  // [G][HD]
  float *sc = qs + MAX_G * HD;                                // [SMAX][MAX_G]
  float *ml = sc + SC_POS * MAX_G;                            // [G][2]
  __shared__ __align__(8) uint64_t bar;
  __shared__ int dead_flag, last_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(&bar, 1);
    dead_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  KV *kc = static_cast<KV *>(A.k_cache), *vc = static_cast<KV *>(A.v_cache);
  const size_t row0 = ((size_t)seq * A.kv_heads + kvh) * A.ctx + p0;
  if (tid == 0 && ncopy > 0) {
    const uint32_t bytes = (uint32_t)((size_t)ncopy * HD * sizeof(KV));
    mbar_expect_tx(&bar, 2 * bytes);
    bulk_g2s(ks, kc + row0 * HD, bytes, &bar);
    bulk_g2s(vs, vc + row0 * HD, bytes, &bar);
  }
  const int qw = A.heads * HD, kw = A.kv_heads * HD;
  const float *row = A.qkv + (size_t)c * (qw + 2 * kw);
  const float *ct = A.cos_t + (size_t)pos * (HD / 2), *st = A.sin_t + (size_t)pos * (HD / 2);
  float cs0 = 0.0f, sn0 = 0.0f;  // rotation factors of this thread's first pair (constant tables)
  if (tid < G * (HD / 2)) {
    cs0 = ct[tid % (HD / 2)];
    sn0 = st[tid % (HD / 2)];
  }
  const bool tr_first = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  if (tid == 0) trace_stamp(trace, 0, tr_first, false);  // CTA started, K / V copies issued
  if (A.early) pdl_wait();
  pdl_launch_dependents();
  if (tid == 0) trace_stamp(trace, 1, tr_first, false);  // grid dependency resolved
  // pairs (2i, 2i+1) of the projection rotate into (i, HD/2 + i) (layer.rs:349-371)
  for (int it = tid; it < G * (HD / 2); it += THREADS) {
    const int gq = it / (HD / 2), i = it - gq * (HD / 2);
    const float2 xv = reinterpret_cast<const float2 *>(row + (size_t)(kvh * G + gq) * HD)[i];
    const float cs = it == tid ? cs0 : ct[i], sn = it == tid ? sn0 : st[i];
    qs[gq * HD + i] = __fsub_rn(__fmul_rn(xv.x, cs), __fmul_rn(xv.y, sn));
    qs[gq * HD + HD / 2 + i] = __fadd_rn(__fmul_rn(xv.y, cs), __fmul_rn(xv.x, sn));
  }
  if (has_new) {
    for (int i = tid; i < HD / 2; i += THREADS) {
      const float2 xv = reinterpret_cast<const float2 *>(row + qw + (size_t)kvh * HD)[i];
      const float cs = i == tid ? cs0 : ct[i], sn = i == tid ? sn0 : st[i];
      const KV y1 = to_kv<KV>(__fsub_rn(__fmul_rn(xv.x, cs), __fmul_rn(xv.y, sn)));
      const KV y2 = to_kv<KV>(__fadd_rn(__fmul_rn(xv.y, cs), __fmul_rn(xv.x, sn)));
      KV *g = kc + (row0 + (np - 1)) * HD, *s = ks + (size_t)(np - 1) * HD;
      g[i] = y1, g[HD / 2 + i] = y2;
      s[i] = y1, s[HD / 2 + i] = y2;
    }
    for (int j = tid; j < HD; j += THREADS) {
      const KV v = to_kv<KV>(row[qw + kw + (size_t)kvh * HD + j]);
      vc[(row0 + (np - 1)) * HD + j] = v;
      vs[(size_t)(np - 1) * HD + j] = v;
    }
  }
  __syncthreads();
  if (ncopy > 0) mbar_wait_bounded(&bar, 0, &dead_flag, status);
  if (tid == 0) trace_stamp(trace, 2, tr_first, false);  // q rotated, K / V spans in shared memory
  // ---- scores: 16 lanes per position; scale = 1 / f32(sqrt(hd)) applied as a division (attention.rs:1183-1188)
  const float inv_scale = (float)(1.0 / (1.0 / sqrt((double)HD)));
  {
    // 16 lanes per position, DPL dims per lane; a K row is converted once and used by GH heads;
    // eight positions per warp in flight (four per half-warp)
    constexpr int GH = G < 4 ? G : 4, NV = 4 * GH;
    const int sub = lane & 15, hi = lane >> 4;
    for (int g0 = 0; g0 < G; g0 += GH) {
      float qr[GH][DPL];
#pragma unroll
      for (int h = 0; h < GH; ++h)
#pragma unroll
        for (int i = 0; i < DPL; ++i) qr[h][i] = qs[(g0 + h) * HD + sub * DPL + i];
      for (int base = 0; base < np; base += 8 * WARPS) {
        float dot[NV];  // index u * GH + h
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int p = base + u * 2 * WARPS + warp * 2 + hi;
#pragma unroll
          for (int h = 0; h < GH; ++h) dot[u * GH + h] = 0.0f;
          if (p < np) {
            float kr[DPL];
            load_n<DPL>(ks + (size_t)p * HD + sub * DPL, kr);
#pragma unroll
            for (int h = 0; h < GH; ++h)
#pragma unroll
              for (int i = 0; i < DPL; ++i) dot[u * GH + h] = fmaf(qr[h][i], kr[i], dot[u * GH + h]);
          }
        }
        const float tot = reduce_scatter16<NV>(dot, sub);
        const int v = sub / (16 / NV), u = v / GH, h = v - u * GH;
        const int p = base + u * 2 * WARPS + warp * 2 + hi;
        if ((sub & (16 / NV - 1)) == 0 && p < np) sc[p * MAX_G + g0 + h] = __fdiv_rn(tot, inv_scale);
      }
    }
  }
  __syncthreads();
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
  __syncthreads();
  // ---- P.V: one thread per (pair of dims, position class p mod PG) for all heads, so a V pair is
  // converted once; the PG partial sums meet in the K staging buffer (free after the scores)
  constexpr int PG = THREADS / (HD / 2);
  static_assert(PG * MAX_G * HD * 4 <= STAGE_BYTES / 2, "partial sums fit the K staging buffer");
  float *pvs = reinterpret_cast<float *>(smem);  // [PG][G][HD]
  {
    const int pg = tid / (HD / 2), dp = tid - pg * (HD / 2);
    float acc[G][2];
#pragma unroll
    for (int h = 0; h < G; ++h) acc[h][0] = acc[h][1] = 0.0f;
#pragma unroll 4
    for (int p = pg; p < np; p += PG) {
      const float2 vv = load2(vs + (size_t)p * HD + 2 * dp);
      float pr[G];
      if constexpr (G % 4 == 0) {
#pragma unroll
        for (int h4 = 0; h4 < G / 4; ++h4) {
          const float4 f = *reinterpret_cast<const float4 *>(sc + p * MAX_G + 4 * h4);
          pr[4 * h4] = f.x, pr[4 * h4 + 1] = f.y, pr[4 * h4 + 2] = f.z, pr[4 * h4 + 3] = f.w;
        }
      } else {
#pragma unroll
        for (int h = 0; h < G; ++h) pr[h] = sc[p * MAX_G + h];
      }
#pragma unroll
      for (int h = 0; h < G; ++h) {
        acc[h][0] = fmaf(pr[h], vv.x, acc[h][0]);
        acc[h][1] = fmaf(pr[h], vv.y, acc[h][1]);
      }
    }
#pragma unroll
    for (int h = 0; h < G; ++h)
      *reinterpret_cast<float2 *>(pvs + ((size_t)pg * G + h) * HD + 2 * dp) = make_float2(acc[h][0], acc[h][1]);
  }
  __syncthreads();
  for (int o = tid; o < G * (HD / 2); o += THREADS) {
    const int gq = o / (HD / 2), dp = o - gq * (HD / 2);
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int pg = 0; pg < PG; ++pg) {
      const float2 f = *reinterpret_cast<const float2 *>(pvs + ((size_t)pg * G + gq) * HD + 2 * dp);
      a0 += f.x;
      a1 += f.y;
    }
    float *dst = A.scratch + (((size_t)c * A.heads + (size_t)(kvh * G + gq)) * A.max_splits + sp) * (HD + 2);
    dst[2 + 2 * dp] = a0;
    dst[2 + 2 * dp + 1] = a1;
    if (dp == 0) {
      dst[0] = ml[gq * 2];
      dst[1] = ml[gq * 2 + 1];
    }
  }
  __syncthreads();
  if (tid == 0) trace_stamp(trace, 3, tr_first, false);  // this span's partial result written
  if (tid == 0) {
    unsigned *counter = A.counters + (size_t)c * A.kv_heads + kvh;
    int last = 1;
    if (nspl > 1) {
      __threadfence();  // this CTA's partial results before its arrival
      const unsigned old = atomicAdd(counter, 1u);
      last = (old == (unsigned)(nspl - 1));
      if (last) {
        *counter = 0u;    // every arrival of this step has happened
        __threadfence();  // the other spans' results before the combine reads them
      }
    }
    last_flag = last;
    trace_stamp(trace, 4, tr_first, false);  // arrival counted
  }
  __syncthreads();
  if (!last_flag) return;
  if (tid == 0 && kvh == 0 && c == 0) trace_stamp(trace, 8, true, false);  // last span of kv head 0 arrived (slot 8)
  // ---- combine.  The span headers (max, sum) and the first CB spans of this thread's output
  // column are requested together, before the weights exist: one round trip to L2 instead of one
  // for the headers and one per batch of spans (a dependent load-use loop would pay it per span).
  constexpr int CB = 40;
  constexpr int HPT = 6;  // headers per thread: 2 * MAX_G * split cap <= HPT * THREADS
  float *hdr = sc;  // [G][nspl][2] then weights [G][nspl]; the scores are no longer needed
  float *wts = sc + 2 * G * nspl;  // 3 * G * nspl floats in all: the launcher caps the number of spans
  const int nh = G * nspl * 2, nout = G * (HD / 2);
  const float *head0 = A.scratch + ((size_t)c * A.heads + (size_t)kvh * G) * A.max_splits * (HD + 2);
  float hreg[HPT];
#pragma unroll
  for (int j = 0; j < HPT; ++j) {
    const int i = tid + j * THREADS;
    hreg[j] = 0.0f;
    if (i < nh) {
      const int gq = i / (nspl * 2), r = i - gq * nspl * 2;
      hreg[j] = __ldcg(head0 + ((size_t)gq * A.max_splits + (r >> 1)) * (HD + 2) + (r & 1));
    }
  }
  auto column = [&](int o) {
    const int gq = o / (HD / 2), d = 2 * (o - gq * (HD / 2));
    return head0 + (size_t)gq * A.max_splits * (HD + 2) + 2 + d;
  };
  float2 v0[CB];
  {
    const float *base = column(tid < nout ? tid : 0);
#pragma unroll
    for (int j = 0; j < CB; ++j)
      v0[j] = (tid < nout && j < nspl) ? __ldcg(reinterpret_cast<const float2 *>(base + (size_t)j * (HD + 2))) : make_float2(0.0f, 0.0f);
  }
#pragma unroll
  for (int j = 0; j < HPT; ++j)
    if (tid + j * THREADS < nh) hdr[tid + j * THREADS] = hreg[j];
  __syncthreads();
  if (tid == 0 && kvh == 0 && c == 0) trace_stamp(trace, 10, true, false);  // span headers gathered (slot 10)
  if (warp < G) {
    const int gq = warp;
    float M = -INFINITY;
    for (int s = lane; s < nspl; s += 32) M = fmaxf(M, hdr[(gq * nspl + s) * 2]);
    M = warp_max(M);
    float L = 0.0f;
    for (int s = lane; s < nspl; s += 32) {
      const float wgt = exp2f(__fmul_rn(__fsub_rn(hdr[(gq * nspl + s) * 2], M), 1.44269504088896340736f));
      wts[gq * nspl + s] = wgt;
      L = fmaf(hdr[(gq * nspl + s) * 2 + 1], wgt, L);
    }
    L = warp_sum(L);
    if (lane == 0) ml[gq * 2 + 1] = __frcp_rn(L);
  }
  __syncthreads();
  if (tid == 0 && kvh == 0 && c == 0) trace_stamp(trace, 11, true, false);  // span weights ready (slot 11)
  for (int o = tid; o < nout; o += THREADS) {
    const int gq = o / (HD / 2), d = 2 * (o - gq * (HD / 2));
    const float *base = column(o);
    float a0 = 0.0f, a1 = 0.0f;
    for (int s0 = 0; s0 < nspl; s0 += CB) {  // spans in order; CB independent loads per round
      if (o != tid || s0 != 0) {             // the first round of the first column is already here
#pragma unroll
        for (int j = 0; j < CB; ++j)
          v0[j] = (s0 + j < nspl) ? __ldcg(reinterpret_cast<const float2 *>(base + (size_t)(s0 + j) * (HD + 2))) : make_float2(0.0f, 0.0f);
      }
#pragma unroll
      for (int j = 0; j < CB; ++j)
        if (s0 + j < nspl) {
          const float wgt = wts[gq * nspl + s0 + j];
          a0 = fmaf(v0[j].x, wgt, a0);
          a1 = fmaf(v0[j].y, wgt, a1);
        }
    }
    float *dst = A.out + (size_t)c * A.heads * HD + (size_t)(kvh * G + gq) * HD + d;
    const float o0 = __fmul_rn(a0, ml[gq * 2 + 1]), o1 = __fmul_rn(a1, ml[gq * 2 + 1]);
    dst[0] = o0;
    dst[1] = o1;
    if (tid == 0 && kvh == 0 && c == 0) trace_stamp(trace, 12, true, false);  // first output pair stored (slot 12)
    if (A.xpack_out) {
      const int e = (kvh * G + gq) * HD + d;
      xpack_store(static_cast<__half *>(A.xpack_out), 2 * A.cols, c, e, o0);
      xpack_store(static_cast<__half *>(A.xpack_out), 2 * A.cols, c, e + 1, o1);
    }
    if (A.pack_out) {
      // The sixteen lanes of a half-warp hold one 32-element block of the output projection's input
      // (lane j: elements 2j, 2j + 1): pack it as block fixed point for the integer GEMV (rg_device.cuh).
      const int e_glob = (kvh * G + gq) * HD + d, kbo = e_glob >> 5, j = lane & 15;
      const int kb_all = A.heads * HD / 32;
      const bool q4 = A.pack_type == RG_TYPE_Q4_0;
      float m = fmaxf(fabsf(o0), fabsf(o1));
#pragma unroll
      for (int off = 1; off < 16; off <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
      const unsigned bad = __ballot_sync(0xffffffffu, !(fabsf(o0) <= 3.0e38f) || !(fabsf(o1) <= 3.0e38f));
      if ((bad >> (lane & 16)) & 0xFFFFu) m = __uint_as_float(0x7f800000u);  // keep NaN / inf visible
      const uint32_t E = __float_as_uint(m) >> 23, XBITS = q4 ? 25u : 29u;
      float sc_b = 0.0f;
      int X0 = 0, X1 = 0;
      if (E >= 40u && E < 255u) {
        sc_b = __uint_as_float((E - XBITS) << 23);
        const float up = __uint_as_float((254u + XBITS - E) << 23);
        X0 = __float2int_rn(o0 * up);
        X1 = __float2int_rn(o1 * up);
      } else if (E == 255u) {
        sc_b = __uint_as_float(0x7fc00000u);
        X0 = j == 0 ? 1 : 0;
      }
      int t_lo = 0, t_hi = 0;
      if (q4) {
        int sum = X0 + X1;
#pragma unroll
        for (int off = 1; off < 16; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        t_lo = (sum & 0x1FF) << 7;
        t_hi = sum >> 9;
        const int p0 = __shfl_xor_sync(0xffffffffu, X0, 8), p1 = __shfl_xor_sync(0xffffffffu, X1, 8);
        if (j < 8) {
          X0 <<= 4;
          X1 <<= 4;
        } else {
          X0 -= p0 << 4;
          X1 -= p1 << 4;
        }
      }
      const uint32_t Y0 = (uint32_t)X0 + 0x80808080u, Y1 = (uint32_t)X1 + 0x80808080u;
      uint8_t *dq = A.pack_out + (size_t)kbo * 128 + ((j & 7) >> 1) * 8 + (j >> 3) * 4 + (j & 1) * 2;
#pragma unroll
      for (int dg = 0; dg < 4; ++dg) {
        const uint32_t b0 = ((Y0 >> (8 * dg)) & 0xFFu) ^ 0x80u, b1 = ((Y1 >> (8 * dg)) & 0xFFu) ^ 0x80u;
        *reinterpret_cast<uint16_t *>(dq + dg * 32) = (uint16_t)(b0 | (b1 << 8));
      }
      if (j == 0)
        *reinterpret_cast<float4 *>(A.pack_out + xq_side_offset(kb_all) + (size_t)kbo * 16) =
            make_float4(sc_b, __int_as_float(t_lo), sc_b, __int_as_float(t_hi));
    }
  }
  if (tid == 0 && kvh == 0 && c == 0) trace_stamp(trace, 9, true, false);  // combined output of kv head 0 stored (slot 9)
}

template <typename KV, int HD, int G>
cudaError_t launch_t(const FusedAttnArgs &a, const LaunchCfg &cfg) {
  auto kernel = attn_fused_kernel<KV, HD, G>;
  constexpr size_t smem = STAGE_BYTES + (MAX_G * HD + SC_POS * MAX_G + 2 * MAX_G) * sizeof(float);
  static_assert(span_max(HD, (int)sizeof(KV)) <= SC_POS, "score buffer");
  static DeviceOnce attr_once;  // per instantiation and device
  bool *attr_flag = attr_once.slot();
  if (!attr_flag || !*attr_flag) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    // same shared-memory / L1 split as the GEMV kernels on either side: no reconfiguration between launches
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    if (attr_flag) *attr_flag = true;
  }
  const int sms = cfg.sm_count > 0 ? cfg.sm_count : 148;
  const int per_head = fused_attn_per_head(sms, a.kv_heads, a.cols);
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3((unsigned)a.max_splits, (unsigned)a.kv_heads, (unsigned)a.cols);
  lc.blockDim = dim3(THREADS);
  lc.dynamicSmemBytes = smem;
  lc.stream = cfg.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = cfg.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&lc, kernel, a, per_head, cfg.status, cfg.trace);
}

template <int G>
cudaError_t launch_g(const FusedAttnArgs &a, const LaunchCfg &cfg) {
  if (a.hd == 128) return a.kv_f32 ? launch_t<float, 128, G>(a, cfg) : launch_t<__half, 128, G>(a, cfg);
  return a.kv_f32 ? launch_t<float, 64, G>(a, cfg) : launch_t<__half, 64, G>(a, cfg);
}

}  // namespace

int fused_attn_per_head(int sm_count, int kv_heads, int cols) {
  static const int waves = [] {
    const char *v = getenv("RG_B200_ATTN_WAVES");
    const int w = v ? atoi(v) : 2;  // two spans per SM in flight: shorter spans, shorter dependent chains
    return w >= 1 && w <= 3 ? w : 1;
  }();
  const int n = waves * sm_count / (kv_heads * (cols > 0 ? cols : 1));
  return n > 1 ? n : 1;
}

int fused_attn_max_splits(int ctx, int hd, bool kv_f32, int sm_count, int kv_heads) {
  const int smax = span_max(hd, kv_f32 ? 4 : 2);
  const int per_head = fused_attn_per_head(sm_count, kv_heads, 1);
  const int by_ctx = (ctx + smax - 1) / smax;
  // span_for never goes below 64 positions once the context exceeds 64 (and a context of up to 64
  // has at most four spans of 16), so few kv heads do not mean hundreds of spans
  int by_floor = (ctx + 63) / 64;
  if (by_floor < 4) by_floor = 4;
  const int spread = per_head < by_floor ? per_head : by_floor;
  return (spread > by_ctx ? spread : by_ctx) + 1;
}

int fused_attn_split_cap() { return SC_POS / 3; }  // span headers + weights of all heads fit the score buffer

bool fused_attention_supported(int heads, int kv_heads, int hd) {
  if (kv_heads < 1 || heads % kv_heads) return false;
  const int g = heads / kv_heads;
  return (hd == 64 || hd == 128) && (g == 1 || g == 2 || g == 4 || g == 8);
}

cudaError_t launch_attention_fused(const FusedAttnArgs &a, const LaunchCfg &cfg) {
  count_launch(LC_ATTN_FUSED);
  if (!fused_attention_supported(a.heads, a.kv_heads, a.hd) || a.cols < 1 || !a.counters || !a.scratch || !a.out ||
      a.max_splits > fused_attn_split_cap())
    return cudaErrorInvalidValue;
  if (a.pack_out && (a.cols != 1 || (reinterpret_cast<uintptr_t>(a.pack_out) & 127))) return cudaErrorInvalidValue;
  switch (a.heads / a.kv_heads) {
    case 1: return launch_g<1>(a, cfg);
    case 2: return launch_g<2>(a, cfg);
    case 4: return launch_g<4>(a, cfg);
    case 8: return launch_g<8>(a, cfg);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace rg
