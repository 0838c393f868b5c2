// Causal GQA attention for a chunk of consecutive prompt tokens of one sequence on the tensor
// cores, for f16 K / V caches (src/ir/attention.rs:946-981,1157-1240 with the mask
// `col <= past + row` of src/models/transformer/layer.rs:374-380; softmax pieces of
// attention.rs:495-558 in the exp2 form, running max / sum across key tiles).
//
// Same work split as the f32 kernel of attn_prefill.cu: one CTA owns 64 score rows = (64 / G) query
// tokens x the G query heads that share one kv head, and walks the keys 0 .. last query position in
// tiles of 64.  Four warps, 16 rows each; all products run as mma.sync.m16n8k16 (f16 operands, f32
// accumulators):
//  * S = Q K^T: K rows are f16 in the cache, so they are exact operands as they lie ([key][hd] is the
//    column-major B operand); the f32 query is split into two f16 planes hi = f16(q), lo = f16(q - hi)
//    and both are multiplied, so the scores carry about 22 bits of the query.
//  * O += P V: the probabilities of a tile leave the score accumulators as the A operand of the next
//    product without passing through shared memory (two adjacent 8-key score tiles are one 16-key A
//    fragment), again as hi + lo planes; V rows are exact f16, read transposed by ldmatrix.
// Every f16 x f16 product is exact in the f32 accumulator, so what differs from the f32 kernel is
// the order of the sums and the 2^-22 tail of q and p.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdint.h>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int HD = 128;
constexpr int ROWS = 64;     // score rows per CTA
constexpr int TK = 64;       // keys per tile
constexpr int THREADS = 128;  // four warps x 16 rows
constexpr int LD = HD + 8;   // shared row pitch in halves: 272 bytes, so eight rows of an 8 x 8 matrix fall in distinct banks

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

// f32 -> f16 as the GEMM operand conversion does it: finite values beyond the f16 range saturate
__device__ __forceinline__ __half f16_sat(float v) {
  if (fabsf(v) > 65504.0f && fabsf(v) < __int_as_float(0x7f800000)) v = copysignf(65504.0f, v);
  return __float2half_rn(v);
}

template <int G>
__global__ void __launch_bounds__(THREADS) attn_prefill_tc_kernel(const PrefillAttnArgs A) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int TQ = ROWS / G;  // query tokens per CTA
  extern __shared__ __align__(16) uint8_t smem[];
  __half *q_hi = reinterpret_cast<__half *>(smem);  // [ROWS][LD]
  __half *q_lo = q_hi + ROWS * LD;
  __half *ks = q_lo + ROWS * LD;                    // [TK][LD]
  __half *vs = ks + TK * LD;                        // [TK][LD]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kvh = blockIdx.y;
  const int t0 = blockIdx.x * TQ;  // first query token of this CTA within the chunk
  if (t0 >= A.cols) return;
  const int nq = min(TQ, A.cols - t0);
  // row r = head * TQ + token  <->  query head kvh * G + head, token t0 + token; two f16 planes
  for (int i = tid; i < ROWS * (HD / 4); i += THREADS) {
    const int r = i / (HD / 4), c4 = i - r * (HD / 4);
    const int head = r / TQ, tok = r - head * TQ;
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (tok < nq) v = reinterpret_cast<const float4 *>(A.q + ((size_t)(t0 + tok) * A.heads + (size_t)(kvh * G + head)) * HD)[c4];
    uint2 hi, lo;
    split2(v.x, v.y, hi.x, lo.x);
    split2(v.z, v.w, hi.y, lo.y);
    *reinterpret_cast<uint2 *>(q_hi + r * LD + 4 * c4) = hi;
    *reinterpret_cast<uint2 *>(q_lo + r * LD + 4 * c4) = lo;
  }
  const __half *kc = static_cast<const __half *>(A.k_cache) + ((size_t)A.seq * A.kv_heads + kvh) * (size_t)A.ctx * HD;
  const __half *vc = static_cast<const __half *>(A.v_cache) + ((size_t)A.seq * A.kv_heads + kvh) * (size_t)A.ctx * HD;
  const int last_q = A.pos0 + t0 + nq - 1;  // last position any row of this CTA may see
  const float inv_scale = (float)(1.0 / (1.0 / sqrt((double)HD)));
  // this thread's two rows: 16 * warp + g and + 8
  int qpos[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = 16 * warp + g + 8 * h, tok = r % TQ;
    qpos[h] = tok < nq ? A.pos0 + t0 + tok : -1;  // -1: padding row, sees nothing
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  // ldmatrix row addresses of this lane (bytes from the start of a tile)
  const uint32_t a_off = (uint32_t)(((16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + (lane >> 4) * 8) * 2);   // A: Q rows
  const uint32_t kb_off = (uint32_t)((((lane & 7) + (lane >> 4) * 8) * LD + ((lane >> 3) & 1) * 8) * 2);              // B: two key tiles
  const uint32_t vb_off = (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * LD + (lane >> 4) * 8) * 2);              // B^T: two hd tiles
  const uint32_t qh_s = smem_u32(q_hi), ql_s = smem_u32(q_lo), ks_s = smem_u32(ks), vs_s = smem_u32(vs);

  for (int k0 = 0; k0 <= last_q; k0 += TK) {
    __syncthreads();  // the previous tile's K / V are no longer read (and Q is in place before the first tile)
    for (int i = tid; i < TK * (HD / 8); i += THREADS) {  // 16-byte pieces; keys beyond the last visible position read as zero
      const int key = i / (HD / 8), c = i - key * (HD / 8);
      uint4 kq = make_uint4(0u, 0u, 0u, 0u), vq = kq;
      if (k0 + key <= last_q) {
        kq = *reinterpret_cast<const uint4 *>(kc + (size_t)(k0 + key) * HD + 8 * c);
        vq = *reinterpret_cast<const uint4 *>(vc + (size_t)(k0 + key) * HD + 8 * c);
      }
      *reinterpret_cast<uint4 *>(ks + key * LD + 8 * c) = kq;
      *reinterpret_cast<uint4 *>(vs + key * LD + 8 * c) = vq;
    }
    __syncthreads();
    // ---- scores of 16 rows x 64 keys
    float s[TK / 8][4];
#pragma unroll
    for (int n = 0; n < TK / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
      uint32_t ah[4], al[4];
      ldsm4(ah, qh_s + a_off + kk * 32);
      ldsm4(al, ql_s + a_off + kk * 32);
#pragma unroll
      for (int n2 = 0; n2 < TK / 16; ++n2) {
        uint32_t b[4];
        ldsm4(b, ks_s + kb_off + (uint32_t)(n2 * 16 * LD * 2) + kk * 32);
        mma_f16(s[2 * n2], al, b[0], b[1]);  // the small plane first
        mma_f16(s[2 * n2], ah, b[0], b[1]);
        mma_f16(s[2 * n2 + 1], al, b[2], b[3]);
        mma_f16(s[2 * n2 + 1], ah, b[2], b[3]);
      }
    }
    // ---- scale, mask, online softmax: the four lanes of a quad share a row
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < TK / 8; ++n)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int kp = k0 + 8 * n + 2 * t + j;
          float &v = s[n][2 * h + j];
          v = kp <= qpos[h] ? __fdiv_rn(v, inv_scale) : -INFINITY;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[h], mx);
      float sum = 0.0f;
      corr[h] = 1.0f;
      if (m_new > -INFINITY) {
        corr[h] = exp2f(__fmul_rn(__fsub_rn(m_run[h], m_new), 1.44269504088896340736f));  // 0 when m_run is -inf
#pragma unroll
        for (int n = 0; n < TK / 8; ++n)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float e = exp2f(__fmul_rn(__fsub_rn(s[n][2 * h + j], m_new), 1.44269504088896340736f));
            s[n][2 * h + j] = e;
            sum += e;
          }
      } else {
#pragma unroll
        for (int n = 0; n < TK / 8; ++n) s[n][2 * h] = s[n][2 * h + 1] = 0.0f;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[h] = fmaf(l_run[h], corr[h], sum);
      m_run[h] = m_new;
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      o[n][0] *= corr[0];
      o[n][1] *= corr[0];
      o[n][2] *= corr[1];
      o[n][3] *= corr[1];
    }
    // ---- O += P V: two adjacent 8-key score tiles are one 16-key A fragment
#pragma unroll
    for (int kt = 0; kt < TK / 16; ++kt) {
      uint32_t ph[4], pl[4];
      split2(s[2 * kt][0], s[2 * kt][1], ph[0], pl[0]);          // row g,     keys 16kt + 2t, +1
      split2(s[2 * kt][2], s[2 * kt][3], ph[1], pl[1]);          // row g + 8
      split2(s[2 * kt + 1][0], s[2 * kt + 1][1], ph[2], pl[2]);  // row g,     keys 16kt + 8 + 2t, +1
      split2(s[2 * kt + 1][2], s[2 * kt + 1][3], ph[3], pl[3]);  // row g + 8
#pragma unroll
      for (int n2 = 0; n2 < HD / 16; ++n2) {
        uint32_t b[4];
        ldsm4_t(b, vs_s + vb_off + (uint32_t)(kt * 16 * LD * 2) + n2 * 32);
        mma_f16(o[2 * n2], pl, b[0], b[1]);
        mma_f16(o[2 * n2], ph, b[0], b[1]);
        mma_f16(o[2 * n2 + 1], pl, b[2], b[3]);
        mma_f16(o[2 * n2 + 1], ph, b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = 16 * warp + g + 8 * h, head = r / TQ, tok = r - head * TQ;
    if (tok >= nq) continue;
    const float inv = __frcp_rn(l_run[h]);
    const size_t col = (size_t)(kvh * G + head) * HD + 2 * t;
    if (A.out16_hi) {  // the operand planes of the output projection, rounded as the f32 -> operand conversion rounds
      const size_t at = (size_t)(t0 + tok) * A.out16_ld + col;
      uint16_t *hi = static_cast<uint16_t *>(A.out16_hi) + at;
      uint16_t *lo = A.out16_lo ? static_cast<uint16_t *>(A.out16_lo) + at : nullptr;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        const float v0 = __fmul_rn(o[n][2 * h], inv), v1 = __fmul_rn(o[n][2 * h + 1], inv);
        if (A.out16_f16) {
          const __half h0 = f16_sat(v0), h1 = f16_sat(v1);
          *reinterpret_cast<uint32_t *>(hi + 8 * n) = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
          if (lo)
            *reinterpret_cast<uint32_t *>(lo + 8 * n) = (uint32_t)__half_as_ushort(f16_sat(v0 - __half2float(h0))) |
                                                         ((uint32_t)__half_as_ushort(f16_sat(v1 - __half2float(h1))) << 16);
        } else {
          *reinterpret_cast<uint32_t *>(hi + 8 * n) = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v0)) |
                                                       ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v1)) << 16);
        }
      }
      continue;
    }
    float *dst = A.out + (size_t)(t0 + tok) * A.heads * HD + col;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
      *reinterpret_cast<float2 *>(dst + 8 * n) = make_float2(__fmul_rn(o[n][2 * h], inv), __fmul_rn(o[n][2 * h + 1], inv));
  }
}

template <int G>
cudaError_t launch_t(const PrefillAttnArgs &a, const LaunchCfg &cfg) {
  auto kernel = attn_prefill_tc_kernel<G>;
  constexpr size_t smem = (size_t)(2 * ROWS + 2 * TK) * LD * sizeof(__half);
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

}  // namespace

// The f16-cache form of launch_attention_prefill (attn_prefill.cu checks the arguments and picks).
cudaError_t launch_attention_prefill_tc(const PrefillAttnArgs &a, const LaunchCfg &cfg) {
  count_launch(LC_ATTN_PREFILL_TC);
  switch (a.heads / a.kv_heads) {
    case 1: return launch_t<1>(a, cfg);
    case 2: return launch_t<2>(a, cfg);
    case 4: return launch_t<4>(a, cfg);
    case 8: return launch_t<8>(a, cfg);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace rg
