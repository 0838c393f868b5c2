// Device-side helpers shared by the sm_100a kernels: IEEE half conversion that is bit-exact with
// rustgrad's f16_to_f32 (src/tensor/scalar.rs:110-135), mbarrier / bulk-copy / PDL wrappers with
// bounded waits, the m16n8k16 tensor-core instruction, and the packed-activation layout.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rg {

// ---------------------------------------------------------------------------------------------
// Status word written by kernels instead of trapping.  Host code reads it after each step.
// ---------------------------------------------------------------------------------------------
enum : int { DEV_OK = 0, DEV_TIMEOUT = 1, DEV_NON_FINITE = 2, DEV_BAD_INDEX = 3 };

// ---------------------------------------------------------------------------------------------
// Scalars
// ---------------------------------------------------------------------------------------------
// The hardware half->float conversion is exact for every bit pattern (subnormals included), which
// is what the reference's software conversion computes.
__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
  return __half2float(__ushort_as_half((unsigned short)bits16));
}

__device__ __forceinline__ bool finite_f32(float v) { return fabsf(v) <= 3.402823466e+38f; }

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of a decode step calls pdl_wait() before it
// touches memory another kernel of the step writes, so completion stays transitive along the
// chain; constant weights may be prefetched before it.
// ---------------------------------------------------------------------------------------------
// Hint that [p, p + bytes) will be read soon: the lines are brought into L2 and nothing waits for
// them.  p and bytes are multiples of 16.
__device__ __forceinline__ void l2_prefetch_bulk(const void *p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// mbarrier + bulk async copy (TMA engine, untiled form)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls, records DEV_TIMEOUT in *status and raises the
// CTA-wide `dead` flag so that later waits of the same CTA return at once.  Returns false on
// timeout; the caller carries on (its results are garbage, the host sees the status).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, volatile int *dead, int *status,
                                                  uint32_t limit = (1u << 22)) {
  if (*dead) return false;
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *dead) return false;
  }
  *dead = 1;
  if (status) atomicExch(status, DEV_TIMEOUT);
  return false;
}
// Global -> shared bulk copy.  Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// Tensor-core tile: D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Same tile with a zero accumulator input (no register clearing needed).
__device__ __forceinline__ void mma_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  const float z = 0.0f;
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}

// (a0, a1) += s * (c0, c1) as one packed f32x2 fused multiply-add: each half is rounded exactly like fmaf.
__device__ __forceinline__ void ffma2_scale(float &a0, float &a1, float s, float c0, float c1) {
  asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%0, %1};\n\tmov.b64 rb, {%2, %2};\n\tmov.b64 rc, {%3, %4};\n\t"
      "fma.rn.f32x2 ra, rc, rb, ra;\n\tmov.b64 {%0, %1}, ra;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "f"(s), "f"(c0), "f"(c1));
}

__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

// ---------------------------------------------------------------------------------------------
// Packed activations ("xpack"): the B operand of the GEMV in tensor-core fragment order.
//
// A vector x[K] of batch column b is split into two f16 parts, hi = f16(x) and
// lo = f16((x - hi) * 2048), stored in column slots 2b and 2b+1 (so one lane of the accumulator
// fragment holds both parts of one output).  For every 32-element block kb, slot s and t in 0..3
// one uint4 holds the four B registers a lane with threadID_in_group t feeds to the two k16
// steps of the block, in the element order that matches a Q4_0 byte word:
//   reg0 = {x[4t],    x[4t+2]}    reg1 = {x[4t+1],    x[4t+3]}
//   reg2 = {x[16+4t], x[16+4t+2]} reg3 = {x[16+4t+1], x[16+4t+3]}
// uint4 index = (kb * S + s) * 4 + t, S = 2 * batch.  Size = K * batch * 4 bytes.
// ---------------------------------------------------------------------------------------------
constexpr float XPACK_LO_SCALE = 2048.0f;
constexpr float XPACK_LO_INV = 1.0f / 2048.0f;

__device__ __forceinline__ size_t xpack_half_index(int S, int k, int slot) {
  int kb = k >> 5, e = k & 31;
  int t = (e & 15) >> 2, r4 = e & 3;
  int reg = (e >> 4) * 2 + (r4 & 1);
  int hsel = r4 >> 1;
  return ((((size_t)kb * S + slot) * 4 + t) * 4 + reg) * 2 + hsel;
}
__device__ __forceinline__ void xpack_store(__half *xpack, int S, int b, int k, float v) {
  __half hi = __float2half_rn(v);
  __half lo = __float2half_rn((v - __half2float(hi)) * XPACK_LO_SCALE);
  xpack[xpack_half_index(S, k, 2 * b)] = hi;
  xpack[xpack_half_index(S, k, 2 * b + 1)] = lo;
}

// ---------------------------------------------------------------------------------------------
// Packed activation vector of the integer GEMV (qgemv_i8.cu) in global memory, batch 1,
// K = 32 * kb elements: written by the kernel that produces the vector, bulk-copied by the GEMV.
//   [kb][128] digit bytes: block fixed point x = s * X, X split into four signed base-256 digits;
//             digit d of element e of a block sits at byte d * 32 + ((e & 15) >> 2) * 8 + (e >> 4) * 4 + (e & 3).
//             For a Q4_0 consumer the stored integers are 16 X[e] (e < 16) and X[e] - 16 X[e - 16] (e >= 16).
//   [kb][4]   side words {s, T_lo, s, T_hi} with 128 * sum(X) = T_lo + 65536 T_hi (Q4_0; zero for Q8_0)
//   [kb]      f32 sum of squares of the block's elements before any norm weight (deferred RMSNorm)
// ---------------------------------------------------------------------------------------------
__host__ __device__ inline size_t xq_side_offset(int kb) { return (size_t)kb * 128; }
__host__ __device__ inline size_t xq_ssq_offset(int kb) { return (size_t)kb * 128 + (((size_t)kb * 16 + 127) & ~(size_t)127); }

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Phase stamp of the development trace: slot 0..7 for the first CTA of a launch, 8..15 for the last.
__device__ __forceinline__ void trace_stamp(unsigned long long *trace, int slot, bool first_cta, bool last_cta) {
  if (trace && (first_cta || last_cta)) trace[(first_cta ? 0 : 8) + slot] = global_ns();
}

// SwiGLU with the reference's operation order (src/ir/elementwise.rs:6772-6830,7046-7050):
// silu(g) = g * (1 / (1 + exp2(g * (-1/ln 2)))), every step rounded to f32.
__device__ __forceinline__ float swiglu(float g, float u) {
  float z = __fmul_rn(g, -1.44269504088896340736f);
  float e = exp2f(z);
  float dn = __fadd_rn(1.0f, e);
  float sg = __frcp_rn(dn);
  float si = __fmul_rn(g, sg);
  return __fmul_rn(si, u);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// One 32-element block of a packed activation vector (rg_device.cuh), lane = element: block fixed point
// of `val`, digits, side words, and (ssq_out) the sum of squares `ssq` the caller reduced.  All 32 lanes call.
__device__ __forceinline__ void pack_block_warp(float val, bool q4, uint8_t *xq, int kbo, int kb_all, int lane, bool ssq_out,
                                                float ssq) {
  float m = warp_max(fabsf(val));
  if (__any_sync(0xffffffffu, !(fabsf(val) <= 3.0e38f))) m = __uint_as_float(0x7f800000u);  // keep NaN / inf visible
  const uint32_t E = __float_as_uint(m) >> 23;
  const uint32_t XBITS = q4 ? 25u : 29u;
  float s = 0.0f;
  int X = 0;
  if (E >= 40u && E < 255u) {
    s = __uint_as_float((E - XBITS) << 23);
    X = __float2int_rn(val * __uint_as_float((254u + XBITS - E) << 23));
  } else if (E == 255u) {
    s = __uint_as_float(0x7fc00000u);
    X = lane == 0 ? 1 : 0;
  }
  int t_lo = 0, t_hi = 0;
  if (q4) {
    int sum = X;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    t_lo = (sum & 0x1FF) << 7;
    t_hi = sum >> 9;
    const int partner = __shfl_xor_sync(0xffffffffu, X, 16);
    X = lane < 16 ? X << 4 : X - (partner << 4);
  }
  const uint32_t Y = (uint32_t)X + 0x80808080u;
  uint8_t *dst = xq + (size_t)kbo * 128 + ((lane & 15) >> 2) * 8 + (lane >> 4) * 4 + (lane & 3);
#pragma unroll
  for (int d = 0; d < 4; ++d) dst[d * 32] = (uint8_t)(((Y >> (8 * d)) & 0xFFu) ^ 0x80u);
  if (lane == 0) {
    *reinterpret_cast<float4 *>(xq + xq_side_offset(kb_all) + (size_t)kbo * 16) =
        make_float4(s, __int_as_float(t_lo), s, __int_as_float(t_hi));
    if (ssq_out) reinterpret_cast<float *>(xq + xq_ssq_offset(kb_all))[kbo] = ssq;
  }
}

}  // namespace rg
