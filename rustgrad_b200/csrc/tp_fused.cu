// Tensor-parallel sum of the f32 partial results of a row-split projection, fused with the residual
// add, over NVLink peer memory: x[col][:] += sum over ranks of partial_r[col][:].
// Stands where rustgrad's sharded plan inserts an all-reduce on the contracting axis
// (src/sharding.rs:642-667, src/collective.rs:441) followed by the residual add of
// src/models/transformer/layer.rs:455-470.
//
// One-shot exchange: every rank's projection kernel has written its partial into a buffer that the
// other ranks map through CUDA IPC.  A CTA of this kernel then
//   1. bumps its own epoch word and stores the epoch into its flag slot on EVERY rank
//      (st.release.sys; the partial itself is complete: the producing kernel has finished);
//   2. waits, bounded, until the slots written by all ranks have reached the epoch;
//   3. reads its slice of every rank's partial with plain peer loads (volatile: the buffers are
//      rewritten every call) and adds the sum, taken in rank order so that every rank computes
//      the identical value, to the residual stream.
// Two buffers alternate (output projection / down projection): a rank that has passed the second
// exchange of a layer knows that every rank has finished reading the first buffer, so it may be
// overwritten by the next layer.  No NCCL call, no separate add kernel; the kernel is an ordinary
// launch and is captured in the decode graph like the others.
#include <stdint.h>

#include "../../include/rg_b200.h"
#include "kernels.h"
#include "rg_device.cuh"

namespace rg {
namespace {

constexpr int THREADS = 256;

__device__ __forceinline__ float4 ld_peer(const float4 *p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_peer1(const float *p) {
  float v;
  asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(THREADS) tp_allreduce_add_kernel(const TpFusedArgs A, int *status) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ unsigned s_epoch;
  __shared__ int s_dead;
  const int tid = threadIdx.x, b = blockIdx.x;
  const int slot = (A.buffer * TP_FUSED_CTAS + b) * TP_FUSED_MAX_WORLD;
  if (tid == 0) {
    s_epoch = ++A.epochs[A.buffer * TP_FUSED_CTAS + b];
    s_dead = 0;
  }
  __syncthreads();
  const unsigned e = s_epoch;
  if (A.peer_recv) {
    // ---- push form: no flag hand-shake and no load from a peer.  Every element travels as an
    // 8-byte word {value, epoch}, stored into the receive area of each peer (an 8-byte store is
    // indivisible); the receiver polls its OWN memory until the word carries this exchange's epoch.
    // One NVLink store latency per exchange; the same thread sends and later sums an element.
    auto recv = [&](int r, int q) {  // receive area of rank r, slot of source rank q
      return reinterpret_cast<uint2 *>(A.peer_recv[r]) + ((size_t)(A.buffer * A.world + q) * TP_PUSH_COLS) * (size_t)A.ldp;
    };
    const float *mine = A.peer_partial[A.rank];
    // The words of all source ranks are requested together and looked at together: a poll round
    // costs one trip to L2 whatever the world size.  Returns the sum in rank order (own rank from `own`).
    auto gather_sum = [&](size_t idx, float own) {
      const uint2 *src[TP_FUSED_MAX_WORLD];
#pragma unroll
      for (int r = 0; r < TP_FUSED_MAX_WORLD; ++r) src[r] = r < A.world && r != A.rank ? recv(A.rank, r) + idx : nullptr;
      uint2 w[TP_FUSED_MAX_WORLD];
      bool all = false;
      for (unsigned i = 0; i < A.poll_limit && !all; ++i) {
#pragma unroll
        for (int r = 0; r < TP_FUSED_MAX_WORLD; ++r)
          if (src[r]) asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(w[r].x), "=r"(w[r].y) : "l"(src[r]) : "memory");
        all = true;
#pragma unroll
        for (int r = 0; r < TP_FUSED_MAX_WORLD; ++r)
          if (src[r] && w[r].y != e) all = false;
        if (!all && i > 256) __nanosleep(32);
      }
      if (!all) atomicExch(status, DEV_TIMEOUT);  // a rank never arrived: the host sees the status and poisons the session
      float sum = 0.0f;
#pragma unroll
      for (int r = 0; r < TP_FUSED_MAX_WORLD; ++r)
        if (r < A.world) sum = __fadd_rn(sum, r == A.rank ? own : (all ? __uint_as_float(w[r].x) : 0.0f));
      return sum;
    };
    if (A.pack_out) {
      const int warp = tid >> 5, lane = tid & 31, nblk = A.n >> 5;
      const bool q4 = A.pack_type == RG_TYPE_Q4_0;
      constexpr int STRIDE = TP_FUSED_CTAS * (THREADS / 32);
      for (int kb = b * (THREADS / 32) + warp; kb < nblk; kb += STRIDE) {
        const int idx = kb * 32 + lane;
        const float v = mine[idx];
        for (int r = 0; r < A.world; ++r)
          if (r != A.rank)
            asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(recv(r, A.rank) + idx), "r"(__float_as_uint(v)), "r"(e) : "memory");
      }
      for (int kb = b * (THREADS / 32) + warp; kb < nblk; kb += STRIDE) {
        const int idx = kb * 32 + lane;
        const float resid = A.x[idx];
        const float w = A.pack_w ? __ldg(A.pack_w + idx) : 1.0f;
        const float v = __fadd_rn(resid, gather_sum((size_t)idx, mine[idx]));
        A.x[idx] = v;
        const float ssq = warp_sum(__fmul_rn(v, v));
        pack_block_warp(__fmul_rn(v, w), q4, A.pack_out, kb, nblk, lane, true, ssq);
      }
      return;
    }
    const int total = A.cols * A.n;
    for (int i = b * THREADS + tid; i < total; i += TP_FUSED_CTAS * THREADS) {
      const int col = i / A.n, j = i - col * A.n;
      const size_t idx = (size_t)col * A.ldp + j;
      const float v = mine[idx];
      for (int r = 0; r < A.world; ++r)
        if (r != A.rank)
          asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(recv(r, A.rank) + idx), "r"(__float_as_uint(v)), "r"(e) : "memory");
    }
    for (int i = b * THREADS + tid; i < total; i += TP_FUSED_CTAS * THREADS) {
      const int col = i / A.n, j = i - col * A.n;
      const size_t idx = (size_t)col * A.ldp + j;
      float *dst = A.x + (size_t)col * A.ldx + j;
      *dst = __fadd_rn(*dst, gather_sum(idx, mine[idx]));
    }
    return;
  }
  if (tid < A.world) {
    st_release_sys(A.peer_flags[tid] + slot + A.rank, e);  // tell rank `tid` that this rank's partial is ready
    const unsigned *mine = A.peer_flags[A.rank] + slot + tid;  // written by rank `tid`
    bool ok = false;
    for (unsigned i = 0; i < A.poll_limit; ++i) {
      if ((int)(ld_acquire_sys(mine) - e) >= 0) {
        ok = true;
        break;
      }
      if (i > 128) __nanosleep(64);
    }
    if (!ok) {
      s_dead = 1;
      atomicExch(status, DEV_TIMEOUT);
    }
  }
  __syncthreads();
  if (s_dead) return;  // a rank never arrived: leave x untouched, the host sees the status
  if (A.pack_out) {
    // one column: a warp owns whole 32-element blocks (lane = element), so that it can also leave the
    // row packed for the next integer GEMV, the same way a residual epilogue on one GPU does
    const int warp = tid >> 5, lane = tid & 31, nblk = A.n >> 5;
    const bool q4 = A.pack_type == RG_TYPE_Q4_0;
    // every block of this warp is requested from every rank before the first sum: one NVLink round
    // trip for the whole exchange
    constexpr int STRIDE = TP_FUSED_CTAS * (THREADS / 32), UB = 4;
    for (int kb0 = b * (THREADS / 32) + warp; kb0 < nblk; kb0 += UB * STRIDE) {
      float p[UB][TP_FUSED_MAX_WORLD], resid[UB], w[UB];
#pragma unroll
      for (int u = 0; u < UB; ++u) {
        const int e = (kb0 + u * STRIDE) * 32 + lane;
        if (kb0 + u * STRIDE < nblk) {
#pragma unroll
          for (int r = 0; r < TP_FUSED_MAX_WORLD; ++r)
            if (r < A.world) p[u][r] = ld_peer1(A.peer_partial[r] + e);
          resid[u] = A.x[e];
          w[u] = A.pack_w ? __ldg(A.pack_w + e) : 1.0f;
        }
      }
#pragma unroll
      for (int u = 0; u < UB; ++u) {
        const int kb = kb0 + u * STRIDE;
        if (kb < nblk) {
          float sum = 0.0f;
#pragma unroll
          for (int r = 0; r < TP_FUSED_MAX_WORLD; ++r)
            if (r < A.world) sum = __fadd_rn(sum, p[u][r]);  // rank order, as below
          const float v = __fadd_rn(resid[u], sum);
          A.x[kb * 32 + lane] = v;
          const float ssq = warp_sum(__fmul_rn(v, v));
          pack_block_warp(__fmul_rn(v, w[u]), q4, A.pack_out, kb, nblk, lane, true, ssq);
        }
      }
    }
    return;
  }
  const int row4 = A.n / 4;
  const int total = A.cols * row4;
  for (int i = b * THREADS + tid; i < total; i += TP_FUSED_CTAS * THREADS) {
    const int col = i / row4, j = i - col * row4;
    // all ranks' slices and the residual are requested before the first sum: one NVLink round trip
    // for the whole exchange instead of one per rank
    float4 p[TP_FUSED_MAX_WORLD];
#pragma unroll
    for (int r = 0; r < TP_FUSED_MAX_WORLD; ++r)
      if (r < A.world)
        p[r] = ld_peer(reinterpret_cast<const float4 *>(A.peer_partial[r] + (size_t)col * A.ldp) + j);
    const float4 resid = *(reinterpret_cast<const float4 *>(A.x + (size_t)col * A.ldx) + j);
    float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int r = 0; r < TP_FUSED_MAX_WORLD; ++r)
      if (r < A.world) {  // rank order: every rank computes the identical value
        sum.x = __fadd_rn(sum.x, p[r].x);
        sum.y = __fadd_rn(sum.y, p[r].y);
        sum.z = __fadd_rn(sum.z, p[r].z);
        sum.w = __fadd_rn(sum.w, p[r].w);
      }
    float4 *dst = reinterpret_cast<float4 *>(A.x + (size_t)col * A.ldx) + j;
    float4 v = resid;
    v.x = __fadd_rn(v.x, sum.x);
    v.y = __fadd_rn(v.y, sum.y);
    v.z = __fadd_rn(v.z, sum.z);
    v.w = __fadd_rn(v.w, sum.w);
    *dst = v;
  }
}

}  // namespace

cudaError_t launch_tp_allreduce_add(const TpFusedArgs &a, const LaunchCfg &cfg) {
  count_launch(LC_TP_EXCHANGE);
  if (!a.x || !a.peer_partial || !a.peer_flags || !a.epochs || a.world < 2 || a.world > TP_FUSED_MAX_WORLD || a.n % 4 ||
      a.ldx % 4 || a.ldp % 4 || a.buffer < 0 || a.buffer > 1)
    return cudaErrorInvalidValue;
  if (a.peer_recv && a.cols > TP_PUSH_COLS) return cudaErrorInvalidValue;
  if (a.pack_out && (a.cols != 1 || a.n % 32 || (reinterpret_cast<uintptr_t>(a.pack_out) & 127) ||
                     (a.pack_type != RG_TYPE_Q4_0 && a.pack_type != RG_TYPE_Q8_0)))
    return cudaErrorInvalidValue;
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3(TP_FUSED_CTAS);
  lc.blockDim = dim3(THREADS);
  lc.stream = cfg.stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = cfg.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&lc, tp_allreduce_add_kernel, a, cfg.status);
}

}  // namespace rg
