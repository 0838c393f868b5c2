// Operator-level C ABI entry points: host buffers in, host buffers out, plus the device-resident
// GEMV benchmark.  Each call uploads its inputs, runs the sm_100a kernels and reads the result
// back; there is no CPU path behind any of them.
#include <cuda_runtime.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "../../include/rg_b200.h"
#include "gguf.h"
#include "kernels.h"

#include <atomic>

namespace rg {
extern thread_local std::string g_last_error;

static std::atomic<uint64_t> g_launch_counts[LC_COUNT];
void count_launch(int which) {
  if (which >= 0 && which < LC_COUNT) g_launch_counts[which].fetch_add(1, std::memory_order_relaxed);
}
}  // namespace rg
using namespace rg;

extern "C" uint64_t rg_b200_launch_count(const char *kernel) {
  static const char *names[LC_COUNT] = {"qgemv_i8", "qgemv", "qgemm_tc", "qgemm_tc_wide", "attn_fused", "attn_prefill",
                                        "attn_split", "tp_exchange", "kquant_gemv", "dense_gemv", "attn_prefill_tc", "qgemv_rows", "attn_decode_tc"};
  if (!kernel) return 0;
  for (int i = 0; i < LC_COUNT; ++i)
    if (!strcmp(kernel, names[i])) return g_launch_counts[i].load(std::memory_order_relaxed);
  return ~0ull;
}

extern "C" int32_t rg_b200_device_info(int32_t device, rg_device_info *out) {
  if (!out || device < 0) {
    g_last_error = "null output or negative device";
    return RG_INVALID_ARGUMENT;
  }
  cudaDeviceProp p{};
  const cudaError_t e = cudaGetDeviceProperties(&p, device);
  if (e != cudaSuccess) {
    g_last_error = std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e);
    return RG_CUDA_ERROR;
  }
  memset(out, 0, sizeof(*out));
  strncpy(out->name, p.name, sizeof(out->name) - 1);
  out->sm_count = p.multiProcessorCount;
  out->cc_major = p.major;
  out->cc_minor = p.minor;
  out->total_memory_bytes = (uint64_t)p.totalGlobalMem;
  out->l2_bytes = (uint64_t)p.l2CacheSize;
  out->shared_memory_per_block = (uint64_t)p.sharedMemPerBlockOptin;
  return RG_OK;
}

namespace {

int32_t fail(int32_t status, const std::string &why) {
  g_last_error = why;
  return status;
}

#define OP_CUDA(expr)                                                                                   \
  do {                                                                                                  \
    cudaError_t e__ = (expr);                                                                           \
    if (e__ != cudaSuccess)                                                                             \
      return fail(e__ == cudaErrorMemoryAllocation ? RG_OUT_OF_MEMORY : RG_CUDA_ERROR,                  \
                  std::string(#expr) + ": " + cudaGetErrorString(e__) + " (" + __FILE__ + ":" +         \
                      std::to_string(__LINE__) + ")");                                                  \
  } while (0)

// Frees device buffers and the stream when an operator call returns, on every path.
struct Scope {
  std::vector<void *> bufs;
  cudaStream_t stream = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  ~Scope() {
    for (void *p : bufs) cudaFree(p);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (stream) cudaStreamDestroy(stream);
  }
  template <typename T>
  cudaError_t alloc(T **p, size_t bytes) {
    void *raw = nullptr;
    cudaError_t e = cudaMalloc(&raw, bytes ? bytes : 16);
    if (e == cudaSuccess) bufs.push_back(raw);
    *p = static_cast<T *>(raw);
    return e;
  }
};

int32_t open_scope(int32_t device, Scope *sc, LaunchCfg *cfg, int **d_status) {
  OP_CUDA(cudaSetDevice(device));
  OP_CUDA(cudaStreamCreateWithFlags(&sc->stream, cudaStreamNonBlocking));
  int sms = 148;
  OP_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  OP_CUDA(sc->alloc(d_status, sizeof(int)));
  OP_CUDA(cudaMemsetAsync(*d_status, 0, sizeof(int), sc->stream));
  cfg->stream = sc->stream;
  cfg->pdl = false;
  cfg->sm_count = sms;
  cfg->status = *d_status;
  return RG_OK;
}

int32_t check_weight(int32_t type, uint64_t n, uint64_t k, size_t *nbytes) {
  if (!block_elements(type)) return fail(RG_UNSUPPORTED_TYPE, "ggml type " + std::to_string(type) + " is not supported");
  if (k % (uint64_t)block_elements(type)) return fail(RG_SHAPE_MISMATCH, "K is not a multiple of the block size");
  *nbytes = (size_t)(n * (k / (uint64_t)block_elements(type)) * (uint64_t)block_bytes(type));
  return RG_OK;
}

int32_t scan_scales(int32_t type, const uint8_t *bytes, size_t nbytes) {
  if (type == RG_TYPE_Q4_K || type == RG_TYPE_Q6_K) {  // d (and dmin) of every super-block must be finite
    const size_t kb = (size_t)block_bytes(type);
    for (size_t b = 0; b < nbytes / kb; ++b) {
      const uint8_t *blk = bytes + b * kb;
      const bool bad = type == RG_TYPE_Q4_K ? (((blk[1] >> 2) & 0x1f) == 0x1f || ((blk[3] >> 2) & 0x1f) == 0x1f)
                                            : (((blk[209] >> 2) & 0x1f) == 0x1f);
      if (bad) return fail(RG_NON_FINITE_SCALE, "block " + std::to_string(b));
    }
    return RG_OK;
  }
  if (type != RG_TYPE_Q4_0 && type != RG_TYPE_Q8_0) return RG_OK;
  const size_t bb = (size_t)block_bytes(type);
  for (size_t b = 0; b < nbytes / bb; ++b)
    if (((bytes[b * bb + 1] >> 2) & 0x1f) == 0x1f) return fail(RG_NON_FINITE_SCALE, "block " + std::to_string(b));
  return RG_OK;
}

// Workspace of the K-split row GEMV (qgemv_rows.cu): partial tiles and zeroed arrival counters.
struct GemvWorkspace {
  float *scratch = nullptr;
  size_t floats = 0;
  unsigned *counters = nullptr;
};
constexpr size_t GEMV_WS_FLOATS = (size_t)256 * 512 * 8;  // up to 256 units of 512 threads x 8 partial sums
cudaError_t alloc_gemv_workspace(Scope *sc, GemvWorkspace *ws) {
  cudaError_t e = sc->alloc(&ws->scratch, sizeof(float) * GEMV_WS_FLOATS);
  if (e != cudaSuccess) return e;
  if ((e = sc->alloc(&ws->counters, sizeof(unsigned) * QGEMV_ROWS_MAX_TILES)) != cudaSuccess) return e;
  ws->floats = GEMV_WS_FLOATS;
  return cudaMemsetAsync(ws->counters, 0, sizeof(unsigned) * QGEMV_ROWS_MAX_TILES, sc->stream);
}

// Activation rows one launch takes: 16 for the packed types (the f16-MMA GEMV), else 8.
int matmul_chunk(int32_t type, uint64_t k) { return ((type == RG_TYPE_Q4_0 || type == RG_TYPE_Q8_0) && k % 256 == 0) ? 16 : 8; }

// Launches y[m,n] = x[m,k] . W[n,k]^T in column chunks of at most matmul_chunk() activation rows.
int32_t run_matmul(int32_t type, const uint8_t *d_w, uint64_t n, uint64_t k, const float *d_x, uint64_t m, float *d_y,
                   void *d_pack, const GemvWorkspace &ws, const LaunchCfg &cfg) {
  const bool packed = (type == RG_TYPE_Q4_0 || type == RG_TYPE_Q8_0);
  const uint64_t chunk = (uint64_t)matmul_chunk(type, k);
  for (uint64_t m0 = 0; m0 < m; m0 += chunk) {
    const int batch = (int)std::min<uint64_t>(chunk, m - m0);
    if (packed && qgemv_i8_supported((int)k, batch)) {
      // batch 1..2: integer tensor-core kernel, packs the f32 activations in its own prologue
      GemvI8Args a;
      a.type = type;
      a.w[0] = d_w;
      a.seg_rows[0] = (int)n;
      a.nseg = 1;
      a.k = (int)k;
      a.x = d_x + m0 * k;
      a.ldx = (int)k;
      a.batch = batch;
      a.epi = EPI_STORE;
      a.y = d_y + m0 * n;
      a.ldy = (int)n;
      OP_CUDA(launch_qgemv_i8(a, cfg));
    } else if (packed) {
      OP_CUDA(launch_pack(d_x + m0 * k, (int)k, (int)k, batch, d_pack, cfg));
      GemvArgs a;
      a.type = type;
      a.w[0] = d_w;
      a.seg_rows[0] = (int)n;
      a.nseg = 1;
      a.k = (int)k;
      a.xpack = d_pack;
      a.batch = batch;
      a.epi = EPI_STORE;
      a.y = d_y + m0 * n;
      a.ldy = (int)n;
      a.split_scratch = ws.scratch;
      a.split_scratch_floats = ws.floats;
      a.split_counters = ws.counters;
      OP_CUDA(launch_qgemv(a, cfg));
    } else {
      DenseGemvArgs a;
      a.type = type;
      a.w = d_w;
      a.rows = (int)n;
      a.k = (int)k;
      a.x = d_x + m0 * k;
      a.ldx = (int)k;
      a.batch = batch;
      a.epi = EPI_STORE;
      a.y = d_y + m0 * n;
      a.ldy = (int)n;
      OP_CUDA(launch_dense_gemv(a, cfg));
    }
  }
  return RG_OK;
}

}  // namespace

extern "C" {

int32_t rg_b200_dequantize(int32_t device, int32_t type, const uint8_t *bytes, size_t elements, float *out) {
  if (!bytes || (!out && elements)) return fail(RG_INVALID_ARGUMENT, "null argument");
  size_t nbytes;
  int32_t rc = check_weight(type, 1, elements, &nbytes);
  if (rc) return rc;
  if (elements == 0) return RG_OK;
  Scope sc;
  LaunchCfg cfg;
  int *d_status;
  if ((rc = open_scope(device, &sc, &cfg, &d_status))) return rc;
  uint8_t *d_in;
  float *d_out;
  OP_CUDA(sc.alloc(&d_in, nbytes));
  OP_CUDA(sc.alloc(&d_out, elements * sizeof(float)));
  OP_CUDA(cudaMemcpyAsync(d_in, bytes, nbytes, cudaMemcpyHostToDevice, sc.stream));
  OP_CUDA(launch_dequantize(type, d_in, elements, d_out, cfg));
  int status = 0;
  OP_CUDA(cudaMemcpyAsync(out, d_out, elements * sizeof(float), cudaMemcpyDeviceToHost, sc.stream));
  OP_CUDA(cudaMemcpyAsync(&status, d_status, sizeof(int), cudaMemcpyDeviceToHost, sc.stream));
  OP_CUDA(cudaStreamSynchronize(sc.stream));
  if (status == 2) return fail(RG_NON_FINITE_SCALE, "a block decodes to a non-finite value");
  if (status) return fail(RG_CUDA_ERROR, "device status " + std::to_string(status));
  return RG_OK;
}

int32_t rg_b200_qmatmul(int32_t device, int32_t type, const uint8_t *weight, uint64_t n, uint64_t k, const float *activation,
                        uint64_t m, float *out) {
  if (!weight || !activation || !out) return fail(RG_INVALID_ARGUMENT, "null argument");
  size_t wbytes;
  int32_t rc = check_weight(type, n, k, &wbytes);
  if (rc) return rc;
  if (n == 0 || m == 0) return RG_OK;
  const bool packed = (type == RG_TYPE_Q4_0 || type == RG_TYPE_Q8_0);
  if (k == 0) {  // empty contraction: zeros (src/matmul/quantized.rs:512-560)
    memset(out, 0, sizeof(float) * m * n);
    return RG_OK;
  }
  if (packed && k % 256) return fail(RG_UNSUPPORTED_GEOMETRY, "packed weights need K to be a multiple of 256");
  if ((rc = scan_scales(type, weight, wbytes))) return rc;
  Scope sc;
  LaunchCfg cfg;
  int *d_status;
  if ((rc = open_scope(device, &sc, &cfg, &d_status))) return rc;
  uint8_t *d_w, *d_pack;
  float *d_x, *d_y;
  OP_CUDA(sc.alloc(&d_w, wbytes));
  OP_CUDA(sc.alloc(&d_x, sizeof(float) * m * k));
  OP_CUDA(sc.alloc(&d_y, sizeof(float) * m * n));
  OP_CUDA(sc.alloc(&d_pack, xpack_bytes((int)k, 16)));
  GemvWorkspace ws;
  OP_CUDA(alloc_gemv_workspace(&sc, &ws));
  OP_CUDA(cudaMemcpyAsync(d_w, weight, wbytes, cudaMemcpyHostToDevice, sc.stream));
  OP_CUDA(cudaMemcpyAsync(d_x, activation, sizeof(float) * m * k, cudaMemcpyHostToDevice, sc.stream));
  if ((rc = run_matmul(type, d_w, n, k, d_x, m, d_y, d_pack, ws, cfg))) return rc;
  int status = 0;
  OP_CUDA(cudaMemcpyAsync(out, d_y, sizeof(float) * m * n, cudaMemcpyDeviceToHost, sc.stream));
  OP_CUDA(cudaMemcpyAsync(&status, d_status, sizeof(int), cudaMemcpyDeviceToHost, sc.stream));
  OP_CUDA(cudaStreamSynchronize(sc.stream));
  if (status == 1) return fail(RG_TIMEOUT, "a bounded device-side wait gave up");
  if (status) return fail(RG_CUDA_ERROR, "device status " + std::to_string(status));
  return RG_OK;
}

int32_t rg_b200_row_gather(int32_t device, int32_t type, const uint8_t *weight, uint64_t rows, uint64_t cols,
                           const int64_t *indices, size_t count, float *out) {
  if (!weight || (!indices && count) || (!out && count)) return fail(RG_INVALID_ARGUMENT, "null argument");
  size_t wbytes;
  int32_t rc = check_weight(type, rows, cols, &wbytes);
  if (rc) return rc;
  // every index is validated before any decode (src/gguf/quantization/row_gather.rs:187-226)
  std::vector<int32_t> ids(count);
  for (size_t i = 0; i < count; ++i) {
    if (indices[i] < 0 || (uint64_t)indices[i] >= rows) return fail(RG_TOKEN_OUT_OF_RANGE, "index " + std::to_string(indices[i]) + " at " + std::to_string(i));
    ids[i] = (int32_t)indices[i];
  }
  if (count == 0 || cols == 0) return RG_OK;
  if ((rc = scan_scales(type, weight, wbytes))) return rc;
  Scope sc;
  LaunchCfg cfg;
  int *d_status;
  if ((rc = open_scope(device, &sc, &cfg, &d_status))) return rc;
  uint8_t *d_w;
  int32_t *d_ids;
  float *d_out;
  OP_CUDA(sc.alloc(&d_w, wbytes));
  OP_CUDA(sc.alloc(&d_ids, sizeof(int32_t) * count));
  OP_CUDA(sc.alloc(&d_out, sizeof(float) * count * cols));
  OP_CUDA(cudaMemcpyAsync(d_w, weight, wbytes, cudaMemcpyHostToDevice, sc.stream));
  OP_CUDA(cudaMemcpyAsync(d_ids, ids.data(), sizeof(int32_t) * count, cudaMemcpyHostToDevice, sc.stream));
  OP_CUDA(launch_row_gather(type, d_w, (int)cols, d_ids, (int)count, d_out, (int)cols, cfg));
  OP_CUDA(cudaMemcpyAsync(out, d_out, sizeof(float) * count * cols, cudaMemcpyDeviceToHost, sc.stream));
  OP_CUDA(cudaStreamSynchronize(sc.stream));
  return RG_OK;
}

int32_t rg_b200_qgemm(int32_t device, int32_t type, const uint8_t *weight, uint64_t n, uint64_t k, const float *activation,
                      uint64_t m, int32_t operand_mode, int32_t iters, float *out, float *kernel_ms) {
  if (!weight || !activation || !out) return fail(RG_INVALID_ARGUMENT, "null argument");
  if (type != RG_TYPE_Q4_0 && type != RG_TYPE_Q8_0) return fail(RG_UNSUPPORTED_TYPE, "the tensor-core GEMM takes Q4_0 or Q8_0 weights");
  size_t wbytes;
  int32_t rc = check_weight(type, n, k, &wbytes);
  if (rc) return rc;
  if (n == 0 || m == 0) return RG_OK;
  if (k == 0 || k % 256) return fail(RG_UNSUPPORTED_GEOMETRY, "packed weights need K to be a multiple of 256");
  if ((rc = scan_scales(type, weight, wbytes))) return rc;
  Scope sc;
  LaunchCfg cfg;
  int *d_status;
  if ((rc = open_scope(device, &sc, &cfg, &d_status))) return rc;
  uint8_t *d_w, *d_xb;
  float *d_x, *d_y;
  OP_CUDA(sc.alloc(&d_w, wbytes));
  OP_CUDA(sc.alloc(&d_x, sizeof(float) * m * k));
  if (operand_mode < 0 || operand_mode > 2) return fail(RG_INVALID_ARGUMENT, "operand_mode must be 0, 1 or 2");
  OP_CUDA(sc.alloc(&d_xb, 4 * m * k));  // hi and lo planes
  OP_CUDA(sc.alloc(&d_y, sizeof(float) * m * n));
  OP_CUDA(cudaMemcpyAsync(d_w, weight, wbytes, cudaMemcpyHostToDevice, sc.stream));
  OP_CUDA(cudaMemcpyAsync(d_x, activation, sizeof(float) * m * k, cudaMemcpyHostToDevice, sc.stream));
  Operand16 op;
  op.hi = d_xb;
  op.lo = operand_mode == QGEMM_F16X3 ? d_xb + 2 * m * k : nullptr;
  op.ld = (int)k;
  op.f16 = operand_mode != QGEMM_BF16;
  OP_CUDA(launch_to16(d_x, (int)k, (int)k, (int)m, op, cfg));
  QGemmArgs a;
  a.type = type;
  a.w = d_w;
  a.n = (int)n;
  a.k = (int)k;
  a.x16 = d_xb;
  a.x16_lo = op.lo;
  a.mode = operand_mode;
  a.ldx = (int)k;
  a.m = (int)m;
  a.out = d_y;
  a.ldc = (int)n;
  OP_CUDA(launch_qgemm_tc(a, cfg));  // first launch also serves as warm-up
  const int reps = iters > 0 ? iters : 0;
  OP_CUDA(cudaEventCreate(&sc.e0));
  OP_CUDA(cudaEventCreate(&sc.e1));
  OP_CUDA(cudaEventRecord(sc.e0, sc.stream));
  for (int i = 0; i < reps; ++i) OP_CUDA(launch_qgemm_tc(a, cfg));
  OP_CUDA(cudaEventRecord(sc.e1, sc.stream));
  int status = 0;
  OP_CUDA(cudaMemcpyAsync(out, d_y, sizeof(float) * m * n, cudaMemcpyDeviceToHost, sc.stream));
  OP_CUDA(cudaMemcpyAsync(&status, d_status, sizeof(int), cudaMemcpyDeviceToHost, sc.stream));
  OP_CUDA(cudaStreamSynchronize(sc.stream));
  if (status == 1) return fail(RG_TIMEOUT, "a bounded device-side wait gave up");
  if (status) return fail(RG_CUDA_ERROR, "device status " + std::to_string(status));
  if (kernel_ms) {
    float ms = 0.0f;
    OP_CUDA(cudaEventElapsedTime(&ms, sc.e0, sc.e1));
    *kernel_ms = reps ? ms / (float)reps : 0.0f;
  }
  return RG_OK;
}

int32_t rg_b200_attention_decode(int32_t device, const float *q, const void *keys, const void *values, int32_t heads,
                                 int32_t kv_heads, int32_t head_dim, int32_t n_pos, int32_t kv_f32, float *out) {
  if (!q || !keys || !values || !out) return fail(RG_INVALID_ARGUMENT, "null argument");
  if (n_pos < 1) return fail(RG_INVALID_ARGUMENT, "n_pos must be at least 1");
  if (heads < 1 || kv_heads < 1 || !attention_supported(heads, kv_heads, head_dim))
    return fail(RG_UNSUPPORTED_GEOMETRY, "head_dim must be 64 or 128 and query heads per kv head 1, 2, 4 or 8");
  Scope sc;
  LaunchCfg cfg;
  int *d_status;
  int32_t rc;
  if ((rc = open_scope(device, &sc, &cfg, &d_status))) return rc;
  const size_t item = kv_f32 ? 4 : 2;
  const size_t kv_bytes = (size_t)kv_heads * n_pos * head_dim * item, q_bytes = sizeof(float) * (size_t)heads * head_dim;
  float *d_q, *d_out, *d_scratch;
  uint8_t *d_k, *d_v;
  int32_t *d_ctl;
  OP_CUDA(sc.alloc(&d_q, q_bytes));
  OP_CUDA(sc.alloc(&d_out, q_bytes));
  OP_CUDA(sc.alloc(&d_k, kv_bytes));
  OP_CUDA(sc.alloc(&d_v, kv_bytes));
  OP_CUDA(sc.alloc(&d_ctl, 2 * sizeof(int32_t)));
  OP_CUDA(sc.alloc(&d_scratch, sizeof(float) * attn_scratch_floats(1, heads, head_dim, n_pos)));
  const int32_t ctl[2] = {0, n_pos - 1};  // sequence 0, position of the new token
  OP_CUDA(cudaMemcpyAsync(d_q, q, q_bytes, cudaMemcpyHostToDevice, sc.stream));
  OP_CUDA(cudaMemcpyAsync(d_k, keys, kv_bytes, cudaMemcpyHostToDevice, sc.stream));
  OP_CUDA(cudaMemcpyAsync(d_v, values, kv_bytes, cudaMemcpyHostToDevice, sc.stream));
  OP_CUDA(cudaMemcpyAsync(d_ctl, ctl, sizeof(ctl), cudaMemcpyHostToDevice, sc.stream));
  AttnArgs a;
  a.q = d_q;
  a.k_cache = d_k;
  a.v_cache = d_v;
  a.kv_f32 = kv_f32 != 0;
  a.cols = 1;
  a.heads = heads;
  a.kv_heads = kv_heads;
  a.hd = head_dim;
  a.ctx = n_pos;
  a.col_seq = d_ctl;
  a.col_pos = d_ctl + 1;
  a.scratch = d_scratch;
  a.out_f32 = d_out;
  OP_CUDA(launch_attention(a, cfg));
  int status = 0;
  OP_CUDA(cudaMemcpyAsync(out, d_out, q_bytes, cudaMemcpyDeviceToHost, sc.stream));
  OP_CUDA(cudaMemcpyAsync(&status, d_status, sizeof(int), cudaMemcpyDeviceToHost, sc.stream));
  OP_CUDA(cudaStreamSynchronize(sc.stream));
  if (status == 1) return fail(RG_TIMEOUT, "a bounded device-side wait gave up");
  if (status) return fail(RG_CUDA_ERROR, "device status " + std::to_string(status));
  return RG_OK;
}

int32_t rg_b200_qmatmul_bench(int32_t device, int32_t type, const uint8_t *weight, uint64_t n, uint64_t k, const float *activation,
                              uint64_t m, int32_t rotate, int32_t iters, int32_t warmup, float *out, float *kernel_ms) {
  if (!weight || !activation || !kernel_ms) return fail(RG_INVALID_ARGUMENT, "null argument");
  if (m < 1 || m > 16 || (m > 8 && matmul_chunk(type, k) < 16) || iters < 1 || rotate < 1)
    return fail(RG_INVALID_ARGUMENT, "m in 1..16, iters >= 1, rotate >= 1");
  size_t wbytes;
  int32_t rc = check_weight(type, n, k, &wbytes);
  if (rc) return rc;
  const bool packed = (type == RG_TYPE_Q4_0 || type == RG_TYPE_Q8_0);
  if (!packed) return fail(RG_UNSUPPORTED_TYPE, "the benchmark covers packed weights");
  if (k == 0 || k % 256) return fail(RG_UNSUPPORTED_GEOMETRY, "packed weights need K to be a multiple of 256");
  Scope sc;
  LaunchCfg cfg;
  int *d_status;
  if ((rc = open_scope(device, &sc, &cfg, &d_status))) return rc;
  std::vector<uint8_t *> copies((size_t)rotate);
  for (int r = 0; r < rotate; ++r) {
    OP_CUDA(sc.alloc(&copies[(size_t)r], wbytes));
    if (r == 0) OP_CUDA(cudaMemcpyAsync(copies[0], weight, wbytes, cudaMemcpyHostToDevice, sc.stream));
    else OP_CUDA(cudaMemcpyAsync(copies[(size_t)r], copies[0], wbytes, cudaMemcpyDeviceToDevice, sc.stream));
  }
  float *d_x, *d_y;
  uint8_t *d_pack;
  OP_CUDA(sc.alloc(&d_x, sizeof(float) * m * k));
  OP_CUDA(sc.alloc(&d_y, sizeof(float) * m * n));
  OP_CUDA(sc.alloc(&d_pack, xpack_bytes((int)k, (int)m)));
  OP_CUDA(cudaMemcpyAsync(d_x, activation, sizeof(float) * m * k, cudaMemcpyHostToDevice, sc.stream));
  OP_CUDA(launch_pack(d_x, (int)k, (int)k, (int)m, d_pack, cfg));
  GemvArgs a;
  a.type = type;
  a.seg_rows[0] = (int)n;
  a.nseg = 1;
  a.k = (int)k;
  a.xpack = d_pack;
  a.batch = (int)m;
  a.epi = EPI_STORE;
  a.y = d_y;
  a.ldy = (int)n;
  GemvWorkspace ws;
  OP_CUDA(alloc_gemv_workspace(&sc, &ws));
  a.split_scratch = ws.scratch;
  a.split_scratch_floats = ws.floats;
  a.split_counters = ws.counters;
  // batch 1..2 runs the integer tensor-core kernel (activations packed by its prologue)
  const bool use_i8 = qgemv_i8_supported((int)k, (int)m);
  GemvI8Args a8;
  a8.type = type;
  a8.seg_rows[0] = (int)n;
  a8.nseg = 1;
  a8.k = (int)k;
  a8.x = d_x;
  a8.ldx = (int)k;
  a8.batch = (int)m;
  a8.epi = EPI_STORE;
  a8.y = d_y;
  a8.ldy = (int)n;
  auto launch_one = [&](const uint8_t *w) {
    if (use_i8) {
      a8.w[0] = w;
      return launch_qgemv_i8(a8, cfg);
    }
    a.w[0] = w;
    return launch_qgemv(a, cfg);
  };
  OP_CUDA(cudaEventCreate(&sc.e0));
  OP_CUDA(cudaEventCreate(&sc.e1));
  for (int i = 0; i < warmup; ++i) OP_CUDA(launch_one(copies[(size_t)(i % rotate)]));
  OP_CUDA(cudaEventRecord(sc.e0, sc.stream));
  for (int i = 0; i < iters; ++i) OP_CUDA(launch_one(copies[(size_t)((warmup + i) % rotate)]));
  OP_CUDA(cudaEventRecord(sc.e1, sc.stream));
  int status = 0;
  if (out) OP_CUDA(cudaMemcpyAsync(out, d_y, sizeof(float) * m * n, cudaMemcpyDeviceToHost, sc.stream));
  OP_CUDA(cudaMemcpyAsync(&status, d_status, sizeof(int), cudaMemcpyDeviceToHost, sc.stream));
  OP_CUDA(cudaStreamSynchronize(sc.stream));
  if (status == 1) return fail(RG_TIMEOUT, "a bounded device-side wait gave up");
  if (status) return fail(RG_CUDA_ERROR, "device status " + std::to_string(status));
  float ms = 0.0f;
  OP_CUDA(cudaEventElapsedTime(&ms, sc.e0, sc.e1));
  *kernel_ms = ms / (float)iters;
  return RG_OK;
}

}  // extern "C"
