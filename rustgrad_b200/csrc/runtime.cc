// Host runtime behind the C ABI: tensor binding with typed rejections, one-time upload of the
// native GGML block bytes (sharded for tensor parallelism), the session with its fixed launch
// sequence, CUDA-graph replay of the decode step, and transactional positions.
//
// It takes the place of rustgrad's CUDA plumbing for this model: src/cuda.rs (driver wrapper),
// src/runtime/cuda_graph.rs (prepared graph replay), src/sharded_cuda_plan.rs /
// src/sharded_cuda_execute.rs (static Megatron split instead of a general sharded plan).
#include <cuda_runtime.h>
#include <math.h>

#include <cmath>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/rg_b200.h"
#include "comm.h"
#include "gguf.h"
#include "kernels.h"

namespace rg {

// ------------------------------------------------------------------------------------------
// Errors and host-side fault injection
// ------------------------------------------------------------------------------------------
thread_local std::string g_last_error;

static int32_t fail(int32_t status, const std::string &why) {
  g_last_error = why;
  return status;
}

// Fail-after-N counters for the wrapped runtime calls, the host-side stand-in for the
// fault knobs of rustgrad's mock driver (src/cuda.rs:5895-5960).  -1 = never fail.
struct FaultKnobs {
  std::atomic<int> malloc_after{-1}, memcpy_after{-1}, launch_after{-1}, sync_after{-1};
};
static FaultKnobs g_faults;

static bool inject(std::atomic<int> &knob) {
  int v = knob.load();
  if (v < 0) return false;
  if (v == 0) {
    knob.store(-1);
    return true;
  }
  knob.store(v - 1);
  return false;
}

#define RG_CUDA(expr)                                                                                        \
  do {                                                                                                       \
    cudaError_t e__ = (expr);                                                                                \
    if (e__ != cudaSuccess)                                                                                  \
      return fail(e__ == cudaErrorMemoryAllocation ? RG_OUT_OF_MEMORY : RG_CUDA_ERROR,                       \
                  std::string(#expr) + ": " + cudaGetErrorString(e__) + " (" + __FILE__ + ":" +              \
                      std::to_string(__LINE__) + ")");                                                       \
  } while (0)

static cudaError_t x_malloc(void **p, size_t n) {
  if (inject(g_faults.malloc_after)) return cudaErrorMemoryAllocation;
  return cudaMalloc(p, n ? n : 16);
}
static cudaError_t x_memcpy_async(void *dst, const void *src, size_t n, cudaMemcpyKind kind, cudaStream_t s) {
  if (inject(g_faults.memcpy_after)) return cudaErrorUnknown;
  return cudaMemcpyAsync(dst, src, n, kind, s);
}
static cudaError_t x_sync(cudaStream_t s) {
  if (inject(g_faults.sync_after)) return cudaErrorUnknown;
  return cudaStreamSynchronize(s);
}
static cudaError_t x_launch(cudaError_t launched) {
  if (inject(g_faults.launch_after)) return cudaErrorLaunchFailure;
  return launched;
}

static bool env_flag(const char *name) {
  const char *v = getenv(name);
  return v && *v && strcmp(v, "0") != 0;
}

// ------------------------------------------------------------------------------------------
// Tensors
// ------------------------------------------------------------------------------------------
struct DevTensor {
  int type = -1;          // -1: absent
  uint64_t rows = 0, cols = 0;  // rank-local shape
  uint8_t *d = nullptr;
  size_t nbytes = 0;
  // served by the tensor-core GEMV / GEMM kernels: Q4_0 / Q8_0 rows of whole 256-element groups.  Block
  // tensors with any other K (a multiple of 32, as the reference requires) take the generic
  // decode-and-multiply GEMV like the dense ones
  bool packed() const { return (type == RG_TYPE_Q4_0 || type == RG_TYPE_Q8_0) && cols % 256 == 0; }
};

struct LayerW {
  DevTensor attn_norm, q, k, v, o, ffn_norm, gate, up, down;
  DevTensor q_norm, k_norm, q_bias, k_bias, v_bias;  // model variants only (f32 vectors)
  // q, k, v (gate, up) lie one after the other in ONE allocation: the tensor-core path then runs
  // them as a single GEMM over the stacked rows, which fills the SMs' waves better than 3 (2) launches
  bool qkv_stacked = false, gu_stacked = false;
};

enum Split { SPLIT_NONE, SPLIT_ROWS, SPLIT_COLS };

struct Slot {
  DevTensor *t = nullptr;
  uint64_t rows = 0, cols = 0;  // full shape
  bool norm = false;
  Split split = SPLIT_NONE;
  bool ignored = false;  // rope_freqs.weight: validated, not used (as in the reference forward)
};

}  // namespace rg

using namespace rg;


struct rg_plan {
  rg_llama_config cfg{};
  rg_options opt{};
  int tp_rank = 0, tp_world = 1;
  cudaStream_t stream = nullptr;
  int *d_status = nullptr;
  int sm_count = 148;
  std::vector<LayerW> layers;
  DevTensor token_embd, output_norm, output;
  uint64_t weight_bytes = 0;
  bool consumed = false;

  ~rg_plan() {
    if (!consumed) {
      auto drop = [](DevTensor &t) {
        if (t.d) cudaFree(t.d);
        t.d = nullptr;
      };
      drop(token_embd);
      drop(output_norm);
      drop(output);
      for (auto &l : layers)
        for (DevTensor *t : {&l.attn_norm, &l.q, &l.k, &l.v, &l.o, &l.ffn_norm, &l.gate, &l.up, &l.down, &l.q_norm, &l.k_norm, &l.q_bias,
                             &l.k_bias, &l.v_bias})
          drop(*t);
    }
    if (d_status) cudaFree(d_status);
    if (stream) cudaStreamDestroy(stream);
  }
};

namespace rg {

// How a tensor is divided over tensor-parallel ranks, by name (Megatron split: the projections that
// produce heads or hidden units by rows, the two that consume them along the contracting axis;
// src/sharding.rs:642-667).
static Split split_of(const std::string &name) {
  auto ends = [&](const char *suffix) {
    const size_t n = strlen(suffix);
    return name.size() >= n && name.compare(name.size() - n, n, suffix) == 0;
  };
  if (name == "output.weight" || ends("attn_q.weight") || ends("attn_k.weight") || ends("attn_v.weight") ||
      ends("ffn_gate.weight") || ends("ffn_up.weight"))
    return SPLIT_ROWS;
  if (ends("attn_output.weight") || ends("ffn_down.weight")) return SPLIT_COLS;
  return SPLIT_NONE;
}

// The rank's share of a [rows, cols] tensor: whole rows, or whole blocks of every row.
static int32_t shard_range(const std::string &name, int32_t type, uint64_t rows, uint64_t cols, Split split, uint64_t W, uint64_t R,
                           uint64_t *r0, uint64_t *lr, uint64_t *c0, uint64_t *lc) {
  *r0 = 0, *lr = rows, *c0 = 0, *lc = cols;
  if (W > 1 && split == SPLIT_ROWS) {
    if (rows % W) return fail(RG_UNSUPPORTED_GEOMETRY, name + ": rows do not divide by the tensor-parallel world size");
    *lr = rows / W;
    *r0 = R * *lr;
  } else if (W > 1 && split == SPLIT_COLS) {
    // a rank owns whole blocks of every row: 32 elements, or a 256-element K-quant super-block
    if (cols % (W * (uint64_t)block_elements(type)))
      return fail(RG_UNSUPPORTED_GEOMETRY, name + ": columns do not split at block boundaries");
    *lc = cols / W;
    *c0 = R * *lc;
  }
  return RG_OK;
}

static bool find_slot(rg_plan *p, const std::string &name, Slot *s) {
  const rg_llama_config &c = p->cfg;
  const uint64_t d = c.d_model, f = c.ffn_dim, qw = (uint64_t)c.n_heads * c.head_dim, kw = (uint64_t)c.n_kv_heads * c.head_dim;
  auto set = [&](DevTensor *t, uint64_t rows, uint64_t cols, bool norm, Split split) {
    s->t = t;
    s->rows = rows;
    s->cols = cols;
    s->norm = norm;
    s->split = split;
    return true;
  };
  if (name == "token_embd.weight") return set(&p->token_embd, c.vocab, d, false, SPLIT_NONE);
  if (name == "output.weight") return set(&p->output, c.vocab, d, false, split_of(name));
  if (name == "output_norm.weight") return set(&p->output_norm, 1, d, true, SPLIT_NONE);
  if (name == "rope_freqs.weight") {
    s->ignored = true;
    return set(nullptr, 1, (uint64_t)(c.rope_dim ? c.rope_dim : c.head_dim) / 2, true, SPLIT_NONE);
  }
  int layer = -1, used = 0;
  if (sscanf(name.c_str(), "blk.%d.%n", &layer, &used) != 1 || layer < 0 || layer >= c.n_layers) return false;
  const std::string suffix = name.substr((size_t)used);
  LayerW &L = p->layers[(size_t)layer];
  if (suffix == "attn_norm.weight") return set(&L.attn_norm, 1, d, true, SPLIT_NONE);
  if (suffix == "ffn_norm.weight") return set(&L.ffn_norm, 1, d, true, SPLIT_NONE);
  if (suffix == "attn_q.weight") return set(&L.q, qw, d, false, split_of(name));
  if (suffix == "attn_k.weight") return set(&L.k, kw, d, false, split_of(name));
  if (suffix == "attn_v.weight") return set(&L.v, kw, d, false, split_of(name));
  if (suffix == "attn_output.weight") return set(&L.o, d, qw, false, split_of(name));
  if (suffix == "ffn_gate.weight") return set(&L.gate, f, d, false, split_of(name));
  if (suffix == "ffn_up.weight") return set(&L.up, f, d, false, split_of(name));
  if (suffix == "ffn_down.weight") return set(&L.down, d, f, false, split_of(name));
  // present only in the variant the configuration names (model.rs:427-449)
  const uint64_t hd = (uint64_t)c.head_dim;
  if (c.qk_norm && suffix == "attn_q_norm.weight") return set(&L.q_norm, 1, c.qk_norm == 1 ? hd : qw, true, SPLIT_NONE);
  if (c.qk_norm && suffix == "attn_k_norm.weight") return set(&L.k_norm, 1, c.qk_norm == 1 ? hd : kw, true, SPLIT_NONE);
  if (c.qkv_bias && suffix == "attn_q.bias") return set(&L.q_bias, 1, qw, true, SPLIT_NONE);
  if (c.qkv_bias && suffix == "attn_k.bias") return set(&L.k_bias, 1, kw, true, SPLIT_NONE);
  if (c.qkv_bias && suffix == "attn_v.bias") return set(&L.v_bias, 1, kw, true, SPLIT_NONE);
  return false;
}

// Shape/type checks shared by uploaded and synthesized tensors.  Computes the rank-local shard.
static int32_t check_tensor(rg_plan *p, const std::string &name, int32_t type, uint64_t rows, uint64_t cols, Slot *slot,
                            uint64_t *r0, uint64_t *lr, uint64_t *c0, uint64_t *lc) {
  if (!find_slot(p, name, slot)) return fail(RG_UNEXPECTED_TENSOR, "unexpected tensor " + name);
  if (!block_elements(type)) return fail(RG_UNSUPPORTED_TYPE, name + ": ggml type " + std::to_string(type) + " is not supported");
  if (slot->norm && type != RG_TYPE_F32 && type != RG_TYPE_F16)
    return fail(RG_UNSUPPORTED_TYPE, name + ": packed tensor where a dense vector is required");
  if (rows != slot->rows || cols != slot->cols)
    return fail(RG_SHAPE_MISMATCH, name + ": expected [" + std::to_string(slot->rows) + "," + std::to_string(slot->cols) +
                                       "], got [" + std::to_string(rows) + "," + std::to_string(cols) + "]");
  if (cols % (uint64_t)block_elements(type)) return fail(RG_SHAPE_MISMATCH, name + ": columns are not a multiple of the block size");
  if (slot->t && slot->t->type >= 0) return fail(RG_INVALID_ARGUMENT, name + ": tensor bound twice");
  return shard_range(name, type, rows, cols, slot->split, (uint64_t)p->tp_world, (uint64_t)p->tp_rank, r0, lr, c0, lc);
}

}  // namespace rg

// ------------------------------------------------------------------------------------------
// Session
// ------------------------------------------------------------------------------------------
static constexpr int MAXC = 16;   // columns of the GEMV paths: decode batches <= 16 (dense-weight GEMVs: <= DENSE_MAXC)
static constexpr int DENSE_MAXC = 8;  // columns the dense-weight GEMV takes; prompt chunk of models with dense tensors
static constexpr int WMAX = 1024;  // columns of the tensor-core path: prefill chunk, decode batch 9..32
static constexpr int SCOLS = 256;  // columns the per-column attention kernels are given scratch for
static constexpr int BMAX = 32;   // independent sequences per session

struct Ctrl {  // device control block, uploaded in one copy per host-driven step
  int32_t tokens[WMAX];
  int32_t pos[WMAX];
  int32_t seq[WMAX];
  int32_t logit_cols[BMAX];
  int32_t step;
  int32_t pad[3];
};

struct rg_session {
  rg_llama_config cfg{};
  rg_options opt{};
  int tp_rank = 0, tp_world = 1;
  int heads_l = 0, kv_l = 0, ffn_l = 0, vocab_l = 0;  // rank-local sizes
  int max_batch = 1, ctx = 0;
  bool kv_f32 = false, use_graph = true, use_pdl = true;
  cudaStream_t stream = nullptr;
  int sm_count = 148;
  Comm comm;
  std::vector<LayerW> layers;
  DevTensor token_embd, output_norm, output;
  const DevTensor *head = nullptr;
  uint64_t weight_bytes = 0, kv_bytes = 0;
  // device buffers
  Ctrl *d_ctrl = nullptr;
  int32_t *d_ids = nullptr, *d_history = nullptr;
  int *d_status = nullptr;
  float *x = nullptr, *xn_f32 = nullptr, *qkv = nullptr, *q_rot = nullptr, *attn_scratch = nullptr, *attn_f32 = nullptr;
  float *partial = nullptr, *gate_f32 = nullptr, *up_f32 = nullptr, *h_f32 = nullptr, *logits = nullptr, *logits_l = nullptr;
  void *xn_pack = nullptr, *attn_pack = nullptr, *h_pack = nullptr, *head_pack = nullptr;
  // batch-1 decode: activation vectors packed by their producers for the integer GEMV that reads them
  // (qgemv_i8.cu): the residual stream after a projection, and the attention output
  uint8_t *xq_x = nullptr, *xq_attn = nullptr, *xq_h = nullptr;
  int32_t *xq_h_fix = nullptr;  // blocks of the SwiGLU output that straddle two CTAs of the gate/up launch
  int xq_h_nfix = 0;
  // Gumbel-max selection for the current step: device rows of uniforms [logit cols][vocab]; null = greedy
  const float *sample_uniforms = nullptr;
  float sample_temperature = 1.0f;
  float *d_uniforms = nullptr;  // [BMAX][vocab], allocated on first use
  const float *sample_temps = nullptr;  // per-column temperatures of a mixed step (device), else null
  float *d_temps = nullptr;             // [BMAX]
  bool chunk_is_prompt = false;  // the columns of the current step are runs of consecutive positions (prompt_segments)
  struct PromptSegment {
    int col0, cols, seq, pos0;
  };
  std::vector<PromptSegment> prompt_segments;  // one run per sequence in the current prompt chunk
  // partial rotary lanes, q / k RMS norms or projection biases: such models take the general
  // q/k/v post-processing kernel and the three-launch attention on every path
  bool variant = false;
  int rope_dim = 0;  // rotary lanes per head (head_dim for the plain layer)
  float *split_scratch = nullptr;  // K-split partial tiles of the tensor-core GEMM at small token counts and of the 3..16-row GEMV
  unsigned *gemv_counters = nullptr;  // arrival counters of the K-split row GEMV, zero between launches
  // deferred RMSNorm of 3..16-row steps: per-CTA sums of squares left by the O (a) and down (b) projections
  float *ssq_a = nullptr, *ssq_b = nullptr;
  bool defer_norm_ok = false;
  bool packed_layers = false;  // one GPU and every layer tensor Q4_0 / Q8_0 with whole 256-element groups: the GEMV paths serve 3..16 rows
  void *xb = nullptr;  // 16-bit operand planes (hi, lo) of the tensor-core path: [2][WMAX][max(d, qw, ffn_l)]
  int gemm_mode = QGEMM_F16X3;
  int xb_ld = 0;
  float *cos_t = nullptr, *sin_t = nullptr;
  std::vector<void *> k_cache, v_cache;
  std::vector<void *> owned;  // everything to cudaFree
  // pinned host staging
  Ctrl *h_ctrl = nullptr;
  int32_t *h_result = nullptr;  // pinned: [status, pad x 3, ids / id history]
  int32_t *h_ids = nullptr;
  int *h_status = nullptr;
  float *h_logits = nullptr;
  int history_cap = 0;
  // state
  std::vector<int32_t> position;
  bool poisoned = false;
  std::map<int, cudaGraphExec_t> graphs;  // by batch
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  rg_report report{};
  uint64_t launches_in_step = 0;
  // profiling pass: only the kernel families in family_mask are launched
  unsigned family_mask = 0xffffffffu;
  int cur_kind = 0;
  // finer selection inside the GEMV family for the per-projection profile (bit = GemvSite); all by default
  unsigned gemv_site_mask = 0xffffffffu;
  int cur_site = 0;
  // development trace (RG_B200_TRACE=1): 16 u64 per launch of a small-batch step, in launch order
  unsigned long long *d_trace = nullptr;
  int trace_cap = 0, trace_next = 0;
  // tensor-parallel partial sums: [0] output projection, [1] down projection.  Fused form: the buffers live
  // in one block that the other ranks map through CUDA IPC (tp_fused.cu); otherwise both point at `partial`
  float *tp_part[2] = {nullptr, nullptr};
  bool tp_fused = false;
  const float **tp_peer_part[2] = {nullptr, nullptr};  // device arrays [world]
  unsigned **tp_peer_flags = nullptr;                  // device array [world]
  float **tp_peer_recv = nullptr;                      // device array [world]: receive areas of the push form (null: pull)
  unsigned *tp_epochs = nullptr;
  std::vector<void *> tp_ipc_opened;
  // one-launch decode attention (attn_fused.cu): arrival counters per (column, kv head); null = not used
  unsigned *attn_counters = nullptr;
  int attn_max_splits = 0;

  ~rg_session() {
    for (auto &g : graphs) cudaGraphExecDestroy(g.second);
    for (void *p : tp_ipc_opened) cudaIpcCloseMemHandle(p);
    for (void *p : owned) cudaFree(p);
    if (h_ctrl) cudaFreeHost(h_ctrl);
    if (h_result) cudaFreeHost(h_result);
    if (h_logits) cudaFreeHost(h_logits);
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
    comm_destroy(&comm);
    if (stream) cudaStreamDestroy(stream);
  }
};

namespace rg {

template <typename T>
static int32_t dalloc(rg_session *s, T **p, size_t count) {
  void *raw = nullptr;
  RG_CUDA(x_malloc(&raw, count * sizeof(T)));
  s->owned.push_back(raw);
  *p = static_cast<T *>(raw);
  return RG_OK;
}

static LaunchCfg lcfg(rg_session *s) {
  LaunchCfg c;
  c.stream = s->stream;
  c.pdl = s->use_pdl;
  c.sm_count = s->sm_count;
  c.status = s->d_status;
  return c;
}
// The next launch's slots of the development trace (null when tracing is off or the buffer is full).
static unsigned long long *next_trace(rg_session *s) {
  if (!s->d_trace || s->trace_next >= s->trace_cap) return nullptr;
  return s->d_trace + (size_t)16 * (size_t)s->trace_next++;
}

#define RG_LAUNCH(s, expr)                                                                       \
  do {                                                                                           \
    if (((s)->family_mask & (1u << (s)->cur_kind)) &&                                            \
        ((s)->cur_kind != 0 || ((s)->gemv_site_mask & (1u << (s)->cur_site)))) {                 \
      cudaError_t e__ = x_launch(expr);                                                          \
      (s)->launches_in_step++;                                                                   \
      if (e__ != cudaSuccess)                                                                    \
        return fail(RG_CUDA_ERROR, std::string(#expr) + ": " + cudaGetErrorString(e__) + " (" +  \
                                       __FILE__ + ":" + std::to_string(__LINE__) + ")");         \
    }                                                                                            \
  } while (0)

enum ProfKind { PROF_GEMV = 0, PROF_ATTN = 1, PROF_OTHER = 2, PROF_END = 3 };
// Which projection a GEMV launch serves (forward_small); SITE_ANY for the other paths.
enum GemvSite { SITE_ANY = 0, SITE_QKV = 1, SITE_O = 2, SITE_GATE_UP = 3, SITE_DOWN = 4, SITE_HEAD = 5, SITE_END = 6 };

// Names the kernel family of the launches that follow; the profiling pass launches one family
// at a time.
static inline void prof_mark(rg_session *s, int kind) { s->cur_kind = kind; }

// Deferred RMSNorm around a packed projection of a batch step (GemvArgs): the input rows come without their
// 1 / rms (ssq_in), and / or the residual rows this projection completes leave packed for the next norm.
struct NormFuse {
  const float *ssq_in = nullptr;
  int ssq_n = 0;
  void *pack_next = nullptr;
  const float *pack_w = nullptr;
  float *ssq_out = nullptr;
};

// y = W x for one projection given as `n` row segments sharing K.  Packed segments of one type go
// out as a single fused launch; dense ones run the dense kernel segment by segment.
static int32_t linear(rg_session *s, const DevTensor *const *w, int n, const void *in_pack, const float *in_f32, int ld_in,
                      int batch, int epi, float *y, int ldy, const NormFuse *nf = nullptr) {
  bool all_packed = true;
  for (int i = 0; i < n; ++i) all_packed = all_packed && w[i]->packed() && w[i]->type == w[0]->type;
  prof_mark(s, PROF_GEMV);
  if (all_packed) {
    GemvArgs a;
    a.type = w[0]->type;
    a.nseg = n;
    for (int i = 0; i < n; ++i) {
      a.w[i] = w[i]->d;
      a.seg_rows[i] = (int)w[i]->rows;
    }
    a.k = (int)w[0]->cols;
    a.xpack = in_pack;
    a.batch = batch;
    a.epi = epi;
    a.y = y;
    a.ldy = ldy;
    a.split_scratch = s->split_scratch;
    a.split_scratch_floats = s->split_scratch ? (size_t)BMAX * 2 * s->sm_count * 256 : 0;
    a.split_counters = s->gemv_counters;
    if (nf) {
      a.ssq_in = nf->ssq_in;
      a.ssq_n = nf->ssq_n;
      a.norm_eps = s->cfg.norm_eps;
      a.pack_next = nf->pack_next;
      a.pack_w = nf->pack_w;
      a.ssq_out = nf->ssq_out;
    }
    RG_LAUNCH(s, launch_qgemv(a, lcfg(s)));
    return RG_OK;
  }
  int row0 = 0;
  for (int i = 0; i < n; ++i) {
    if (w[i]->packed()) {
      GemvArgs a;
      a.type = w[i]->type;
      a.nseg = 1;
      a.w[0] = w[i]->d;
      a.seg_rows[0] = (int)w[i]->rows;
      a.k = (int)w[i]->cols;
      a.xpack = in_pack;
      a.batch = batch;
      a.epi = epi;
      a.y = y + row0;
      a.ldy = ldy;
      a.split_scratch = s->split_scratch;
      a.split_scratch_floats = s->split_scratch ? (size_t)BMAX * 2 * s->sm_count * 256 : 0;
      a.split_counters = s->gemv_counters;
      if (nf) {  // (pack_next needs the one-launch form: whole rows of the residual stream)
        if (nf->pack_next) return fail(RG_INVALID_ARGUMENT, "deferred norm output on a segmented projection");
        a.ssq_in = nf->ssq_in;
        a.ssq_n = nf->ssq_n;
        a.norm_eps = s->cfg.norm_eps;
      }
      RG_LAUNCH(s, launch_qgemv(a, lcfg(s)));
    } else {
      if (nf && (nf->ssq_in || nf->pack_next)) return fail(RG_INVALID_ARGUMENT, "deferred norm on a dense projection");
      DenseGemvArgs a;
      a.type = w[i]->type;
      a.w = w[i]->d;
      a.rows = (int)w[i]->rows;
      a.k = (int)w[i]->cols;
      a.x = in_f32;
      a.ldx = ld_in;
      a.batch = batch;
      a.epi = epi;
      a.y = y + row0;
      a.ldy = ldy;
      RG_LAUNCH(s, launch_dense_gemv(a, lcfg(s)));
    }
    row0 += (int)w[i]->rows;
  }
  return RG_OK;
}

// x += sum over ranks of the partial projection in buffer `which` (0: output projection, 1: down
// projection).  Fused form: one kernel over NVLink peer memory; otherwise NCCL all-reduce + add.
// pack_*: also leave the new residual row packed for the GEMV that reads it next (one column, peer-memory exchange only)
static int32_t tp_reduce_add(rg_session *s, int ncols, int which, uint8_t *pack_out = nullptr, const float *pack_w = nullptr,
                             int pack_type = 0) {
  const int d = s->cfg.d_model;
  std::string err;
  prof_mark(s, PROF_OTHER);
  if (!(s->family_mask & (1u << PROF_OTHER))) return RG_OK;
  // The one-shot peer-memory kernel is tuned for the latency of a decode step (16 CTAs, every rank
  // pulls every rank's whole partial).  A prompt chunk moves megabytes per exchange, which is
  // bandwidth work: it goes through the ring / tree of ncclAllReduce, then one add kernel.
  if (s->tp_fused && ncols <= BMAX) {
    TpFusedArgs a;
    a.x = s->x;
    a.ldx = d;
    a.n = d;
    a.cols = ncols;
    a.peer_partial = s->tp_peer_part[which];
    a.ldp = d;
    a.peer_flags = s->tp_peer_flags;
    a.epochs = s->tp_epochs;
    a.rank = s->tp_rank;
    a.world = s->tp_world;
    a.buffer = which;
    a.pack_out = pack_out;
    a.pack_w = pack_w;
    a.pack_type = pack_type;
    a.peer_recv = ncols <= TP_PUSH_COLS ? s->tp_peer_recv : nullptr;
    RG_LAUNCH(s, launch_tp_allreduce_add(a, lcfg(s)));
    s->report.peer_reduce_launches++;
    return RG_OK;
  }
  int32_t rc = comm_allreduce_sum_f32(&s->comm, s->tp_part[which], (size_t)ncols * d, s->stream, &err);
  if (rc) return fail(rc, err);
  LaunchCfg c = lcfg(s);
  c.pdl = false;  // follows a library kernel
  RG_LAUNCH(s, launch_add_rows(s->x, d, s->tp_part[which], d, d, ncols, c));
  return RG_OK;
}

// Variant fields of the q/k/v post-processing launch (no-ops for the plain layer).
static void rope_variant(const rg_session *s, const LayerW &W, RopeArgs *ra) {
  ra->rope_dim = s->rope_dim;
  ra->qk_norm = s->cfg.qk_norm;
  ra->eps = s->cfg.norm_eps;
  ra->q_norm = reinterpret_cast<const float *>(W.q_norm.d);
  ra->k_norm = reinterpret_cast<const float *>(W.k_norm.d);
  ra->q_bias = reinterpret_cast<const float *>(W.q_bias.d);
  ra->k_bias = reinterpret_cast<const float *>(W.k_bias.d);
  ra->v_bias = reinterpret_cast<const float *>(W.v_bias.d);
}

// Decode rows of distinct sequences on f16 caches: from eight rows on, the tensor-core attention with per-warp
// cp.async rings (attn_decode_tc.cu) streams K / V faster than the one-launch kernel, whose CTAs load, score and
// combine one after the other.  Measured on the 8B shape, attention ms per step, new against one-launch: 16 rows
// 1.52 / 1.88 at context 2100; 8 rows 0.63 / 0.72 at context 1024 and 0.43 / 0.45 at 200; 6 rows 0.59 / 0.57;
// 4 rows 0.54 / 0.48.  So seven rows and fewer keep the one-launch kernel.
static bool decode_tc_attention(const rg_session *s, int ncols) {
  static const bool off = env_flag("RG_B200_NO_ATTN_DECODE_TC");
  static const int min_cols = [] {
    const char *v = getenv("RG_B200_ATTN_TC_MIN_COLS");
    const int n = v ? atoi(v) : 0;
    return n > 0 ? n : 8;
  }();
  if (off || s->chunk_is_prompt || ncols < min_cols || ncols > BMAX) return false;
  AttnArgs a;
  a.kv_f32 = s->kv_f32;
  a.heads = s->heads_l;
  a.kv_heads = s->kv_l;
  a.hd = s->cfg.head_dim;
  return attention_decode_tc_supported(a) &&
         attention_decode_tc_scratch_floats(s->sm_count, s->heads_l, s->kv_l, ncols, s->ctx) <=
             attn_scratch_floats(SCOLS, s->heads_l, s->cfg.head_dim, s->ctx);
}

// True when every projection of the model can run the integer tensor-core GEMV at this width.
static bool small_batch_path(const rg_session *s, int ncols) {
  if (ncols > 2 || s->opt.general_path_only || s->variant) return false;
  const int d = s->cfg.d_model, qw = s->heads_l * s->cfg.head_dim;
  if (!qgemv_i8_supported(d, ncols) || !qgemv_i8_supported(qw, ncols) || !qgemv_i8_supported(s->ffn_l, ncols)) return false;
  for (const LayerW &W : s->layers) {
    if (!W.q.packed() || W.k.type != W.q.type || W.v.type != W.q.type || !W.o.packed() || !W.gate.packed() ||
        W.up.type != W.gate.type || !W.down.packed())
      return false;
  }
  return s->head->packed();
}

// Packed input / output of one integer GEMV launch of a batch-1 step (see GemvI8Args).
struct PackedIo {
  int site = SITE_ANY;
  const uint8_t *xq = nullptr;
  bool xq_norm = false;
  const int32_t *xq_fix = nullptr;
  int xq_nfix = 0;
  uint8_t *pack_out = nullptr;
  const float *pack_w = nullptr;
  int pack_type = 0;
  // the packed tensors the next GEMV of the step streams (asked into L2 by this launch)
  const DevTensor *const *next_w = nullptr;
  int next_n = 0;
  int next_lead = 0;  // the first next_lead tensors are read before the others
};

// How much of the next kernel's weights a GEMV launch asks into L2 (all tensors together).
static size_t l2_prefetch_budget() {
  static const size_t bytes = [] {
    const char *e = getenv("RG_B200_L2_PREFETCH_MB");
    return (size_t)(e ? atoi(e) : 40) << 20;
  }();
  return bytes;
}

static int32_t gemv_i8(rg_session *s, const DevTensor *const *w, int n, const float *x, int ldx, const int32_t *col_map,
                       const float *norm_w, int batch, int epi, float *y, int ldy, const LaunchCfg &L,
                       const PackedIo &io = PackedIo()) {
  GemvI8Args a;
  a.xq = io.xq;
  a.xq_norm = io.xq_norm;
  a.xq_fix = io.xq_fix;
  a.xq_nfix = io.xq_nfix;
  a.pack_out = io.pack_out;
  a.pack_w = io.pack_w;
  a.pack_type = io.pack_type;
  {
    // split the budget over the tensors in proportion (gate and up are consumed side by side)
    size_t budget = l2_prefetch_budget(), total = 0;
    for (int i = 0; i < io.next_n && i < 3; ++i) {
      if (!io.next_w[i]->packed()) continue;
      a.next_w[i] = io.next_w[i]->d;
      if (i < io.next_lead) {  // read first: taken whole as far as the budget goes
        a.next_bytes[i] = std::min(io.next_w[i]->nbytes, budget);
        budget -= a.next_bytes[i];
      } else {
        total += io.next_w[i]->nbytes;
      }
    }
    for (int i = io.next_lead; i < io.next_n && i < 3; ++i)
      if (a.next_w[i]) a.next_bytes[i] = total <= budget ? io.next_w[i]->nbytes : (size_t)((double)io.next_w[i]->nbytes * budget / total);
  }
  a.type = w[0]->type;
  a.nseg = n;
  for (int i = 0; i < n; ++i) {
    a.w[i] = w[i]->d;
    a.seg_rows[i] = (int)w[i]->rows;
  }
  a.k = (int)w[0]->cols;
  a.x = x;
  a.ldx = ldx;
  a.col_map = col_map;
  a.norm_w = norm_w;
  a.eps = s->cfg.norm_eps;
  a.batch = batch;
  a.epi = epi;
  a.y = y;
  a.ldy = ldy;
  prof_mark(s, PROF_GEMV);
  s->cur_site = io.site;
  LaunchCfg Lt = L;
  Lt.trace = next_trace(s);
  RG_LAUNCH(s, launch_qgemv_i8(a, Lt));
  s->cur_site = SITE_ANY;
  return RG_OK;
}

// Decode forward for one or two columns: RMSNorm and activation packing live in the GEMV
// prologues, so a layer is seven launches (QKV, RoPE+append, attention split, combine, O, gate/up
// with SwiGLU, down).
static int32_t forward_small(rg_session *s, int ncols, int n_logit_cols, bool advance) {
  const rg_llama_config &c = s->cfg;
  const int d = c.d_model, hd = c.head_dim;
  const int qw = s->heads_l * hd, kw = s->kv_l * hd, qkv_w = qw + 2 * kw;
  Ctrl *ctl = s->d_ctrl;
  LaunchCfg L = lcfg(s);
  LaunchCfg plain = L;
  plain.pdl = false;
  const bool tp = s->tp_world > 1;
  const bool tp_lib = tp && !s->tp_fused;  // a library collective precedes some kernels: no dependent launch there
  int32_t rc;
  // One column on one GPU: the residual epilogues (output and down projection) leave the new residual
  // stream packed, with the next norm weight folded in, for the projection that reads it, whose
  // prologue is then a single bulk copy; the norm's scalar factor is applied to that projection's results.
  s->trace_next = 0;
  // (under tensor parallelism the peer-memory exchange kernel, which adds the residual, is that producer)
  const bool pre = ncols == 1 && (!tp || s->tp_fused) && s->xq_x && !env_flag("RG_B200_NO_PREPACK");
  // likewise the one-launch attention packs its output for the output projection (any world size:
  // the heads are rank-local)
  const bool pre_attn = ncols == 1 && s->xq_attn && s->attn_counters && !env_flag("RG_B200_NO_PREPACK");
  prof_mark(s, PROF_OTHER);
  RG_LAUNCH(s, launch_row_gather(s->token_embd.type, s->token_embd.d, d, ctl->tokens, ncols, s->x, d, plain));
  for (int l = 0; l < c.n_layers; ++l) {
    const LayerW &W = s->layers[(size_t)l];
    const DevTensor *qkvw[3] = {&W.q, &W.k, &W.v};
    const DevTensor *ow[1] = {&W.o};
    const DevTensor *guw[2] = {&W.gate, &W.up};
    const DevTensor *dw[1] = {&W.down};
    const DevTensor *hw_next[1] = {s->head};
    const DevTensor *qkv_next[3] = {nullptr, nullptr, nullptr};
    if (l + 1 < c.n_layers) {
      const LayerW &N = s->layers[(size_t)l + 1];
      qkv_next[0] = &N.q;
      qkv_next[1] = &N.k;
      qkv_next[2] = &N.v;
    }
    PackedIo qkv_io;
    qkv_io.site = SITE_QKV;
    // the attention launch between this projection and the next reads little: ask for the output
    // projection and, with what is left of the budget, the start of gate / up
    const DevTensor *after_qkv[3] = {&W.o, &W.gate, &W.up};
    qkv_io.next_w = after_qkv;
    qkv_io.next_n = env_flag("RG_B200_PF_QKV_O_ONLY") ? 1 : 3;
    qkv_io.next_lead = 1;
    if (pre && l > 0) {  // layer 0 reads the embedding row, which nothing packed
      qkv_io.xq = s->xq_x;
      qkv_io.xq_norm = true;
    }
    // the first GEMV of a layer follows a collective (library kernel) under tensor parallelism
    if ((rc = gemv_i8(s, qkvw, 3, s->x, d, nullptr, reinterpret_cast<const float *>(W.attn_norm.d), ncols, EPI_STORE, s->qkv,
                      qkv_w, (tp_lib && l > 0) ? plain : L, qkv_io)))
      return rc;
    prof_mark(s, PROF_ATTN);
    // Two columns of ONE sequence (a two-token prompt chunk) must not share the one-launch kernel:
    // column 1 reads the cache row that column 0 appends in the same launch.  Such a chunk takes
    // the append-then-attend launches below; columns of distinct sequences never read each other's rows.
    if (s->attn_counters && (!s->chunk_is_prompt || ncols == 1)) {
      // RoPE, cache append, split attention and the combine in one launch
      FusedAttnArgs fa;
      fa.qkv = s->qkv;
      fa.cols = ncols;
      fa.heads = s->heads_l;
      fa.kv_heads = s->kv_l;
      fa.hd = hd;
      fa.ctx = s->ctx;
      fa.col_seq = ctl->seq;
      fa.col_pos = ctl->pos;
      fa.cos_t = s->cos_t;
      fa.sin_t = s->sin_t;
      fa.k_cache = s->k_cache[(size_t)l];
      fa.v_cache = s->v_cache[(size_t)l];
      fa.kv_f32 = s->kv_f32;
      fa.scratch = s->attn_scratch;
      fa.max_splits = s->attn_max_splits;
      fa.counters = s->attn_counters;
      fa.out = s->attn_f32;
      fa.early = l > 0;  // layer 0 follows the kernels that set the positions
      if (pre_attn) {
        fa.pack_out = s->xq_attn;
        fa.pack_type = W.o.type;
      }
      LaunchCfg Lt = L;
      Lt.trace = next_trace(s);
      RG_LAUNCH(s, launch_attention_fused(fa, Lt));
    } else {
      RopeArgs ra;
      ra.qkv = s->qkv;
      ra.cols = ncols;
      ra.heads = s->heads_l;
      ra.kv_heads = s->kv_l;
      ra.hd = hd;
      ra.ctx = s->ctx;
      ra.col_seq = ctl->seq;
      ra.col_pos = ctl->pos;
      ra.cos_t = s->cos_t;
      ra.sin_t = s->sin_t;
      ra.q_out = s->q_rot;
      ra.k_cache = s->k_cache[(size_t)l];
      ra.v_cache = s->v_cache[(size_t)l];
      ra.kv_f32 = s->kv_f32;
      rope_variant(s, W, &ra);
    RG_LAUNCH(s, launch_rope_append(ra, L));
      AttnArgs aa;
      aa.q = s->q_rot;
      aa.k_cache = ra.k_cache;
      aa.v_cache = ra.v_cache;
      aa.kv_f32 = s->kv_f32;
      aa.cols = ncols;
      aa.heads = s->heads_l;
      aa.kv_heads = s->kv_l;
      aa.hd = hd;
      aa.ctx = s->ctx;
      aa.col_seq = ctl->seq;
      aa.col_pos = ctl->pos;
      aa.scratch = s->attn_scratch;
      aa.out_f32 = s->attn_f32;
      RG_LAUNCH(s, launch_attention(aa, L));
      if (s->family_mask & (1u << PROF_ATTN)) s->launches_in_step++;  // split + combine
    }
    PackedIo o_in;
    o_in.site = SITE_O;
    o_in.next_w = guw;
    o_in.next_n = 2;
    if (pre_attn) o_in.xq = s->xq_attn;
    if (tp) {
      if ((rc = gemv_i8(s, ow, 1, s->attn_f32, qw, nullptr, nullptr, ncols, EPI_STORE, s->tp_part[0], d, L, o_in))) return rc;
      if ((rc = tp_reduce_add(s, ncols, 0, pre ? s->xq_x : nullptr, reinterpret_cast<const float *>(W.ffn_norm.d), W.gate.type)))
        return rc;
    } else {
      PackedIo io = o_in;
      if (pre) {
        io.pack_out = s->xq_x;
        io.pack_w = reinterpret_cast<const float *>(W.ffn_norm.d);
        io.pack_type = W.gate.type;
      }
      if ((rc = gemv_i8(s, ow, 1, s->attn_f32, qw, nullptr, nullptr, ncols, EPI_RESIDUAL, s->x, d, L, io))) return rc;
    }
    PackedIo gu_io;
    gu_io.site = SITE_GATE_UP;
    gu_io.next_w = dw;
    gu_io.next_n = 1;
    if (pre) {
      gu_io.xq = s->xq_x;
      gu_io.xq_norm = true;
    }
    PackedIo down_in;  // the SwiGLU epilogue packs the blocks that lie inside one of its CTAs, the down projection the rest
    down_in.site = SITE_DOWN;
    if (l + 1 < c.n_layers) {
      down_in.next_w = qkv_next;
      down_in.next_n = 3;
    } else if (n_logit_cols > 0) {
      down_in.next_w = hw_next;
      down_in.next_n = 1;
    }
    if (pre_attn && s->xq_h) {
      gu_io.pack_out = s->xq_h;
      gu_io.pack_type = W.down.type;
      down_in.xq = s->xq_h;
      down_in.xq_fix = s->xq_h_fix;
      down_in.xq_nfix = s->xq_h_nfix;
    }
    if ((rc = gemv_i8(s, guw, 2, s->x, d, nullptr, reinterpret_cast<const float *>(W.ffn_norm.d), ncols, EPI_SWIGLU, s->h_f32,
                      s->ffn_l, tp_lib ? plain : L, gu_io)))
      return rc;
    if (tp) {
      if ((rc = gemv_i8(s, dw, 1, s->h_f32, s->ffn_l, nullptr, nullptr, ncols, EPI_STORE, s->tp_part[1], d, L, down_in))) return rc;
      const bool last = l + 1 == c.n_layers;
      if ((rc = tp_reduce_add(s, ncols, 1, pre ? s->xq_x : nullptr,
                              reinterpret_cast<const float *>(last ? s->output_norm.d : s->layers[(size_t)l + 1].attn_norm.d),
                              last ? s->head->type : s->layers[(size_t)l + 1].q.type)))
        return rc;
    } else {
      PackedIo io = down_in;
      if (pre) {  // read next by the following layer's q/k/v projection, or by the head after the last layer
        const bool last = l + 1 == c.n_layers;
        io.pack_out = s->xq_x;
        io.pack_w = reinterpret_cast<const float *>(last ? s->output_norm.d : s->layers[(size_t)l + 1].attn_norm.d);
        io.pack_type = last ? s->head->type : s->layers[(size_t)l + 1].q.type;
      }
      if ((rc = gemv_i8(s, dw, 1, s->h_f32, s->ffn_l, nullptr, nullptr, ncols, EPI_RESIDUAL, s->x, d, L, io))) return rc;
    }
  }
  if (n_logit_cols > 0) {
    const DevTensor *hw[1] = {s->head};
    const bool split_head = tp && s->head == &s->output;
    float *dst = split_head ? s->logits_l : s->logits;
    const int ld = split_head ? s->vocab_l : c.vocab;
    PackedIo head_io;
    head_io.site = SITE_HEAD;
    if (pre) {  // one column: the logit column is column 0
      head_io.xq = s->xq_x;
      head_io.xq_norm = true;
    }
    if ((rc = gemv_i8(s, hw, 1, s->x, d, ctl->logit_cols, reinterpret_cast<const float *>(s->output_norm.d), n_logit_cols,
                      EPI_STORE, dst, ld, tp_lib ? plain : L, head_io)))
      return rc;
    LaunchCfg am = L;
    prof_mark(s, PROF_OTHER);
    if (split_head && (s->family_mask & (1u << PROF_OTHER))) {
      std::string err;
      if ((rc = comm_group_start(&err))) return fail(rc, err);
      for (int col = 0; col < n_logit_cols; ++col)
        if ((rc = comm_allgather_f32(&s->comm, s->logits_l + (size_t)col * s->vocab_l, s->logits + (size_t)col * c.vocab,
                                     (size_t)s->vocab_l, s->stream, &err)))
          return fail(rc, err);
      if ((rc = comm_group_end(&err))) return fail(rc, err);
      am.pdl = false;
    }
    RG_LAUNCH(s, launch_select(s->logits, c.vocab, c.vocab, n_logit_cols, s->sample_uniforms, s->sample_temperature, s->d_ids, am, s->sample_temps));
    if (advance) RG_LAUNCH(s, launch_advance(s->d_ids, ctl->tokens, ctl->pos, s->d_history, &ctl->step, ncols, L));
  }
  return RG_OK;
}

// True when every projection can run the tensor-core GEMM (packed, K a multiple of 256).
static bool wide_path_ok(const rg_session *s) {
  if (s->opt.general_path_only) return false;
  for (const LayerW &W : s->layers)
    for (const DevTensor *t : {&W.q, &W.k, &W.v, &W.o, &W.gate, &W.up, &W.down})
      if (!t->packed() || t->cols % 256) return false;
  return s->head->packed() && s->head->cols % 256 == 0;
}

// Operand planes of the tensor-core path.  The default mode is the compensated one: single bf16 or
// f16 operands leave the logits of a prompt 1e-2 .. 1e-1 away from the f32 arithmetic.
static Operand16 wide_operand(const rg_session *s) {
  Operand16 o;
  o.hi = s->xb;
  o.lo = s->gemm_mode == QGEMM_F16X3 ? static_cast<uint8_t *>(s->xb) + (size_t)WMAX * s->xb_ld * 2 : nullptr;
  o.ld = s->xb_ld;
  o.f16 = s->gemm_mode != QGEMM_BF16;
  return o;
}

static int32_t gemm_tc(rg_session *s, const DevTensor &w, int m, float *out, int ldc, const LaunchCfg &L, bool accumulate = false) {
  QGemmArgs a;
  a.accumulate = accumulate;
  a.type = w.type;
  a.w = w.d;
  a.n = (int)w.rows;
  a.k = (int)w.cols;
  const Operand16 op = wide_operand(s);
  a.x16 = op.hi;
  a.x16_lo = op.lo;
  a.mode = s->gemm_mode;
  a.ldx = s->xb_ld;
  a.m = m;
  a.out = out;
  a.ldc = ldc;
  prof_mark(s, PROF_GEMV);
  // Few tokens (decode batches of 9..32): one CTA per 128 weight rows would leave most SMs without
  // weights to stream, so K is split until about two CTAs per SM exist and the partial tiles are summed.
  const int rows_per_cta = qgemm_rows_per_cta(s->gemm_mode);
  const int tiles = ((int)w.rows + rows_per_cta - 1) / rows_per_cta;  // CTAs along the weight rows
  int splits = (m <= BMAX && s->split_scratch) ? (2 * s->sm_count) / tiles : 1;
  splits = qgemm_effective_splits(a.k, splits);
  while (splits > 1 && (size_t)splits * (size_t)m * (size_t)a.n > (size_t)BMAX * 2 * (size_t)s->sm_count * 256) --splits;  // never past the scratch
  splits = qgemm_effective_splits(a.k, splits);  // the launcher's own count: the reduction sums exactly the tiles it writes
  if (splits > 1) {
    if (accumulate) return fail(RG_INVALID_ARGUMENT, "a split-K GEMM cannot add into its output");
    a.out = s->split_scratch;
    a.ldc = a.n;
    a.splits = splits;
    a.split_stride = (size_t)m * a.n;
    RG_LAUNCH(s, launch_qgemm_tc(a, L));
    RG_LAUNCH(s, launch_reduce_splits(s->split_scratch, splits, a.split_stride, a.n, m, out, ldc, L));
    return RG_OK;
  }
  RG_LAUNCH(s, launch_qgemm_tc(a, L));
  return RG_OK;
}

// Forward for 9..1024 columns (a prefill chunk, or decode of 9..32 rows): the projections run on
// the tcgen05 tensor cores (compensated f16 operands by default); norms, RoPE, attention and residuals stay f32.
static int32_t forward_wide(rg_session *s, int ncols, int n_logit_cols, bool advance) {
  const rg_llama_config &c = s->cfg;
  const int d = c.d_model, hd = c.head_dim;
  const int qw = s->heads_l * hd, kw = s->kv_l * hd, qkv_w = qw + 2 * kw;
  Ctrl *ctl = s->d_ctrl;
  LaunchCfg L = lcfg(s);
  LaunchCfg plain = L;
  plain.pdl = false;
  const bool tp = s->tp_world > 1;
  const bool tp_lib = tp && !s->tp_fused;  // a library collective precedes some kernels: no dependent launch there
  const Operand16 xop = wide_operand(s);
  int32_t rc;
  prof_mark(s, PROF_OTHER);
  RG_LAUNCH(s, launch_row_gather(s->token_embd.type, s->token_embd.d, d, ctl->tokens, ncols, s->x, d, plain));
  for (int l = 0; l < c.n_layers; ++l) {
    const LayerW &W = s->layers[(size_t)l];
    prof_mark(s, PROF_OTHER);
    RG_LAUNCH(s, launch_rmsnorm16(s->x, d, reinterpret_cast<const float *>(W.attn_norm.d), d, c.norm_eps, ncols, xop,
                                  (tp_lib && l > 0) ? plain : L));
    if (W.qkv_stacked && ncols > BMAX) {  // one GEMM over the stacked rows of q | k | v
      DevTensor all = W.q;
      all.rows = W.q.rows + W.k.rows + W.v.rows;
      all.nbytes = W.q.nbytes + W.k.nbytes + W.v.nbytes;
      if ((rc = gemm_tc(s, all, ncols, s->qkv, qkv_w, L))) return rc;
    } else {
      if ((rc = gemm_tc(s, W.q, ncols, s->qkv, qkv_w, L))) return rc;
      if ((rc = gemm_tc(s, W.k, ncols, s->qkv + qw, qkv_w, L))) return rc;
      if ((rc = gemm_tc(s, W.v, ncols, s->qkv + qw + kw, qkv_w, L))) return rc;
    }
    prof_mark(s, PROF_ATTN);
    bool attn_in_operand = false;
    const bool tc_attn = decode_tc_attention(s, ncols);
    if (!tc_attn && !s->chunk_is_prompt && ncols <= BMAX && s->attn_counters && !s->variant) {
      // a decode batch: RoPE, cache append, split attention and the combine in one launch
      FusedAttnArgs fa;
      fa.qkv = s->qkv;
      fa.cols = ncols;
      fa.heads = s->heads_l;
      fa.kv_heads = s->kv_l;
      fa.hd = hd;
      fa.ctx = s->ctx;
      fa.col_seq = ctl->seq;
      fa.col_pos = ctl->pos;
      fa.cos_t = s->cos_t;
      fa.sin_t = s->sin_t;
      fa.k_cache = s->k_cache[(size_t)l];
      fa.v_cache = s->v_cache[(size_t)l];
      fa.kv_f32 = s->kv_f32;
      fa.scratch = s->attn_scratch;
      fa.max_splits = s->attn_max_splits;
      fa.counters = s->attn_counters;
      fa.out = s->attn_f32;
      RG_LAUNCH(s, launch_attention_fused(fa, L));
    } else {
    RopeArgs ra;
    ra.qkv = s->qkv;
    ra.cols = ncols;
    ra.heads = s->heads_l;
    ra.kv_heads = s->kv_l;
    ra.hd = hd;
    ra.ctx = s->ctx;
    ra.col_seq = ctl->seq;
    ra.col_pos = ctl->pos;
    ra.cos_t = s->cos_t;
    ra.sin_t = s->sin_t;
    ra.q_out = s->q_rot;
    ra.k_cache = s->k_cache[(size_t)l];
    ra.v_cache = s->v_cache[(size_t)l];
    ra.kv_f32 = s->kv_f32;
    rope_variant(s, W, &ra);
    RG_LAUNCH(s, launch_rope_append(ra, L));
    if (s->chunk_is_prompt && prefill_attention_supported(s->heads_l, s->kv_l, hd)) {  // q and the caches are post-processed already
      // consecutive positions of one sequence: the tiled causal kernel reads each K / V row once per CTA
      // (a chunk of several prompts holds one run per sequence: one launch per run)
      bool to_operand = true;  // every run wrote the operand planes of the output projection itself
      for (const auto &seg : s->prompt_segments) {
        PrefillAttnArgs pa;
        pa.q = s->q_rot + (size_t)seg.col0 * qw;
        pa.k_cache = ra.k_cache;
        pa.v_cache = ra.v_cache;
        pa.kv_f32 = s->kv_f32;
        pa.cols = seg.cols;
        pa.heads = s->heads_l;
        pa.kv_heads = s->kv_l;
        pa.ctx = s->ctx;
        pa.seq = seg.seq;
        pa.pos0 = seg.pos0;
        pa.out = s->attn_f32 + (size_t)seg.col0 * qw;
        if (prefill_attention_uses_tc(pa)) {
          pa.out16_hi = static_cast<uint16_t *>(xop.hi) + (size_t)seg.col0 * xop.ld;
          pa.out16_lo = xop.lo ? static_cast<uint16_t *>(xop.lo) + (size_t)seg.col0 * xop.ld : nullptr;
          pa.out16_ld = xop.ld;
          pa.out16_f16 = xop.f16;
        } else {
          to_operand = false;
        }
        RG_LAUNCH(s, launch_attention_prefill(pa, L));
      }
      attn_in_operand = to_operand;
    } else {
      AttnArgs aa;
      aa.q = s->q_rot;
      aa.k_cache = ra.k_cache;
      aa.v_cache = ra.v_cache;
      aa.kv_f32 = s->kv_f32;
      aa.cols = ncols;
      aa.heads = s->heads_l;
      aa.kv_heads = s->kv_l;
      aa.hd = hd;
      aa.ctx = s->ctx;
      aa.col_seq = ctl->seq;
      aa.col_pos = ctl->pos;
      aa.scratch = s->attn_scratch;
      aa.out_f32 = s->attn_f32;
      if (tc_attn) {
        RG_LAUNCH(s, launch_attention_decode_tc(aa, L));
      } else {
        RG_LAUNCH(s, launch_attention(aa, L));
      }
      if (s->family_mask & (1u << PROF_ATTN)) s->launches_in_step++;  // split + combine
    }
    }
    if (!attn_in_operand) RG_LAUNCH(s, launch_to16(s->attn_f32, qw, qw, ncols, xop, L));
    const bool add_in_gemm = !tp && ncols > BMAX;  // one GPU, no K split: the projection adds into the residual stream itself
    if (add_in_gemm) {
      if ((rc = gemm_tc(s, W.o, ncols, s->x, d, L, true))) return rc;
    } else {
      if ((rc = gemm_tc(s, W.o, ncols, s->tp_part[0], d, L))) return rc;
      if (tp) {
        if ((rc = tp_reduce_add(s, ncols, 0))) return rc;
      } else {
        prof_mark(s, PROF_OTHER);
        RG_LAUNCH(s, launch_add_rows(s->x, d, s->tp_part[0], d, d, ncols, L));
      }
    }
    prof_mark(s, PROF_OTHER);
    RG_LAUNCH(s, launch_rmsnorm16(s->x, d, reinterpret_cast<const float *>(W.ffn_norm.d), d, c.norm_eps, ncols, xop,
                                  tp_lib ? plain : L));
    if (W.gu_stacked && ncols > BMAX) {  // one GEMM over gate | up: token rows of [gate, up] side by side
      DevTensor all = W.gate;
      all.rows = W.gate.rows + W.up.rows;
      all.nbytes = W.gate.nbytes + W.up.nbytes;
      if ((rc = gemm_tc(s, all, ncols, s->gate_f32, 2 * s->ffn_l, L))) return rc;
      prof_mark(s, PROF_OTHER);
      RG_LAUNCH(s, launch_swiglu16(s->gate_f32, s->gate_f32 + s->ffn_l, s->ffn_l, 2 * s->ffn_l, ncols, xop, L));
    } else {
      if ((rc = gemm_tc(s, W.gate, ncols, s->gate_f32, s->ffn_l, L))) return rc;
      if ((rc = gemm_tc(s, W.up, ncols, s->up_f32, s->ffn_l, L))) return rc;
      prof_mark(s, PROF_OTHER);
      RG_LAUNCH(s, launch_swiglu16(s->gate_f32, s->up_f32, s->ffn_l, s->ffn_l, ncols, xop, L));
    }
    if (add_in_gemm) {
      if ((rc = gemm_tc(s, W.down, ncols, s->x, d, L, true))) return rc;
    } else {
      if ((rc = gemm_tc(s, W.down, ncols, s->tp_part[1], d, L))) return rc;
      if (tp) {
        if ((rc = tp_reduce_add(s, ncols, 1))) return rc;
      } else {
        prof_mark(s, PROF_OTHER);
        RG_LAUNCH(s, launch_add_rows(s->x, d, s->tp_part[1], d, d, ncols, L));
      }
    }
  }
  if (n_logit_cols > 0) {
    const bool split_head = tp && s->head == &s->output;
    float *dst = split_head ? s->logits_l : s->logits;
    const int ld = split_head ? s->vocab_l : c.vocab;
    if (n_logit_cols <= 2) {
      // a prompt's last token: the integer GEMV with the final norm in its prologue
      const DevTensor *hw[1] = {s->head};
      if ((rc = gemv_i8(s, hw, 1, s->x, d, ctl->logit_cols, reinterpret_cast<const float *>(s->output_norm.d), n_logit_cols,
                        EPI_STORE, dst, ld, tp_lib ? plain : L)))
        return rc;
    } else {
      // decode of many rows: logit column i is row i.  A chunk of several prompts wants the last
      // column of each prompt instead: those rows are gathered first
      prof_mark(s, PROF_OTHER);
      const float *head_in = s->x;
      if (s->chunk_is_prompt) {
        RG_LAUNCH(s, launch_row_gather(RG_TYPE_F32, reinterpret_cast<const uint8_t *>(s->x), d, ctl->logit_cols, n_logit_cols,
                                       s->partial, d, tp_lib ? plain : L));
        head_in = s->partial;
      }
      RG_LAUNCH(s, launch_rmsnorm16(head_in, d, reinterpret_cast<const float *>(s->output_norm.d), d, c.norm_eps, n_logit_cols, xop,
                                    (tp_lib && !s->chunk_is_prompt) ? plain : L));
      if ((rc = gemm_tc(s, *s->head, n_logit_cols, dst, ld, L))) return rc;
    }
    LaunchCfg am = L;
    prof_mark(s, PROF_OTHER);
    if (split_head && (s->family_mask & (1u << PROF_OTHER))) {
      std::string err;
      if ((rc = comm_group_start(&err))) return fail(rc, err);
      for (int col = 0; col < n_logit_cols; ++col)
        if ((rc = comm_allgather_f32(&s->comm, s->logits_l + (size_t)col * s->vocab_l, s->logits + (size_t)col * c.vocab,
                                     (size_t)s->vocab_l, s->stream, &err)))
          return fail(rc, err);
      if ((rc = comm_group_end(&err))) return fail(rc, err);
      am.pdl = false;
    }
    RG_LAUNCH(s, launch_select(s->logits, c.vocab, c.vocab, n_logit_cols, s->sample_uniforms, s->sample_temperature, s->d_ids, am, s->sample_temps));
    if (advance) RG_LAUNCH(s, launch_advance(s->d_ids, ctl->tokens, ctl->pos, s->d_history, &ctl->step, ncols, L));
  }
  return RG_OK;
}

// Peer-memory exchange for the tensor-parallel partial sums: allocates this rank's block (two
// partial buffers + flag words), trades CUDA IPC handles through the NCCL communicator and maps the
// other ranks' blocks.  Every rank learns whether ALL ranks succeeded (one more all-reduce) and only
// then switches to the fused kernel; otherwise the NCCL all-reduce path stays in place.
static int32_t tp_fused_setup(rg_session *s) {
  const int W = s->tp_world, d = s->cfg.d_model;
  if (W > TP_FUSED_MAX_WORLD || d % 4) return RG_OK;
  const size_t part_floats = (size_t)WMAX * d;
  // two partial buffers, the flag words, then the receive area of the push form
  const size_t recv_off = 2 * part_floats * sizeof(float) + ((TP_FUSED_FLAG_WORDS * sizeof(unsigned) + 255) & ~(size_t)255);
  const size_t recv_floats = (size_t)2 * 2 * W * TP_PUSH_COLS * d;  // 8-byte words {value, epoch}
  const size_t block_bytes = recv_off + recv_floats * sizeof(float);
  uint8_t *block = nullptr;
  float *xchg = nullptr;  // [16 floats of handle + 1 ok flag] * (1 + W)
  int32_t rc;
  if ((rc = dalloc(s, &block, block_bytes))) return rc;
  if ((rc = dalloc(s, &xchg, (size_t)17 * (1 + W)))) return rc;
  RG_CUDA(cudaMemset(block, 0, block_bytes));
  cudaIpcMemHandle_t mine;
  float host[17 * (1 + TP_FUSED_MAX_WORLD)] = {0};
  float ok = cudaIpcGetMemHandle(&mine, block) == cudaSuccess ? 1.0f : 0.0f;
  cudaGetLastError();
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(host, &mine, sizeof(mine));
  host[16] = ok;
  RG_CUDA(cudaMemcpy(xchg, host, 17 * sizeof(float), cudaMemcpyHostToDevice));
  std::string err;
  if ((rc = comm_allgather_f32(&s->comm, xchg, xchg + 17, 17, s->stream, &err))) return fail(rc, err);
  RG_CUDA(cudaStreamSynchronize(s->stream));
  RG_CUDA(cudaMemcpy(host + 17, xchg + 17, (size_t)17 * W * sizeof(float), cudaMemcpyDeviceToHost));
  std::vector<uint8_t *> base((size_t)W, nullptr);
  for (int r = 0; r < W; ++r) ok = std::min(ok, host[17 + 17 * r + 16]);
  if (ok > 0.5f) {
    for (int r = 0; r < W; ++r) {
      if (r == s->tp_rank) {
        base[(size_t)r] = block;
        continue;
      }
      cudaIpcMemHandle_t h;
      memcpy(&h, host + 17 + 17 * r, sizeof(h));
      void *ptr = nullptr;
      if (cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        ok = 0.0f;
        break;
      }
      s->tp_ipc_opened.push_back(ptr);
      base[(size_t)r] = static_cast<uint8_t *>(ptr);
    }
  }
  // agreement: the fused path is used only if every rank mapped every block
  host[0] = ok;
  RG_CUDA(cudaMemcpy(xchg, host, sizeof(float), cudaMemcpyHostToDevice));
  if ((rc = comm_allreduce_sum_f32(&s->comm, xchg, 1, s->stream, &err))) return fail(rc, err);
  RG_CUDA(cudaStreamSynchronize(s->stream));
  RG_CUDA(cudaMemcpy(host, xchg, sizeof(float), cudaMemcpyDeviceToHost));
  if (host[0] < (float)W - 0.5f) return RG_OK;  // some rank could not: everyone keeps the NCCL path
  std::vector<const float *> pa((size_t)W), pb((size_t)W);
  std::vector<unsigned *> pf((size_t)W);
  std::vector<float *> pr((size_t)W);
  for (int r = 0; r < W; ++r) {
    pa[(size_t)r] = reinterpret_cast<const float *>(base[(size_t)r]);
    pb[(size_t)r] = reinterpret_cast<const float *>(base[(size_t)r]) + part_floats;
    pf[(size_t)r] = reinterpret_cast<unsigned *>(base[(size_t)r] + 2 * part_floats * sizeof(float));
    pr[(size_t)r] = reinterpret_cast<float *>(base[(size_t)r] + recv_off);
  }
  const float **d_pa, **d_pb;
  unsigned **d_pf;
  float **d_pr;
  if ((rc = dalloc(s, &d_pa, (size_t)W))) return rc;
  if ((rc = dalloc(s, &d_pb, (size_t)W))) return rc;
  if ((rc = dalloc(s, &d_pf, (size_t)W))) return rc;
  if ((rc = dalloc(s, &d_pr, (size_t)W))) return rc;
  RG_CUDA(cudaMemcpy(d_pr, pr.data(), sizeof(void *) * (size_t)W, cudaMemcpyHostToDevice));
  s->tp_peer_recv = env_flag("RG_B200_TP_PULL") ? nullptr : d_pr;
  if ((rc = dalloc(s, &s->tp_epochs, (size_t)2 * TP_FUSED_CTAS))) return rc;
  RG_CUDA(cudaMemcpy(d_pa, pa.data(), sizeof(void *) * (size_t)W, cudaMemcpyHostToDevice));
  RG_CUDA(cudaMemcpy(d_pb, pb.data(), sizeof(void *) * (size_t)W, cudaMemcpyHostToDevice));
  RG_CUDA(cudaMemcpy(d_pf, pf.data(), sizeof(void *) * (size_t)W, cudaMemcpyHostToDevice));
  RG_CUDA(cudaMemset(s->tp_epochs, 0, sizeof(unsigned) * 2 * TP_FUSED_CTAS));
  s->tp_peer_part[0] = d_pa;
  s->tp_peer_part[1] = d_pb;
  s->tp_peer_flags = d_pf;
  s->tp_part[0] = reinterpret_cast<float *>(block);
  s->tp_part[1] = reinterpret_cast<float *>(block) + part_floats;
  s->tp_fused = true;
  return RG_OK;
}

// One forward over `ncols` columns described by the device control block.  n_logit_cols columns
// (indices in ctrl.logit_cols) get logits + greedy ids; 0 skips the head (non-final prefill chunk).
static int32_t forward(rg_session *s, int ncols, int n_logit_cols, bool advance) {
  if (small_batch_path(s, ncols)) return forward_small(s, ncols, n_logit_cols, advance);
  // Decode batches of 9..16 rows stream the weights once through the f16-MMA GEMV (four column
  // tiles); prompt chunks of that size and everything wider run on the tcgen05 GEMM.
  const bool gemv16 = ncols > DENSE_MAXC && ncols <= MAXC && !s->chunk_is_prompt && wide_path_ok(s) && !env_flag("RG_B200_NO_GEMV16");
  if (ncols > DENSE_MAXC && !gemv16) {
    if (!wide_path_ok(s))
      return fail(RG_UNSUPPORTED_GEOMETRY, "more than 8 columns need packed projections with K a multiple of 256");
    return forward_wide(s, ncols, n_logit_cols, advance);
  }
  const rg_llama_config &c = s->cfg;
  const int d = c.d_model, hd = c.head_dim;
  const int qw = s->heads_l * hd, kw = s->kv_l * hd, qkv_w = qw + 2 * kw;
  Ctrl *ctl = s->d_ctrl;
  LaunchCfg L = lcfg(s);
  LaunchCfg first = L;
  first.pdl = false;  // follows a memcpy, not a kernel
  prof_mark(s, PROF_OTHER);
  RG_LAUNCH(s, launch_row_gather(s->token_embd.type, s->token_embd.d, d, ctl->tokens, ncols, s->x, d, first));
  const bool defer = s->defer_norm_ok && ncols >= 3 && ncols <= 16;
  const int ssq_n = qgemv_grid(d, s->sm_count);  // CTAs of a projection with d output rows
  for (int l = 0; l < c.n_layers; ++l) {
    const LayerW &W = s->layers[(size_t)l];
    const bool qkv_dense = !W.q.packed() || !W.k.packed() || !W.v.packed();
    // 3..16 rows on packed weights: only the first norm of the step is a launch of its own; afterwards the O and
    // down projections leave the new residual rows packed (times the next norm's weight) with their sums of
    // squares, and the projection that consumes them applies 1 / rms to its outputs
    NormFuse qkv_in;
    if (defer && l > 0) {
      qkv_in.ssq_in = s->ssq_b;
      qkv_in.ssq_n = ssq_n;
    } else {
      prof_mark(s, PROF_OTHER);
      RG_LAUNCH(s, launch_rmsnorm_pack(s->x, d, reinterpret_cast<const float *>(W.attn_norm.d), d, c.norm_eps, ncols, nullptr,
                                       s->xn_pack, qkv_dense ? s->xn_f32 : nullptr, d, L));
    }
    const DevTensor *qkvw[3] = {&W.q, &W.k, &W.v};
    int32_t rc = linear(s, qkvw, 3, s->xn_pack, s->xn_f32, d, ncols, EPI_STORE, s->qkv, qkv_w, &qkv_in);
    if (rc) return rc;
    prof_mark(s, PROF_ATTN);
    const bool tc_attn = decode_tc_attention(s, ncols);
    if (!tc_attn && (gemv16 || (ncols >= 3 && !s->chunk_is_prompt && !env_flag("RG_B200_SPLIT_ATTENTION_SMALL"))) &&
        s->attn_counters && !s->variant) {
      // rows of distinct sequences: RoPE, cache append, split attention and the combine in one launch
      FusedAttnArgs fa;
      fa.qkv = s->qkv;
      fa.cols = ncols;
      fa.heads = s->heads_l;
      fa.kv_heads = s->kv_l;
      fa.hd = hd;
      fa.ctx = s->ctx;
      fa.col_seq = ctl->seq;
      fa.col_pos = ctl->pos;
      fa.cos_t = s->cos_t;
      fa.sin_t = s->sin_t;
      fa.k_cache = s->k_cache[(size_t)l];
      fa.v_cache = s->v_cache[(size_t)l];
      fa.kv_f32 = s->kv_f32;
      fa.scratch = s->attn_scratch;
      fa.max_splits = s->attn_max_splits;
      fa.counters = s->attn_counters;
      fa.out = s->attn_f32;
      fa.xpack_out = s->attn_pack;  // the O projection's packed input comes out of the same launch
      RG_LAUNCH(s, launch_attention_fused(fa, L));
    } else {
    RopeArgs ra;
    ra.qkv = s->qkv;
    ra.cols = ncols;
    ra.heads = s->heads_l;
    ra.kv_heads = s->kv_l;
    ra.hd = hd;
    ra.ctx = s->ctx;
    ra.col_seq = ctl->seq;
    ra.col_pos = ctl->pos;
    ra.cos_t = s->cos_t;
    ra.sin_t = s->sin_t;
    ra.q_out = s->q_rot;
    ra.k_cache = s->k_cache[(size_t)l];
    ra.v_cache = s->v_cache[(size_t)l];
    ra.kv_f32 = s->kv_f32;
    rope_variant(s, W, &ra);
    RG_LAUNCH(s, launch_rope_append(ra, L));
    AttnArgs aa;
    aa.q = s->q_rot;
    aa.k_cache = ra.k_cache;
    aa.v_cache = ra.v_cache;
    aa.kv_f32 = s->kv_f32;
    aa.cols = ncols;
    aa.heads = s->heads_l;
    aa.kv_heads = s->kv_l;
    aa.hd = hd;
    aa.ctx = s->ctx;
    aa.col_seq = ctl->seq;
    aa.col_pos = ctl->pos;
    aa.scratch = s->attn_scratch;
    aa.out_pack = s->attn_pack;
    aa.out_f32 = W.o.packed() ? nullptr : s->attn_f32;
    if (tc_attn) {
      RG_LAUNCH(s, launch_attention_decode_tc(aa, L));
    } else {
      RG_LAUNCH(s, launch_attention(aa, L));
    }
    if (s->family_mask & (1u << PROF_ATTN)) s->launches_in_step++;  // split + combine
    }
    const DevTensor *ow[1] = {&W.o};
    if (s->tp_world > 1) {
      if ((rc = linear(s, ow, 1, s->attn_pack, s->attn_f32, qw, ncols, EPI_STORE, s->tp_part[0], d))) return rc;
      if ((rc = tp_reduce_add(s, ncols, 0))) return rc;
    } else {
      NormFuse o_out;
      if (defer) {
        o_out.pack_next = s->xn_pack;
        o_out.pack_w = reinterpret_cast<const float *>(W.ffn_norm.d);
        o_out.ssq_out = s->ssq_a;
      }
      if ((rc = linear(s, ow, 1, s->attn_pack, s->attn_f32, qw, ncols, EPI_RESIDUAL, s->x, d, &o_out))) return rc;
    }
    LaunchCfg after = L;
    if (s->tp_world > 1 && !s->tp_fused) after.pdl = false;
    const bool gu_dense = !W.gate.packed() || !W.up.packed() || W.gate.type != W.up.type;
    if (!defer) {
      prof_mark(s, PROF_OTHER);
      RG_LAUNCH(s, launch_rmsnorm_pack(s->x, d, reinterpret_cast<const float *>(W.ffn_norm.d), d, c.norm_eps, ncols, nullptr,
                                       s->xn_pack, gu_dense ? s->xn_f32 : nullptr, d, after));
    }
    if (!gu_dense) {
      prof_mark(s, PROF_GEMV);
      GemvArgs a;
      a.type = W.gate.type;
      a.nseg = 2;
      a.w[0] = W.gate.d;
      a.w[1] = W.up.d;
      a.seg_rows[0] = a.seg_rows[1] = s->ffn_l;
      a.k = d;
      a.xpack = s->xn_pack;
      a.batch = ncols;
      a.epi = EPI_SWIGLU;
      a.ypack = s->h_pack;
      if (defer) {
        a.ssq_in = s->ssq_a;
        a.ssq_n = ssq_n;
        a.norm_eps = c.norm_eps;
      }
      RG_LAUNCH(s, launch_qgemv(a, L));
      if (!W.down.packed()) RG_LAUNCH(s, launch_unpack(s->h_pack, s->ffn_l, ncols, s->h_f32, s->ffn_l, L));
    } else {
      const DevTensor *gw[1] = {&W.gate}, *uw[1] = {&W.up};
      if ((rc = linear(s, gw, 1, s->xn_pack, s->xn_f32, d, ncols, EPI_STORE, s->gate_f32, s->ffn_l))) return rc;
      if ((rc = linear(s, uw, 1, s->xn_pack, s->xn_f32, d, ncols, EPI_STORE, s->up_f32, s->ffn_l))) return rc;
      RG_LAUNCH(s, launch_swiglu(s->gate_f32, s->up_f32, s->ffn_l, s->ffn_l, ncols, s->h_pack, s->h_f32, s->ffn_l, L));
    }
    const DevTensor *dw[1] = {&W.down};
    if (s->tp_world > 1) {
      if ((rc = linear(s, dw, 1, s->h_pack, s->h_f32, s->ffn_l, ncols, EPI_STORE, s->tp_part[1], d))) return rc;
      if ((rc = tp_reduce_add(s, ncols, 1))) return rc;
    } else {
      NormFuse d_out;
      if (defer && l + 1 < c.n_layers) {
        d_out.pack_next = s->xn_pack;
        d_out.pack_w = reinterpret_cast<const float *>(s->layers[(size_t)l + 1].attn_norm.d);
        d_out.ssq_out = s->ssq_b;
      }
      if ((rc = linear(s, dw, 1, s->h_pack, s->h_f32, s->ffn_l, ncols, EPI_RESIDUAL, s->x, d, &d_out))) return rc;
    }
  }
  if (n_logit_cols > 0) {
    LaunchCfg after = L;
    if (s->tp_world > 1 && !s->tp_fused) after.pdl = false;
    prof_mark(s, PROF_OTHER);
    RG_LAUNCH(s, launch_rmsnorm_pack(s->x, d, reinterpret_cast<const float *>(s->output_norm.d), d, c.norm_eps, n_logit_cols,
                                     ctl->logit_cols, s->head_pack, s->head->packed() ? nullptr : s->xn_f32, d, after));
    const DevTensor *hw[1] = {s->head};
    const bool split_head = s->tp_world > 1 && s->head == &s->output;
    float *dst = split_head ? s->logits_l : s->logits;
    const int ld = split_head ? s->vocab_l : c.vocab;
    int32_t rc = linear(s, hw, 1, s->head_pack, s->xn_f32, d, n_logit_cols, EPI_STORE, dst, ld);
    if (rc) return rc;
    LaunchCfg am = L;
    prof_mark(s, PROF_OTHER);
    if (split_head && (s->family_mask & (1u << PROF_OTHER))) {
      std::string err;
      if ((rc = comm_group_start(&err))) return fail(rc, err);
      for (int col = 0; col < n_logit_cols; ++col)
        if ((rc = comm_allgather_f32(&s->comm, s->logits_l + (size_t)col * s->vocab_l, s->logits + (size_t)col * c.vocab,
                                     (size_t)s->vocab_l, s->stream, &err)))
          return fail(rc, err);
      if ((rc = comm_group_end(&err))) return fail(rc, err);
      am.pdl = false;
    }
    RG_LAUNCH(s, launch_select(s->logits, c.vocab, c.vocab, n_logit_cols, s->sample_uniforms, s->sample_temperature, s->d_ids, am, s->sample_temps));
    if (advance) RG_LAUNCH(s, launch_advance(s->d_ids, ctl->tokens, ctl->pos, s->d_history, &ctl->step, ncols, L));
  }
  return RG_OK;
}

// Captures the decode step for `batch` rows once and returns the executable graph.
static int32_t decode_graph(rg_session *s, int batch, cudaGraphExec_t *out) {
  auto it = s->graphs.find(batch);
  if (it != s->graphs.end()) {
    *out = it->second;
    return RG_OK;
  }
  // Run every kernel once outside capture so lazy module loading and function attributes are
  // done.  The run uses the control block already uploaded; what it writes (KV rows at the
  // current positions, advanced control block) is rewritten by the upload and the replay below.
  s->launches_in_step = 0;
  int32_t warm = forward(s, batch, batch, true);
  if (warm) return warm;
  RG_CUDA(x_memcpy_async(s->d_ctrl, s->h_ctrl, sizeof(Ctrl), cudaMemcpyHostToDevice, s->stream));
  RG_CUDA(cudaStreamSynchronize(s->stream));
  RG_CUDA(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
  s->launches_in_step = 0;
  int32_t rc = forward(s, batch, batch, true);
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(s->stream, &graph);
  if (rc) {
    if (graph) cudaGraphDestroy(graph);
    return rc;
  }
  if (e != cudaSuccess) return fail(RG_CUDA_ERROR, std::string("cudaStreamEndCapture: ") + cudaGetErrorString(e));
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return fail(RG_CUDA_ERROR, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
  s->graphs[batch] = exec;
  *out = exec;
  return RG_OK;
}

static int32_t run_step(rg_session *s, int ncols, int n_logit_cols, bool advance, bool allow_graph) {
  if (allow_graph && s->use_graph) {
    cudaGraphExec_t exec;
    int32_t rc = decode_graph(s, ncols, &exec);
    if (rc) return rc;
    if (inject(g_faults.launch_after)) return fail(RG_CUDA_ERROR, "injected graph launch failure");
    RG_CUDA(cudaGraphLaunch(exec, s->stream));
    s->report.graph_replays++;
    s->report.kernel_launches += s->launches_in_step;
    return RG_OK;
  }
  s->launches_in_step = 0;
  int32_t rc = forward(s, ncols, n_logit_cols, advance);
  s->report.kernel_launches += s->launches_in_step;
  return rc;
}

static int32_t upload_ctrl(rg_session *s) {
  RG_CUDA(x_memcpy_async(s->d_ctrl, s->h_ctrl, sizeof(Ctrl), cudaMemcpyHostToDevice, s->stream));
  s->report.h2d_calls++;
  s->report.h2d_bytes += sizeof(Ctrl);
  return RG_OK;
}

// Reads back the status word and `n` greedy ids; maps device findings to typed statuses.
static int32_t finish_step(rg_session *s, int n_ids, float *logits_out, int n_logit_rows) {
  // status word and ids lie side by side on both sides: one copy
  const size_t res_bytes = sizeof(int32_t) * (n_ids > 0 ? 4 + (size_t)n_ids : 1);
  RG_CUDA(x_memcpy_async(s->h_result, s->d_status, res_bytes, cudaMemcpyDeviceToHost, s->stream));
  s->report.d2h_calls += 1;
  s->report.d2h_bytes += res_bytes;
  if (logits_out && n_logit_rows > 0) {
    const size_t bytes = sizeof(float) * (size_t)n_logit_rows * (size_t)s->cfg.vocab;
    RG_CUDA(x_memcpy_async(s->h_logits, s->logits, bytes, cudaMemcpyDeviceToHost, s->stream));
    s->report.d2h_calls++;
    s->report.d2h_bytes += bytes;
  }
  cudaError_t e = x_sync(s->stream);
  if (e != cudaSuccess) {
    s->poisoned = true;  // completion cannot be proven (src/runtime/cuda_graph.rs:542-546)
    return fail(RG_POISONED, std::string("stream synchronize: ") + cudaGetErrorString(e));
  }
  if (*s->h_status == 1) {
    s->poisoned = true;
    return fail(RG_TIMEOUT, "a bounded device-side wait gave up");
  }
  if (*s->h_status != 0) return fail(RG_CUDA_ERROR, "device status " + std::to_string(*s->h_status));
  if (logits_out && n_logit_rows > 0) memcpy(logits_out, s->h_logits, sizeof(float) * (size_t)n_logit_rows * (size_t)s->cfg.vocab);
  for (int i = 0; i < n_ids; ++i)
    if (s->h_ids[i] < 0) return fail(RG_NON_FINITE_LOGITS, "non-finite logits in row " + std::to_string(i));
  return RG_OK;
}

static int32_t check_live(const rg_session *s) {
  if (!s) return fail(RG_INVALID_ARGUMENT, "null session");
  if (s->poisoned) return fail(RG_POISONED, "session poisoned by an earlier failure");
  return RG_OK;
}

}  // namespace rg

// ==========================================================================================
// C ABI
// ==========================================================================================
extern "C" {

const char *rg_b200_version(void) { return "rg_b200 0.1 (sm_100a)"; }

const char *rg_b200_status_string(int32_t st) {
  static const char *names[] = {"OK", "INVALID_ARGUMENT", "UNSUPPORTED_TYPE", "SHAPE_MISMATCH", "NON_FINITE_SCALE",
                                "TOKEN_OUT_OF_RANGE", "CONTEXT_EXHAUSTED", "NON_FINITE_LOGITS", "FRESH_SESSION_REQUIRED",
                                "CUDA_ERROR", "NCCL_ERROR", "OUT_OF_MEMORY", "TIMEOUT", "POISONED", "MALFORMED_GGUF",
                                "MISSING_TENSOR", "UNEXPECTED_TENSOR", "UNSUPPORTED_VARIANT", "MISSING_METADATA", "EMPTY_PROMPT",
                                "UNSUPPORTED_GEOMETRY"};
  if (st < 0 || st > 20) return "UNKNOWN";
  return names[st];
}

const char *rg_b200_last_error(void) { return g_last_error.c_str(); }

// Test hook: make the n-th next call of a wrapped CUDA entry fail ("malloc", "memcpy", "launch",
// "sync"); n < 0 disarms.  Host-side fault injection in the manner of src/cuda.rs:5895-5960.
int32_t rg_b200_test_fail_after(const char *what, int32_t n) {
  if (!what) return RG_INVALID_ARGUMENT;
  if (!strcmp(what, "malloc")) g_faults.malloc_after = n;
  else if (!strcmp(what, "memcpy")) g_faults.memcpy_after = n;
  else if (!strcmp(what, "launch")) g_faults.launch_after = n;
  else if (!strcmp(what, "sync")) g_faults.sync_after = n;
  else return RG_INVALID_ARGUMENT;
  return RG_OK;
}

// Test hook: makes a bounded device-side wait of this session run out, without faulting or hanging
// anything.  The partial-sum exchange kernel is launched on the session's stream as rank 0 of a
// pretended world of two whose flag words all live in local memory; nothing ever writes the slot of
// rank 1, the poll limit is cut to a few thousand polls, so the kernel records DEV_TIMEOUT in the
// session's status word and returns.  The session's next step reports RG_TIMEOUT and is poisoned.
int32_t rg_b200_test_expire_device_wait(rg_session *s) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  RG_CUDA(cudaSetDevice(s->opt.device));
  const int d = s->cfg.d_model;
  if (d % 4) return fail(RG_UNSUPPORTED_GEOMETRY, "d_model must be a multiple of 4");
  float *part = nullptr, *x = nullptr;
  unsigned *flags = nullptr, *epochs = nullptr;
  const float **d_parts = nullptr;
  unsigned **d_flags = nullptr;
  if ((rc = dalloc(s, &part, (size_t)d)) || (rc = dalloc(s, &x, (size_t)d)) || (rc = dalloc(s, &flags, (size_t)TP_FUSED_FLAG_WORDS)) ||
      (rc = dalloc(s, &epochs, (size_t)2 * TP_FUSED_CTAS)) || (rc = dalloc(s, &d_parts, (size_t)2)) || (rc = dalloc(s, &d_flags, (size_t)2)))
    return rc;
  RG_CUDA(cudaMemsetAsync(part, 0, sizeof(float) * (size_t)d, s->stream));
  RG_CUDA(cudaMemsetAsync(x, 0, sizeof(float) * (size_t)d, s->stream));
  RG_CUDA(cudaMemsetAsync(flags, 0, sizeof(unsigned) * TP_FUSED_FLAG_WORDS, s->stream));
  RG_CUDA(cudaMemsetAsync(epochs, 0, sizeof(unsigned) * 2 * TP_FUSED_CTAS, s->stream));
  const float *hp[2] = {part, part};
  unsigned *hf[2] = {flags, flags};
  RG_CUDA(cudaMemcpyAsync(d_parts, hp, sizeof(hp), cudaMemcpyHostToDevice, s->stream));
  RG_CUDA(cudaMemcpyAsync(d_flags, hf, sizeof(hf), cudaMemcpyHostToDevice, s->stream));
  RG_CUDA(cudaStreamSynchronize(s->stream));
  TpFusedArgs a;
  a.x = x;
  a.ldx = d;
  a.n = d;
  a.cols = 1;
  a.peer_partial = d_parts;
  a.ldp = d;
  a.peer_flags = d_flags;
  a.epochs = epochs;
  a.rank = 0;
  a.world = 2;
  a.buffer = 0;
  a.poll_limit = 4096;
  LaunchCfg c = lcfg(s);
  c.pdl = false;
  RG_CUDA(launch_tp_allreduce_add(a, c));
  return RG_OK;
}

// ------------------------------------------------------------------------------ GGUF
int32_t rg_b200_gguf_open(const uint8_t *bytes, size_t len, rg_gguf **out) {
  if (!bytes || !out) return fail(RG_INVALID_ARGUMENT, "null argument");
  auto g = std::make_unique<rg_gguf>();
  std::string err;
  int32_t rc = gguf_parse(bytes, len, &g->g, &err);
  if (rc) return fail(rc, err);
  *out = g.release();
  return RG_OK;
}
void rg_b200_gguf_close(rg_gguf *g) { delete g; }
size_t rg_b200_gguf_tensor_count(const rg_gguf *g) { return g ? g->g.tensors.size() : 0; }
int32_t rg_b200_gguf_tensor_info(const rg_gguf *g, size_t index, const char **name, int32_t *type, int32_t *rank, uint64_t dims[4],
                                 const uint8_t **data, size_t *nbytes) {
  if (!g || index >= g->g.tensors.size()) return fail(RG_INVALID_ARGUMENT, "tensor index out of range");
  const GgufTensorInfo &t = g->g.tensors[index];
  if (name) *name = t.name.c_str();
  if (type) *type = t.ggml_type;
  if (rank) *rank = (int32_t)t.shape.size();
  if (dims)
    for (size_t i = 0; i < t.shape.size(); ++i) dims[i] = t.shape[i];
  if (data) *data = g->g.bytes + t.offset;
  if (nbytes) *nbytes = t.nbytes;
  return RG_OK;
}
int32_t rg_b200_gguf_llama_config(const rg_gguf *g, rg_llama_config *out) {
  if (!g || !out) return fail(RG_INVALID_ARGUMENT, "null argument");
  std::string err;
  int32_t rc = gguf_llama_config(g->g, out, &err);
  return rc ? fail(rc, err) : RG_OK;
}

// ------------------------------------------------------------------------------ plan
int32_t rg_b200_plan_create(const rg_llama_config *c, const rg_options *o, rg_plan **out) {
  if (!c || !out) return fail(RG_INVALID_ARGUMENT, "null argument");
  if (c->n_layers <= 0 || c->d_model <= 0 || c->n_heads <= 0 || c->n_kv_heads <= 0 || c->head_dim <= 0 || c->ffn_dim <= 0 ||
      c->vocab <= 0 || c->max_context <= 0 || c->n_heads % c->n_kv_heads || !(c->norm_eps >= 0.0f) || !(c->rope_theta > 0.0))
    return fail(RG_INVALID_ARGUMENT, "invalid model configuration");
  if (c->rope_dim < 0 || c->rope_dim > c->head_dim || (c->rope_dim & 1) || c->qk_norm < 0 || c->qk_norm > 2 ||
      (c->qk_norm == 2 && c->n_heads != c->n_kv_heads))
    return fail(RG_INVALID_ARGUMENT, "invalid rotary width or q/k normalisation kind");
  if (!attention_supported(c->n_heads, c->n_kv_heads, c->head_dim))
    return fail(RG_UNSUPPORTED_GEOMETRY, "head_dim must be 64 or 128 and query heads per kv head 1, 2, 4 or 8");
  auto p = std::make_unique<rg_plan>();
  p->cfg = *c;
  if (o) p->opt = *o;
  p->tp_world = p->opt.tp_world > 1 ? p->opt.tp_world : 1;
  p->tp_rank = p->tp_world > 1 ? p->opt.tp_rank : 0;
  if (p->tp_rank < 0 || p->tp_rank >= p->tp_world) return fail(RG_INVALID_ARGUMENT, "tensor-parallel rank out of range");
  if (p->tp_world > 1 && (c->n_heads % p->tp_world || c->n_kv_heads % p->tp_world || c->ffn_dim % p->tp_world))
    return fail(RG_UNSUPPORTED_GEOMETRY, "heads, kv heads and ffn width must divide by the tensor-parallel world size");
  if (p->opt.max_batch > BMAX) return fail(RG_UNSUPPORTED_GEOMETRY, "max_batch above 32 is not supported");
  if (p->tp_world > 1 && ((c->rope_dim && c->rope_dim != c->head_dim) || c->qk_norm || c->qkv_bias))
    return fail(RG_UNSUPPORTED_GEOMETRY, "partial rotary, q/k normalisation and projection biases run on one GPU only");
  RG_CUDA(cudaSetDevice(p->opt.device));
  int sms = 0;
  RG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p->opt.device));
  p->sm_count = sms;
  RG_CUDA(cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking));
  RG_CUDA(x_malloc(reinterpret_cast<void **>(&p->d_status), sizeof(int)));
  RG_CUDA(cudaMemsetAsync(p->d_status, 0, sizeof(int), p->stream));
  p->layers.resize((size_t)c->n_layers);
  *out = p.release();
  return RG_OK;
}

int32_t rg_b200_tp_shard(const char *name, int32_t type, uint64_t rows, uint64_t cols, int32_t rank, int32_t world, uint64_t *row0,
                         uint64_t *n_rows, uint64_t *col0, uint64_t *n_cols) {
  if (!name || !row0 || !n_rows || !col0 || !n_cols) return fail(RG_INVALID_ARGUMENT, "null argument");
  if (world < 1 || rank < 0 || rank >= world) return fail(RG_INVALID_ARGUMENT, "rank out of range");
  if (!block_elements(type)) return fail(RG_UNSUPPORTED_TYPE, std::string(name) + ": ggml type " + std::to_string(type) + " is not supported");
  if (cols % (uint64_t)block_elements(type)) return fail(RG_SHAPE_MISMATCH, std::string(name) + ": columns are not a multiple of the block size");
  return shard_range(name, type, rows, cols, split_of(name), (uint64_t)world, (uint64_t)rank, row0, n_rows, col0, n_cols);
}

int32_t rg_b200_plan_add_tensor(rg_plan *p, const char *name, int32_t type, uint64_t rows, uint64_t cols, const uint8_t *bytes,
                                size_t nbytes) {
  if (!p || !name || !bytes) return fail(RG_INVALID_ARGUMENT, "null argument");
  if (p->consumed) return fail(RG_INVALID_ARGUMENT, "plan already prepared");
  Slot slot;
  uint64_t r0, lr, c0, lc;
  int32_t rc = check_tensor(p, name, type, rows, cols, &slot, &r0, &lr, &c0, &lc);
  if (rc) return rc;
  const uint64_t be = (uint64_t)block_elements(type), bb = (uint64_t)block_bytes(type);
  const uint64_t row_bytes = cols / be * bb;
  if (nbytes != rows * row_bytes) return fail(RG_SHAPE_MISMATCH, std::string(name) + ": byte length does not match its geometry");
  if (type == RG_TYPE_Q4_0 || type == RG_TYPE_Q8_0) {
    // a non-finite scale is rejected before any device work (src/gguf/quantization/data.rs:325-327)
    const uint64_t blocks = rows * cols / 32;
    for (uint64_t b = 0; b < blocks; ++b) {
      const uint8_t *blk = bytes + b * bb;
      if (((blk[1] >> 2) & 0x1f) == 0x1f) return fail(RG_NON_FINITE_SCALE, std::string(name) + ": block " + std::to_string(b));
    }
  }
  if (type == RG_TYPE_Q4_K || type == RG_TYPE_Q6_K) {
    const uint64_t blocks = rows * cols / 256;
    for (uint64_t b = 0; b < blocks; ++b) {
      const uint8_t *blk = bytes + b * bb;
      const bool bad = type == RG_TYPE_Q4_K ? (((blk[1] >> 2) & 0x1f) == 0x1f || ((blk[3] >> 2) & 0x1f) == 0x1f)
                                            : (((blk[209] >> 2) & 0x1f) == 0x1f);
      if (bad) return fail(RG_NON_FINITE_SCALE, std::string(name) + ": block " + std::to_string(b));
    }
  }
  if (slot.ignored) return RG_OK;
  RG_CUDA(cudaSetDevice(p->opt.device));
  DevTensor t;
  t.rows = lr;
  t.cols = lc;
  if (slot.norm) {
    std::vector<float> v((size_t)cols);
    if (type == RG_TYPE_F32) {
      memcpy(v.data(), bytes, (size_t)cols * 4);
    } else {
      for (uint64_t i = 0; i < cols; ++i) {  // IEEE half -> float, exact (src/tensor/scalar.rs:110-135)
        const uint16_t h = (uint16_t)(bytes[2 * i] | (bytes[2 * i + 1] << 8));
        uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, mant = h & 0x3ffu, o;
        if (exp == 0) {
          if (!mant) o = sign;
          else {
            int e = -14;
            while (!(mant & 0x400u)) { mant <<= 1; --e; }
            o = sign | ((uint32_t)(e + 127) << 23) | ((mant & 0x3ffu) << 13);
          }
        } else if (exp == 31) o = sign | 0x7f800000u | (mant << 13);
        else o = sign | ((exp + 112u) << 23) | (mant << 13);
        memcpy(&v[(size_t)i], &o, 4);
      }
    }
    t.type = RG_TYPE_F32;
    t.nbytes = (size_t)cols * 4;
    RG_CUDA(x_malloc(reinterpret_cast<void **>(&t.d), t.nbytes));
    RG_CUDA(cudaMemcpy(t.d, v.data(), t.nbytes, cudaMemcpyHostToDevice));
  } else {
    const uint64_t local_row_bytes = lc / be * bb;
    t.type = type;
    t.nbytes = (size_t)(lr * local_row_bytes);
    RG_CUDA(x_malloc(reinterpret_cast<void **>(&t.d), t.nbytes));
    const uint8_t *src = bytes + r0 * row_bytes + c0 / be * bb;
    if (inject(g_faults.memcpy_after)) {
      cudaFree(t.d);
      return fail(RG_CUDA_ERROR, "injected upload failure");
    }
    cudaError_t e = cudaMemcpy2D(t.d, (size_t)local_row_bytes, src, (size_t)row_bytes, (size_t)local_row_bytes, (size_t)lr,
                                 cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      cudaFree(t.d);
      return fail(RG_CUDA_ERROR, std::string("upload of ") + name + ": " + cudaGetErrorString(e));
    }
  }
  p->weight_bytes += t.nbytes;
  *slot.t = t;
  return RG_OK;
}

int32_t rg_b200_plan_synth_tensor(rg_plan *p, const char *name, int32_t type, uint64_t rows, uint64_t cols, uint64_t seed,
                                  float std) {
  if (!p || !name) return fail(RG_INVALID_ARGUMENT, "null argument");
  if (p->consumed) return fail(RG_INVALID_ARGUMENT, "plan already prepared");
  Slot slot;
  uint64_t r0, lr, c0, lc;
  int32_t rc = check_tensor(p, name, type, rows, cols, &slot, &r0, &lr, &c0, &lc);
  if (rc) return rc;
  if (slot.ignored) return RG_OK;
  RG_CUDA(cudaSetDevice(p->opt.device));
  LaunchCfg cfg;
  cfg.stream = p->stream;
  DevTensor t;
  t.rows = lr;
  t.cols = lc;
  if (slot.norm) {
    t.type = RG_TYPE_F32;
    t.nbytes = (size_t)cols * 4;
    RG_CUDA(x_malloc(reinterpret_cast<void **>(&t.d), t.nbytes));
    RG_CUDA(launch_fill_f32(reinterpret_cast<float *>(t.d), (size_t)cols, 1.0f, cfg));
  } else {
    t.type = type;
    t.nbytes = (size_t)(lr * (lc / (uint64_t)block_elements(type)) * (uint64_t)block_bytes(type));
    RG_CUDA(x_malloc(reinterpret_cast<void **>(&t.d), t.nbytes));
    RG_CUDA(launch_synth(type, t.d, seed, std, cols, r0, lr, c0, lc, cfg));
  }
  RG_CUDA(cudaStreamSynchronize(p->stream));
  p->weight_bytes += t.nbytes;
  *slot.t = t;
  return RG_OK;
}

int32_t rg_b200_plan_from_gguf(const rg_gguf *g, const rg_options *o, rg_plan **out) {
  if (!g || !out) return fail(RG_INVALID_ARGUMENT, "null argument");
  rg_llama_config cfg;
  int32_t rc = rg_b200_gguf_llama_config(g, &cfg);
  if (rc) return rc;
  rg_plan *p = nullptr;
  if ((rc = rg_b200_plan_create(&cfg, o, &p))) return rc;
  for (const GgufTensorInfo &t : g->g.tensors) {
    uint64_t rows = 1, cols = 0;
    if (t.shape.size() == 1) cols = t.shape[0];
    else if (t.shape.size() == 2) { rows = t.shape[0]; cols = t.shape[1]; }
    else {
      delete p;
      return fail(RG_SHAPE_MISMATCH, t.name + ": rank " + std::to_string(t.shape.size()));
    }
    if ((rc = rg_b200_plan_add_tensor(p, t.name.c_str(), t.ggml_type, rows, cols, g->g.bytes + t.offset, t.nbytes))) {
      delete p;
      return rc;
    }
  }
  *out = p;
  return RG_OK;
}

static const DevTensor *plan_tensor(const rg_plan *p, const char *name) {
  Slot s;
  if (!find_slot(const_cast<rg_plan *>(p), name, &s) || !s.t || s.t->type < 0) return nullptr;
  return s.t;
}
int32_t rg_b200_plan_tensor_nbytes(const rg_plan *p, const char *name, size_t *nbytes) {
  if (!p || !name || !nbytes) return fail(RG_INVALID_ARGUMENT, "null argument");
  const DevTensor *t = plan_tensor(p, name);
  if (!t) return fail(RG_MISSING_TENSOR, std::string("tensor not bound: ") + name);
  *nbytes = t->nbytes;
  return RG_OK;
}
int32_t rg_b200_plan_read_tensor(const rg_plan *p, const char *name, uint8_t *out, size_t nbytes) {
  if (!p || !name || !out) return fail(RG_INVALID_ARGUMENT, "null argument");
  if (p->consumed) return fail(RG_INVALID_ARGUMENT, "plan already prepared");
  const DevTensor *t = plan_tensor(p, name);
  if (!t) return fail(RG_MISSING_TENSOR, std::string("tensor not bound: ") + name);
  if (nbytes != t->nbytes) return fail(RG_INVALID_ARGUMENT, "buffer size differs from the tensor's byte length");
  RG_CUDA(cudaSetDevice(p->opt.device));
  RG_CUDA(cudaMemcpy(out, t->d, nbytes, cudaMemcpyDeviceToHost));
  return RG_OK;
}
void rg_b200_plan_destroy(rg_plan *p) { delete p; }

// ------------------------------------------------------------------------------ session
int32_t rg_b200_session_prepare(rg_plan *p, rg_session **out) {
  if (!p || !out) return fail(RG_INVALID_ARGUMENT, "null argument");
  if (p->consumed) return fail(RG_INVALID_ARGUMENT, "plan already prepared");
  const rg_llama_config &c = p->cfg;
  // exact inventory (src/models/transformer/model.rs:384-455)
  if (p->token_embd.type < 0) return fail(RG_MISSING_TENSOR, "token_embd.weight");
  if (p->output_norm.type < 0) return fail(RG_MISSING_TENSOR, "output_norm.weight");
  for (int l = 0; l < c.n_layers; ++l) {
    LayerW &L = p->layers[(size_t)l];
    const char *names[] = {"attn_norm", "attn_q", "attn_k", "attn_v", "attn_output", "ffn_norm", "ffn_gate", "ffn_up", "ffn_down"};
    DevTensor *ts[] = {&L.attn_norm, &L.q, &L.k, &L.v, &L.o, &L.ffn_norm, &L.gate, &L.up, &L.down};
    for (int i = 0; i < 9; ++i)
      if (ts[i]->type < 0) return fail(RG_MISSING_TENSOR, "blk." + std::to_string(l) + "." + names[i] + ".weight");
  }
  for (int l = 0; l < c.n_layers; ++l) {
    LayerW &L = p->layers[(size_t)l];
    const std::string pre = "blk." + std::to_string(l) + ".";
    if (c.qk_norm && L.q_norm.type < 0) return fail(RG_MISSING_TENSOR, pre + "attn_q_norm.weight");
    if (c.qk_norm && L.k_norm.type < 0) return fail(RG_MISSING_TENSOR, pre + "attn_k_norm.weight");
    if (c.qkv_bias && L.q_bias.type < 0) return fail(RG_MISSING_TENSOR, pre + "attn_q.bias");
    if (c.qkv_bias && L.k_bias.type < 0) return fail(RG_MISSING_TENSOR, pre + "attn_k.bias");
    if (c.qkv_bias && L.v_bias.type < 0) return fail(RG_MISSING_TENSOR, pre + "attn_v.bias");
  }
  const bool tied = p->output.type < 0;
  RG_CUDA(cudaSetDevice(p->opt.device));
  auto s = std::make_unique<rg_session>();
  s->cfg = c;
  s->opt = p->opt;
  s->tp_rank = p->tp_rank;
  s->tp_world = p->tp_world;
  s->heads_l = c.n_heads / s->tp_world;
  s->kv_l = c.n_kv_heads / s->tp_world;
  s->ffn_l = c.ffn_dim / s->tp_world;
  s->vocab_l = (!tied && s->tp_world > 1) ? c.vocab / s->tp_world : c.vocab;
  s->max_batch = p->opt.max_batch > 0 ? p->opt.max_batch : 1;
  s->ctx = p->opt.max_context > 0 ? p->opt.max_context : c.max_context;
  if (s->ctx > c.max_context) return fail(RG_INVALID_ARGUMENT, "max_context above the model's context length");
  s->kv_f32 = p->opt.kv_f32 != 0;
  s->rope_dim = c.rope_dim ? c.rope_dim : c.head_dim;
  s->variant = s->rope_dim != c.head_dim || c.qk_norm || c.qkv_bias;
  s->use_graph = !p->opt.disable_graph && !env_flag("RG_B200_DISABLE_GRAPH");
  s->use_pdl = !p->opt.disable_pdl && !env_flag("RG_B200_DISABLE_PDL");
  s->sm_count = p->sm_count;
  RG_CUDA(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
  RG_CUDA(cudaEventCreate(&s->ev0));
  RG_CUDA(cudaEventCreate(&s->ev1));
  if (s->tp_world > 1) {
    std::string err;
    int32_t rc = comm_init(&s->comm, p->opt.nccl_id, s->tp_rank, s->tp_world, &err);
    if (rc) return fail(rc, err);
  }
  const int d = c.d_model, hd = c.head_dim;
  const int qw = s->heads_l * hd, kw = s->kv_l * hd;
  int32_t rc;
#define RG_TRY(e)            \
  if ((rc = (e))) return rc;
  RG_TRY(dalloc(s.get(), &s->d_ctrl, 1));
  {
    // status word and selected ids side by side: a host-driven step reads both back with one copy
    int32_t *res = nullptr;
    RG_TRY(dalloc(s.get(), &res, 4 + BMAX));
    s->d_status = reinterpret_cast<int *>(res);
    s->d_ids = res + 4;
  }
  s->history_cap = 8192;
  RG_TRY(dalloc(s.get(), &s->d_history, (size_t)s->history_cap * BMAX));

  // per-column buffers are sized for the widest forward (a 1024-token prefill chunk)
  RG_TRY(dalloc(s.get(), &s->x, (size_t)WMAX * d));
  RG_TRY(dalloc(s.get(), &s->xn_f32, (size_t)MAXC * d));
  RG_TRY(dalloc(s.get(), &s->qkv, (size_t)WMAX * (qw + 2 * kw)));
  RG_TRY(dalloc(s.get(), &s->q_rot, (size_t)WMAX * qw));
  RG_TRY(dalloc(s.get(), &s->attn_scratch, attn_scratch_floats(SCOLS, s->heads_l, hd, s->ctx)));
  RG_TRY(dalloc(s.get(), &s->attn_f32, (size_t)WMAX * qw));
  if (fused_attention_supported(s->heads_l, s->kv_l, hd) && !env_flag("RG_B200_SPLIT_ATTENTION")) {
    s->attn_max_splits = fused_attn_max_splits(s->ctx, hd, s->kv_f32, s->sm_count, s->kv_l);
    if (s->attn_max_splits <= fused_attn_split_cap() &&
        (size_t)BMAX * s->heads_l * s->attn_max_splits * (hd + 2) <= attn_scratch_floats(SCOLS, s->heads_l, hd, s->ctx)) {
      RG_TRY(dalloc(s.get(), &s->attn_counters, (size_t)BMAX * s->kv_l));
      RG_CUDA(cudaMemsetAsync(s->attn_counters, 0, sizeof(unsigned) * BMAX * (size_t)s->kv_l, s->stream));
    }
  }
  RG_TRY(dalloc(s.get(), &s->partial, (size_t)WMAX * d));
  s->tp_part[0] = s->tp_part[1] = s->partial;
  // one allocation: two [WMAX][ffn] halves, or (stacked gate|up GEMM) [tokens][2 ffn] rows
  RG_TRY(dalloc(s.get(), &s->gate_f32, (size_t)2 * WMAX * s->ffn_l));
  s->up_f32 = s->gate_f32 + (size_t)WMAX * s->ffn_l;
  RG_TRY(dalloc(s.get(), &s->h_f32, (size_t)MAXC * s->ffn_l));
  RG_TRY(dalloc(s.get(), &s->logits, (size_t)BMAX * c.vocab));
  RG_TRY(dalloc(s.get(), &s->logits_l, (size_t)BMAX * s->vocab_l));
  uint8_t *raw;
  s->xb_ld = std::max(d, std::max(qw, s->ffn_l));
  RG_TRY(dalloc(s.get(), &raw, (size_t)2 * WMAX * s->xb_ld * 2));
  // splits <= 2 * SMs / tiles and rows <= tiles * rows_per_cta (256 with two row tiles per CTA)
  RG_TRY(dalloc(s.get(), &s->split_scratch, (size_t)BMAX * 2 * s->sm_count * 256));
  RG_TRY(dalloc(s.get(), &s->ssq_a, (size_t)256 * 16));
  RG_TRY(dalloc(s.get(), &s->ssq_b, (size_t)256 * 16));
  RG_CUDA(cudaMemsetAsync(s->ssq_a, 0, sizeof(float) * 256 * 16, s->stream));
  RG_CUDA(cudaMemsetAsync(s->ssq_b, 0, sizeof(float) * 256 * 16, s->stream));
  RG_TRY(dalloc(s.get(), &s->gemv_counters, (size_t)QGEMV_ROWS_MAX_TILES));
  RG_CUDA(cudaMemsetAsync(s->gemv_counters, 0, sizeof(unsigned) * QGEMV_ROWS_MAX_TILES, s->stream));
  s->gemm_mode = (s->opt.gemm_operand_mode >= 1 && s->opt.gemm_operand_mode <= 3) ? s->opt.gemm_operand_mode - 1 : QGEMM_F16X3;
  s->xb = raw;
  RG_TRY(dalloc(s.get(), &raw, xpack_bytes(d, MAXC)));
  s->xn_pack = raw;
  RG_TRY(dalloc(s.get(), &raw, xpack_bytes(qw, MAXC)));
  s->attn_pack = raw;
  RG_TRY(dalloc(s.get(), &raw, xpack_bytes(s->ffn_l, MAXC)));
  s->h_pack = raw;
  RG_TRY(dalloc(s.get(), &raw, xpack_bytes(d, MAXC)));
  s->head_pack = raw;
  RG_TRY(dalloc(s.get(), &s->xq_x, qgemv_i8_xq_bytes(d)));
  RG_TRY(dalloc(s.get(), &s->xq_attn, qgemv_i8_xq_bytes(qw)));
  if (env_flag("RG_B200_TRACE")) {
    s->trace_cap = 5 * c.n_layers + 2;
    RG_TRY(dalloc(s.get(), &s->d_trace, (size_t)16 * (size_t)s->trace_cap));
    RG_CUDA(cudaMemsetAsync(s->d_trace, 0, sizeof(unsigned long long) * 16 * (size_t)s->trace_cap, s->stream));
  }
  if (s->ffn_l % 32 == 0) {
    RG_TRY(dalloc(s.get(), &s->xq_h, qgemv_i8_xq_bytes(s->ffn_l)));
    // the gate/up launch gives each CTA rows_per_cta rows of the SwiGLU output: a 32-row block that
    // holds a CTA boundary is packed by the down projection instead
    const int rpc = qgemv_i8_rows_per_cta(s->ffn_l, s->sm_count, false);
    std::vector<int32_t> fix;
    for (int b = rpc; b < s->ffn_l; b += rpc)
      if (b % 32) fix.push_back(b / 32);
    s->xq_h_nfix = (int)fix.size();
    RG_TRY(dalloc(s.get(), &s->xq_h_fix, fix.size() + 1));
    if (!fix.empty()) RG_CUDA(cudaMemcpy(s->xq_h_fix, fix.data(), fix.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
  }
  if (s->tp_world > 1 && !p->opt.disable_fused_allreduce && !env_flag("RG_B200_DISABLE_FUSED_ALLREDUCE")) RG_TRY(tp_fused_setup(s.get()));
  // RoPE tables in f64 on the host, cast to f32 (src/models/transformer/layer.rs:541-556)
  {
    const int half = s->rope_dim / 2;  // angle(p, i) = p / theta^(2i / rope_dim)
    std::vector<float> cs((size_t)s->ctx * half), sn((size_t)s->ctx * half);
    for (int i = 0; i < half; ++i) {
      const double freq = 1.0 / pow(c.rope_theta, (double)(2 * i) / (double)s->rope_dim);
      for (int pos = 0; pos < s->ctx; ++pos) {
        const double ang = (double)pos * freq;
        cs[(size_t)pos * half + i] = (float)cos(ang);
        sn[(size_t)pos * half + i] = (float)sin(ang);
      }
    }
    RG_TRY(dalloc(s.get(), &s->cos_t, cs.size()));
    RG_TRY(dalloc(s.get(), &s->sin_t, sn.size()));
    RG_CUDA(cudaMemcpy(s->cos_t, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
    RG_CUDA(cudaMemcpy(s->sin_t, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice));
  }
  const size_t kv_elems = (size_t)s->max_batch * s->kv_l * s->ctx * hd;
  const size_t kv_item = s->kv_f32 ? 4 : 2;
  for (int l = 0; l < c.n_layers; ++l) {
    uint8_t *k, *v;
    RG_TRY(dalloc(s.get(), &k, kv_elems * kv_item));
    RG_TRY(dalloc(s.get(), &v, kv_elems * kv_item));
    RG_CUDA(cudaMemsetAsync(k, 0, kv_elems * kv_item, s->stream));
    RG_CUDA(cudaMemsetAsync(v, 0, kv_elems * kv_item, s->stream));
    s->k_cache.push_back(k);
    s->v_cache.push_back(v);
    s->kv_bytes += 2 * kv_elems * kv_item;
  }
  RG_CUDA(cudaMemsetAsync(s->d_status, 0, sizeof(int), s->stream));
  RG_CUDA(cudaMemsetAsync(s->d_ctrl, 0, sizeof(Ctrl), s->stream));
  RG_CUDA(cudaMallocHost(reinterpret_cast<void **>(&s->h_ctrl), sizeof(Ctrl)));
  RG_CUDA(cudaMallocHost(reinterpret_cast<void **>(&s->h_result), sizeof(int32_t) * (4 + (size_t)s->history_cap * BMAX)));
  s->h_status = reinterpret_cast<int *>(s->h_result);  // same head as the device block: [status, pad x 3, ids ...]
  s->h_ids = s->h_result + 4;
  RG_CUDA(cudaMallocHost(reinterpret_cast<void **>(&s->h_logits), sizeof(float) * (size_t)BMAX * c.vocab));
  memset(s->h_ctrl, 0, sizeof(Ctrl));
  RG_CUDA(cudaStreamSynchronize(s->stream));
#undef RG_TRY
  // take ownership of the weights
  s->layers = p->layers;
  {
    bool ok = s->tp_world == 1 && s->cfg.d_model % 256 == 0;
    for (const LayerW &W : s->layers)
      ok = ok && W.q.packed() && W.k.packed() && W.v.packed() && W.o.packed() && W.gate.packed() && W.up.packed() &&
           W.down.packed() && W.gate.type == W.up.type;
    s->packed_layers = ok;
    s->defer_norm_ok = ok && s->sm_count <= 256 && !qgemv_rows_enabled() && !env_flag("RG_B200_NO_DEFERRED_NORM");
  }
  s->token_embd = p->token_embd;
  s->output_norm = p->output_norm;
  s->output = p->output;
  s->head = tied ? &s->token_embd : &s->output;
  s->weight_bytes = p->weight_bytes;
  auto own = [&](DevTensor &t) {
    if (t.d) s->owned.push_back(t.d);
  };
  own(s->token_embd);
  own(s->output_norm);
  own(s->output);
  // Tensors that one tensor-core GEMM can take together are copied into one allocation (device to
  // device, once): same block type, same K, every part a whole number of 256-row tiles.
  auto stack = [&](std::initializer_list<DevTensor *> parts) -> bool {
    const DevTensor *first = *parts.begin();
    size_t total = 0;
    for (const DevTensor *t : parts) {
      if (!t->packed() || t->type != first->type || t->cols != first->cols || t->rows % 256) return false;
      total += t->nbytes;
    }
    uint8_t *block = nullptr;
    if (x_malloc(reinterpret_cast<void **>(&block), total) != cudaSuccess) {
      cudaGetLastError();
      return false;  // not enough memory for the second copy during the move: the tensors stay where they are
    }
    size_t off = 0;
    for (DevTensor *t : parts) {
      if (cudaMemcpy(block + off, t->d, t->nbytes, cudaMemcpyDeviceToDevice) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(block);
        return false;
      }
      off += t->nbytes;
    }
    off = 0;
    for (DevTensor *t : parts) {
      cudaFree(t->d);
      t->d = block + off;
      off += t->nbytes;
    }
    s->owned.push_back(block);
    return true;
  };
  const bool stacking = wide_path_ok(s.get()) && !env_flag("RG_B200_NO_STACKED_GEMM");
  for (auto &L : s->layers) {
    if (stacking) {
      L.qkv_stacked = stack({&L.q, &L.k, &L.v});
      L.gu_stacked = stack({&L.gate, &L.up});
    }
    for (DevTensor *t : {&L.attn_norm, &L.o, &L.ffn_norm, &L.down, &L.q_norm, &L.k_norm, &L.q_bias, &L.k_bias, &L.v_bias}) own(*t);
    if (!L.qkv_stacked)
      for (DevTensor *t : {&L.q, &L.k, &L.v}) own(*t);
    if (!L.gu_stacked)
      for (DevTensor *t : {&L.gate, &L.up}) own(*t);
  }
  p->consumed = true;
  s->position.assign((size_t)s->max_batch, 0);
  s->report.weight_bytes = s->weight_bytes;
  s->report.kv_bytes = s->kv_bytes;
  *out = s.release();
  return RG_OK;
}

void rg_b200_session_destroy(rg_session *s) {
  if (!s) return;
  cudaSetDevice(s->opt.device);
  cudaStreamSynchronize(s->stream);
  delete s;
}

int32_t rg_b200_position(const rg_session *s, int32_t row) {
  if (!s || row < 0 || row >= s->max_batch) return -1;
  return s->position[(size_t)row];
}
int32_t rg_b200_max_context(const rg_session *s) { return s ? s->ctx : -1; }
int32_t rg_b200_vocab_size(const rg_session *s) { return s ? s->cfg.vocab : -1; }
int32_t rg_b200_is_full(const rg_session *s) {
  if (!s) return -1;
  for (int32_t p : s->position)
    if (p >= s->ctx) return 1;
  return 0;
}
// Rewinds every row to position 0.  The cache is not cleared: stale rows lie beyond the causal
// horizon and each row is rewritten before it is read (metal_generation.rs:847-859).
int32_t rg_b200_reset_sequence(rg_session *s) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  std::fill(s->position.begin(), s->position.end(), 0);
  return RG_OK;
}

// Uploads `rows` rows of uniforms and arms Gumbel-max selection for the next step(s); null disarms.
static int32_t arm_sampling(rg_session *s, float temperature, const float *uniforms, int rows) {
  s->sample_uniforms = nullptr;
  if (!uniforms) return RG_OK;
  if (!s->d_uniforms) {
    int32_t rc = dalloc(s, &s->d_uniforms, (size_t)BMAX * (size_t)s->cfg.vocab);
    if (rc) return rc;
  }
  const size_t bytes = sizeof(float) * (size_t)rows * (size_t)s->cfg.vocab;
  RG_CUDA(x_memcpy_async(s->d_uniforms, uniforms, bytes, cudaMemcpyHostToDevice, s->stream));
  s->report.h2d_calls++;
  s->report.h2d_bytes += bytes;
  s->sample_uniforms = s->d_uniforms;
  s->sample_temperature = temperature;
  return RG_OK;
}

static int32_t prefill_impl(rg_session *s, int32_t row, const int32_t *ids, size_t n, float *last_logits, float temperature,
                            const float *uniforms) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  if (!ids) return fail(RG_INVALID_ARGUMENT, "null ids");
  if (row < 0 || row >= s->max_batch) return fail(RG_INVALID_ARGUMENT, "row out of range");
  if (n == 0) return fail(RG_EMPTY_PROMPT, "empty token list");
  const int base = s->position[(size_t)row];
  if ((size_t)base + n > (size_t)s->ctx) return fail(RG_CONTEXT_EXHAUSTED, "position " + std::to_string(base) + " + " + std::to_string(n) + " tokens exceeds " + std::to_string(s->ctx));
  for (size_t i = 0; i < n; ++i)
    if (ids[i] < 0 || ids[i] >= s->cfg.vocab) return fail(RG_TOKEN_OUT_OF_RANGE, "token " + std::to_string(ids[i]) + " at index " + std::to_string(i));
  RG_CUDA(cudaSetDevice(s->opt.device));
  if ((rc = arm_sampling(s, temperature, uniforms, 1))) return rc;
  struct Disarm {
    rg_session *s;
    ~Disarm() { s->sample_uniforms = nullptr; }
  } disarm{s};
  RG_CUDA(cudaEventRecord(s->ev0, s->stream));
  const bool wide_ok = wide_path_ok(s);  // prompt chunks of up to 1024 tokens on the tensor cores
  for (size_t done = 0; done < n;) {
    const int wide_chunk = prefill_attention_supported(s->heads_l, s->kv_l, s->cfg.head_dim) && !env_flag("RG_B200_SPLIT_ATTENTION") ? WMAX : SCOLS;
    const int chunk = (int)std::min<size_t>(wide_ok ? wide_chunk : DENSE_MAXC, n - done);
    const bool last = done + (size_t)chunk == n;
    Ctrl *h = s->h_ctrl;
    for (int i = 0; i < chunk; ++i) {
      h->tokens[i] = ids[done + (size_t)i];
      h->pos[i] = base + (int)done + i;
      h->seq[i] = row;
    }
    h->logit_cols[0] = chunk - 1;
    h->step = 0;
    if ((rc = upload_ctrl(s))) return rc;
    s->chunk_is_prompt = !env_flag("RG_B200_SPLIT_ATTENTION");
    s->prompt_segments.assign(1, {0, chunk, row, base + (int)done});
    rc = run_step(s, chunk, last ? 1 : 0, false, false);
    s->chunk_is_prompt = false;
    if (rc) return rc;
    // the pinned control block is reused by the next chunk: wait for the upload to be consumed
    if (!last) RG_CUDA(x_sync(s->stream));
    done += (size_t)chunk;
  }
  RG_CUDA(cudaEventRecord(s->ev1, s->stream));
  if ((rc = finish_step(s, 1, last_logits, last_logits ? 1 : 0))) return rc;
  cudaEventElapsedTime(&s->report.last_prefill_ms, s->ev0, s->ev1);
  s->position[(size_t)row] = base + (int)n;  // commit only after the whole call succeeded
  return RG_OK;
}

int32_t rg_b200_prefill(rg_session *s, int32_t row, const int32_t *ids, size_t n, float *last_logits) {
  return prefill_impl(s, row, ids, n, last_logits, 1.0f, nullptr);
}

// Several prompts in one pass (the batch prefill of batch.rs:177-325, batch_generation.rs:104-189,
// without its right padding: the chunk simply holds one run of columns per prompt).  Chunks of up
// to 1024 columns are cut from the prompts laid end to end, so short prompts share every weight
// tile; attention runs per prompt, and the last column of each prompt yields its logits.
int32_t rg_b200_prefill_rows(rg_session *s, const int32_t *rows, const int32_t *ids, const size_t *lens, int32_t n_rows,
                             float *last_logits, int32_t *greedy) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  if (!rows || !ids || !lens) return fail(RG_INVALID_ARGUMENT, "null argument");
  if (n_rows < 1 || n_rows > s->max_batch) return fail(RG_INVALID_ARGUMENT, "row count out of range");
  std::vector<char> seen((size_t)s->max_batch, 0);
  size_t total = 0;
  for (int r = 0; r < n_rows; ++r) {
    if (rows[r] < 0 || rows[r] >= s->max_batch) return fail(RG_INVALID_ARGUMENT, "row out of range");
    if (seen[(size_t)rows[r]]) return fail(RG_INVALID_ARGUMENT, "row " + std::to_string(rows[r]) + " listed twice");
    seen[(size_t)rows[r]] = 1;
    if (lens[r] == 0) return fail(RG_EMPTY_PROMPT, "empty token list for row " + std::to_string(rows[r]));
    const int base = s->position[(size_t)rows[r]];
    if ((size_t)base + lens[r] > (size_t)s->ctx)
      return fail(RG_CONTEXT_EXHAUSTED, "row " + std::to_string(rows[r]) + ": position " + std::to_string(base) + " + " +
                                            std::to_string(lens[r]) + " tokens exceeds " + std::to_string(s->ctx));
    total += lens[r];
  }
  for (size_t i = 0; i < total; ++i)
    if (ids[i] < 0 || ids[i] >= s->cfg.vocab) return fail(RG_TOKEN_OUT_OF_RANGE, "token " + std::to_string(ids[i]) + " at index " + std::to_string(i));
  const size_t vocab = (size_t)s->cfg.vocab;
  const bool shared = wide_path_ok(s) && !env_flag("RG_B200_SPLIT_ATTENTION");
  if (!shared) {
    // models that do not run on the tensor-core path: one prompt after the other, all or nothing
    const std::vector<int32_t> before = s->position;
    size_t off = 0;
    for (int r = 0; r < n_rows; ++r) {
      rc = prefill_impl(s, rows[r], ids + off, lens[r], last_logits ? last_logits + (size_t)r * vocab : nullptr, 1.0f, nullptr);
      if (!rc && greedy) greedy[r] = s->h_ids[0];
      if (rc) {
        s->position = before;
        return rc;
      }
      off += lens[r];
    }
    return RG_OK;
  }
  RG_CUDA(cudaSetDevice(s->opt.device));
  s->sample_uniforms = nullptr;
  RG_CUDA(cudaEventRecord(s->ev0, s->stream));
  const int cap = prefill_attention_supported(s->heads_l, s->kv_l, s->cfg.head_dim) ? WMAX : SCOLS;
  int r = 0;             // prompt the next column comes from
  size_t taken = 0;      // tokens of prompt r already placed
  size_t id_off = 0;     // index of prompt r's first token in ids
  int first_done = 0;    // prompts finished before the current chunk
  while (r < n_rows) {
    Ctrl *h = s->h_ctrl;
    s->prompt_segments.clear();
    int cols = 0, n_logit = 0;
    while (r < n_rows && cols < cap && n_logit < BMAX) {
      const int base = s->position[(size_t)rows[r]];
      const int take = (int)std::min<size_t>((size_t)(cap - cols), lens[r] - taken);
      for (int i = 0; i < take; ++i) {
        h->tokens[cols + i] = ids[id_off + taken + (size_t)i];
        h->pos[cols + i] = base + (int)taken + i;
        h->seq[cols + i] = rows[r];
      }
      s->prompt_segments.push_back({cols, take, rows[r], base + (int)taken});
      cols += take;
      taken += (size_t)take;
      if (taken == lens[r]) {
        h->logit_cols[n_logit++] = cols - 1;
        id_off += lens[r];
        taken = 0;
        ++r;
      }
    }
    h->step = 0;
    if ((rc = upload_ctrl(s))) return rc;
    s->chunk_is_prompt = true;
    rc = run_step(s, cols, n_logit, false, false);
    s->chunk_is_prompt = false;
    if (rc) return rc;
    // the pinned control block and the logits buffer are reused by the next chunk
    rc = finish_step(s, n_logit, last_logits ? last_logits + (size_t)first_done * vocab : nullptr, last_logits ? n_logit : 0);
    if (rc) return rc;
    if (greedy) memcpy(greedy + first_done, s->h_ids, sizeof(int32_t) * (size_t)n_logit);
    first_done += n_logit;
  }
  RG_CUDA(cudaEventRecord(s->ev1, s->stream));
  RG_CUDA(cudaEventSynchronize(s->ev1));
  cudaEventElapsedTime(&s->report.last_prefill_ms, s->ev0, s->ev1);
  for (int i = 0; i < n_rows; ++i) s->position[(size_t)rows[i]] += (int)lens[i];  // commit only after the whole call succeeded
  return RG_OK;
}

// More than 16 decode rows on packed weights: the 16-row kernels (GEMV with four column tiles, tensor-core decode
// attention) run two half-size steps faster than the 17..32-row path runs one (8B shape: 3.8 against 3.1 thousand
// tokens/s at 32 rows), so such a step is cut into equal chunks of at most 16 rows.  The rows are independent
// sequences, so the result is the same; positions move only when every chunk has succeeded.
static int decode_chunk_rows(const rg_session *s, int n) {
  if (n <= 16 || !s->packed_layers || env_flag("RG_B200_WIDE_DECODE_ONE_STEP")) return n;
  const int chunks = (n + 15) / 16;
  return (n + chunks - 1) / chunks;
}

static int32_t decode_impl(rg_session *s, const int32_t *tokens, int32_t batch, float *logits, int32_t *greedy, float temperature,
                           const float *uniforms) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  if (!tokens) return fail(RG_INVALID_ARGUMENT, "null tokens");
  if (batch < 1 || batch > s->max_batch) return fail(RG_INVALID_ARGUMENT, "batch out of range");
  for (int i = 0; i < batch; ++i) {
    if (tokens[i] < 0 || tokens[i] >= s->cfg.vocab) return fail(RG_TOKEN_OUT_OF_RANGE, "token " + std::to_string(tokens[i]) + " in row " + std::to_string(i));
    if (s->position[(size_t)i] >= s->ctx) return fail(RG_CONTEXT_EXHAUSTED, "row " + std::to_string(i) + " is at position " + std::to_string(s->position[(size_t)i]) + " of " + std::to_string(s->ctx));
  }
  RG_CUDA(cudaSetDevice(s->opt.device));
  struct Disarm {
    rg_session *s;
    ~Disarm() { s->sample_uniforms = nullptr; }
  } disarm{s};
  // (timed with the host clock: two event records and a query would cost a step several microseconds)
  const auto t0 = std::chrono::steady_clock::now();
  const int per = decode_chunk_rows(s, batch);
  const size_t vocab = (size_t)s->cfg.vocab;
  for (int off = 0; off < batch; off += per) {
    const int m = std::min(per, batch - off);
    Ctrl *h = s->h_ctrl;
    for (int i = 0; i < m; ++i) {
      h->tokens[i] = tokens[off + i];
      h->pos[i] = s->position[(size_t)(off + i)];
      h->seq[i] = off + i;
      h->logit_cols[i] = i;
    }
    h->step = 0;
    if ((rc = arm_sampling(s, temperature, uniforms ? uniforms + (size_t)off * vocab : nullptr, m))) return rc;
    if ((rc = upload_ctrl(s))) return rc;
    if ((rc = run_step(s, m, m, true, uniforms == nullptr))) return rc;  // the captured graph selects greedily
    rc = finish_step(s, m, logits ? logits + (size_t)off * vocab : nullptr, logits ? m : 0);
    if (rc && rc != RG_NON_FINITE_LOGITS) return rc;
    s->report.last_decode_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    if (rc) return rc;  // non-finite logits: position unchanged (metal_generation.rs:892-898)
    if (greedy) memcpy(greedy + off, s->h_ids, sizeof(int32_t) * (size_t)m);
  }
  for (int i = 0; i < batch; ++i) s->position[(size_t)i] += 1;
  return RG_OK;
}

int32_t rg_b200_decode(rg_session *s, const int32_t *tokens, int32_t batch, float *logits, int32_t *greedy) {
  return decode_impl(s, tokens, batch, logits, greedy, 1.0f, nullptr);
}

int32_t rg_b200_decode_sampled(rg_session *s, const int32_t *tokens, int32_t batch, float temperature, const float *uniforms,
                               float *logits, int32_t *ids) {
  if (!uniforms) return fail(RG_INVALID_ARGUMENT, "null uniforms");
  return decode_impl(s, tokens, batch, logits, ids, temperature, uniforms);
}

// ---- verbs of a continuous-batching step (serving/mod.rs:557-690 runs over these) --------------
// Uploads per-column temperatures and the uniform tape of a mixed step.  A column with a
// non-positive temperature is greedy; with no positive temperature at all nothing is armed.
static int32_t arm_mixed(rg_session *s, const float *temps, const float *uniforms, int n) {
  s->sample_uniforms = nullptr;
  s->sample_temps = nullptr;
  if (!temps) return RG_OK;
  bool any = false;
  for (int i = 0; i < n; ++i) {
    if (temps[i] > 0.0f && !std::isfinite(temps[i])) return fail(RG_INVALID_ARGUMENT, "temperature must be finite");
    any = any || temps[i] > 0.0f;
  }
  if (!any) return RG_OK;
  if (!uniforms) return fail(RG_INVALID_ARGUMENT, "a sampled column needs the uniform tape");
  int32_t rc = arm_sampling(s, 1.0f, uniforms, n);
  if (rc) return rc;
  if (!s->d_temps && (rc = dalloc(s, &s->d_temps, (size_t)BMAX))) return rc;
  RG_CUDA(x_memcpy_async(s->d_temps, temps, sizeof(float) * (size_t)n, cudaMemcpyHostToDevice, s->stream));
  s->report.h2d_calls++;
  s->report.h2d_bytes += sizeof(float) * (size_t)n;
  s->sample_temps = s->d_temps;
  return RG_OK;
}

int32_t rg_b200_reset_row(rg_session *s, int32_t row) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  if (row < 0 || row >= s->max_batch) return fail(RG_INVALID_ARGUMENT, "row out of range");
  s->position[(size_t)row] = 0;
  return RG_OK;
}

int32_t rg_b200_prefill_select(rg_session *s, int32_t row, const int32_t *ids, size_t n, float temperature, const float *uniforms,
                               float *last_logits, int32_t *selected) {
  const bool sampled = temperature > 0.0f && uniforms;
  const int32_t rc = prefill_impl(s, row, ids, n, last_logits, sampled ? temperature : 1.0f, sampled ? uniforms : nullptr);
  if (rc == RG_OK && selected) *selected = s->h_ids[0];
  return rc;
}

int32_t rg_b200_decode_rows(rg_session *s, const int32_t *rows, const int32_t *tokens, int32_t n, const float *temperatures,
                            const float *uniforms, float *logits, int32_t *ids) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  if (!rows || !tokens) return fail(RG_INVALID_ARGUMENT, "null rows or tokens");
  if (n < 1 || n > s->max_batch) return fail(RG_INVALID_ARGUMENT, "batch out of range");
  for (int i = 0; i < n; ++i) {
    if (rows[i] < 0 || rows[i] >= s->max_batch) return fail(RG_INVALID_ARGUMENT, "row out of range");
    for (int j = 0; j < i; ++j)
      if (rows[j] == rows[i]) return fail(RG_INVALID_ARGUMENT, "row " + std::to_string(rows[i]) + " appears twice in one step");
    if (tokens[i] < 0 || tokens[i] >= s->cfg.vocab) return fail(RG_TOKEN_OUT_OF_RANGE, "token " + std::to_string(tokens[i]) + " in column " + std::to_string(i));
    if (s->position[(size_t)rows[i]] >= s->ctx) return fail(RG_CONTEXT_EXHAUSTED, "row " + std::to_string(rows[i]) + " is full");
  }
  RG_CUDA(cudaSetDevice(s->opt.device));
  struct Disarm {
    rg_session *s;
    ~Disarm() { s->sample_uniforms = nullptr, s->sample_temps = nullptr; }
  } disarm{s};
  const auto t0 = std::chrono::steady_clock::now();
  const int per = decode_chunk_rows(s, n);
  const size_t vocab = (size_t)s->cfg.vocab;
  for (int off = 0; off < n; off += per) {
    const int m = std::min(per, n - off);
    Ctrl *h = s->h_ctrl;
    for (int i = 0; i < m; ++i) {
      h->tokens[i] = tokens[off + i];
      h->pos[i] = s->position[(size_t)rows[off + i]];
      h->seq[i] = rows[off + i];
      h->logit_cols[i] = i;
    }
    h->step = 0;
    if ((rc = arm_mixed(s, temperatures ? temperatures + off : nullptr, uniforms ? uniforms + (size_t)off * vocab : nullptr, m)))
      return rc;
    if ((rc = upload_ctrl(s))) return rc;
    if ((rc = run_step(s, m, m, true, s->sample_uniforms == nullptr))) return rc;
    rc = finish_step(s, m, logits ? logits + (size_t)off * vocab : nullptr, logits ? m : 0);
    if (rc && rc != RG_NON_FINITE_LOGITS) return rc;
    s->report.last_decode_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    if (rc) return rc;
    if (ids) memcpy(ids + off, s->h_ids, sizeof(int32_t) * (size_t)m);
  }
  for (int i = 0; i < n; ++i) s->position[(size_t)rows[i]] += 1;
  return RG_OK;
}

int32_t rg_b200_select(rg_session *s, const float *logits, int32_t n, const float *temperatures, const float *uniforms, int32_t *ids) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  if (!logits || !ids || n < 1 || n > s->max_batch) return fail(RG_INVALID_ARGUMENT, "bad selection arguments");
  RG_CUDA(cudaSetDevice(s->opt.device));
  const size_t bytes = sizeof(float) * (size_t)n * (size_t)s->cfg.vocab;
  RG_CUDA(x_memcpy_async(s->logits, logits, bytes, cudaMemcpyHostToDevice, s->stream));
  s->report.h2d_calls++;
  s->report.h2d_bytes += bytes;
  if ((rc = arm_mixed(s, temperatures, uniforms, n))) return rc;
  struct Disarm {
    rg_session *s;
    ~Disarm() { s->sample_uniforms = nullptr, s->sample_temps = nullptr; }
  } disarm{s};
  LaunchCfg am = lcfg(s);
  am.pdl = false;
  RG_LAUNCH(s, launch_select(s->logits, s->cfg.vocab, s->cfg.vocab, n, s->sample_uniforms, s->sample_temperature, s->d_ids, am,
                             s->sample_temps));
  if ((rc = finish_step(s, n, nullptr, 0))) return rc;
  memcpy(ids, s->h_ids, sizeof(int32_t) * (size_t)n);
  return RG_OK;
}

// An immutable copy of the first `length` cached positions of one row, all layers
// (LlamaNativePrefixSnapshot of serving/mod.rs:182-190): [layer][K, V][kv head][length][head_dim].
struct rg_kv_snapshot {
  int device = 0;
  int length = 0;
  size_t bytes = 0;
  size_t row_bytes = 0;  // length * head_dim * element size
  int n_layers = 0, kv_heads = 0;
  uint8_t *data = nullptr;
};

static size_t kv_esize(const rg_session *s) { return s->kv_f32 ? 4 : 2; }

int32_t rg_b200_kv_snapshot_create(rg_session *s, int32_t row, int32_t length, rg_kv_snapshot **out) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  if (!out || row < 0 || row >= s->max_batch || length < 1 || length > s->position[(size_t)row])
    return fail(RG_INVALID_ARGUMENT, "snapshot of positions the row does not hold");
  RG_CUDA(cudaSetDevice(s->opt.device));
  auto snap = std::make_unique<rg_kv_snapshot>();
  const size_t hd = (size_t)s->cfg.head_dim, es = kv_esize(s);
  snap->device = s->opt.device;
  snap->length = length;
  snap->n_layers = s->cfg.n_layers;
  snap->kv_heads = s->kv_l;
  snap->row_bytes = (size_t)length * hd * es;
  snap->bytes = 2 * (size_t)snap->n_layers * (size_t)snap->kv_heads * snap->row_bytes;
  void *p = nullptr;
  if (x_malloc(&p, snap->bytes) != cudaSuccess) return fail(RG_OUT_OF_MEMORY, "KV snapshot of " + std::to_string(snap->bytes) + " bytes");
  snap->data = static_cast<uint8_t *>(p);
  const size_t src_pitch = (size_t)s->ctx * hd * es, head_block = (size_t)snap->kv_heads * snap->row_bytes;
  for (int l = 0; l < snap->n_layers; ++l)
    for (int kv = 0; kv < 2; ++kv) {
      const uint8_t *src = static_cast<const uint8_t *>(kv ? s->v_cache[(size_t)l] : s->k_cache[(size_t)l]) +
                           (size_t)row * (size_t)snap->kv_heads * src_pitch;
      uint8_t *dst = snap->data + ((size_t)l * 2 + (size_t)kv) * head_block;
      cudaError_t e = cudaMemcpy2DAsync(dst, snap->row_bytes, src, src_pitch, snap->row_bytes, (size_t)snap->kv_heads,
                                        cudaMemcpyDeviceToDevice, s->stream);
      if (e != cudaSuccess) {
        cudaFree(snap->data);
        return fail(RG_CUDA_ERROR, std::string("snapshot copy: ") + cudaGetErrorString(e));
      }
    }
  cudaError_t e = x_sync(s->stream);
  if (e != cudaSuccess) {
    cudaFree(snap->data);
    s->poisoned = true;
    return fail(RG_POISONED, std::string("stream synchronize: ") + cudaGetErrorString(e));
  }
  *out = snap.release();
  return RG_OK;
}

int32_t rg_b200_kv_snapshot_length(const rg_kv_snapshot *k) { return k ? k->length : -1; }
size_t rg_b200_kv_snapshot_bytes(const rg_kv_snapshot *k) { return k ? k->bytes : 0; }

int32_t rg_b200_kv_snapshot_restore(rg_session *s, const rg_kv_snapshot *k, int32_t row) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  if (!k || row < 0 || row >= s->max_batch) return fail(RG_INVALID_ARGUMENT, "bad restore arguments");
  const size_t hd = (size_t)s->cfg.head_dim, es = kv_esize(s);
  if (k->device != s->opt.device || k->n_layers != s->cfg.n_layers || k->kv_heads != s->kv_l || k->length > s->ctx ||
      k->row_bytes != (size_t)k->length * hd * es)
    return fail(RG_SHAPE_MISMATCH, "snapshot was taken from a session of another shape");
  RG_CUDA(cudaSetDevice(s->opt.device));
  const size_t dst_pitch = (size_t)s->ctx * hd * es, head_block = (size_t)k->kv_heads * k->row_bytes;
  for (int l = 0; l < k->n_layers; ++l)
    for (int kv = 0; kv < 2; ++kv) {
      uint8_t *dst = static_cast<uint8_t *>(kv ? s->v_cache[(size_t)l] : s->k_cache[(size_t)l]) + (size_t)row * (size_t)k->kv_heads * dst_pitch;
      const uint8_t *src = k->data + ((size_t)l * 2 + (size_t)kv) * head_block;
      RG_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, src, k->row_bytes, k->row_bytes, (size_t)k->kv_heads, cudaMemcpyDeviceToDevice, s->stream));
    }
  cudaError_t e = x_sync(s->stream);
  if (e != cudaSuccess) {
    s->poisoned = true;
    return fail(RG_POISONED, std::string("stream synchronize: ") + cudaGetErrorString(e));
  }
  s->position[(size_t)row] = k->length;  // the row now holds exactly the snapshot's positions
  return RG_OK;
}

void rg_b200_kv_snapshot_free(rg_kv_snapshot *k) {
  if (!k) return;
  cudaSetDevice(k->device);
  cudaFree(k->data);
  delete k;
}

static int32_t generate_impl(rg_session *s, const int32_t *prompt, size_t n_prompt, size_t max_new, int32_t *out, size_t *n_out,
                             int32_t *stopped, bool sampled, float temperature, const float *uniforms) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  if (!n_out || !stopped || (!out && max_new)) return fail(RG_INVALID_ARGUMENT, "null output");
  *n_out = 0;
  *stopped = 0;
  if (!prompt || n_prompt == 0) return fail(RG_EMPTY_PROMPT, "empty prompt");
  if (s->position[0] != 0) return fail(RG_FRESH_SESSION_REQUIRED, "sequence 0 is at position " + std::to_string(s->position[0]));
  if (n_prompt + max_new > (size_t)s->ctx) return fail(RG_CONTEXT_EXHAUSTED, std::to_string(n_prompt + max_new) + " tokens requested of " + std::to_string(s->ctx));
  for (size_t i = 0; i < n_prompt; ++i)
    if (prompt[i] < 0 || prompt[i] >= s->cfg.vocab) return fail(RG_TOKEN_OUT_OF_RANGE, "token " + std::to_string(prompt[i]) + " at index " + std::to_string(i));
  if (max_new == 0) return RG_OK;
  if (sampled && !uniforms) return fail(RG_INVALID_ARGUMENT, "null uniforms");
  const size_t V = (size_t)s->cfg.vocab;  // the tape is row-major [step, vocabulary] (generation.rs:7-9)
  if ((rc = prefill_impl(s, 0, prompt, n_prompt, nullptr, temperature, sampled ? uniforms : nullptr))) return rc;
  int32_t token = s->h_ids[0];
  for (size_t step = 0; step < max_new; ++step) {
    out[(*n_out)++] = token;
    if (token == s->cfg.eos_id || token == s->cfg.eot_id) {
      *stopped = 1;
      break;
    }
    if (step + 1 < max_new) {
      int32_t next;
      if ((rc = decode_impl(s, &token, 1, nullptr, &next, temperature, sampled ? uniforms + (step + 1) * V : nullptr))) return rc;
      token = next;
    }
  }
  return RG_OK;
}

int32_t rg_b200_generate_greedy(rg_session *s, const int32_t *prompt, size_t n_prompt, size_t max_new, int32_t *out, size_t *n_out,
                                int32_t *stopped) {
  return generate_impl(s, prompt, n_prompt, max_new, out, n_out, stopped, false, 1.0f, nullptr);
}

int32_t rg_b200_generate_sampled(rg_session *s, const int32_t *prompt, size_t n_prompt, size_t max_new, float temperature,
                                 const float *uniforms, int32_t *out, size_t *n_out, int32_t *stopped) {
  return generate_impl(s, prompt, n_prompt, max_new, out, n_out, stopped, true, temperature, uniforms);
}

int32_t rg_b200_decode_loop(rg_session *s, const int32_t *first, int32_t batch, int32_t steps, int32_t *out, float *gpu_ms) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  if (!first || batch < 1 || batch > s->max_batch || steps < 1) return fail(RG_INVALID_ARGUMENT, "bad arguments");
  if (steps > s->history_cap) return fail(RG_INVALID_ARGUMENT, "steps above the history capacity of " + std::to_string(s->history_cap));
  for (int i = 0; i < batch; ++i) {
    if (first[i] < 0 || first[i] >= s->cfg.vocab) return fail(RG_TOKEN_OUT_OF_RANGE, "token in row " + std::to_string(i));
    if (s->position[(size_t)i] + steps > s->ctx) return fail(RG_CONTEXT_EXHAUSTED, "row " + std::to_string(i));
  }
  RG_CUDA(cudaSetDevice(s->opt.device));
  // rows are independent sequences: a batch beyond 16 rows runs its chunks one after the other, each for all steps
  const int per = decode_chunk_rows(s, batch);
  float total_ms = 0.0f;
  for (int off = 0; off < batch; off += per) {
    const int m = std::min(per, batch - off);
    Ctrl *h = s->h_ctrl;
    for (int i = 0; i < m; ++i) {
      h->tokens[i] = first[off + i];
      h->pos[i] = s->position[(size_t)(off + i)];
      h->seq[i] = off + i;
      h->logit_cols[i] = i;
    }
    h->step = 0;
    if ((rc = upload_ctrl(s))) return rc;
    if (s->use_graph) {
      cudaGraphExec_t exec;
      if ((rc = decode_graph(s, m, &exec))) return rc;  // capture outside the timed region
    }
    RG_CUDA(cudaEventRecord(s->ev0, s->stream));
    for (int i = 0; i < steps; ++i)
      if ((rc = run_step(s, m, m, true, true))) {
        s->poisoned = true;
        return rc;
      }
    RG_CUDA(cudaEventRecord(s->ev1, s->stream));
    const size_t hist_bytes = sizeof(int32_t) * (size_t)steps * (size_t)m;
    RG_CUDA(x_memcpy_async(s->h_ids, s->d_history, hist_bytes, cudaMemcpyDeviceToHost, s->stream));
    s->report.d2h_calls++;
    s->report.d2h_bytes += hist_bytes;
    rc = finish_step(s, 0, nullptr, 0);
    if (rc) {
      if (off > 0) s->poisoned = true;  // earlier chunks have moved on
      return rc;
    }
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, s->ev0, s->ev1);
    total_ms += ms;
    for (size_t i = 0; i < (size_t)steps * (size_t)m; ++i)
      if (s->h_ids[i] < 0) {
        s->poisoned = true;  // later steps consumed a sentinel token; the cache content is unproven
        return fail(RG_NON_FINITE_LOGITS, "non-finite logits at step " + std::to_string(i / (size_t)m));
      }
    if (out)
      for (int st = 0; st < steps; ++st)
        memcpy(out + (size_t)st * batch + off, s->h_ids + (size_t)st * m, sizeof(int32_t) * (size_t)m);
    for (int i = 0; i < m; ++i) s->position[(size_t)(off + i)] += steps;
  }
  if (gpu_ms) *gpu_ms = total_ms;
  s->report.last_decode_ms = total_ms / (float)steps;
  return RG_OK;
}

static int32_t decode_profile_impl(rg_session *s, const int32_t *first, int32_t batch, int32_t steps, float out_ms[4],
                                   uint64_t out_launches[4], bool serialized, float *site_ms = nullptr) {
  int32_t rc = check_live(s);
  if (rc) return rc;
  if (!first || (!out_ms && !site_ms) || batch < 1 || batch > s->max_batch || steps < 1) return fail(RG_INVALID_ARGUMENT, "bad arguments");
  for (int i = 0; i < batch; ++i) {
    if (first[i] < 0 || first[i] >= s->cfg.vocab) return fail(RG_TOKEN_OUT_OF_RANGE, "token in row " + std::to_string(i));
    if (s->position[(size_t)i] >= s->ctx) return fail(RG_CONTEXT_EXHAUSTED, "row " + std::to_string(i));
  }
  RG_CUDA(cudaSetDevice(s->opt.device));
  Ctrl *h = s->h_ctrl;
  for (int i = 0; i < batch; ++i) {
    h->tokens[i] = first[i];
    h->pos[i] = s->position[(size_t)i];
    h->seq[i] = i;
    h->logit_cols[i] = i;
  }
  h->step = 0;
  if ((rc = upload_ctrl(s))) return rc;
  const bool saved_pdl = s->use_pdl;
  if (serialized) s->use_pdl = false;  // serialized launches: every kernel runs alone
  s->launches_in_step = 0;
  rc = forward(s, batch, batch, false);  // loads every kernel before capture; nothing is committed
  // one selection of the step's launches, captured as a graph and replayed `steps` times between two events
  auto time_selection = [&](unsigned family_mask, unsigned site_mask, float *ms_out, uint64_t *launches_out) -> int32_t {
    cudaGraphExec_t exec = nullptr;
    s->family_mask = family_mask;
    s->gemv_site_mask = site_mask;
    s->launches_in_step = 0;
    int32_t r = RG_OK;
    cudaError_t e = cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
      r = forward(s, batch, batch, false);
      cudaGraph_t graph = nullptr;
      e = cudaStreamEndCapture(s->stream, &graph);
      if (e == cudaSuccess && !r) e = cudaGraphInstantiate(&exec, graph, 0);
      if (graph) cudaGraphDestroy(graph);
    }
    s->family_mask = 0xffffffffu;
    s->gemv_site_mask = 0xffffffffu;
    if (!r && e != cudaSuccess) r = fail(RG_CUDA_ERROR, std::string("profile graph: ") + cudaGetErrorString(e));
    if (r) {
      if (exec) cudaGraphExecDestroy(exec);
      return r;
    }
    if (launches_out) *launches_out = s->launches_in_step;
    e = cudaGraphLaunch(exec, s->stream);  // warm replay
    if (e == cudaSuccess) e = cudaEventRecord(s->ev0, s->stream);
    for (int it = 0; it < steps && e == cudaSuccess; ++it) e = cudaGraphLaunch(exec, s->stream);
    if (e == cudaSuccess) e = cudaEventRecord(s->ev1, s->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->stream);
    float ms = 0.0f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, s->ev0, s->ev1);
    cudaGraphExecDestroy(exec);
    if (e != cudaSuccess) {
      s->poisoned = true;
      return fail(RG_CUDA_ERROR, std::string("profile replay: ") + cudaGetErrorString(e));
    }
    *ms_out = ms / (float)steps;
    return RG_OK;
  };
  double total = 0.0;
  if (site_ms) {
    // the projections of the GEMV family one at a time: q+k+v, output, gate+up, down, head
    for (int site = SITE_QKV; site < SITE_END && !rc; ++site) rc = time_selection(1u << PROF_GEMV, 1u << site, &site_ms[site - 1], nullptr);
  } else {
    for (int fam = 0; fam < 3 && !rc; ++fam) {
      rc = time_selection(1u << fam, 0xffffffffu, &out_ms[fam], out_launches ? &out_launches[fam] : nullptr);
      if (!rc) total += out_ms[fam];
    }
  }
  s->use_pdl = saved_pdl;
  if (rc) return rc;
  if (!site_ms) {
    out_ms[3] = (float)total;
    if (out_launches) out_launches[3] = out_launches[0] + out_launches[1] + out_launches[2];
  }
  return finish_step(s, 0, nullptr, 0);
}

int32_t rg_b200_decode_profile(rg_session *s, const int32_t *first, int32_t batch, int32_t steps, float out_ms[4],
                               uint64_t out_launches[4]) {
  return decode_profile_impl(s, first, batch, steps, out_ms, out_launches, true);
}

int32_t rg_b200_decode_profile_in_step(rg_session *s, const int32_t *first, int32_t batch, int32_t steps, float out_ms[4],
                                       uint64_t out_launches[4]) {
  return decode_profile_impl(s, first, batch, steps, out_ms, out_launches, false);
}

int32_t rg_b200_decode_profile_projections(rg_session *s, const int32_t *first, int32_t batch, int32_t steps, float out_ms[5]) {
  return decode_profile_impl(s, first, batch, steps, nullptr, nullptr, false, out_ms);
}

// Development aid: copies the phase stamps of the last small-batch step (RG_B200_TRACE=1 at prepare)
// to `out` (16 u64 per launch); returns the launch count.
int32_t rg_b200_debug_read_trace(rg_session *s, unsigned long long *out, int32_t max_launches) {
  if (!s || !out || !s->d_trace) return 0;
  cudaSetDevice(s->opt.device);
  const int n = std::min(max_launches, s->trace_cap);
  cudaStreamSynchronize(s->stream);
  cudaMemcpy(out, s->d_trace, sizeof(unsigned long long) * 16 * (size_t)n, cudaMemcpyDeviceToHost);
  return n;
}

int32_t rg_b200_report(const rg_session *s, rg_report *out) {
  if (!s || !out) return fail(RG_INVALID_ARGUMENT, "null argument");
  *out = s->report;
  return RG_OK;
}
void *rg_b200_session_stream(const rg_session *s) { return s ? (void *)s->stream : nullptr; }

int32_t rg_b200_nccl_unique_id(uint8_t out[128]) {
  if (!out) return fail(RG_INVALID_ARGUMENT, "null argument");
  std::string err;
  int32_t rc = comm_unique_id(out, &err);
  return rc ? fail(rc, err) : RG_OK;
}

}  // extern "C"
