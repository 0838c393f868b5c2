/*
 * rg_b200 — C ABI of the B200-native GGUF-quantized Llama session.
 *
 * This is the boundary a rustgrad CUDA session target binds through FFI.  Every entry point
 * names the rustgrad interface it stands in for (paths relative to the rustgrad tree).  All
 * pointers are plain host pointers unless a parameter is documented as a device pointer; no
 * C++ or torch type crosses the boundary; every function returns an rg_status and never throws.
 *
 * Threading: a plan or session is driven by one host thread at a time (rustgrad sessions are
 * `&mut self`, src/models/transformer/metal_generation.rs:1052).  Distinct sessions may be used
 * from distinct threads.
 */
#ifndef RG_B200_H
#define RG_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Typed, fail-closed statuses.  They fold rustgrad's error enums for this path:
 * GgufErrorKind (src/gguf/mod.rs:70-134), LlamaModelError (src/models/transformer/model.rs:1073-1153),
 * LlamaMetalStepError (src/models/transformer/metal_step.rs:161-170) and CudaError (src/cuda.rs:478-511). */
typedef enum {
  RG_OK = 0,
  RG_INVALID_ARGUMENT = 1,
  RG_UNSUPPORTED_TYPE = 2,      /* ggml type outside {F32, F16, Q4_0, Q8_0}; packed norm tensor */
  RG_SHAPE_MISMATCH = 3,        /* tensor shape differs from the configuration's inventory */
  RG_NON_FINITE_SCALE = 4,      /* a packed block carries an inf/NaN scale */
  RG_TOKEN_OUT_OF_RANGE = 5,
  RG_CONTEXT_EXHAUSTED = 6,
  RG_NON_FINITE_LOGITS = 7,
  RG_FRESH_SESSION_REQUIRED = 8,
  RG_CUDA_ERROR = 9,
  RG_NCCL_ERROR = 10,
  RG_OUT_OF_MEMORY = 11,
  RG_TIMEOUT = 12,              /* a bounded device-side wait gave up */
  RG_POISONED = 13,             /* an earlier step could not be proven complete */
  RG_MALFORMED_GGUF = 14,
  RG_MISSING_TENSOR = 15,
  RG_UNEXPECTED_TENSOR = 16,
  RG_UNSUPPORTED_VARIANT = 17,  /* rope scaling, experts, MLA, LoRA, partial q/k-norm or bias families */
  RG_MISSING_METADATA = 18,
  RG_EMPTY_PROMPT = 19,
  RG_UNSUPPORTED_GEOMETRY = 20  /* a shape the sm_100a kernels do not cover (K % 256 != 0 for packed) */
} rg_status;

/* GGML tensor types on this path (src/gguf/tensor.rs:33-59). */
enum { RG_TYPE_F32 = 0, RG_TYPE_F16 = 1, RG_TYPE_Q4_0 = 2, RG_TYPE_Q8_0 = 8,
       /* 256-element super-blocks (blocks.rs:1164-1187,1219-1240): decoded bit-exactly; projections in these
        * types run a plain decode-and-multiply GEMV (correct, not yet tuned), one GPU only */
       RG_TYPE_Q4_K = 12, RG_TYPE_Q6_K = 14 };

/* Mirror of LlamaModelConfig (src/models/transformer/model.rs:109-121). */
typedef struct {
  int32_t n_layers;
  int32_t d_model;
  int32_t n_heads;
  int32_t n_kv_heads;
  int32_t head_dim;
  int32_t ffn_dim;
  int32_t vocab;
  int32_t max_context;
  float norm_eps;
  double rope_theta;
  int32_t eos_id; /* -1 = none */
  int32_t eot_id; /* -1 = none */
  /* Variants of the layer the reference's binder accepts (model.rs:160-175,253-282,
   * layer.rs:274-346,481-571); all zero for the plain Llama layer.  They run on one GPU. */
  int32_t rope_dim; /* rotary lanes per head (llama.rope.dimension_count), even, <= head_dim; 0 = head_dim.
                     * The query is de-interleaved over its last rope_dim lanes, the key over the whole
                     * head, and lanes [0, rope_dim) of both rotate (layer.rs:481-571). */
  int32_t qk_norm;  /* 0 none; 1 per head: blk.N.attn_{q,k}_norm.weight [head_dim];
                     * 2 per projection: weights [heads * head_dim], query and key widths equal */
  int32_t qkv_bias; /* 1: blk.N.attn_{q,k,v}.bias, added after the lane permutation */
} rg_llama_config;

/* Session options.  Zero-initialise, then set what differs.  (rustgrad has no config framework:
 * builders and plain structs such as MetalPlanOptions; src/session/target.rs:165-213.) */
typedef struct {
  int32_t device;        /* CUDA ordinal of this process's GPU */
  int32_t max_batch;     /* independent sequences decoded together; 0 -> 1 */
  int32_t max_context;   /* KV positions per sequence; 0 -> config.max_context */
  int32_t kv_f32;        /* 0: f16 KV cache; 1: f32 cache like the reference's (model.rs:879-922) */
  int32_t tp_rank;       /* tensor-parallel rank of this process */
  int32_t tp_world;      /* 0 or 1: single GPU */
  uint8_t nccl_id[128];  /* rg_b200_nccl_unique_id() of rank 0, identical on every rank */
  int32_t disable_graph; /* 1: launch decode kernels directly instead of replaying a CUDA graph */
  int32_t disable_pdl;   /* 1: no programmatic dependent launch between kernels */
  int32_t disable_fused_allreduce; /* 1: TP all-reduce through NCCL only */
  int32_t general_path_only; /* 1: never take the fused small-batch decode path nor the tensor-core
                              * path (every step runs the 3..8-column kernels; used by tests) */
  int32_t gemm_operand_mode; /* operands of the tensor-core path, as in rg_b200_qgemm offset by one:
                              * 0 = default = compensated half, 1 = bf16, 2 = half, 3 = compensated half */
  int32_t reserved[6];       /* must be zero */
} rg_options;

/* Per-run evidence in the vocabulary of MetalDeviceRunReport
 * (src/runtime/metal/session.rs:145-185) and BenchmarkMetrics (src/benchmark.rs:290-305). */
typedef struct {
  uint64_t kernel_launches;   /* kernels launched (graph nodes count once per replay) */
  uint64_t graph_replays;
  uint64_t h2d_calls, h2d_bytes;
  uint64_t d2h_calls, d2h_bytes;
  uint64_t weight_bytes;      /* packed bytes resident in HBM on this rank */
  uint64_t kv_bytes;          /* KV cache bytes on this rank */
  uint64_t fallback_count;    /* always 0: there is no CPU or library fallback */
  float last_prefill_ms;      /* CUDA-event time of the last prefill call */
  float last_decode_ms;       /* last decode: host-clock time of the call (host-driven verbs), CUDA-event time per step (decode_loop) */
  uint64_t peer_reduce_launches; /* tensor-parallel partial sums done by the peer-memory kernel (0: NCCL path) */
} rg_report;

typedef struct rg_gguf rg_gguf;
typedef struct rg_plan rg_plan;
typedef struct rg_session rg_session;

const char *rg_b200_version(void);
const char *rg_b200_status_string(int32_t status);
/* Detail of the most recent failure on the calling thread (CUDA/NCCL code and call site). */
const char *rg_b200_last_error(void);

/* Host-side fault injection for tests: the n-th next call of a wrapped CUDA entry ("malloc",
 * "memcpy", "launch", "sync") fails; n < 0 disarms.  Stands where rustgrad's mock driver has its
 * fail-after-N knobs (src/cuda.rs:5895-5960).  Never makes the GPU itself fault. */
int32_t rg_b200_test_fail_after(const char *what, int32_t n);
/* How many launches of a kernel family this process has made: "qgemv_i8", "qgemv", "qgemm_tc",
 * "qgemm_tc_wide", "attn_fused", "attn_prefill" (both forms; "attn_prefill_tc" the tensor-core form alone), "attn_split", "tp_exchange", "kquant_gemv",
 * "dense_gemv", "qgemv_rows" (the opt-in 3..16-row form, not counted under "qgemv"), "attn_decode_tc"; UINT64_MAX for an unknown name.  Evidence for tests and reports of which kernel
 * served a call (the role of MetalDeviceRunReport's dispatch counts, src/runtime/metal/session.rs:145-185). */
uint64_t rg_b200_launch_count(const char *kernel);
/* What a session on CUDA ordinal `device` would run on (the role of MetalDeviceInfo,
 * src/runtime/metal/dispatch.rs:33-40, reached through LlamaMetalSession::device_info): name, SM count, compute
 * capability and the memory sizes the kernels are laid out for.  RG_CUDA_ERROR when there is no such device. */
typedef struct {
  char name[128];                  /* NUL-terminated */
  int32_t sm_count;
  int32_t cc_major, cc_minor;
  uint64_t total_memory_bytes;
  uint64_t l2_bytes;
  uint64_t shared_memory_per_block; /* opt-in maximum of dynamic shared memory per block */
} rg_device_info;
int32_t rg_b200_device_info(int32_t device, rg_device_info *out);
/* Test hook for the device-side time-out path (bounded waits that end in a status word, the
 * stand-in for rustgrad's unprovable-completion rule, src/runtime/cuda_graph.rs:542-546): enqueues
 * on the session's stream one launch of the partial-sum exchange kernel whose peer flag is never
 * written and whose poll limit is a few thousand polls.  The wait runs out, nothing faults or
 * hangs, and the session's next step returns RG_TIMEOUT and leaves the session poisoned. */
int32_t rg_b200_test_expire_device_wait(rg_session *s);
/* Development aid: with RG_B200_TRACE=1 in the environment at prepare, the kernels of a one- or
 * two-column decode step stamp the global nanosecond timer at their phases (CTA started, grid
 * dependency resolved, activations in shared memory, last weight stage consumed, first / last row
 * group stored, first weight stage landed, all loads issued), first CTA in words 0-7 and last CTA in
 * words 8-15 of each launch.  Copies the stamps of the last step (16 words per launch, launch order)
 * and returns the number of launches copied; 0 when tracing is off. */
int32_t rg_b200_debug_read_trace(rg_session *s, unsigned long long *out, int32_t max_launches);

/* ---- GGUF container: replaces read_gguf / GgufFile (src/gguf/mod.rs:166-173,256-384,
 * src/gguf/reader.rs:8-301).  The bytes are borrowed and must outlive the handle. ---- */
int32_t rg_b200_gguf_open(const uint8_t *bytes, size_t len, rg_gguf **out);
void rg_b200_gguf_close(rg_gguf *g);
size_t rg_b200_gguf_tensor_count(const rg_gguf *g);
/* dims are logical (outermost first), as GgufTensor::shape (src/gguf/reader.rs:144-146). */
int32_t rg_b200_gguf_tensor_info(const rg_gguf *g, size_t index, const char **name, int32_t *ggml_type,
                                 int32_t *rank, uint64_t dims[4], const uint8_t **data, size_t *nbytes);
/* LlamaModelConfig::from_gguf (src/models/transformer/model.rs:126-298). */
int32_t rg_b200_gguf_llama_config(const rg_gguf *g, rg_llama_config *out);

/* ---- Plan: replaces LlamaModelState::bind (model.rs:352-529) + LlamaMetalPlan::from_workflow_on
 * (metal_generation.rs:276-281).  Tensors are validated on the host before any device work and
 * uploaded once, in their native block bytes, with no host dequantisation.  Unlike the Metal
 * plan the upload happens per tensor at add time, so a 39 GB model never has two host copies. ---- */
int32_t rg_b200_plan_create(const rg_llama_config *config, const rg_options *options, rg_plan **out);
int32_t rg_b200_plan_add_tensor(rg_plan *plan, const char *name, int32_t ggml_type, uint64_t rows,
                                uint64_t cols, const uint8_t *bytes, size_t nbytes);
/* Binds every tensor of an open GGUF file (exact inventory, unexpected tensors rejected). */
int32_t rg_b200_plan_from_gguf(const rg_gguf *g, const rg_options *options, rg_plan **out);
/* Synthetic weights generated and quantized on the device: N(0, std) from a counter-based
 * generator keyed by (seed, element index of the full tensor), so a tensor-parallel rank
 * produces exactly its shard of the single-GPU tensor.  No counterpart in rustgrad (it has no
 * encoder and no synthetic-model tool); exists so 8B/70B-shape models need no 39 GB host file.
 * norm tensors: std is ignored and the value 1.0 is written. */
int32_t rg_b200_plan_synth_tensor(rg_plan *plan, const char *name, int32_t ggml_type, uint64_t rows,
                                  uint64_t cols, uint64_t seed, float std);
/* Copies the rank-local packed bytes of a bound tensor back to the host (tests, checker input). */
int32_t rg_b200_plan_tensor_nbytes(const rg_plan *plan, const char *name, size_t *nbytes);
int32_t rg_b200_plan_read_tensor(const rg_plan *plan, const char *name, uint8_t *out, size_t nbytes);
void rg_b200_plan_destroy(rg_plan *plan);

/* ---- Session: replaces SessionTarget::prepare for the Llama plan
 * (src/session/target.rs:13-18, metal_generation.rs:453-500,702-715).  Consumes the plan's device
 * tensors; the plan handle stays valid only for rg_b200_plan_destroy. ---- */
int32_t rg_b200_session_prepare(rg_plan *plan, rg_session **out);
void rg_b200_session_destroy(rg_session *s);

/* metal_generation.rs:837-882 */
int32_t rg_b200_position(const rg_session *s, int32_t row);
int32_t rg_b200_max_context(const rg_session *s);
int32_t rg_b200_vocab_size(const rg_session *s);
int32_t rg_b200_is_full(const rg_session *s);
int32_t rg_b200_reset_sequence(rg_session *s);

/* prefill_ids (metal_generation.rs:913-1047): appends n prompt tokens to sequence `row`;
 * last_logits ([vocab], nullable) receives the logits of the final prompt token. */
int32_t rg_b200_prefill(rg_session *s, int32_t row, const int32_t *ids, size_t n, float *last_logits);
/* Several prompts in one pass: the batch prefill of LlamaBatchGenerator (src/models/transformer/
 * batch.rs:177-325, batch_generation.rs:104-189) without its right padding.  Prompt i (lens[i] ids,
 * the prompts laid end to end in `ids`) continues cache row rows[i] from that row's position; the
 * rows must be distinct.  Chunks of up to 1024 columns are cut across the prompts, so short prompts
 * share every weight tile.  last_logits (nullable) receives [n_rows, vocab], the logits after each
 * prompt's last token; greedy (nullable) the token selected from them.  Everything is validated
 * before any device work, and no row's position advances unless the whole call succeeded. */
int32_t rg_b200_prefill_rows(rg_session *s, const int32_t *rows, const int32_t *ids, const size_t *lens, int32_t n_rows,
                             float *last_logits, int32_t *greedy);
/* run_token (metal_generation.rs:1123-1138) generalised to `batch` rows (batch.rs:140-162):
 * tokens[batch] in; logits [batch, vocab] and/or greedy ids [batch] out (either may be NULL).
 * Rows 0..batch-1 advance by one position only when the whole step succeeds.  The rows are independent
 * sequences: on Q4_0 / Q8_0 weights a step of more than 16 rows runs as equal chunks of at most 16 rows (the
 * same results; rg_b200_decode_rows and rg_b200_decode_loop likewise). */
int32_t rg_b200_decode(rg_session *s, const int32_t *tokens, int32_t batch, float *logits, int32_t *greedy);
/* generate_ids with greedy selection (generation.rs:106-160, metal_generation.rs:1052-1175):
 * requires a fresh sequence, prefill then one-token steps, stops on EOS/EOT, the last token is
 * not fed back.  out has room for max_new ids. */
int32_t rg_b200_generate_greedy(rg_session *s, const int32_t *prompt, size_t n_prompt, size_t max_new,
                                int32_t *out, size_t *n_out, int32_t *stopped);
/* LlamaSampling::GumbelMax (src/models/transformer/generation.rs:10-19,227-287): the selected id of
 * every row maximises logit / max(temperature, 1e-12) - ln(-ln(max(u, 1e-12))) in f32 with strict
 * '>' (lowest id among equal scores); any non-finite LOGIT is RG_NON_FINITE_LOGITS.  Randomness is an
 * explicit tape of uniforms supplied by the caller: `uniforms` holds one row of vocab_size floats per
 * decoded row for rg_b200_decode_sampled, and max_new rows (row-major [step, vocabulary]; row 0 picks
 * the first token from the prompt's logits) for rg_b200_generate_sampled.  Otherwise these behave as
 * rg_b200_decode / rg_b200_generate_greedy. */
int32_t rg_b200_decode_sampled(rg_session *s, const int32_t *tokens, int32_t batch, float temperature,
                               const float *uniforms, float *logits, int32_t *ids);
int32_t rg_b200_generate_sampled(rg_session *s, const int32_t *prompt, size_t n_prompt, size_t max_new,
                                 float temperature, const float *uniforms, int32_t *out, size_t *n_out,
                                 int32_t *stopped);

/* Device-resident greedy loop for rows 0..batch-1: `steps` replays of the decode graph with the
 * selected token fed back on the device (the device-greedy session of
 * metal_greedy_generation.rs:52-72).  first_tokens[batch] seeds it; out [steps, batch] (nullable)
 * receives the ids after the last step.  gpu_ms (nullable) is the CUDA-event time of the loop (summed over
 * the chunks of a batch beyond 16 rows, which run one after the other, each for all steps). */
int32_t rg_b200_decode_loop(rg_session *s, const int32_t *first_tokens, int32_t batch, int32_t steps,
                            int32_t *out, float *gpu_ms);
/* Profiling pass in the vocabulary of rustgrad's CUDA event recorder (src/cuda_profile.rs:15-60).
 * The launches of one decode step are replayed one kernel family at a time, serialized (no
 * programmatic overlap), `steps` times between two CUDA events on the session's stream.
 * out_ms / out_launches: [0] quantized GEMV launches, [1] RoPE + KV append + attention,
 * [2] norms, embedding, selection and collectives, [3] their sum; milliseconds per step and
 * kernels per step.  Positions are not advanced and nothing is committed. */
int32_t rg_b200_decode_profile(rg_session *s, const int32_t *first_tokens, int32_t batch, int32_t steps,
                               float out_ms[4], uint64_t out_launches[4]);
/* The same pass with the launch attributes of the real step: consecutive launches of a family
 * keep their programmatic dependent-launch edges, so a kernel's weight prefetch overlaps the end
 * of the kernel before it as it does inside a decode step (src/cuda_profile.rs:15-60). */
int32_t rg_b200_decode_profile_in_step(rg_session *s, const int32_t *first_tokens, int32_t batch, int32_t steps,
                                       float out_ms[4], uint64_t out_launches[4]);
/* The GEMV family split by projection (batch 1 or 2, the integer tensor-core path): milliseconds per
 * step of the launches of [0] q+k+v, [1] attention output, [2] gate+up, [3] down, [4] logits head,
 * each set replayed alone with the step's launch attributes (src/cuda_profile.rs:15-60). */
int32_t rg_b200_decode_profile_projections(rg_session *s, const int32_t *first_tokens, int32_t batch, int32_t steps,
                                           float out_ms[5]);
int32_t rg_b200_report(const rg_session *s, rg_report *out);
/* cudaStream_t the session launches on (for CUDA-event timing by the caller). */
void *rg_b200_session_stream(const rg_session *s);

/* The share of one tensor a tensor-parallel rank keeps (the rule rg_b200_plan_add_tensor applies):
 * q / k / v, gate / up and the vocabulary head by output rows, attn_output / ffn_down along the
 * contracting axis at whole blocks (32 elements, 256 for K-quants), everything else whole
 * (src/sharding.rs:642-667).  Host arithmetic only. */
int32_t rg_b200_tp_shard(const char *name, int32_t ggml_type, uint64_t rows, uint64_t cols, int32_t rank, int32_t world,
                         uint64_t *row0, uint64_t *n_rows, uint64_t *col0, uint64_t *n_cols);
/* ---- Tensor parallel plumbing (replaces CudaCollectiveGroup, src/collective.rs:322-345,441). ---- */
int32_t rg_b200_nccl_unique_id(uint8_t out[128]);

/* ---- Operator-level entry points (host buffers in, host buffers out). ---- */
/* QuantizedTensorData::dequantize_f32 (src/gguf/quantization/data.rs:415-428): bit-exact. */
int32_t rg_b200_dequantize(int32_t device, int32_t ggml_type, const uint8_t *bytes, size_t elements, float *out);
/* QuantizedMatmulPlan::execute (src/matmul/quantized.rs:126-182): activation f32 [m,k] x packed
 * or dense [n,k] -> f32 [m,n], through the decode GEMVs in chunks of at most 16 activation rows (8 for
 * types other than Q4_0 / Q8_0). */
int32_t rg_b200_qmatmul(int32_t device, int32_t ggml_type, const uint8_t *weight, uint64_t n, uint64_t k,
                        const float *activation, uint64_t m, float *out);
/* QuantizedRowGatherPlan::execute (src/gguf/quantization/row_gather.rs:149-226). */
int32_t rg_b200_row_gather(int32_t device, int32_t ggml_type, const uint8_t *weight, uint64_t rows,
                           uint64_t cols, const int64_t *indices, size_t count, float *out);

/* The same product for many activation rows on the tcgen05 tensor cores (prefill): activations are
 * rounded to a 16-bit operand type and the weights are dequantised to tiles of that type,
 * accumulation is f32 (the per-layer linear of src/models/transformer/layer.rs:445-448 for a whole
 * prompt chunk).  operand_mode 0: bf16 operands (Q4_0 weights enter as bf16(bf16(d) * (n - 8)));
 * 1: IEEE half operands (f16(d * (n - 8)); finite activations beyond +-65504 saturate);
 * 2: compensated half, the session's default: each operand is split into f16 hi + f16 lo and three
 * products per K step (hi.hi + hi.lo + lo.hi) give f32-grade accuracy at three times the
 * tensor-core work.  iters > 0 additionally repeats the launch `iters` times between CUDA events
 * and stores the mean kernel time in kernel_ms (nullable). */
int32_t rg_b200_qgemm(int32_t device, int32_t ggml_type, const uint8_t *weight, uint64_t n, uint64_t k,
                      const float *activation, uint64_t m, int32_t operand_mode, int32_t iters, float *out,
                      float *kernel_ms);

/* One decode token of scaled_dot_product_attention with GQA (src/ir/attention.rs:946-981,1157-1240;
 * mask `col <= past + row` of src/models/transformer/layer.rs:374-380 for a single new row): q is
 * [heads, head_dim] f32, already rotated; keys / values are caches [kv_heads, n_pos, head_dim] of
 * f32 (kv_f32 != 0) or IEEE half; the token sits at position n_pos - 1 and attends to all n_pos
 * positions.  out [heads, head_dim] f32. */
int32_t rg_b200_attention_decode(int32_t device, const float *q, const void *keys, const void *values, int32_t heads,
                                 int32_t kv_heads, int32_t head_dim, int32_t n_pos, int32_t kv_f32, float *out);

/* The same decode attention for callers that must not allocate device memory: a runtime that
 * carved up all of its HBM into its own arena at start-up, a serving loop that cannot afford the
 * device-wide stall of a cudaMalloc, or code between the begin and end of a stream capture.  It
 * has no counterpart in rustgrad (whose CUDA layer always draws scratch from its pooled
 * allocator).  All pointers are DEVICE pointers owned by the caller: q [heads, head_dim] f32,
 * caches [kv_heads, ctx, head_dim] (ctx = rows allocated per kv head, of which the first n_pos are
 * used; the new token sits at n_pos - 1), out [heads, head_dim] f32.  keys_dev and values_dev must
 * be 16-byte aligned (they are fetched by bulk copies), q_dev and out_dev 4-byte aligned; a pointer
 * that is not is refused with RG_INVALID_ARGUMENT before anything is launched.  The split-context partials
 * live in a 4 MiB array inside the library image, held by every GPU that loads the library until
 * the process ends; heads * ceil(ctx / 128) * (head_dim + 2) may not exceed 1 048 576 floats, and
 * anything larger is refused with RG_UNSUPPORTED_GEOMETRY.  The call makes no cudaMalloc, cudaFree
 * or other allocating call.  The first call on a device resolves the array's device address and
 * prepares the kernels: make it before any stream capture.  Every call on a device shares the
 * array, so calls whose kernels could overlap on the GPU must be ordered by the caller.  Work is
 * enqueued on `stream` (a cudaStream_t, NULL for the default stream); with wait != 0 the call
 * also synchronises the stream and reports a device-side time-out as RG_TIMEOUT. */
int32_t rg_b200_attention_decode_noalloc(const float *q_dev, const void *keys_dev, const void *values_dev, int32_t heads,
                                         int32_t kv_heads, int32_t head_dim, int32_t ctx, int32_t n_pos, int32_t kv_f32,
                                         float *out_dev, void *stream, int32_t wait);

/* ---- Verbs of a continuous-batching step.  rustgrad's serving scheduler
 * (src/models/transformer/serving/mod.rs:557-690) rebuilds a batch from per-request K/V
 * snapshots at every step; here a request keeps one cache row of the session while it runs, and a
 * step is one decode launch over an arbitrary set of rows plus one prefill per newly admitted
 * prompt.  rg_b200_serving.h declares the scheduler that drives them. ---- */
typedef struct rg_kv_snapshot rg_kv_snapshot;
/* Forgets the cached positions of one row (a finished request's slot is handed to the next). */
int32_t rg_b200_reset_row(rg_session *s, int32_t row);
/* rg_b200_prefill that also returns the token selected from the last row's logits: greedy when
 * temperature <= 0 or uniforms is NULL, else Gumbel-max with one row of `vocab` uniforms
 * (serving/mod.rs:649-665). */
int32_t rg_b200_prefill_select(rg_session *s, int32_t row, const int32_t *ids, size_t n, float temperature,
                               const float *uniforms, float *last_logits, int32_t *selected);
/* One decode step over n distinct rows, each at its own position: column i feeds tokens[i] to
 * row rows[i].  temperatures (nullable) holds one value per column, <= 0 meaning greedy; uniforms
 * is [n, vocab] and is only read for sampled columns.  logits (nullable) receives [n, vocab].
 * Positions advance only when the whole step succeeded. */
int32_t rg_b200_decode_rows(rg_session *s, const int32_t *rows, const int32_t *tokens, int32_t n,
                            const float *temperatures, const float *uniforms, float *logits, int32_t *ids);
/* Selection alone on host logits [n, vocab] (a prompt fully covered by a cached prefix needs no
 * forward pass, serving/mod.rs:591-603), same rules as above, on the device. */
int32_t rg_b200_select(rg_session *s, const float *logits, int32_t n, const float *temperatures, const float *uniforms,
                       int32_t *ids);
/* Immutable device copy of the first `length` cached positions of a row, all layers
 * (LlamaNativePrefixSnapshot, serving/mod.rs:182-190); restore writes it into any row of a
 * session of the same shape and sets that row's position to its length. */
int32_t rg_b200_kv_snapshot_create(rg_session *s, int32_t row, int32_t length, rg_kv_snapshot **out);
int32_t rg_b200_kv_snapshot_length(const rg_kv_snapshot *k);
size_t rg_b200_kv_snapshot_bytes(const rg_kv_snapshot *k);
int32_t rg_b200_kv_snapshot_restore(rg_session *s, const rg_kv_snapshot *k, int32_t row);
void rg_b200_kv_snapshot_free(rg_kv_snapshot *k);

/* Device-resident operator benchmark: weight uploaded once, `iters` launches timed with CUDA
 * events on the library's stream; `rotate` distinct weight copies are cycled so that each launch
 * reads HBM rather than L2.  kernel_ms receives the mean time of one launch.  m in 1..16. */
int32_t rg_b200_qmatmul_bench(int32_t device, int32_t ggml_type, const uint8_t *weight, uint64_t n, uint64_t k,
                              const float *activation, uint64_t m, int32_t rotate, int32_t iters,
                              int32_t warmup, float *out, float *kernel_ms);

#ifdef __cplusplus
}
#endif
#endif
