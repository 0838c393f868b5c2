/*
 * CPU restatement of rustgrad's GGUF-quantized Llama path.  TEST INFRASTRUCTURE ONLY.
 *
 * This library is the checker that the CUDA path is compared against.  It is never linked
 * into, imported by or called from the shipped library; only the test-suite, the smoke entry
 * point and the benchmark's CPU-baseline leg load it.
 *
 * Parity pin: every block decoder and the blockwise matmul are checked against the
 * known-answer vectors of the reference's own tests (src/gguf/tests.rs:105-187,
 * src/matmul/quantized.rs:254-264,356-416) and the strict forward is checked against an
 * independent f64 forward on the reference's formula-defined 2-layer fixture
 * (src/models/transformer/model_tests.rs:16-20,343-377).
 *
 * Every function cites the reference file:line (paths relative to the rustgrad tree) it follows.
 */
#ifndef RG_ORACLE_H
#define RG_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML tensor type ids accepted on this path (src/gguf/tensor.rs:33-59). */
enum { RGO_F32 = 0, RGO_F16 = 1, RGO_Q4_0 = 2, RGO_Q8_0 = 8, RGO_Q4_K = 12, RGO_Q6_K = 14 };

/* Status codes. */
enum {
  RGO_OK = 0,
  RGO_ERR_ARG = 1,
  RGO_ERR_TYPE = 2,
  RGO_ERR_NON_FINITE = 3,
  RGO_ERR_TOKEN_RANGE = 4,
  RGO_ERR_CONTEXT = 5,
  RGO_ERR_NON_FINITE_LOGITS = 6,
  RGO_ERR_INDEX = 7
};

/* src/tensor/scalar.rs:110-135 and :137-174 */
float rgo_f16_to_f32(uint16_t bits);
uint16_t rgo_f32_to_f16(float value);

/* src/gguf/tensor.rs:88-155: (block elements, block bytes); 0 for unsupported. */
int rgo_block_elements(int ggml_type);
int rgo_block_bytes(int ggml_type);

/* src/gguf/quantization/blocks.rs:1244-1257 and :1493-1505 */
int rgo_decode_q4_0_block(const uint8_t *block, float out[32]);
int rgo_decode_q8_0_block(const uint8_t *block, float out[32]);

/* src/gguf/quantization/data.rs:415-428: decode `elements` values of a packed or dense tensor. */
int rgo_dequantize(int ggml_type, const uint8_t *bytes, size_t elements, float *out);

/* src/gguf/quantization/row_gather.rs:149-226: every index is validated before any decode. */
int rgo_row_gather(int ggml_type, const uint8_t *bytes, size_t rows, size_t cols,
                   const int64_t *indices, size_t count, float *out);

/* src/matmul/quantized.rs:126-182: out[m,n] = f32(sum_k f64(a[m,k]) * f64(w[n,k])), k ascending. */
int rgo_quantized_matmul(int ggml_type, const uint8_t *weight, size_t n, size_t k,
                         const float *activation, size_t m, float *out);

/* src/backend/cpu.rs:3484-3532 with a dense f32 weight [n,k]: acc = f32(acc + f32(a*w)), k ascending. */
void rgo_dense_matmul_strict(const float *weight, size_t n, size_t k, const float *activation,
                             size_t m, float *out);

/* ---- Llama model (src/models/transformer/model.rs, layer.rs) ---- */

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
  /* model variants (src/models/transformer/model.rs:160-175,253-282); zero = the plain Llama layer */
  int32_t rope_dim; /* rotary lanes per head, even, <= head_dim; 0 = head_dim */
  int32_t qk_norm;  /* 0 none, 1 per head (weights [head_dim]), 2 per projection (weights [width]) */
  int32_t qkv_bias; /* 1: blk.N.attn_{q,k,v}.bias are bound */
} rgo_config;

typedef struct rgo_model rgo_model;
typedef struct rgo_cache rgo_cache;

/* Execution modes of the forward. */
enum {
  RGO_MODE_STRICT = 0, /* op-by-op f32 commits, sequential non-FMA sums: the faithful restatement */
  RGO_MODE_FAST = 1    /* same algorithm, rows spread over threads and 8-lane partial sums */
};

rgo_model *rgo_model_create(const rgo_config *config);
void rgo_model_destroy(rgo_model *model);
/* Names follow src/models/transformer/model.rs:384-455.  Bytes are borrowed: the caller keeps
 * them alive for the model's lifetime.  A missing output.weight ties the head to token_embd
 * (model.rs:517-521). */
int rgo_model_set_tensor(rgo_model *model, const char *name, int ggml_type, size_t rows,
                         size_t cols, const uint8_t *bytes);
/* Returns RGO_OK when the whole inventory of model.rs:384-455 is present. */
int rgo_model_check(const rgo_model *model);

/* kv_f16 != 0 rounds K and V to IEEE half when they enter the cache (the GPU session's cache
 * type); 0 keeps the reference's f32 cache (model.rs:879-922). */
rgo_cache *rgo_cache_create(const rgo_model *model, int kv_f16);
void rgo_cache_destroy(rgo_cache *cache);
void rgo_cache_clear(rgo_cache *cache);
int rgo_cache_len(const rgo_cache *cache);
/* Timing aid: `n_pos` positions of seeded pseudo-random K / V rows; the cache length becomes n_pos. */
int rgo_cache_fill_seeded(rgo_cache *cache, int n_pos, uint64_t seed);

/* src/models/transformer/model.rs:909-921 -> plan_with_past :740-836 -> execute_all :959-1064.
 * logits: [n_tokens, vocab] (all rows) when all_logits != 0, else [vocab] (last row). */
int rgo_forward(const rgo_model *model, rgo_cache *cache, const int32_t *tokens, int n_tokens,
                int mode, int threads, int all_logits, float *logits);

/* src/models/transformer/generation.rs:260-287: strict '>' so the lowest id wins ties; any
 * non-finite logit is an error. */
int rgo_decode_q4_k_block(const uint8_t *block, float out[256]);
int rgo_decode_q6_k_block(const uint8_t *block, float out[256]);
int rgo_select_greedy(const float *row, int vocab, int32_t *token);
int rgo_select_gumbel(const float *row, int vocab, float temperature, const float *uniforms, int32_t *token);

/* src/models/transformer/generation.rs:106-160. */
int rgo_generate_greedy(const rgo_model *model, rgo_cache *cache, const int32_t *prompt,
                        int n_prompt, int max_new, int mode, int threads, int32_t *out,
                        int *n_out, int *stopped);

/* One decode token of src/ir/attention.rs:1157-1240: q [heads][hd] (rotated), caches
 * [kv_heads][n_pos][hd], the token attends to all n_pos positions; out [heads][hd]. */
int rgo_attention_decode(const float *q, const float *keys, const float *values, int heads, int kv_heads, int hd,
                         int n_pos, float *out);

/* Independent f64 forward (no f32 commits) used only to pin the strict mode, in the manner of
 * the in-test oracle of src/models/transformer/model_tests.rs:827-997.  Full sequence, no cache. */
int rgo_forward_f64(const rgo_model *model, const int32_t *tokens, int n_tokens, double *logits);

#ifdef __cplusplus
}
#endif
#endif
