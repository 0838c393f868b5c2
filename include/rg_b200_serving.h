/* Continuous batching with a prefix cache over one CUDA session: the C ABI a binding uses in place
 * of rustgrad's `LlamaServingScheduler` (src/models/transformer/serving/mod.rs:371-690), with its
 * verbs (submit_ids / submit_text / submit_chat / status / result / remove / step / prefix_stats /
 * invalidate_prefix_cache) and its policy: requests are served in arrival order, at most
 * batch_size per step, one token per selected request per step.
 *
 * What differs, because the caches live in HBM rather than in per-request host tensors:
 *  - a request keeps one cache row of the session from its first step to its last, instead of a
 *    batch being rebuilt from snapshots at every step;
 *  - a prefix entry is taken when a prompt has been prefilled, as a device-to-device copy of the
 *    row's K/V; decode steps add no entries;
 *  - the decode columns of one step run as ONE launch sequence over all running rows; the greedy
 *    prompts admitted in a step are prefilled together in one pass (rg_b200_prefill_rows), so short
 *    prompts share every weight tile; sampled ones one after the other.
 * The scheduler only decides what runs: all device work goes through the verbs of rg_b200.h
 * (prefill_select, decode_rows, select, kv_snapshot_*, reset_row), reached through the table of
 * rg_serving_backend so that the policy can be driven without a device.
 */
#ifndef RG_B200_SERVING_H
#define RG_B200_SERVING_H

#include <stddef.h>
#include <stdint.h>

#include "rg_b200.h"
#include "rg_b200_tokenizer.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rg_scheduler rg_scheduler;

/* LlamaServingError by kind (serving/mod.rs:792-860). */
typedef enum rg_serving_status {
  RG_SERVING_OK = 0,
  RG_SERVING_EMPTY_BATCH = 1,          /* batch_size 0, or fewer cache rows than batch_size */
  RG_SERVING_EMPTY_PROMPT = 2,
  RG_SERVING_CONTEXT_LENGTH = 3,       /* value = requested, value2 = maximum */
  RG_SERVING_TOKEN_OUT_OF_RANGE = 4,   /* value = token, value2 = vocabulary */
  RG_SERVING_INVALID_TEMPERATURE = 5,
  RG_SERVING_UNIFORM_TAPE_LENGTH = 6,  /* value = required, value2 = actual */
  RG_SERVING_INVALID_UNIFORM = 7,      /* value = index of the first bad entry */
  RG_SERVING_UNKNOWN_REQUEST = 8,
  RG_SERVING_SESSION = 9,              /* a session verb failed: value = its rg_status; rg_b200_last_error has the text */
  RG_SERVING_TOKENIZER = 10,           /* value = rg_tok_status */
  RG_SERVING_INVALID_ARGUMENT = 11,
  RG_SERVING_NOT_COMPLETE = 12,        /* result asked of a request that has not finished */
  RG_SERVING_ACTIVE_REQUESTS = 13      /* rebind of a scheduler that still has unfinished requests */
} rg_serving_status;

typedef struct rg_serving_error {
  int32_t kind;
  int64_t value, value2;
} rg_serving_error;

typedef struct rg_serving_options {
  int32_t batch_size;          /* requests selected per step */
  int32_t max_rows;            /* cache rows the scheduler may hand out; 0 = batch_size */
  size_t prefix_max_entries;   /* 0 switches the prefix cache off */
  size_t prefix_max_bytes;
  const int32_t *stop_ids;     /* generation stops after one of these (borrowed for the call) */
  size_t n_stop_ids;
  int32_t has_bos;             /* submit_text puts bos_id in front of the encoded prompt */
  int32_t bos_id;
} rg_serving_options;

/* LlamaServingSampling (serving/mod.rs:28-38): greedy, or Gumbel-max at `temperature` with an
 * explicit row-major [generation_step, vocabulary] tape of uniforms in [0, 1). */
typedef struct rg_serving_sampling {
  int32_t greedy;
  float temperature;
  const float *uniforms;   /* copied at submission */
  size_t n_uniforms;
} rg_serving_sampling;

/* LlamaTokenEvent (serving/mod.rs:98-129). */
typedef struct rg_token_event {
  uint64_t request_id;
  uint64_t arrival_order;
  int32_t generation_step;
  int32_t token_id;
  int32_t stopped;
  int32_t complete;
} rg_token_event;

/* LlamaServingResult (serving/mod.rs:131-155); the pointers stay valid until the request is removed. */
typedef struct rg_serving_result {
  uint64_t request_id;
  const int32_t *prompt_ids;
  size_t n_prompt_ids;
  const int32_t *generated_ids;
  size_t n_generated_ids;
  const char *decoded;     /* UTF-8, NUL-terminated; empty without a tokenizer */
  size_t decoded_bytes;
  int32_t stopped;
} rg_serving_result;

typedef struct rg_prefix_stats {
  uint64_t entries, bytes, hits, misses, stale_rejections, evictions, generation;
} rg_prefix_stats;

enum { RG_REQUEST_QUEUED = 0, RG_REQUEST_RUNNING = 1, RG_REQUEST_COMPLETE = 2 };

/* The session verbs a step is made of.  rg_b200_scheduler_new fills this table with the functions
 * of rg_b200.h over one rg_session; a test (or another device back end) supplies its own.  Every
 * function returns an rg_status.  A snapshot is an opaque handle owned by the scheduler. */
typedef struct rg_serving_backend {
  void *ctx;
  int32_t vocab, max_context;
  int32_t (*reset_row)(void *ctx, int32_t row);
  int32_t (*prefill_select)(void *ctx, int32_t row, const int32_t *ids, size_t n, float temperature, const float *uniforms,
                            float *last_logits, int32_t *selected);
  int32_t (*decode_rows)(void *ctx, const int32_t *rows, const int32_t *tokens, int32_t n, const float *temperatures,
                         const float *uniforms, int32_t *ids);
  int32_t (*select)(void *ctx, const float *logits, float temperature, const float *uniforms, int32_t *id);
  int32_t (*snapshot_create)(void *ctx, int32_t row, int32_t length, void **snapshot, size_t *bytes);
  int32_t (*snapshot_restore)(void *ctx, const void *snapshot, int32_t row);
  void (*snapshot_free)(void *ctx, void *snapshot);
  /* Optional (may be NULL): several greedy prompts in one pass, rg_b200_prefill_rows.  Prompt i (lens[i]
   * ids, laid end to end) continues cache row rows[i]; last_logits is [n, vocab], selected [n]. */
  int32_t (*prefill_rows)(void *ctx, const int32_t *rows, const int32_t *ids, const size_t *lens, int32_t n, float *last_logits,
                          int32_t *selected);
} rg_serving_backend;

/* LlamaServingScheduler::new (serving/mod.rs:371-406).  The session (and the tokenizer, nullable,
 * needed by submit_text / submit_chat and for decoded results) must outlive the scheduler. */
int32_t rg_b200_scheduler_new(rg_session *session, const rg_tokenizer *tokenizer, const rg_serving_options *options,
                              rg_scheduler **out, rg_serving_error *err);
int32_t rg_b200_scheduler_new_with_backend(const rg_serving_backend *backend, const rg_tokenizer *tokenizer,
                                           const rg_serving_options *options, rg_scheduler **out, rg_serving_error *err);
void rg_b200_scheduler_free(rg_scheduler *s);

/* Admission (serving/mod.rs:408-477; validate_request :726-790): the request is checked as a whole
 * before it gets an id.  max_new_tokens 0 completes at once with an empty result. */
int32_t rg_b200_scheduler_submit_ids(rg_scheduler *s, const int32_t *prompt, size_t n, size_t max_new_tokens,
                                     const rg_serving_sampling *sampling, uint64_t *request_id, rg_serving_error *err);
int32_t rg_b200_scheduler_submit_text(rg_scheduler *s, const char *prompt, size_t prompt_len, size_t max_new_tokens,
                                      const rg_serving_sampling *sampling, uint64_t *request_id, rg_serving_error *err);
/* Renders the checked chat template with the generation prompt (roles: rg_chat_role). */
int32_t rg_b200_scheduler_submit_chat(rg_scheduler *s, const int32_t *roles, const char *const *contents,
                                      const size_t *content_len, size_t n_messages, size_t max_new_tokens,
                                      const rg_serving_sampling *sampling, uint64_t *request_id, rg_serving_error *err);

int32_t rg_b200_scheduler_status(const rg_scheduler *s, uint64_t request_id, int32_t *status);
int32_t rg_b200_scheduler_result(const rg_scheduler *s, uint64_t request_id, rg_serving_result *out);
int32_t rg_b200_scheduler_remove(rg_scheduler *s, uint64_t request_id);
size_t rg_b200_scheduler_pending(const rg_scheduler *s);
/* Ids of the finished requests in arrival order; returns how many there are, writes at most cap. */
size_t rg_b200_scheduler_completed(const rg_scheduler *s, uint64_t *ids, size_t cap);
void rg_b200_scheduler_prefix_stats(const rg_scheduler *s, rg_prefix_stats *out);
void rg_b200_scheduler_invalidate_prefix_cache(rg_scheduler *s);
/* LlamaServingScheduler::rebind (serving/mod.rs:528-547): an idle scheduler (no unfinished request, else
 * RG_SERVING_ACTIVE_REQUESTS) takes another session and tokenizer.  When the session differs from the bound
 * one (another object, vocabulary or context length; for a backend table also any other verb) every cached prefix is dropped -- its snapshots are freed
 * through the OLD session -- before a new request can be admitted; *changed (nullable) is then 1, else 0.
 * Finished requests keep their results.  The new session must hold as many cache rows as the scheduler was
 * created with.  `options` (nullable) replaces the stop ids and the BOS rule; its other fields are ignored. */
int32_t rg_b200_scheduler_rebind(rg_scheduler *s, rg_session *session, const rg_tokenizer *tokenizer,
                                 const rg_serving_options *options, int32_t *changed, rg_serving_error *err);
int32_t rg_b200_scheduler_rebind_with_backend(rg_scheduler *s, const rg_serving_backend *backend,
                                              const rg_tokenizer *tokenizer, const rg_serving_options *options,
                                              int32_t *changed, rg_serving_error *err);

/* One step (serving/mod.rs:557-690): selects up to batch_size unfinished requests in arrival order,
 * admits the new ones (longest cached prefix, then a prefill of the rest), decodes one token for
 * all running ones in one launch sequence, and reports one event per selected request.  events
 * must hold batch_size entries.  When a session verb fails the step returns RG_SERVING_SESSION;
 * requests it had not reached keep their state. */
int32_t rg_b200_scheduler_step(rg_scheduler *s, rg_token_event *events, size_t cap, size_t *n_events, rg_serving_error *err);

/* ---- Fixed-size batch generation: LlamaBatchGenerator (src/models/transformer/batch_generation.rs:58-189) ----
 * `batch_size` cache rows; every generate starts from empty rows, runs all prompts together (one batched
 * prefill where the session offers it, then one decode launch sequence per step over the rows that have not
 * stopped) and commits the rows' lengths only when every row, sample and decode succeeded.  The rows are
 * independent: each produces exactly what it produces alone. */
typedef struct rg_batch_generator rg_batch_generator;

/* LlamaBatchGenerationError (batch_generation.rs:251-279). */
typedef enum rg_batch_status {
  RG_BATCH_OK = 0,
  RG_BATCH_SESSION = 1,              /* a session verb failed (Model / non-finite logits): value = its rg_status */
  RG_BATCH_INVALID_TEMPERATURE = 2,
  RG_BATCH_TOKENIZER = 3,            /* value = rg_tok_status */
  RG_BATCH_BATCH_SIZE = 4,           /* value = expected, value2 = actual */
  RG_BATCH_EMPTY_PROMPT = 5,         /* row */
  RG_BATCH_CONTEXT_OVERFLOW = 6,
  RG_BATCH_CONTEXT_LENGTH = 7,       /* row; value = requested, value2 = maximum */
  RG_BATCH_UNIFORM_TAPE_LENGTH = 8,  /* value = required, value2 = actual */
  RG_BATCH_INVALID_UNIFORM = 9,      /* value = index of the first bad entry */
  RG_BATCH_TOKEN_OUT_OF_RANGE = 10,  /* row; value = token, value2 = vocabulary */
  RG_BATCH_INVALID_ARGUMENT = 11
} rg_batch_status;

typedef struct rg_batch_error {
  int32_t kind;
  int32_t row;
  int64_t value, value2;
} rg_batch_error;

/* LlamaBatchGenerator::new.  Of `options` (nullable) the stop ids and the BOS rule are used.  The session
 * (rows 0 .. batch_size-1 of it) and the tokenizer (nullable: no text in, decoded results empty) must outlive
 * the generator. */
int32_t rg_b200_batch_generator_new(rg_session *session, const rg_tokenizer *tokenizer, int32_t batch_size,
                                    const rg_serving_options *options, rg_batch_generator **out, rg_batch_error *err);
int32_t rg_b200_batch_generator_new_with_backend(const rg_serving_backend *backend, const rg_tokenizer *tokenizer,
                                                 int32_t batch_size, const rg_serving_options *options,
                                                 rg_batch_generator **out, rg_batch_error *err);
void rg_b200_batch_generator_free(rg_batch_generator *g);
/* cache_lengths: returns batch_size, writes at most cap committed row lengths.  clear: all rows empty. */
size_t rg_b200_batch_generator_cache_lengths(const rg_batch_generator *g, size_t *lengths, size_t cap);
void rg_b200_batch_generator_clear(rg_batch_generator *g);
/* generate_ids (batch_generation.rs:104-189).  Prompt r is lens[r] ids of `ids` (laid end to end);
 * n_prompts must equal batch_size.  Checks in the reference's order: batch size; per row empty prompt, context
 * overflow, context length; token ids; the sampling (temperature, tape length, tape values) -- all before any
 * device work.  Gumbel-max reads the [step, batch, vocabulary] row-major tape of `sampling`.  A row stops at a
 * stop id (the stop token is reported, not fed back); the last generated token is never fed back.  On failure
 * the committed lengths are the ones from before the call. */
int32_t rg_b200_batch_generate_ids(rg_batch_generator *g, const int32_t *ids, const size_t *lens, size_t n_prompts,
                                   size_t max_new_tokens, const rg_serving_sampling *sampling, rg_batch_error *err);
/* generate_texts (batch_generation.rs:85-102): encodes every text, puts the BOS id in front when configured. */
int32_t rg_b200_batch_generate_texts(rg_batch_generator *g, const char *const *texts, const size_t *text_bytes, size_t n_prompts,
                                     size_t max_new_tokens, const rg_serving_sampling *sampling, rg_batch_error *err);
/* Row `row` of the last successful generation (LlamaBatchSequence); request_id carries the row.  The pointers
 * stay valid until the next generate or free.  RG_BATCH_INVALID_ARGUMENT when there is none. */
int32_t rg_b200_batch_sequence(const rg_batch_generator *g, size_t row, rg_serving_result *out);

#ifdef __cplusplus
}
#endif
#endif
