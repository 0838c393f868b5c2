/* Prompt-to-tokens facade over the CUDA session: the C ABI a binding uses in place of rustgrad's
 * `LlamaPromptWorkflow` (src/models/transformer/workflow.rs:18-147) joined to the accelerated
 * session's text verbs (`LlamaMetalSession::generate_text / generate_chat`,
 * src/models/transformer/metal_generation.rs:1177-1215).  One handle owns the validated model on
 * the GPU, its GGUF tokenizer and the one checked chat template; a request is text in, token ids
 * and text out, greedy, on a fresh sequence.  Nothing falls back to a CPU path.
 */
#ifndef RG_B200_WORKFLOW_H
#define RG_B200_WORKFLOW_H

#include <stddef.h>
#include <stdint.h>

#include "rg_b200.h"
#include "rg_b200_tokenizer.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rg_workflow rg_workflow;

/* Called once per generated token with the text that token completed (possibly empty: an
 * incomplete UTF-8 sequence is held back, StreamingDecoder, src/tokenizer/mod.rs:459-470), and once
 * more with token_id = -1 for what the end of the stream flushes. */
typedef void (*rg_text_callback)(void *user, int32_t token_id, const char *text, size_t text_len);

/* Sizes and flags of the last request; the arrays and strings stay readable through the accessors
 * below until the next request on the same handle. */
typedef struct rg_prompt_output {
  size_t n_prompt_ids;    /* ids the prompt encoded to, the configured BOS included */
  size_t n_generated_ids;
  size_t decoded_bytes;   /* UTF-8 bytes of the decoded generated ids */
  size_t rendered_bytes;  /* UTF-8 bytes of the prompt as given to the tokenizer (chat: the rendered template) */
  int32_t stopped;        /* 1 when the last generated id is the EOS or EOT id */
  int32_t tokenizer_status; /* rg_tok_status of a tokenizer / chat failure (the call then returns RG_INVALID_ARGUMENT), else 0 */
} rg_prompt_output;

/* LlamaPromptWorkflow::from_gguf_bytes (workflow.rs:30-40) followed by
 * LlamaMetalPlan::from_workflow_on + SessionTarget::prepare (metal_generation.rs:276-281,702-715):
 * parses and validates the container, builds the tokenizer (which also supplies the stop ids),
 * accepts only an absent or the one supported chat template, binds and uploads the tensors and
 * prepares a session.  The bytes are borrowed for the call only.  options may be NULL. */
int32_t rg_b200_workflow_open(const uint8_t *gguf_bytes, size_t len, const rg_options *options, rg_workflow **out);
void rg_b200_workflow_close(rg_workflow *w);

/* The parts, owned by the workflow (the session for the id-level verbs of rg_b200.h). */
rg_session *rg_b200_workflow_session(rg_workflow *w);
const rg_tokenizer *rg_b200_workflow_tokenizer(const rg_workflow *w);

/* generate_text (generation.rs:92-103; metal_generation.rs:1177-1190): encode, put the configured
 * BOS id in front, generate up to max_new_tokens greedy ids from position 0, stop on EOS / EOT
 * (the last generated id is not fed back), decode.  on_text may be NULL.  The context bound
 * (prompt ids + max_new_tokens <= context) is checked before any device work. */
int32_t rg_b200_workflow_generate_text(rg_workflow *w, const char *prompt, size_t prompt_len, size_t max_new_tokens,
                                       rg_text_callback on_text, void *user, rg_prompt_output *out);
/* generate_chat (workflow.rs:83-98; metal_generation.rs:1192-1207): renders the checked template
 * with the generation prompt (roles: rg_chat_role), then as generate_text. */
int32_t rg_b200_workflow_generate_chat(rg_workflow *w, const int32_t *roles, const char *const *contents,
                                       const size_t *content_len, size_t n_messages, size_t max_new_tokens,
                                       rg_text_callback on_text, void *user, rg_prompt_output *out);

/* Results of the last request (LlamaGeneration, generation.rs:40-60; LlamaPromptOutput,
 * workflow.rs:150-170). */
const int32_t *rg_b200_workflow_prompt_ids(const rg_workflow *w);
const int32_t *rg_b200_workflow_generated_ids(const rg_workflow *w);
const char *rg_b200_workflow_decoded(const rg_workflow *w);          /* decoded_bytes bytes, also NUL-terminated */
const char *rg_b200_workflow_rendered_prompt(const rg_workflow *w);  /* rendered_bytes bytes, also NUL-terminated */

#ifdef __cplusplus
}
#endif
#endif
