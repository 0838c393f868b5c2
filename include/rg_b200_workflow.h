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

/* ---- LlamaConversation (src/models/transformer/conversation.rs:29-85): a transcript over one workflow. ----
 * send() renders the committed history plus the new user message through the chat template, generates
 * greedily from position 0 and appends the user and the assistant message only when everything succeeded. */
typedef struct rg_conversation rg_conversation;

/* LlamaConversationError. */
enum {
  RG_CONVERSATION_OK = 0,
  RG_CONVERSATION_EMPTY_INPUT = 1,
  RG_CONVERSATION_CHAT = 2,            /* template / tokenizer / message bound: *detail = rg_tok_status */
  RG_CONVERSATION_GENERATION = 3,      /* the generation failed: *detail = rg_status */
  RG_CONVERSATION_INVALID_ARGUMENT = 4
};

/* The workflow verbs a turn is made of; rg_b200_conversation_new binds them to an rg_workflow, a test supplies
 * its own.  generate_chat has the contract of rg_b200_workflow_generate_chat; decoded returns the
 * decoded_bytes bytes of the last request. */
typedef struct rg_chat_backend {
  void *ctx;
  int32_t (*generate_chat)(void *ctx, const int32_t *roles, const char *const *contents, const size_t *content_len,
                           size_t n_messages, size_t max_new_tokens, rg_text_callback on_text, void *user, rg_prompt_output *out);
  const char *(*decoded)(void *ctx);
} rg_chat_backend;

/* LlamaPromptWorkflow::conversation (workflow.rs:136-139).  The workflow must outlive the conversation, and
 * requests made on the workflow in between do not disturb the transcript (every turn starts from position 0). */
int32_t rg_b200_conversation_new(rg_workflow *w, rg_conversation **out);
int32_t rg_b200_conversation_new_with_backend(const rg_chat_backend *backend, rg_conversation **out);
void rg_b200_conversation_free(rg_conversation *c);
/* history(): messages committed so far (user, assistant, user, ...); the content pointer stays valid until the
 * next send or reset. */
size_t rg_b200_conversation_history_len(const rg_conversation *c);
int32_t rg_b200_conversation_message(const rg_conversation *c, size_t index, int32_t *role, const char **content, size_t *content_len);
/* cache_len(): positions the last successful turn left in the cache (its prompt and all but the last generated
 * id); reset(): empty transcript, cache length 0. */
size_t rg_b200_conversation_cache_len(const rg_conversation *c);
void rg_b200_conversation_reset(rg_conversation *c);
/* send (conversation.rs:58-84): message bound, then empty input, then render + generate on the staged transcript.
 * `out` and the workflow's accessors describe the turn's generation; on any failure the transcript and the
 * cache length are what they were.  detail (nullable) receives the status named above. */
int32_t rg_b200_conversation_send(rg_conversation *c, const char *content, size_t content_len, size_t max_new_tokens,
                                  rg_text_callback on_text, void *user, rg_prompt_output *out, int32_t *detail);

#ifdef __cplusplus
}
#endif
#endif
