// Prompt-to-tokens facade behind include/rg_b200_workflow.h: one GGUF file becomes a validated
// model on the GPU, its tokenizer and the checked chat template; a request encodes text, runs the
// session's greedy generation from position 0 and decodes the ids, streaming the text token by
// token.  Composition only: every step goes through the public entry points of rg_b200.h and
// rg_b200_tokenizer.h (src/models/transformer/workflow.rs:18-147,
// src/models/transformer/metal_generation.rs:1177-1215).
#include <string.h>

#include <string>
#include <vector>

#include "../../include/rg_b200_workflow.h"
#include "gguf.h"

namespace rg {
extern thread_local std::string g_last_error;
}

struct rg_workflow {
  rg_session *session = nullptr;
  rg_tokenizer *tokenizer = nullptr;
  rg_tok_config tok_cfg{};
  rg_llama_config model_cfg{};
  int32_t context = 0;
  // last request
  std::vector<int32_t> prompt_ids, generated_ids;
  std::string decoded, rendered;
};

namespace {

int32_t fail(int32_t status, const std::string &why) {
  rg::g_last_error = why;
  return status;
}

int32_t tok_fail(rg_prompt_output *out, int32_t tok_status, const rg_tok_error &e, const char *what) {
  if (out) out->tokenizer_status = tok_status;
  const size_t n = e.text_len < sizeof(e.text) ? e.text_len : sizeof(e.text);
  return fail(RG_INVALID_ARGUMENT, std::string(what) + ": tokenizer status " + std::to_string(tok_status) + " (" +
                                       std::string(e.text, n) + ", " + std::to_string(e.value) + ", " + std::to_string(e.value2) + ")");
}

// Encodes `text`, inserts the configured BOS id, generates and decodes.  `text` is what the tokenizer sees.
int32_t run_request(rg_workflow *w, const std::string &text, size_t max_new, rg_text_callback on_text, void *user,
                    rg_prompt_output *out) {
  rg_tok_error terr{};
  // encode (sizing call, then the real one)
  size_t n_ids = 0;
  int32_t trc = rg_b200_tokenizer_encode(w->tokenizer, text.data(), text.size(), nullptr, 0, &n_ids, &terr);
  if (trc != RG_TOK_OK && !(trc == RG_TOK_INVALID_ARGUMENT && n_ids > 0)) return tok_fail(out, trc, terr, "encode");
  std::vector<uint32_t> ids(n_ids ? n_ids : 1);
  if (n_ids) {
    trc = rg_b200_tokenizer_encode(w->tokenizer, text.data(), text.size(), ids.data(), ids.size(), &n_ids, &terr);
    if (trc != RG_TOK_OK) return tok_fail(out, trc, terr, "encode");
  }
  w->prompt_ids.clear();
  if (w->tok_cfg.has_bos) w->prompt_ids.push_back((int32_t)w->tok_cfg.bos_id);
  for (size_t i = 0; i < n_ids; ++i) w->prompt_ids.push_back((int32_t)ids[i]);
  w->rendered = text;
  if (out) {
    out->n_prompt_ids = w->prompt_ids.size();
    out->rendered_bytes = w->rendered.size();
  }
  // generate_ids on a fresh sequence (generation.rs:106-160): bounds before any device work
  if (w->prompt_ids.empty()) return fail(RG_EMPTY_PROMPT, "the prompt encodes to no token and no BOS id is configured");
  if (w->prompt_ids.size() + max_new > (size_t)w->context)
    return fail(RG_CONTEXT_EXHAUSTED, std::to_string(w->prompt_ids.size() + max_new) + " tokens requested of " + std::to_string(w->context));
  int32_t rc = rg_b200_reset_sequence(w->session);
  if (rc) return rc;
  if (max_new == 0) return RG_OK;
  rg_tok_stream *stream = nullptr;
  if (on_text && rg_b200_tok_stream_new(w->tokenizer, &stream) != RG_TOK_OK) return fail(RG_INVALID_ARGUMENT, "streaming decoder");
  struct StreamGuard {
    rg_tok_stream *s;
    ~StreamGuard() { rg_b200_tok_stream_free(s); }
  } guard{stream};
  std::string piece;
  auto emit = [&](int32_t token) -> int32_t {
    if (!on_text) return RG_OK;
    size_t need = 0;
    piece.resize(64);
    int32_t t = rg_b200_tok_stream_push(stream, (uint32_t)token, &piece[0], piece.size(), &need, &terr);
    if (t == RG_TOK_INVALID_ARGUMENT && need > piece.size()) {  // nothing was consumed: repeat with room
      piece.resize(need);
      t = rg_b200_tok_stream_push(stream, (uint32_t)token, &piece[0], piece.size(), &need, &terr);
    }
    if (t != RG_TOK_OK) return tok_fail(out, t, terr, "streaming decode");
    on_text(user, token, piece.data(), need);
    return RG_OK;
  };
  int32_t token = -1;
  rc = rg_b200_prefill_select(w->session, 0, w->prompt_ids.data(), w->prompt_ids.size(), 0.0f, nullptr, nullptr, &token);
  if (rc) return rc;
  for (size_t step = 0; step < max_new; ++step) {
    w->generated_ids.push_back(token);
    if ((rc = emit(token))) return rc;
    if (token == w->model_cfg.eos_id || token == w->model_cfg.eot_id) {
      if (out) out->stopped = 1;
      break;
    }
    if (step + 1 < max_new) {
      int32_t next = -1;
      if ((rc = rg_b200_decode(w->session, &token, 1, nullptr, &next))) return rc;
      token = next;
    }
  }
  if (on_text) {
    char tail[8];
    size_t need = 0;
    if (rg_b200_tok_stream_finish(stream, tail, sizeof(tail), &need) == RG_TOK_OK && need) on_text(user, -1, tail, need);
  }
  // the decoded text of the whole generation (generation.rs:152)
  std::vector<uint32_t> gen(w->generated_ids.begin(), w->generated_ids.end());
  size_t bytes = 0;
  trc = rg_b200_tokenizer_decode(w->tokenizer, gen.data(), gen.size(), nullptr, 0, &bytes, &terr);
  if (trc != RG_TOK_OK && !(trc == RG_TOK_INVALID_ARGUMENT && bytes > 0)) return tok_fail(out, trc, terr, "decode");
  w->decoded.resize(bytes);
  if (bytes) {
    trc = rg_b200_tokenizer_decode(w->tokenizer, gen.data(), gen.size(), &w->decoded[0], bytes, &bytes, &terr);
    if (trc != RG_TOK_OK) return tok_fail(out, trc, terr, "decode");
  }
  if (out) {
    out->n_generated_ids = w->generated_ids.size();
    out->decoded_bytes = w->decoded.size();
  }
  return RG_OK;
}

void begin_request(rg_workflow *w, rg_prompt_output *out) {
  w->prompt_ids.clear();
  w->generated_ids.clear();
  w->decoded.clear();
  w->rendered.clear();
  if (out) memset(out, 0, sizeof(*out));
}

}  // namespace

extern "C" {

int32_t rg_b200_workflow_open(const uint8_t *bytes, size_t len, const rg_options *options, rg_workflow **out) {
  if (!bytes || !out) return fail(RG_INVALID_ARGUMENT, "null argument");
  rg_gguf *g = nullptr;
  int32_t rc = rg_b200_gguf_open(bytes, len, &g);
  if (rc) return rc;
  struct GgufGuard {
    rg_gguf *g;
    ~GgufGuard() { rg_b200_gguf_close(g); }
  } gg{g};
  auto w = new rg_workflow();
  struct WfGuard {
    rg_workflow *w;
    ~WfGuard() {
      if (w) rg_b200_workflow_close(w);
    }
  } wg{w};
  if ((rc = rg_b200_gguf_llama_config(g, &w->model_cfg))) return rc;  // builds the tokenizer once to validate it
  rg_tok_error terr{};
  int32_t trc = rg_b200_tokenizer_from_gguf(g, &w->tokenizer, &terr);
  if (trc != RG_TOK_OK) return tok_fail(nullptr, trc, terr, "tokenizer");
  rg_b200_tokenizer_config(w->tokenizer, &w->tok_cfg);
  int32_t present = 0;
  trc = rg_b200_chat_template_from_gguf(g, &present, &terr);
  if (trc != RG_TOK_OK) return tok_fail(nullptr, trc, terr, "chat template");
  rg_plan *plan = nullptr;
  if ((rc = rg_b200_plan_from_gguf(g, options, &plan))) return rc;
  rc = rg_b200_session_prepare(plan, &w->session);
  rg_b200_plan_destroy(plan);
  if (rc) return rc;
  w->context = rg_b200_max_context(w->session);
  *out = w;
  wg.w = nullptr;
  return RG_OK;
}

void rg_b200_workflow_close(rg_workflow *w) {
  if (!w) return;
  if (w->session) rg_b200_session_destroy(w->session);
  if (w->tokenizer) rg_b200_tokenizer_free(w->tokenizer);
  delete w;
}

rg_session *rg_b200_workflow_session(rg_workflow *w) { return w ? w->session : nullptr; }
const rg_tokenizer *rg_b200_workflow_tokenizer(const rg_workflow *w) { return w ? w->tokenizer : nullptr; }

int32_t rg_b200_workflow_generate_text(rg_workflow *w, const char *prompt, size_t prompt_len, size_t max_new_tokens,
                                       rg_text_callback on_text, void *user, rg_prompt_output *out) {
  if (!w || (!prompt && prompt_len)) return fail(RG_INVALID_ARGUMENT, "null argument");
  begin_request(w, out);
  return run_request(w, std::string(prompt ? prompt : "", prompt_len), max_new_tokens, on_text, user, out);
}

int32_t rg_b200_workflow_generate_chat(rg_workflow *w, const int32_t *roles, const char *const *contents,
                                       const size_t *content_len, size_t n_messages, size_t max_new_tokens,
                                       rg_text_callback on_text, void *user, rg_prompt_output *out) {
  if (!w || (n_messages && (!roles || !contents || !content_len))) return fail(RG_INVALID_ARGUMENT, "null argument");
  begin_request(w, out);
  rg_tok_error terr{};
  size_t bytes = 0;
  int32_t trc = rg_b200_chat_render(w->tokenizer, roles, contents, content_len, n_messages, 1, nullptr, 0, &bytes, &terr);
  if (trc != RG_TOK_OK && !(trc == RG_TOK_INVALID_ARGUMENT && bytes > 0)) return tok_fail(out, trc, terr, "chat render");
  std::string rendered(bytes, '\0');
  if (bytes) {
    trc = rg_b200_chat_render(w->tokenizer, roles, contents, content_len, n_messages, 1, &rendered[0], bytes, &bytes, &terr);
    if (trc != RG_TOK_OK) return tok_fail(out, trc, terr, "chat render");
  }
  return run_request(w, rendered, max_new_tokens, on_text, user, out);
}

const int32_t *rg_b200_workflow_prompt_ids(const rg_workflow *w) { return w ? w->prompt_ids.data() : nullptr; }
const int32_t *rg_b200_workflow_generated_ids(const rg_workflow *w) { return w ? w->generated_ids.data() : nullptr; }
const char *rg_b200_workflow_decoded(const rg_workflow *w) { return w ? w->decoded.c_str() : nullptr; }
const char *rg_b200_workflow_rendered_prompt(const rg_workflow *w) { return w ? w->rendered.c_str() : nullptr; }

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// LlamaConversation (src/models/transformer/conversation.rs:29-85)
// ---------------------------------------------------------------------------------------------
struct rg_conversation {
  rg_chat_backend be{};
  std::vector<int32_t> roles;
  std::vector<std::string> contents;
  size_t cache_len = 0;
};

namespace {

const size_t CONVERSATION_MESSAGE_BYTES = 1024 * 1024;  // LlamaChatMessage::new (chat.rs:45-55)

int32_t wf_generate_chat(void *ctx, const int32_t *roles, const char *const *contents, const size_t *content_len, size_t n,
                         size_t max_new, rg_text_callback on_text, void *user, rg_prompt_output *out) {
  return rg_b200_workflow_generate_chat(static_cast<rg_workflow *>(ctx), roles, contents, content_len, n, max_new, on_text, user, out);
}
const char *wf_decoded(void *ctx) { return rg_b200_workflow_decoded(static_cast<rg_workflow *>(ctx)); }

}  // namespace

extern "C" {

int32_t rg_b200_conversation_new_with_backend(const rg_chat_backend *backend, rg_conversation **out) {
  if (!backend || !backend->generate_chat || !backend->decoded || !out) return RG_CONVERSATION_INVALID_ARGUMENT;
  auto c = new rg_conversation();
  c->be = *backend;
  *out = c;
  return RG_CONVERSATION_OK;
}

int32_t rg_b200_conversation_new(rg_workflow *w, rg_conversation **out) {
  if (!w) return RG_CONVERSATION_INVALID_ARGUMENT;
  rg_chat_backend be{};
  be.ctx = w;
  be.generate_chat = wf_generate_chat;
  be.decoded = wf_decoded;
  return rg_b200_conversation_new_with_backend(&be, out);
}

void rg_b200_conversation_free(rg_conversation *c) { delete c; }

size_t rg_b200_conversation_history_len(const rg_conversation *c) { return c ? c->roles.size() : 0; }

int32_t rg_b200_conversation_message(const rg_conversation *c, size_t index, int32_t *role, const char **content, size_t *content_len) {
  if (!c || index >= c->roles.size()) return RG_CONVERSATION_INVALID_ARGUMENT;
  if (role) *role = c->roles[index];
  if (content) *content = c->contents[index].c_str();
  if (content_len) *content_len = c->contents[index].size();
  return RG_CONVERSATION_OK;
}

size_t rg_b200_conversation_cache_len(const rg_conversation *c) { return c ? c->cache_len : 0; }

void rg_b200_conversation_reset(rg_conversation *c) {
  if (!c) return;
  c->roles.clear();
  c->contents.clear();
  c->cache_len = 0;
}

int32_t rg_b200_conversation_send(rg_conversation *c, const char *content, size_t content_len, size_t max_new_tokens,
                                  rg_text_callback on_text, void *user, rg_prompt_output *out, int32_t *detail) {
  if (detail) *detail = 0;
  if (!c || (content_len && !content)) return RG_CONVERSATION_INVALID_ARGUMENT;
  if (content_len > CONVERSATION_MESSAGE_BYTES) {
    if (detail) *detail = RG_TOK_MESSAGE_TOO_LONG;
    return RG_CONVERSATION_CHAT;
  }
  if (content_len == 0) return RG_CONVERSATION_EMPTY_INPUT;
  // the staged transcript: committed history + the new user message
  const size_t n = c->roles.size() + 1;
  std::vector<int32_t> roles(c->roles);
  roles.push_back(RG_CHAT_USER);
  std::vector<const char *> ptrs(n);
  std::vector<size_t> lens(n);
  for (size_t i = 0; i + 1 < n; ++i) {
    ptrs[i] = c->contents[i].data();
    lens[i] = c->contents[i].size();
  }
  ptrs[n - 1] = content;
  lens[n - 1] = content_len;
  rg_prompt_output local{};
  rg_prompt_output *o = out ? out : &local;
  const int32_t rc = c->be.generate_chat(c->be.ctx, roles.data(), ptrs.data(), lens.data(), n, max_new_tokens, on_text, user, o);
  if (rc != RG_OK) {
    if (o->tokenizer_status) {
      if (detail) *detail = o->tokenizer_status;
      return RG_CONVERSATION_CHAT;
    }
    if (detail) *detail = rc;
    return RG_CONVERSATION_GENERATION;
  }
  if (o->decoded_bytes > CONVERSATION_MESSAGE_BYTES) {  // the assistant message is bounded like any other
    if (detail) *detail = RG_TOK_MESSAGE_TOO_LONG;
    return RG_CONVERSATION_CHAT;
  }
  const char *text = c->be.decoded(c->be.ctx);
  std::string assistant(text ? text : "", text ? o->decoded_bytes : 0);
  c->roles.push_back(RG_CHAT_USER);
  c->contents.emplace_back(content, content_len);
  c->roles.push_back(RG_CHAT_ASSISTANT);
  c->contents.push_back(std::move(assistant));
  // a generation of no tokens returns before any cache work (generation.rs:127-134)
  if (o->n_generated_ids > 0) c->cache_len = o->n_prompt_ids + o->n_generated_ids - 1;
  return RG_CONVERSATION_OK;
}

}  // extern "C"

