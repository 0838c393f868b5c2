/* Host-side tokenizer of the GGUF Llama path: the C ABI a binding uses in place of rustgrad's
 * `SimpleTokenizer` (src/tokenizer/mod.rs).  Same contract: GPT-2 byte alphabet for normal
 * tokens (mod.rs:505-528), ordered special tokens that split the text first (mod.rs:379-391),
 * the Unicode word pre-tokeniser of mod.rs:24-48,393-424, rank-ordered greedy merges where the
 * rank of a merge is the id of the merged token (mod.rs:426-456), byte-concatenating decode with
 * U+FFFD for malformed UTF-8 (mod.rs:340-346) and an incremental decoder that holds back an
 * incomplete trailing sequence (mod.rs:459-470,530-566).  No device work: nothing here touches
 * a GPU, and nothing here is part of a timed region.
 *
 * Strings cross the boundary as (pointer, byte length) pairs of UTF-8; no terminator is assumed.
 */
#ifndef RG_B200_TOKENIZER_H
#define RG_B200_TOKENIZER_H

#include <stddef.h>
#include <stdint.h>

#include "rg_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* TokenizerErrorKind (src/tokenizer/mod.rs:103-139); 0 is success. */
typedef enum rg_tok_status {
  RG_TOK_OK = 0,
  RG_TOK_INVALID_ARGUMENT = 1,            /* null pointer, output capacity too small (needed size is still reported) */
  RG_TOK_UNSUPPORTED_PRESET = 2,          /* detail.text = the preset string */
  RG_TOK_MISSING_METADATA = 3,            /* detail.text = the key */
  RG_TOK_MALFORMED_METADATA = 4,          /* detail.text = the key, detail.value = GGUF type id found */
  RG_TOK_METADATA_LENGTH_MISMATCH = 5,    /* detail.value = tokens, detail.value2 = token types */
  RG_TOK_TOKEN_ID_OUT_OF_RANGE = 6,       /* a metadata id that does not fit 32 bits: detail.text = key, detail.value */
  RG_TOK_CONFIGURED_ID_OUT_OF_RANGE = 7,  /* detail.text = key, detail.value = id, detail.value2 = token count */
  RG_TOK_INVALID_NORMAL_TOKEN_CHARACTER = 8, /* detail.value = token id, detail.value2 = code point */
  RG_TOK_EMPTY_SPECIAL_TOKEN = 9,         /* detail.value = token id */
  RG_TOK_TOKEN_NOT_FOUND = 10,            /* detail.text = the bytes no token covers */
  RG_TOK_UNKNOWN_TOKEN_ID = 11,           /* detail.value = the id */
  /* LlamaChatError (src/models/transformer/chat.rs:163-174) */
  RG_TOK_TEMPLATE_TOO_LONG = 12,          /* detail.value = bytes, detail.value2 = maximum */
  RG_TOK_UNSUPPORTED_JINJA = 13,
  RG_TOK_UNSUPPORTED_TEMPLATE = 14,
  RG_TOK_CHAT_UNSUPPORTED_PRESET = 15,    /* detail.value = the tokenizer's preset */
  RG_TOK_MESSAGE_TOO_LONG = 16,           /* detail.value = bytes, detail.value2 = maximum */
  RG_TOK_CHAT_TOO_LONG = 17,              /* detail.value = bytes, detail.value2 = maximum */
  RG_TOK_CHAT_OVERFLOW = 18
} rg_tok_status;

/* TokenizerPreset (mod.rs:50-62): the `tokenizer.ggml.pre` values accepted, aliases normalised. */
typedef enum rg_tok_preset {
  RG_TOK_PRESET_LLAMA3 = 0,
  RG_TOK_PRESET_LLAMA_V3 = 1,
  RG_TOK_PRESET_LLAMA_BPE = 2,
  RG_TOK_PRESET_QWEN2 = 3, /* "qwen2", "qwen35", "qwen35moe" */
  RG_TOK_PRESET_OLMO = 4,
  RG_TOK_PRESET_KIMI_K2 = 5,
  RG_TOK_PRESET_TEKKEN = 6,
  RG_TOK_PRESET_GLM4 = 7
} rg_tok_preset;

/* TokenizerConfig (mod.rs:82-101).  has_bos / has_eot play the role of Option. */
typedef struct rg_tok_config {
  int32_t preset;
  int32_t has_bos;
  uint32_t bos_id;
  uint32_t eos_id;
  int32_t has_eot;
  uint32_t eot_id;
} rg_tok_config;

/* What went wrong, in the fields the status names.  text is truncated to its capacity. */
typedef struct rg_tok_error {
  int32_t status;
  uint64_t value;
  uint64_t value2;
  size_t text_len;
  char text[128];
} rg_tok_error;

typedef struct rg_tokenizer rg_tokenizer;
typedef struct rg_tok_stream rg_tok_stream;

/* SimpleTokenizer::new (mod.rs:176-231).  Token strings are in the byte alphabet for normal
 * tokens and literal text for special tokens; a repeated string keeps its first position among the
 * specials and its last id.  cfg may be NULL (defaults of mod.rs:91-100).  err may be NULL. */
int32_t rg_b200_tokenizer_new(const char *const *normal, const size_t *normal_len, const uint32_t *normal_ids,
                              size_t n_normal, const char *const *special, const size_t *special_len,
                              const uint32_t *special_ids, size_t n_special, const rg_tok_config *cfg,
                              rg_tokenizer **out, rg_tok_error *err);
/* SimpleTokenizer::from_gguf (mod.rs:233-308): token type 1 is normal, every other type special;
 * bos only when `tokenizer.ggml.add_bos_token` is absent or true; eot falls back to the last
 * special named <|im_end|>; configured ids must index the vocabulary. */
int32_t rg_b200_tokenizer_from_gguf(const rg_gguf *gguf, rg_tokenizer **out, rg_tok_error *err);
void rg_b200_tokenizer_free(rg_tokenizer *t);

void rg_b200_tokenizer_config(const rg_tokenizer *t, rg_tok_config *out);
/* is_end (mod.rs:356-358): the eos id or the eot id. */
int32_t rg_b200_tokenizer_is_end(const rg_tokenizer *t, uint32_t token_id);
/* TokenizerPreset::parse (mod.rs:64-79); RG_TOK_UNSUPPORTED_PRESET otherwise. */
int32_t rg_b200_tokenizer_parse_preset(const char *value, size_t len, int32_t *preset);

/* encode (mod.rs:328-338).  *n_ids receives the number of ids the text encodes to even when it
 * exceeds `capacity` (then nothing past capacity is written and the status is
 * RG_TOK_INVALID_ARGUMENT); call with capacity 0 to size the buffer. */
int32_t rg_b200_tokenizer_encode(const rg_tokenizer *t, const char *text, size_t len, uint32_t *ids, size_t capacity,
                                 size_t *n_ids, rg_tok_error *err);
/* decode (mod.rs:340-346); same sizing rule, in bytes of UTF-8. */
int32_t rg_b200_tokenizer_decode(const rg_tokenizer *t, const uint32_t *ids, size_t n_ids, char *text, size_t capacity,
                                 size_t *n_bytes, rg_tok_error *err);

/* StreamingDecoder (mod.rs:459-470): push returns the text completed by this token, keeping only
 * an incomplete trailing UTF-8 sequence; finish flushes it as U+FFFD and later pushes return
 * nothing.  A push or finish whose text does not fit `capacity` consumes nothing: *n_bytes holds
 * the size needed and the call can be repeated.  The stream borrows the tokenizer, which must
 * outlive it. */
int32_t rg_b200_tok_stream_new(const rg_tokenizer *t, rg_tok_stream **out);
int32_t rg_b200_tok_stream_push(rg_tok_stream *s, uint32_t token_id, char *text, size_t capacity, size_t *n_bytes,
                                rg_tok_error *err);
int32_t rg_b200_tok_stream_finish(rg_tok_stream *s, char *text, size_t capacity, size_t *n_bytes);
void rg_b200_tok_stream_free(rg_tok_stream *s);

/* ---- Llama chat prompt (src/models/transformer/chat.rs) ---- */
typedef enum rg_chat_role { RG_CHAT_SYSTEM = 0, RG_CHAT_USER = 1, RG_CHAT_ASSISTANT = 2 } rg_chat_role;

/* LlamaChatTemplate::from_gguf (chat.rs:69-97): `tokenizer.chat_template` may be absent
 * (*metadata_present = 0) or exactly the one supported Llama template (1); anything else is
 * refused, never approximated: RG_TOK_UNSUPPORTED_JINJA when it holds template syntax,
 * RG_TOK_UNSUPPORTED_TEMPLATE otherwise, RG_TOK_TEMPLATE_TOO_LONG beyond 64 KiB,
 * RG_TOK_MALFORMED_METADATA when the value is not a string. */
int32_t rg_b200_chat_template_from_gguf(const rg_gguf *gguf, int32_t *metadata_present, rg_tok_error *err);
/* The supported template text (chat.rs:16), NUL-terminated, owned by the library. */
const char *rg_b200_chat_template_text(void);
/* LlamaChatTemplate::render (chat.rs:104-160): bos text, then for each message
 * "<|start_header_id|>" role "<|end_header_id|>\n\n" content eos text, then the assistant header
 * when add_generation_prompt is set.  Only the three Llama presets; a message may hold at most
 * 1 MiB and the prompt 4 MiB.  Sizing rule as for decode. */
int32_t rg_b200_chat_render(const rg_tokenizer *t, const int32_t *roles, const char *const *contents,
                            const size_t *content_len, size_t n_messages, int32_t add_generation_prompt, char *text,
                            size_t capacity, size_t *n_bytes, rg_tok_error *err);

#ifdef __cplusplus
}
#endif
#endif
