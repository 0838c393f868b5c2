// Bounded GGUF v2/v3 container reader (host only).  Same acceptance rules as rustgrad's
// reader::parse (src/gguf/reader.rs:8-301) and GgmlType::byte_len (src/gguf/tensor.rs:222-263);
// rejections surface as RG_MALFORMED_GGUF / RG_UNSUPPORTED_TYPE with a message.
#pragma once

#include <stdint.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/rg_b200.h"

namespace rg {

struct GgufValue {
  uint32_t type = 0;        // GGUF metadata type id (0..12)
  uint64_t u = 0;           // integer / bool payload
  double f = 0.0;           // float payload
  std::string s;            // string payload
  uint32_t elem_type = 0;   // arrays
  uint64_t count = 0;       // arrays
  size_t array_offset = 0;  // byte offset of the first array item
};

struct GgufTensorInfo {
  std::string name;
  int32_t ggml_type = 0;
  std::vector<uint64_t> shape;  // logical, outermost first
  uint64_t elements = 0;
  size_t offset = 0;  // absolute byte offset in the file
  size_t nbytes = 0;
};

struct Gguf {
  const uint8_t *bytes = nullptr;
  size_t len = 0;
  uint32_t version = 0;
  size_t alignment = 32;
  std::map<std::string, GgufValue> metadata;
  std::vector<GgufTensorInfo> tensors;
  std::map<std::string, size_t> by_name;
};

// Returns RG_OK or a typed status; `err` receives the reason.
int32_t gguf_parse(const uint8_t *bytes, size_t len, Gguf *out, std::string *err);
// LlamaModelConfig::from_gguf (src/models/transformer/model.rs:126-298).
int32_t gguf_llama_config(const Gguf &g, rg_llama_config *out, std::string *err);

// Stop ids as the reference's tokenizer derives them from the same file (tokenizer.cc).
int32_t gguf_tokenizer_stop_ids(const Gguf &g, int32_t *eos, int32_t *eot, std::string *why);

// (block elements, block bytes) of a ggml type on this path; 0 when unsupported.
int block_elements(int32_t ggml_type);
int block_bytes(int32_t ggml_type);

}  // namespace rg

// The handle of rg_b200_gguf_open.
struct rg_gguf {
  rg::Gguf g;
};
