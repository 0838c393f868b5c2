#include "gguf.h"

#include <math.h>
#include <string.h>

#include <algorithm>
#include <set>

namespace rg {

int block_elements(int32_t t) {
  switch (t) {
    case RG_TYPE_F32:
    case RG_TYPE_F16: return 1;
    case RG_TYPE_Q4_0:
    case RG_TYPE_Q8_0: return 32;
    case RG_TYPE_Q4_K:
    case RG_TYPE_Q6_K: return 256;
    default: return 0;
  }
}
int block_bytes(int32_t t) {
  switch (t) {
    case RG_TYPE_F32: return 4;
    case RG_TYPE_F16: return 2;
    case RG_TYPE_Q4_0: return 18;
    case RG_TYPE_Q8_0: return 34;
    case RG_TYPE_Q4_K: return 144;
    case RG_TYPE_Q6_K: return 210;
    default: return 0;
  }
}

namespace {

// Limits of GgufLimits::default (src/gguf/mod.rs:56-66).
constexpr uint64_t MAX_METADATA = 131072, MAX_TENSORS = 1000000, MAX_STRING = 64ull << 20;
constexpr uint64_t MAX_ARRAY = 16ull << 20, MAX_VALUES = 32ull << 20, MAX_DEPTH = 8;

// Every ggml type id the container format knows: (block elements, block bytes).  Types outside
// {F32,F16,Q4_0,Q8_0} parse (their byte ranges are needed for the layout checks) but cannot be bound.
bool known_type_geometry(uint32_t raw, uint64_t *be, uint64_t *bb) {
  switch (raw) {
    case 0: *be = 1; *bb = 4; return true;
    case 1: *be = 1; *bb = 2; return true;
    case 2: *be = 32; *bb = 18; return true;
    case 3: *be = 32; *bb = 20; return true;
    case 6: *be = 32; *bb = 22; return true;
    case 7: *be = 32; *bb = 24; return true;
    case 8: *be = 32; *bb = 34; return true;
    case 12: *be = 256; *bb = 144; return true;
    case 13: *be = 256; *bb = 176; return true;
    case 14: *be = 256; *bb = 210; return true;
    case 24: *be = 1; *bb = 1; return true;
    case 25: *be = 1; *bb = 2; return true;
    case 26: *be = 1; *bb = 4; return true;
    case 27: *be = 1; *bb = 8; return true;
    case 28: *be = 1; *bb = 8; return true;
    case 30: *be = 1; *bb = 2; return true;
    default: return false;
  }
}

struct Reader {
  const uint8_t *b;
  size_t len, pos = 0;
  uint64_t values = 0;
  std::string *err;
  bool fail(const char *why) {
    if (err && err->empty()) *err = std::string(why) + " at byte " + std::to_string(pos);
    return false;
  }
  bool take(size_t n, const uint8_t **p) {
    if (n > len - pos) return fail("truncated");
    *p = b + pos;
    pos += n;
    return true;
  }
  template <typename T>
  bool num(T *v) {
    const uint8_t *p;
    if (!take(sizeof(T), &p)) return false;
    memcpy(v, p, sizeof(T));
    return true;
  }
  bool count(uint64_t limit, uint64_t *v, const char *field) {
    if (!num(v)) return false;
    if (*v > limit) return fail(field);
    return true;
  }
  bool str(uint64_t limit, std::string *s, const char *field) {
    uint64_t n;
    if (!count(limit, &n, field)) return false;
    const uint8_t *p;
    if (!take((size_t)n, &p)) return false;
    // UTF-8 well-formedness (src/gguf/reader.rs:378-386)
    for (size_t i = 0; i < n;) {
      uint8_t c = p[i];
      int extra = c < 0x80 ? 0 : (c >> 5) == 6 ? 1 : (c >> 4) == 14 ? 2 : (c >> 3) == 30 ? 3 : -1;
      if (extra < 0 || i + (size_t)extra >= n) return fail("invalid utf-8");
      for (int j = 1; j <= extra; ++j)
        if ((p[i + j] & 0xC0) != 0x80) return fail("invalid utf-8");
      i += 1 + (size_t)extra;
    }
    s->assign(reinterpret_cast<const char *>(p), (size_t)n);
    return true;
  }
  bool value(uint32_t type, GgufValue *v, uint64_t depth) {
    if (++values > MAX_VALUES) return fail("metadata value limit");
    v->type = type;
    switch (type) {
      case 0: { uint8_t x; if (!num(&x)) return false; v->u = x; return true; }
      case 1: { int8_t x; if (!num(&x)) return false; v->u = (uint64_t)(int64_t)x; v->f = x; return true; }
      case 2: { uint16_t x; if (!num(&x)) return false; v->u = x; return true; }
      case 3: { int16_t x; if (!num(&x)) return false; v->u = (uint64_t)(int64_t)x; return true; }
      case 4: { uint32_t x; if (!num(&x)) return false; v->u = x; return true; }
      case 5: { int32_t x; if (!num(&x)) return false; v->u = (uint64_t)(int64_t)x; return true; }
      case 6: { float x; if (!num(&x)) return false; v->f = x; return true; }
      case 7: { uint8_t x; if (!num(&x)) return false; if (x > 1) return fail("invalid bool"); v->u = x; return true; }
      case 8: return str(MAX_STRING, &v->s, "string length");
      case 9: {
        if (depth >= MAX_DEPTH) return fail("array depth");
        if (!num(&v->elem_type)) return false;
        if (v->elem_type > 12) return fail("unknown metadata type");
        if (!count(MAX_ARRAY, &v->count, "array length")) return false;
        v->array_offset = pos;
        for (uint64_t i = 0; i < v->count; ++i) {
          GgufValue item;
          if (!value(v->elem_type, &item, depth + 1)) return false;
        }
        return true;
      }
      case 10: { uint64_t x; if (!num(&x)) return false; v->u = x; return true; }
      case 11: { int64_t x; if (!num(&x)) return false; v->u = (uint64_t)x; return true; }
      case 12: { double x; if (!num(&x)) return false; v->f = x; return true; }
      default: return fail("unknown metadata type");
    }
  }
};

bool valid_key(const std::string &key) {
  if (key.empty()) return false;
  size_t start = 0;
  while (true) {
    size_t dot = key.find('.', start);
    std::string seg = key.substr(start, dot == std::string::npos ? std::string::npos : dot - start);
    if (seg.empty() || seg.front() == '_' || seg.back() == '_') return false;
    for (unsigned char c : seg)
      if (!((c >= 'a' && c <= 'z') || (c >= '0' && c <= '9') || c == '_')) return false;
    if (dot == std::string::npos) return true;
    start = dot + 1;
  }
}

}  // namespace

int32_t gguf_parse(const uint8_t *bytes, size_t len, Gguf *out, std::string *err) {
  if (!bytes || !out) return RG_INVALID_ARGUMENT;
  Reader r{bytes, len, 0, 0, err};
  auto bad = [&](const char *why) {
    r.fail(why);
    return RG_MALFORMED_GGUF;
  };
  const uint8_t *magic;
  if (!r.take(4, &magic)) return RG_MALFORMED_GGUF;
  if (memcmp(magic, "GGUF", 4)) return bad("invalid magic");
  uint32_t version;
  if (!r.num(&version)) return RG_MALFORMED_GGUF;
  if (version != 2 && version != 3) return bad("unsupported version");
  uint64_t n_tensors, n_kv;
  if (!r.count(MAX_TENSORS, &n_tensors, "tensor count") || !r.count(MAX_METADATA, &n_kv, "metadata count"))
    return RG_MALFORMED_GGUF;
  out->bytes = bytes;
  out->len = len;
  out->version = version;
  out->metadata.clear();
  out->tensors.clear();
  out->by_name.clear();
  for (uint64_t i = 0; i < n_kv; ++i) {
    std::string key;
    if (!r.str(std::min<uint64_t>(MAX_STRING, 65535), &key, "metadata key")) return RG_MALFORMED_GGUF;
    if (!valid_key(key)) return bad("invalid metadata key");
    if (out->metadata.count(key)) return bad("duplicate metadata key");
    uint32_t type;
    if (!r.num(&type)) return RG_MALFORMED_GGUF;
    GgufValue v;
    if (!r.value(type, &v, 0)) return RG_MALFORMED_GGUF;
    out->metadata.emplace(key, std::move(v));
  }
  size_t alignment = 32;
  auto al = out->metadata.find("general.alignment");
  if (al != out->metadata.end()) {
    if (al->second.type != 4) return bad("general.alignment must be u32");
    alignment = (size_t)al->second.u;
  }
  if (alignment == 0 || alignment % 8) return bad("invalid alignment");
  out->alignment = alignment;

  struct Pending {
    GgufTensorInfo info;
    uint64_t relative;
  };
  std::vector<Pending> pending;
  pending.reserve((size_t)n_tensors);
  std::set<std::string> names;
  for (uint64_t i = 0; i < n_tensors; ++i) {
    Pending p;
    if (!r.str(64, &p.info.name, "tensor name")) return RG_MALFORMED_GGUF;
    if (p.info.name.empty()) return bad("empty tensor name");
    if (!names.insert(p.info.name).second) return bad("duplicate tensor");
    uint32_t rank;
    if (!r.num(&rank)) return RG_MALFORMED_GGUF;
    if (rank == 0 || rank > 4) return bad("invalid rank");
    std::vector<uint64_t> dims(rank);
    uint64_t elements = 1;
    for (uint32_t a = 0; a < rank; ++a) {
      if (!r.num(&dims[a])) return RG_MALFORMED_GGUF;
      if (dims[a] == 0) return bad("invalid dimension");
      if (elements > UINT64_MAX / dims[a]) return bad("shape overflow");
      elements *= dims[a];
    }
    uint32_t raw_type;
    if (!r.num(&raw_type)) return RG_MALFORMED_GGUF;
    uint64_t be, bb;
    if (!known_type_geometry(raw_type, &be, &bb)) return bad("unknown tensor type");
    if (!r.num(&p.relative)) return RG_MALFORMED_GGUF;
    if (elements % be) return bad("element count is not a multiple of the block size");
    p.info.ggml_type = (int32_t)raw_type;
    p.info.elements = elements;
    p.info.nbytes = (size_t)(elements / be * bb);
    p.info.shape.assign(dims.rbegin(), dims.rend());
    pending.push_back(std::move(p));
  }
  size_t data_offset = r.pos;
  if (n_tensors) data_offset += (alignment - r.pos % alignment) % alignment;
  if (data_offset > len) return bad("truncated");
  for (size_t i = r.pos; i < data_offset; ++i)
    if (bytes[i]) return bad("non-zero header padding");
  for (auto &p : pending) {
    if (p.relative % alignment) return bad("misaligned tensor offset");
    if (p.relative > len - data_offset || p.info.nbytes > len - data_offset - p.relative) return bad("tensor range out of bounds");
    p.info.offset = data_offset + (size_t)p.relative;
    out->by_name[p.info.name] = out->tensors.size();
    out->tensors.push_back(p.info);
  }
  std::vector<const GgufTensorInfo *> order;
  for (auto &t : out->tensors) order.push_back(&t);
  std::sort(order.begin(), order.end(), [](auto *a, auto *b) { return a->offset < b->offset; });
  size_t cursor = data_offset;
  for (auto *t : order) {
    if (t->offset < cursor) return bad("overlapping tensors");
    for (size_t i = cursor; i < t->offset; ++i)
      if (bytes[i]) return bad("non-zero tensor padding");
    cursor = t->offset + t->nbytes;
  }
  size_t padded_end = cursor;
  if (!order.empty()) padded_end = data_offset + ((cursor - data_offset) + alignment - 1) / alignment * alignment;
  if (len > padded_end) return bad("trailing data");
  for (size_t i = cursor; i < len; ++i)
    if (bytes[i]) return bad("non-zero trailing padding");
  return RG_OK;
}

namespace {
const GgufValue *find(const Gguf &g, const std::string &key) {
  auto it = g.metadata.find(key);
  return it == g.metadata.end() ? nullptr : &it->second;
}
bool is_int(const GgufValue &v) { return v.type <= 5 || v.type == 10 || v.type == 11; }
int32_t req_usize(const Gguf &g, const std::string &key, int64_t *out, std::string *err) {
  const GgufValue *v = find(g, key);
  if (!v) {
    *err = "missing metadata " + key;
    return RG_MISSING_METADATA;
  }
  if (!is_int(*v) || (int64_t)v->u < 0 || v->u > 0x7fffffffull) {
    *err = "metadata out of range: " + key;
    return RG_INVALID_ARGUMENT;
  }
  *out = (int64_t)v->u;
  return RG_OK;
}
int32_t req_float(const Gguf &g, const std::string &key, double *out, std::string *err) {
  const GgufValue *v = find(g, key);
  if (!v) {
    *err = "missing metadata " + key;
    return RG_MISSING_METADATA;
  }
  if (v->type != 6 && v->type != 12) {
    *err = "metadata is not a float: " + key;
    return RG_INVALID_ARGUMENT;
  }
  *out = v->f;
  return RG_OK;
}
bool nonzero(const Gguf &g, const std::string &key) {
  const GgufValue *v = find(g, key);
  return v && is_int(*v) && v->u != 0;
}
}  // namespace

int32_t gguf_llama_config(const Gguf &g, rg_llama_config *out, std::string *err) {
  std::string local;
  if (!err) err = &local;
  const GgufValue *arch = find(g, "general.architecture");
  if (!arch || arch->type != 8) {
    *err = "missing metadata general.architecture";
    return RG_MISSING_METADATA;
  }
  if (arch->s != "llama") {
    *err = "unsupported architecture " + arch->s;
    return RG_UNSUPPORTED_VARIANT;
  }
  // the tokenizer is built first and supplies the stop ids (model.rs:133; mod.rs:284-296)
  int32_t stop_eos = 0, stop_eot = -1;
  int32_t rc;
  if ((rc = gguf_tokenizer_stop_ids(g, &stop_eos, &stop_eot, err))) return rc;
  const GgufValue *tokens = find(g, "tokenizer.ggml.tokens");
  if (!tokens || tokens->type != 9 || tokens->elem_type != 8) {
    *err = "missing metadata tokenizer.ggml.tokens";
    return RG_MISSING_METADATA;
  }
  int64_t layers, d, ffn, heads, kv, ctx;
  const std::string p = "llama.";
  if ((rc = req_usize(g, p + "block_count", &layers, err))) return rc;
  if ((rc = req_usize(g, p + "embedding_length", &d, err))) return rc;
  if ((rc = req_usize(g, p + "feed_forward_length", &ffn, err))) return rc;
  if ((rc = req_usize(g, p + "attention.head_count", &heads, err))) return rc;
  if ((rc = req_usize(g, p + "attention.head_count_kv", &kv, err))) return rc;
  if ((rc = req_usize(g, p + "context_length", &ctx, err))) return rc;
  if (heads == 0 || d % heads) {
    *err = "embedding_length is not a multiple of head_count";
    return RG_INVALID_ARGUMENT;
  }
  int64_t hd = d / heads, vd, rope;
  if (find(g, p + "attention.key_length") && (rc = req_usize(g, p + "attention.key_length", &hd, err))) return rc;
  vd = hd;
  if (find(g, p + "attention.value_length") && (rc = req_usize(g, p + "attention.value_length", &vd, err))) return rc;
  if (vd != hd) {
    *err = "value head width differs from key head width";
    return RG_UNSUPPORTED_VARIANT;
  }
  rope = hd;
  if (find(g, p + "rope.dimension_count") && (rc = req_usize(g, p + "rope.dimension_count", &rope, err))) return rc;
  if (rope == 0 || rope > hd || rope % 2) {
    *err = "invalid partial rotary dimensions";
    return RG_UNSUPPORTED_VARIANT;
  }
  if (rope != hd && hd % 2) {
    *err = "partial rotary dimensions with odd key head width";
    return RG_UNSUPPORTED_VARIANT;
  }
  for (auto &kvp : g.metadata)
    if (kvp.first.rfind(p + "rope.scaling.", 0) == 0 || kvp.first == p + "rope.freq_scale") {
      *err = "RoPE frequency scaling metadata";
      return RG_UNSUPPORTED_VARIANT;
    }
  if (nonzero(g, p + "nextn_predict_layers") || nonzero(g, p + "expert_count") || nonzero(g, p + "attention.kv_lora_rank") ||
      nonzero(g, p + "attention.q_lora_rank")) {
    *err = "experts, MLA, LoRA or next-token layers";
    return RG_UNSUPPORTED_VARIANT;
  }
  double eps, theta;
  if ((rc = req_float(g, p + "attention.layer_norm_rms_epsilon", &eps, err))) return rc;
  if ((rc = req_float(g, p + "rope.freq_base", &theta, err))) return rc;
  if (!isfinite(eps) || eps < 0 || !isfinite(theta) || theta <= 0 || layers == 0 || ctx == 0 || kv == 0 || heads % kv) {
    *err = "invalid configuration value";
    return RG_INVALID_ARGUMENT;
  }
  // q/k normalisation and projection biases: complete families only, shapes decide the kind (model.rs:253-282)
  auto tensor_dims = [&](const char *name) -> const std::vector<uint64_t> * {
    auto it = g.by_name.find(name);
    return it == g.by_name.end() ? nullptr : &g.tensors[it->second].shape;
  };
  const uint64_t qw = (uint64_t)heads * (uint64_t)hd, kw = (uint64_t)kv * (uint64_t)hd;
  const std::vector<uint64_t> *qn = tensor_dims("blk.0.attn_q_norm.weight"), *kn = tensor_dims("blk.0.attn_k_norm.weight");
  int32_t qk_norm = 0;
  if (qn || kn) {
    auto is1 = [](const std::vector<uint64_t> *v, uint64_t n) { return v && v->size() == 1 && (*v)[0] == n; };
    if (is1(qn, (uint64_t)hd) && is1(kn, (uint64_t)hd)) qk_norm = 1;
    else if (qw == kw && is1(qn, qw) && is1(kn, kw)) qk_norm = 2;
    else {
      *err = "partial or incompatible q/k normalization";
      return RG_UNSUPPORTED_VARIANT;
    }
  }
  const bool qb = tensor_dims("blk.0.attn_q.bias"), kb = tensor_dims("blk.0.attn_k.bias"), vb = tensor_dims("blk.0.attn_v.bias");
  if (qb != kb || qb != vb) {
    *err = "partial q/k/v projection bias family";
    return RG_UNSUPPORTED_VARIANT;
  }
  out->rope_dim = rope == hd ? 0 : (int32_t)rope;
  out->qk_norm = qk_norm;
  out->qkv_bias = qb ? 1 : 0;
  out->n_layers = (int32_t)layers;
  out->d_model = (int32_t)d;
  out->n_heads = (int32_t)heads;
  out->n_kv_heads = (int32_t)kv;
  out->head_dim = (int32_t)hd;
  out->ffn_dim = (int32_t)ffn;
  out->vocab = (int32_t)tokens->count;
  out->max_context = (int32_t)ctx;
  out->norm_eps = (float)eps;
  out->rope_theta = theta;
  out->eos_id = stop_eos;
  out->eot_id = stop_eot;
  return RG_OK;
}

}  // namespace rg
