// Host-side tokenizer behind include/rg_b200_tokenizer.h: the `SimpleTokenizer` contract of
// src/tokenizer/mod.rs restated without a regex engine.  The two patterns of mod.rs:32-44 are
// matched by hand with the leftmost-first, greedy, backtracking meaning they have there; the
// character classes come from generated range tables (unicode_tables.inc).
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../../include/rg_b200_tokenizer.h"
#include "gguf.h"

namespace {

#include "unicode_tables.inc"

bool in_ranges(const uint32_t (*table)[2], int count, uint32_t cp) {
  int lo = 0, hi = count - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    if (cp < table[mid][0])
      hi = mid - 1;
    else if (cp > table[mid][1])
      lo = mid + 1;
    else
      return true;
  }
  return false;
}
bool is_letter(uint32_t cp) { return in_ranges(UNI_LETTER, UNI_LETTER_COUNT, cp); }
bool is_number(uint32_t cp) { return in_ranges(UNI_NUMBER, UNI_NUMBER_COUNT, cp); }
// the whitespace class of mod.rs:33,42: \t \n \x0B \x0C \r U+0085 and the separators
bool is_space(uint32_t cp) {
  return (cp >= 0x09 && cp <= 0x0D) || cp == 0x85 || in_ranges(UNI_SEPARATOR, UNI_SEPARATOR_COUNT, cp);
}
bool is_newline(uint32_t cp) { return cp == '\r' || cp == '\n'; }

// One code point of valid UTF-8 (the caller validated the text).
struct Cp {
  uint32_t cp;
  int len;
};
Cp cp_at(const unsigned char *p, size_t n) {
  if (n == 0) return {0, 0};
  const unsigned char b = p[0];
  if (b < 0x80) return {b, 1};
  if (b < 0xE0 && n >= 2) return {(uint32_t)(b & 0x1F) << 6 | (p[1] & 0x3Fu), 2};
  if (b < 0xF0 && n >= 3) return {(uint32_t)(b & 0x0F) << 12 | (uint32_t)(p[1] & 0x3F) << 6 | (p[2] & 0x3Fu), 3};
  if (n >= 4)
    return {(uint32_t)(b & 0x07) << 18 | (uint32_t)(p[1] & 0x3F) << 12 | (uint32_t)(p[2] & 0x3F) << 6 | (p[3] & 0x3Fu), 4};
  return {0xFFFD, (int)n};
}

// Length of the valid UTF-8 prefix of [p, p+n) and what stops it, with the meaning of
// core::str::from_utf8's error: error_len = bytes of the ill-formed sequence (1..3), or 0 when
// the input merely ends inside a sequence.
struct Utf8Scan {
  size_t valid_up_to;
  bool ok;
  int error_len;
};
Utf8Scan scan_utf8(const unsigned char *p, size_t n) {
  size_t i = 0;
  while (i < n) {
    const unsigned char b = p[i];
    if (b < 0x80) {
      ++i;
      continue;
    }
    int need;
    unsigned char lo = 0x80, hi = 0xBF;
    if (b >= 0xC2 && b <= 0xDF) {
      need = 1;
    } else if (b >= 0xE0 && b <= 0xEF) {
      need = 2;
      if (b == 0xE0) lo = 0xA0;
      if (b == 0xED) hi = 0x9F;
    } else if (b >= 0xF0 && b <= 0xF4) {
      need = 3;
      if (b == 0xF0) lo = 0x90;
      if (b == 0xF4) hi = 0x8F;
    } else {
      return {i, false, 1};
    }
    for (int j = 1; j <= need; ++j) {
      if (i + (size_t)j >= n) return {i, false, 0};
      const unsigned char c = p[i + (size_t)j];
      const unsigned char l = j == 1 ? lo : 0x80, h = j == 1 ? hi : 0xBF;
      if (c < l || c > h) return {i, false, j};
    }
    i += (size_t)need + 1;
  }
  return {n, true, 0};
}

void push_replacement(std::string *out) { out->append("\xEF\xBF\xBD"); }

// drain_utf8 (mod.rs:530-566): move the decodable prefix of `pending` to the result; an
// incomplete tail stays unless this is the final chunk.
std::string drain_utf8(std::string *pending, bool final_chunk) {
  std::string out;
  size_t consumed = 0;
  const unsigned char *p = reinterpret_cast<const unsigned char *>(pending->data());
  while (consumed < pending->size()) {
    const Utf8Scan s = scan_utf8(p + consumed, pending->size() - consumed);
    out.append(pending->data() + consumed, s.valid_up_to);
    if (s.ok) {
      consumed = pending->size();
      break;
    }
    const size_t valid_end = consumed + s.valid_up_to;
    if (s.error_len > 0) {
      push_replacement(&out);
      consumed = valid_end + (size_t)s.error_len;
    } else if (final_chunk) {
      push_replacement(&out);
      consumed = pending->size();
    } else {
      consumed = valid_end;
      break;
    }
  }
  pending->erase(0, consumed);
  return out;
}

// byte_decoder (mod.rs:505-528): code point of the GPT-2 byte alphabet -> byte, or -1.
int alphabet_byte(uint32_t cp) {
  static const std::vector<int> table = [] {
    std::vector<int> t(512, -1);
    std::vector<bool> direct(256, false);
    for (int b = 33; b < 127; ++b) direct[(size_t)b] = true;
    for (int b = 161; b < 173; ++b) direct[(size_t)b] = true;
    for (int b = 174; b < 256; ++b) direct[(size_t)b] = true;
    int next = 0;
    for (int b = 0; b < 256; ++b) {
      if (direct[(size_t)b])
        t[(size_t)b] = b;
      else
        t[(size_t)(256 + next++)] = b;
    }
    return t;
  }();
  return cp < table.size() ? table[cp] : -1;
}

void set_error(rg_tok_error *err, int32_t status, uint64_t value = 0, uint64_t value2 = 0, const std::string &text = std::string()) {
  if (!err) return;
  err->status = status;
  err->value = value;
  err->value2 = value2;
  err->text_len = std::min(text.size(), sizeof(err->text));
  memset(err->text, 0, sizeof(err->text));
  memcpy(err->text, text.data(), err->text_len);
}

// ---- the word pre-tokeniser -------------------------------------------------------------------
// Length in bytes of the match of WORD_PREFIX (mod.rs:32-39) at the start of [p, p+n), 0 for no
// match.  Alternatives are tried in the pattern's order; the first that matches wins.
size_t word_prefix(const unsigned char *p, size_t n) {
  const Cp c0 = cp_at(p, n);
  // 1. (?i:'s|'t|'re|'ve|'m|'ll|'d); case-insensitive in the Unicode sense, so U+017F (long s)
  //    and U+212A (Kelvin sign) fold onto s and k; only s occurs here
  if (c0.cp == '\'' && n >= 2) {
    auto fold = [](uint32_t cp) -> uint32_t {
      if (cp >= 'A' && cp <= 'Z') return cp + 32;
      if (cp == 0x17F) return 's';
      return cp;
    };
    const Cp a = cp_at(p + 1, n - 1);
    const uint32_t fa = fold(a.cp);
    const size_t after_a = 1 + (size_t)a.len;
    const Cp b = after_a < n ? cp_at(p + after_a, n - after_a) : Cp{0, 0};
    const uint32_t fb = b.len ? fold(b.cp) : 0;
    if (fa == 's' || fa == 't') return after_a;
    if (fa == 'r' && fb == 'e') return after_a + (size_t)b.len;
    if (fa == 'v' && fb == 'e') return after_a + (size_t)b.len;
    if (fa == 'm') return after_a;
    if (fa == 'l' && fb == 'l') return after_a + (size_t)b.len;
    if (fa == 'd') return after_a;
  }
  // 2. [^\r\n N L]? L+
  {
    size_t i = 0;
    if (!is_letter(c0.cp)) {
      if (!is_newline(c0.cp) && !is_number(c0.cp)) i = (size_t)c0.len;  // the optional leading character
    }
    size_t j = i;
    while (j < n) {
      const Cp c = cp_at(p + j, n - j);
      if (!is_letter(c.cp)) break;
      j += (size_t)c.len;
    }
    if (j > i) return j;
  }
  // 3. N{1,3}
  if (is_number(c0.cp)) {
    size_t j = (size_t)c0.len;
    for (int k = 1; k < 3 && j < n; ++k) {
      const Cp c = cp_at(p + j, n - j);
      if (!is_number(c.cp)) break;
      j += (size_t)c.len;
    }
    return j;
  }
  // 4.  ?[^ws N L]+[\r\n]*
  {
    size_t i = c0.cp == ' ' ? 1 : 0;
    size_t j = i;
    while (j < n) {
      const Cp c = cp_at(p + j, n - j);
      if (is_space(c.cp) || is_number(c.cp) || is_letter(c.cp)) break;
      j += (size_t)c.len;
    }
    if (j > i) {
      while (j < n && (p[j] == '\r' || p[j] == '\n')) ++j;
      return j;
    }
    // without the optional space the class cannot match a space either: no match
  }
  // 5. [ws]*[\r\n]+ : the greedy run gives characters back until a newline can follow, so the
  //    match ends just after the last newline of the leading whitespace run
  {
    size_t j = 0, last_newline_end = 0;
    while (j < n) {
      const Cp c = cp_at(p + j, n - j);
      if (!is_space(c.cp)) break;
      j += (size_t)c.len;
      if (is_newline(c.cp)) last_newline_end = j;
    }
    if (last_newline_end > 0) return last_newline_end;
  }
  return 0;
}

// The fallback of encode_sentence (mod.rs:399-419): a whitespace run that reaches the end is one
// word; otherwise its last character is left for the next word (unless it is the only one); any
// other character stands alone.
size_t next_word(const unsigned char *p, size_t n) {
  const size_t w = word_prefix(p, n);
  if (w) return w;
  size_t j = 0, last_len = 0, count = 0;
  while (j < n) {
    const Cp c = cp_at(p + j, n - j);
    if (!is_space(c.cp)) break;
    j += (size_t)c.len;
    last_len = (size_t)c.len;
    ++count;
  }
  if (j > 0) {
    if (j == n || count <= 1) return j;
    return j - last_len;
  }
  return (size_t)cp_at(p, n).len;
}

}  // namespace

struct rg_tokenizer {
  std::unordered_map<std::string, uint32_t> normal;     // token bytes -> id (last id of a repeated string)
  std::vector<std::pair<std::string, uint32_t>> special;  // source order, first position of a repeated string
  std::unordered_map<uint32_t, std::string> tok2bytes;
  rg_tok_config cfg{};
};

struct rg_tok_stream {
  const rg_tokenizer *tok = nullptr;
  std::string pending;  // incomplete trailing sequence
  bool finished = false;
};

namespace {

// encode_word (mod.rs:426-456)
int32_t encode_word(const rg_tokenizer &t, const std::string &word, std::vector<uint32_t> *out, rg_tok_error *err) {
  auto whole = t.normal.find(word);
  if (whole != t.normal.end()) {
    out->push_back(whole->second);
    return RG_TOK_OK;
  }
  std::vector<std::string> parts;
  parts.reserve(word.size());
  for (char c : word) parts.emplace_back(1, c);
  std::string merged;
  while (true) {
    bool found = false;
    uint32_t best_rank = 0;
    size_t best_pos = 0;
    for (size_t i = 0; i + 1 < parts.size(); ++i) {
      merged.assign(parts[i]);
      merged.append(parts[i + 1]);
      auto it = t.normal.find(merged);
      if (it != t.normal.end() && (!found || it->second < best_rank)) {  // ties keep the leftmost position
        found = true;
        best_rank = it->second;
        best_pos = i;
      }
    }
    if (!found) break;
    parts[best_pos].append(parts[best_pos + 1]);
    parts.erase(parts.begin() + (ptrdiff_t)best_pos + 1);
  }
  for (const std::string &part : parts) {
    auto it = t.normal.find(part);
    if (it == t.normal.end()) {
      set_error(err, RG_TOK_TOKEN_NOT_FOUND, 0, 0, part);
      return RG_TOK_TOKEN_NOT_FOUND;
    }
    out->push_back(it->second);
  }
  return RG_TOK_OK;
}

int32_t encode_sentence(const rg_tokenizer &t, const char *p, size_t n, std::vector<uint32_t> *out, rg_tok_error *err) {
  size_t pos = 0;
  while (pos < n) {
    const size_t w = next_word(reinterpret_cast<const unsigned char *>(p) + pos, n - pos);
    const int32_t rc = encode_word(t, std::string(p + pos, w), out, err);
    if (rc != RG_TOK_OK) return rc;
    pos += w;
  }
  return RG_TOK_OK;
}

}  // namespace

namespace {

int32_t build(const std::vector<std::pair<std::string, uint32_t>> &normal, const std::vector<std::pair<std::string, uint32_t>> &special,
              const rg_tok_config &cfg, rg_tokenizer **out, rg_tok_error *err) {
  auto t = new rg_tokenizer();
  t->cfg = cfg;
  std::vector<std::string> order;  // first appearance of each byte string
  for (const auto &kv : normal) {
    const unsigned char *p = reinterpret_cast<const unsigned char *>(kv.first.data());
    const size_t n = kv.first.size();
    if (!scan_utf8(p, n).ok) {
      delete t;
      set_error(err, RG_TOK_INVALID_ARGUMENT, kv.second);
      return RG_TOK_INVALID_ARGUMENT;
    }
    std::string bytes;
    for (size_t i = 0; i < n;) {
      const Cp c = cp_at(p + i, n - i);
      const int b = alphabet_byte(c.cp);
      if (b < 0) {
        delete t;
        set_error(err, RG_TOK_INVALID_NORMAL_TOKEN_CHARACTER, kv.second, c.cp);
        return RG_TOK_INVALID_NORMAL_TOKEN_CHARACTER;
      }
      bytes.push_back((char)b);
      i += (size_t)c.len;
    }
    auto ins = t->normal.emplace(bytes, kv.second);
    if (ins.second)
      order.push_back(bytes);
    else
      ins.first->second = kv.second;
  }
  std::unordered_map<std::string, size_t> position;
  for (const auto &kv : special) {
    if (kv.first.empty()) {
      delete t;
      set_error(err, RG_TOK_EMPTY_SPECIAL_TOKEN, kv.second);
      return RG_TOK_EMPTY_SPECIAL_TOKEN;
    }
    auto it = position.find(kv.first);
    if (it != position.end()) {
      t->special[it->second].second = kv.second;
    } else {
      position.emplace(kv.first, t->special.size());
      t->special.push_back(kv);
    }
  }
  // later insertions win, as in the reference's map: normal tokens in first-appearance order, then specials
  for (const std::string &bytes : order) t->tok2bytes[t->normal[bytes]] = bytes;
  for (const auto &kv : t->special) t->tok2bytes[kv.second] = kv.first;
  *out = t;
  return RG_TOK_OK;
}

int32_t parse_preset(const std::string &v, int32_t *preset) {
  static const std::pair<const char *, int32_t> names[] = {
      {"llama3", RG_TOK_PRESET_LLAMA3}, {"llama-v3", RG_TOK_PRESET_LLAMA_V3}, {"llama-bpe", RG_TOK_PRESET_LLAMA_BPE},
      {"qwen2", RG_TOK_PRESET_QWEN2},   {"qwen35", RG_TOK_PRESET_QWEN2},      {"qwen35moe", RG_TOK_PRESET_QWEN2},
      {"olmo", RG_TOK_PRESET_OLMO},     {"kimi-k2", RG_TOK_PRESET_KIMI_K2},   {"tekken", RG_TOK_PRESET_TEKKEN},
      {"glm4", RG_TOK_PRESET_GLM4}};
  for (const auto &kv : names)
    if (v == kv.first) {
      *preset = kv.second;
      return RG_TOK_OK;
    }
  return RG_TOK_UNSUPPORTED_PRESET;
}

bool is_int_type(uint32_t type) { return type <= 5 || type == 10 || type == 11; }
bool is_signed_type(uint32_t type) { return type == 1 || type == 3 || type == 5 || type == 11; }
size_t int_width(uint32_t type) {
  switch (type) {
    case 0: case 1: return 1;
    case 2: case 3: return 2;
    case 4: case 5: return 4;
    default: return 8;
  }
}

// lookup_u64 (src/gguf/metadata.rs:199-234): any non-negative integer scalar.
int32_t optional_id(const rg::Gguf &g, const char *key, bool *present, uint32_t *id, rg_tok_error *err) {
  *present = false;
  auto it = g.metadata.find(key);
  if (it == g.metadata.end()) return RG_TOK_OK;
  const rg::GgufValue &v = it->second;
  if (!is_int_type(v.type) || (is_signed_type(v.type) && (int64_t)v.u < 0)) {
    set_error(err, RG_TOK_MALFORMED_METADATA, v.type, 0, key);
    return RG_TOK_MALFORMED_METADATA;
  }
  if (v.u > 0xFFFFFFFFull) {
    set_error(err, RG_TOK_TOKEN_ID_OUT_OF_RANGE, v.u, 0, key);
    return RG_TOK_TOKEN_ID_OUT_OF_RANGE;
  }
  *present = true;
  *id = (uint32_t)v.u;
  return RG_TOK_OK;
}

int32_t copy_out(const std::string &s, char *text, size_t capacity, size_t *n_bytes) {
  if (n_bytes) *n_bytes = s.size();
  if (s.size() > capacity || (!text && !s.empty())) return RG_TOK_INVALID_ARGUMENT;
  if (!s.empty()) memcpy(text, s.data(), s.size());
  return RG_TOK_OK;
}

}  // namespace

extern "C" {

int32_t rg_b200_tokenizer_parse_preset(const char *value, size_t len, int32_t *preset) {
  if (!value || !preset) return RG_TOK_INVALID_ARGUMENT;
  return parse_preset(std::string(value, len), preset);
}

int32_t rg_b200_tokenizer_new(const char *const *normal, const size_t *normal_len, const uint32_t *normal_ids,
                              size_t n_normal, const char *const *special, const size_t *special_len,
                              const uint32_t *special_ids, size_t n_special, const rg_tok_config *cfg,
                              rg_tokenizer **out, rg_tok_error *err) {
  if (!out || (n_normal && (!normal || !normal_len || !normal_ids)) || (n_special && (!special || !special_len || !special_ids))) {
    set_error(err, RG_TOK_INVALID_ARGUMENT);
    return RG_TOK_INVALID_ARGUMENT;
  }
  std::vector<std::pair<std::string, uint32_t>> nv, sv;
  nv.reserve(n_normal);
  for (size_t i = 0; i < n_normal; ++i) nv.emplace_back(std::string(normal[i] ? normal[i] : "", normal[i] ? normal_len[i] : 0), normal_ids[i]);
  for (size_t i = 0; i < n_special; ++i) sv.emplace_back(std::string(special[i] ? special[i] : "", special[i] ? special_len[i] : 0), special_ids[i]);
  rg_tok_config c{};
  c.preset = RG_TOK_PRESET_LLAMA3;
  if (cfg) c = *cfg;
  return build(nv, sv, c, out, err);
}

static int32_t tokenizer_from_gguf_impl(const rg::Gguf &g, rg_tokenizer **out, rg_tok_error *err) {
  static const char *TOKENS = "tokenizer.ggml.tokens", *TYPES = "tokenizer.ggml.token_type", *PRE = "tokenizer.ggml.pre";
  static const char *BOS = "tokenizer.ggml.bos_token_id", *EOS = "tokenizer.ggml.eos_token_id";
  static const char *EOT = "tokenizer.ggml.eot_token_id", *ADD_BOS = "tokenizer.ggml.add_bos_token";
  auto fail = [&](int32_t status, uint64_t v, uint64_t v2, const std::string &text) {
    set_error(err, status, v, v2, text);
    return status;
  };
  auto tk = g.metadata.find(TOKENS);
  if (tk == g.metadata.end()) return fail(RG_TOK_MISSING_METADATA, 0, 0, TOKENS);
  if (tk->second.type != 9) return fail(RG_TOK_MALFORMED_METADATA, tk->second.type, 0, TOKENS);
  if (tk->second.elem_type != 8) return fail(RG_TOK_MALFORMED_METADATA, tk->second.elem_type, 0, TOKENS);
  auto ty = g.metadata.find(TYPES);
  if (ty == g.metadata.end()) return fail(RG_TOK_MISSING_METADATA, 0, 0, TYPES);
  if (ty->second.type != 9) return fail(RG_TOK_MALFORMED_METADATA, ty->second.type, 0, TYPES);
  if (!is_int_type(ty->second.elem_type)) return fail(RG_TOK_MALFORMED_METADATA, ty->second.elem_type, 0, TYPES);
  if (tk->second.count != ty->second.count)
    return fail(RG_TOK_METADATA_LENGTH_MISMATCH, tk->second.count, ty->second.count, std::string());
  const uint64_t count = tk->second.count;
  auto pre = g.metadata.find(PRE);
  if (pre == g.metadata.end()) return fail(RG_TOK_MISSING_METADATA, 0, 0, PRE);
  if (pre->second.type != 8) return fail(RG_TOK_MALFORMED_METADATA, pre->second.type, 0, PRE);
  rg_tok_config cfg{};
  if (parse_preset(pre->second.s, &cfg.preset) != RG_TOK_OK) return fail(RG_TOK_UNSUPPORTED_PRESET, 0, 0, pre->second.s);

  // the reader validated both arrays; walk their items in the file bytes
  std::vector<std::pair<std::string, uint32_t>> normal, special;
  size_t spos = tk->second.array_offset, tpos = ty->second.array_offset;
  const size_t tw = int_width(ty->second.elem_type);
  for (uint64_t i = 0; i < count; ++i) {
    if (i > 0xFFFFFFFFull) return fail(RG_TOK_TOKEN_ID_OUT_OF_RANGE, i, 0, TOKENS);
    uint64_t slen = 0;
    memcpy(&slen, g.bytes + spos, 8);
    std::string token(reinterpret_cast<const char *>(g.bytes + spos + 8), (size_t)slen);
    spos += 8 + (size_t)slen;
    uint64_t raw = 0;
    memcpy(&raw, g.bytes + tpos, tw);
    tpos += tw;
    int64_t type = (int64_t)raw;
    if (is_signed_type(ty->second.elem_type) && tw < 8) {
      const int shift = 64 - 8 * (int)tw;
      type = (int64_t)(raw << shift) >> shift;
    }
    (type == 1 ? normal : special).emplace_back(std::move(token), (uint32_t)i);
  }

  bool add_bos = true;
  auto ab = g.metadata.find(ADD_BOS);
  if (ab != g.metadata.end()) {
    if (ab->second.type != 7) return fail(RG_TOK_MALFORMED_METADATA, ab->second.type, 0, ADD_BOS);
    add_bos = ab->second.u != 0;
  }
  bool present = false;
  uint32_t id = 0;
  int32_t rc;
  if (add_bos) {
    if ((rc = optional_id(g, BOS, &present, &id, err)) != RG_TOK_OK) return rc;
    cfg.has_bos = present;
    cfg.bos_id = present ? id : 0;
  }
  if ((rc = optional_id(g, EOS, &present, &id, err)) != RG_TOK_OK) return rc;
  cfg.eos_id = present ? id : 0;
  if ((rc = optional_id(g, EOT, &present, &id, err)) != RG_TOK_OK) return rc;
  if (present) {
    cfg.has_eot = 1;
    cfg.eot_id = id;
  } else {
    for (auto it = special.rbegin(); it != special.rend(); ++it)
      if (it->first == "<|im_end|>") {
        cfg.has_eot = 1;
        cfg.eot_id = it->second;
        break;
      }
  }
  if (cfg.eos_id >= count) return fail(RG_TOK_CONFIGURED_ID_OUT_OF_RANGE, cfg.eos_id, count, EOS);
  if (cfg.has_bos && cfg.bos_id >= count) return fail(RG_TOK_CONFIGURED_ID_OUT_OF_RANGE, cfg.bos_id, count, BOS);
  if (cfg.has_eot && cfg.eot_id >= count) return fail(RG_TOK_CONFIGURED_ID_OUT_OF_RANGE, cfg.eot_id, count, EOT);
  return build(normal, special, cfg, out, err);
}

int32_t rg_b200_tokenizer_from_gguf(const rg_gguf *gguf, rg_tokenizer **out, rg_tok_error *err) {
  if (!gguf || !out) {
    set_error(err, RG_TOK_INVALID_ARGUMENT);
    return RG_TOK_INVALID_ARGUMENT;
  }
  return tokenizer_from_gguf_impl(gguf->g, out, err);
}

void rg_b200_tokenizer_free(rg_tokenizer *t) { delete t; }

void rg_b200_tokenizer_config(const rg_tokenizer *t, rg_tok_config *out) {
  if (t && out) *out = t->cfg;
}

int32_t rg_b200_tokenizer_is_end(const rg_tokenizer *t, uint32_t token_id) {
  return t && (token_id == t->cfg.eos_id || (t->cfg.has_eot && token_id == t->cfg.eot_id)) ? 1 : 0;
}

int32_t rg_b200_tokenizer_encode(const rg_tokenizer *t, const char *text, size_t len, uint32_t *ids, size_t capacity,
                                 size_t *n_ids, rg_tok_error *err) {
  if (!t || (!text && len) || !n_ids || !scan_utf8(reinterpret_cast<const unsigned char *>(text), len).ok) {
    set_error(err, RG_TOK_INVALID_ARGUMENT);
    return RG_TOK_INVALID_ARGUMENT;
  }
  std::vector<uint32_t> out;
  size_t pos = 0;
  while (true) {
    // next_special (mod.rs:379-391): earliest start, then source order
    bool found = false;
    size_t best_start = 0, best_len = 0;
    uint32_t best_id = 0;
    for (const auto &kv : t->special) {
      if (kv.first.size() > len - pos) continue;
      const char *hay = text + pos, *end = text + len;
      const char *hit = std::search(hay, end, kv.first.begin(), kv.first.end());
      if (hit == end) continue;
      const size_t start = (size_t)(hit - text);
      if (!found || start < best_start) {
        found = true;
        best_start = start;
        best_len = kv.first.size();
        best_id = kv.second;
      }
    }
    const size_t stop = found ? best_start : len;
    const int32_t rc = encode_sentence(*t, text + pos, stop - pos, &out, err);
    if (rc != RG_TOK_OK) return rc;
    if (!found) break;
    out.push_back(best_id);
    pos = best_start + best_len;
  }
  *n_ids = out.size();
  if (out.size() > capacity || (!ids && !out.empty())) {
    set_error(err, RG_TOK_INVALID_ARGUMENT, out.size());
    return RG_TOK_INVALID_ARGUMENT;
  }
  if (!out.empty()) memcpy(ids, out.data(), out.size() * sizeof(uint32_t));
  return RG_TOK_OK;
}

int32_t rg_b200_tokenizer_decode(const rg_tokenizer *t, const uint32_t *ids, size_t n_ids, char *text, size_t capacity,
                                 size_t *n_bytes, rg_tok_error *err) {
  if (!t || (!ids && n_ids) || !n_bytes) {
    set_error(err, RG_TOK_INVALID_ARGUMENT);
    return RG_TOK_INVALID_ARGUMENT;
  }
  std::string bytes;
  for (size_t i = 0; i < n_ids; ++i) {
    auto it = t->tok2bytes.find(ids[i]);
    if (it == t->tok2bytes.end()) {
      set_error(err, RG_TOK_UNKNOWN_TOKEN_ID, ids[i]);
      return RG_TOK_UNKNOWN_TOKEN_ID;
    }
    bytes.append(it->second);
  }
  const std::string s = drain_utf8(&bytes, true);  // String::from_utf8_lossy: one U+FFFD per ill-formed sequence
  const int32_t rc = copy_out(s, text, capacity, n_bytes);
  if (rc != RG_TOK_OK) set_error(err, rc, s.size());
  return rc;
}

int32_t rg_b200_tok_stream_new(const rg_tokenizer *t, rg_tok_stream **out) {
  if (!t || !out) return RG_TOK_INVALID_ARGUMENT;
  auto s = new rg_tok_stream();
  s->tok = t;
  *out = s;
  return RG_TOK_OK;
}

int32_t rg_b200_tok_stream_push(rg_tok_stream *s, uint32_t token_id, char *text, size_t capacity, size_t *n_bytes,
                                rg_tok_error *err) {
  if (!s || !n_bytes) {
    set_error(err, RG_TOK_INVALID_ARGUMENT);
    return RG_TOK_INVALID_ARGUMENT;
  }
  std::string produced;
  const std::string before = s->pending;
  if (!s->finished) {
    auto it = s->tok->tok2bytes.find(token_id);
    if (it == s->tok->tok2bytes.end()) {
      set_error(err, RG_TOK_UNKNOWN_TOKEN_ID, token_id);
      return RG_TOK_UNKNOWN_TOKEN_ID;
    }
    s->pending.append(it->second);
    produced = drain_utf8(&s->pending, false);
  }
  const int32_t rc = copy_out(produced, text, capacity, n_bytes);
  if (rc != RG_TOK_OK) {  // the token is not consumed: the caller repeats the push with a larger buffer
    s->pending = before;
    set_error(err, rc, produced.size());
  }
  return rc;
}

int32_t rg_b200_tok_stream_finish(rg_tok_stream *s, char *text, size_t capacity, size_t *n_bytes) {
  if (!s || !n_bytes) return RG_TOK_INVALID_ARGUMENT;
  // at most one replacement character (3 bytes) is left to flush; it stays until it fits
  std::string tail = s->pending;
  const std::string produced = s->finished ? std::string() : drain_utf8(&tail, true);
  const int32_t rc = copy_out(produced, text, capacity, n_bytes);
  if (rc == RG_TOK_OK) {
    s->finished = true;
    s->pending.clear();
  }
  return rc;
}

void rg_b200_tok_stream_free(rg_tok_stream *s) { delete s; }

// ---- chat prompt (src/models/transformer/chat.rs) ---------------------------------------------
static const char CHAT_TEMPLATE[] =
    "{{ bos_token }}{% for message in messages %}{{ '<|start_header_id|>' + message['role'] + "
    "'<|end_header_id|>\\n\\n' + message['content'] + eos_token }}{% endfor %}{% if add_generation_prompt %}"
    "{{ '<|start_header_id|>assistant<|end_header_id|>\\n\\n' }}{% endif %}";
static const size_t MAX_TEMPLATE_BYTES = 64 * 1024, MAX_MESSAGE_BYTES = 1024 * 1024, MAX_CHAT_BYTES = 4 * 1024 * 1024;

const char *rg_b200_chat_template_text(void) { return CHAT_TEMPLATE; }

int32_t rg_b200_chat_template_from_gguf(const rg_gguf *gguf, int32_t *metadata_present, rg_tok_error *err) {
  if (!gguf || !metadata_present) {
    set_error(err, RG_TOK_INVALID_ARGUMENT);
    return RG_TOK_INVALID_ARGUMENT;
  }
  static const char *KEY = "tokenizer.chat_template";
  *metadata_present = 0;
  auto it = gguf->g.metadata.find(KEY);
  if (it == gguf->g.metadata.end()) return RG_TOK_OK;
  if (it->second.type != 8) {
    set_error(err, RG_TOK_MALFORMED_METADATA, it->second.type, 0, KEY);
    return RG_TOK_MALFORMED_METADATA;
  }
  const std::string &tpl = it->second.s;
  if (tpl.size() > MAX_TEMPLATE_BYTES) {
    set_error(err, RG_TOK_TEMPLATE_TOO_LONG, tpl.size(), MAX_TEMPLATE_BYTES);
    return RG_TOK_TEMPLATE_TOO_LONG;
  }
  if (tpl != CHAT_TEMPLATE) {
    const bool jinja = tpl.find("{{") != std::string::npos || tpl.find("{%") != std::string::npos || tpl.find("{#") != std::string::npos;
    const int32_t rc = jinja ? RG_TOK_UNSUPPORTED_JINJA : RG_TOK_UNSUPPORTED_TEMPLATE;
    set_error(err, rc);
    return rc;
  }
  *metadata_present = 1;
  return RG_TOK_OK;
}

int32_t rg_b200_chat_render(const rg_tokenizer *t, const int32_t *roles, const char *const *contents,
                            const size_t *content_len, size_t n_messages, int32_t add_generation_prompt, char *text,
                            size_t capacity, size_t *n_bytes, rg_tok_error *err) {
  if (!t || !n_bytes || (n_messages && (!roles || !contents || !content_len))) {
    set_error(err, RG_TOK_INVALID_ARGUMENT);
    return RG_TOK_INVALID_ARGUMENT;
  }
  static const char *ROLE[] = {"system", "user", "assistant"};
  static const std::string HEADER_START = "<|start_header_id|>", HEADER_END = "<|end_header_id|>\n\n";
  for (size_t i = 0; i < n_messages; ++i) {
    if (roles[i] < 0 || roles[i] > 2 || (!contents[i] && content_len[i]) ||
        !scan_utf8(reinterpret_cast<const unsigned char *>(contents[i]), content_len[i]).ok) {
      set_error(err, RG_TOK_INVALID_ARGUMENT, i);
      return RG_TOK_INVALID_ARGUMENT;
    }
    if (content_len[i] > MAX_MESSAGE_BYTES) {  // LlamaChatMessage::new (chat.rs:45-55)
      set_error(err, RG_TOK_MESSAGE_TOO_LONG, content_len[i], MAX_MESSAGE_BYTES);
      return RG_TOK_MESSAGE_TOO_LONG;
    }
  }
  if (t->cfg.preset != RG_TOK_PRESET_LLAMA3 && t->cfg.preset != RG_TOK_PRESET_LLAMA_V3 && t->cfg.preset != RG_TOK_PRESET_LLAMA_BPE) {
    set_error(err, RG_TOK_CHAT_UNSUPPORTED_PRESET, (uint64_t)t->cfg.preset);
    return RG_TOK_CHAT_UNSUPPORTED_PRESET;
  }
  auto token_text = [&](uint32_t id, std::string *out) -> int32_t {
    auto it = t->tok2bytes.find(id);
    if (it == t->tok2bytes.end()) {
      set_error(err, RG_TOK_UNKNOWN_TOKEN_ID, id);
      return RG_TOK_UNKNOWN_TOKEN_ID;
    }
    std::string bytes = it->second;
    *out = drain_utf8(&bytes, true);
    return RG_TOK_OK;
  };
  std::string bos, eos;
  int32_t rc;
  if (t->cfg.has_bos && (rc = token_text(t->cfg.bos_id, &bos)) != RG_TOK_OK) return rc;
  if ((rc = token_text(t->cfg.eos_id, &eos)) != RG_TOK_OK) return rc;
  size_t required = bos.size();
  bool overflow = false;
  auto add = [&](size_t n) {
    if (n > SIZE_MAX - required) overflow = true;
    required += n;
  };
  for (size_t i = 0; i < n_messages; ++i) {
    add(HEADER_START.size());
    add(strlen(ROLE[roles[i]]));
    add(HEADER_END.size());
    add(content_len[i]);
    add(eos.size());
  }
  if (add_generation_prompt) {
    add(HEADER_START.size());
    add(strlen("assistant"));
    add(HEADER_END.size());
  }
  if (overflow) {
    set_error(err, RG_TOK_CHAT_OVERFLOW);
    return RG_TOK_CHAT_OVERFLOW;
  }
  if (required > MAX_CHAT_BYTES) {
    set_error(err, RG_TOK_CHAT_TOO_LONG, required, MAX_CHAT_BYTES);
    return RG_TOK_CHAT_TOO_LONG;
  }
  std::string out;
  out.reserve(required);
  out.append(bos);
  for (size_t i = 0; i < n_messages; ++i) {
    out.append(HEADER_START).append(ROLE[roles[i]]).append(HEADER_END);
    out.append(contents[i] ? contents[i] : "", content_len[i]);
    out.append(eos);
  }
  if (add_generation_prompt) out.append(HEADER_START).append("assistant").append(HEADER_END);
  rc = copy_out(out, text, capacity, n_bytes);
  if (rc != RG_TOK_OK) set_error(err, rc, out.size());
  return rc;
}

}  // extern "C"

namespace rg {

// The model configuration takes its stop ids from the tokenizer built from the same file
// (src/models/transformer/model.rs:133,288-292 with src/tokenizer/mod.rs:284-296): eos is the
// metadata value or 0, eot the metadata value or the last special token named <|im_end|>, and a
// file whose tokenizer does not build has no model configuration either.
int32_t gguf_tokenizer_stop_ids(const Gguf &g, int32_t *eos, int32_t *eot, std::string *why) {
  rg_tokenizer *t = nullptr;
  rg_tok_error e{};
  const int32_t rc = tokenizer_from_gguf_impl(g, &t, &e);
  if (rc != RG_TOK_OK) {
    if (why)
      *why = "tokenizer: status " + std::to_string(rc) + " (" + std::string(e.text, e.text_len < sizeof(e.text) ? e.text_len : sizeof(e.text)) +
             ", " + std::to_string(e.value) + ", " + std::to_string(e.value2) + ")";
    if (rc == RG_TOK_MISSING_METADATA) return RG_MISSING_METADATA;
    if (rc == RG_TOK_UNSUPPORTED_PRESET) return RG_UNSUPPORTED_VARIANT;
    return RG_INVALID_ARGUMENT;
  }
  *eos = (int32_t)t->cfg.eos_id;
  *eot = t->cfg.has_eot ? (int32_t)t->cfg.eot_id : -1;
  delete t;
  return RG_OK;
}

}  // namespace rg
