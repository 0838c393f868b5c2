// Continuous-batching scheduler behind include/rg_b200_serving.h: admission, arrival-order
// selection, cache-row bookkeeping and the prefix cache of rustgrad's LlamaServingScheduler
// (src/models/transformer/serving/mod.rs:192-352 PrefixCache, :371-690 scheduler, :726-790
// validate_request).  Host policy only: a step is composed from the session verbs in the
// rg_serving_backend table (prefill_select, decode_rows, select, kv snapshots).
#include <math.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "../../include/rg_b200_serving.h"

namespace {

int32_t fail(rg_serving_error *err, int32_t kind, int64_t value = 0, int64_t value2 = 0) {
  if (err) *err = rg_serving_error{kind, value, value2};
  return kind;
}

// A device K/V copy shared by the cache and by the requests that lean on it.
struct Snapshot {
  const rg_serving_backend *be;
  void *handle;
  int32_t length;
  size_t bytes;
  Snapshot(const rg_serving_backend *b, void *h, int32_t n, size_t sz) : be(b), handle(h), length(n), bytes(sz) {}
  Snapshot(const Snapshot &) = delete;
  Snapshot &operator=(const Snapshot &) = delete;
  ~Snapshot() {
    if (handle) be->snapshot_free(be->ctx, handle);
  }
};
using SnapshotRef = std::shared_ptr<Snapshot>;
using Key = std::vector<int32_t>;

struct Entry {
  uint64_t generation;
  SnapshotRef snapshot;
  std::vector<float> logits;
  size_t bytes;
  uint64_t last_used;
  uint64_t references = 0;
};

// PrefixCache (serving/mod.rs:192-352): longest-prefix lookup, least-recently-used eviction of
// unreferenced entries under an entry and a byte budget, generation counter for invalidation.
struct PrefixCache {
  size_t max_entries = 0, max_bytes = 0;
  uint64_t generation = 0, clock = 0, bytes = 0, hits = 0, misses = 0, stale_rejections = 0, evictions = 0;
  std::map<Key, Entry> entries;

  void invalidate() {
    ++generation;
    bytes = 0;
    entries.clear();
  }
  void release(const Key &key) {
    auto it = entries.find(key);
    if (it != entries.end() && it->second.references) --it->second.references;
  }
  // The longest entry that is a prefix of `tokens`; the caller holds a reference until release().
  const Key *longest(const Key &tokens, Entry **found) {
    for (auto it = entries.begin(); it != entries.end();) {
      if (it->second.generation != generation) {
        bytes -= it->second.bytes;
        ++stale_rejections;
        it = entries.erase(it);
      } else {
        ++it;
      }
    }
    const Key *best = nullptr;
    Entry *best_entry = nullptr;
    for (auto &kv : entries) {
      const Key &k = kv.first;
      if (k.size() <= tokens.size() && std::equal(k.begin(), k.end(), tokens.begin()) && (!best || k.size() > best->size())) {
        best = &k;
        best_entry = &kv.second;
      }
    }
    if (!best) {
      ++misses;
      return nullptr;
    }
    best_entry->last_used = ++clock;
    ++best_entry->references;
    ++hits;
    *found = best_entry;
    return best;
  }
  bool insert(const Key &tokens, SnapshotRef snapshot, const float *logits, size_t n_logits) {
    if (max_entries == 0 || max_bytes == 0) return false;
    const size_t size = snapshot->bytes + n_logits * 4 + tokens.size() * 4;
    if (size > max_bytes) return false;
    auto old = entries.find(tokens);
    if (old != entries.end()) {
      bytes -= old->second.bytes;
      entries.erase(old);
    }
    while (entries.size() >= max_entries || bytes + size > max_bytes) {
      auto victim = entries.end();
      for (auto it = entries.begin(); it != entries.end(); ++it)
        if (it->second.references == 0 && (victim == entries.end() || it->second.last_used < victim->second.last_used)) victim = it;
      if (victim == entries.end()) return false;
      bytes -= victim->second.bytes;
      entries.erase(victim);
      ++evictions;
    }
    Entry e;
    e.generation = generation;
    e.snapshot = std::move(snapshot);
    e.logits.assign(logits, logits + n_logits);
    e.bytes = size;
    e.last_used = ++clock;
    bytes += size;
    entries.emplace(tokens, std::move(e));
    return true;
  }
};

struct Request {
  uint64_t id = 0, arrival = 0;
  Key prompt;
  size_t max_new = 0;
  bool greedy = true;
  float temperature = 0.f;
  std::vector<float> uniforms;  // [max_new, vocab]
  int32_t status = RG_REQUEST_QUEUED;
  std::vector<int32_t> generated;
  bool stopped = false;
  int32_t row = -1;
  bool has_pending = false;
  int32_t pending_token = 0;
  bool has_result = false;
  std::string decoded;
};

}  // namespace

struct rg_scheduler {
  rg_serving_backend be{};
  const rg_tokenizer *tokenizer = nullptr;
  int32_t batch_size = 0;
  std::set<int32_t> stop_ids;
  bool has_bos = false;
  int32_t bos_id = 0;
  std::set<int32_t> free_rows;
  uint64_t next_id = 0, next_arrival = 0;
  std::vector<uint64_t> order;
  std::map<uint64_t, Request> requests;
  PrefixCache prefixes;

  const float *tape_row(const Request &r) const {
    return r.greedy ? nullptr : r.uniforms.data() + r.generated.size() * (size_t)be.vocab;
  }
  int32_t release_row(Request &r) {
    if (r.row < 0) return RG_OK;
    const int32_t rc = be.reset_row(be.ctx, r.row);
    free_rows.insert(r.row);
    r.row = -1;
    return rc;
  }
};

namespace {

// The table over one rg_session.
int32_t be_reset_row(void *c, int32_t row) { return rg_b200_reset_row((rg_session *)c, row); }
int32_t be_prefill_select(void *c, int32_t row, const int32_t *ids, size_t n, float t, const float *u, float *last, int32_t *sel) {
  return rg_b200_prefill_select((rg_session *)c, row, ids, n, t, u, last, sel);
}
int32_t be_decode_rows(void *c, const int32_t *rows, const int32_t *toks, int32_t n, const float *t, const float *u, int32_t *ids) {
  return rg_b200_decode_rows((rg_session *)c, rows, toks, n, t, u, nullptr, ids);
}
int32_t be_select(void *c, const float *logits, float t, const float *u, int32_t *id) {
  return rg_b200_select((rg_session *)c, logits, 1, &t, u, id);
}
int32_t be_snapshot_create(void *c, int32_t row, int32_t length, void **snap, size_t *bytes) {
  rg_kv_snapshot *k = nullptr;
  const int32_t rc = rg_b200_kv_snapshot_create((rg_session *)c, row, length, &k);
  if (rc) return rc;
  *snap = k;
  *bytes = rg_b200_kv_snapshot_bytes(k);
  return RG_OK;
}
int32_t be_snapshot_restore(void *c, const void *snap, int32_t row) {
  return rg_b200_kv_snapshot_restore((rg_session *)c, (const rg_kv_snapshot *)snap, row);
}
void be_snapshot_free(void *, void *snap) { rg_b200_kv_snapshot_free((rg_kv_snapshot *)snap); }
int32_t be_prefill_rows(void *c, const int32_t *rows, const int32_t *ids, const size_t *lens, int32_t n, float *last, int32_t *sel) {
  return rg_b200_prefill_rows((rg_session *)c, rows, ids, lens, n, last, sel);
}

int32_t encode_text(const rg_tokenizer *tok, const char *text, size_t len, Key *out, rg_serving_error *err) {
  rg_tok_error terr{};
  size_t n = 0;
  int32_t trc = rg_b200_tokenizer_encode(tok, text, len, nullptr, 0, &n, &terr);
  if (trc != RG_TOK_OK && !(trc == RG_TOK_INVALID_ARGUMENT && n > 0)) return fail(err, RG_SERVING_TOKENIZER, trc);
  std::vector<uint32_t> ids(n ? n : 1);
  if (n && (trc = rg_b200_tokenizer_encode(tok, text, len, ids.data(), ids.size(), &n, &terr)) != RG_TOK_OK)
    return fail(err, RG_SERVING_TOKENIZER, trc);
  for (size_t i = 0; i < n; ++i) out->push_back((int32_t)ids[i]);
  return RG_SERVING_OK;
}

}  // namespace

extern "C" {

int32_t rg_b200_scheduler_new_with_backend(const rg_serving_backend *backend, const rg_tokenizer *tokenizer,
                                           const rg_serving_options *o, rg_scheduler **out, rg_serving_error *err) {
  if (!backend || !o || !out) return fail(err, RG_SERVING_INVALID_ARGUMENT);
  if (o->batch_size <= 0) return fail(err, RG_SERVING_EMPTY_BATCH, o->batch_size);
  const int32_t rows = o->max_rows > 0 ? o->max_rows : o->batch_size;
  if (rows < o->batch_size) return fail(err, RG_SERVING_EMPTY_BATCH, rows, o->batch_size);
  if (o->n_stop_ids && !o->stop_ids) return fail(err, RG_SERVING_INVALID_ARGUMENT);
  auto s = new rg_scheduler();
  s->be = *backend;
  s->tokenizer = tokenizer;
  s->batch_size = o->batch_size;
  s->stop_ids.insert(o->stop_ids, o->stop_ids + o->n_stop_ids);
  s->has_bos = o->has_bos != 0;
  s->bos_id = o->bos_id;
  for (int32_t r = 0; r < rows; ++r) s->free_rows.insert(r);
  s->prefixes.max_entries = o->prefix_max_entries;
  s->prefixes.max_bytes = o->prefix_max_bytes;
  *out = s;
  return RG_SERVING_OK;
}

static rg_serving_backend session_backend(rg_session *session) {
  rg_serving_backend be{};
  be.ctx = session;
  be.vocab = rg_b200_vocab_size(session);
  be.max_context = rg_b200_max_context(session);
  be.reset_row = be_reset_row;
  be.prefill_select = be_prefill_select;
  be.decode_rows = be_decode_rows;
  be.select = be_select;
  be.snapshot_create = be_snapshot_create;
  be.snapshot_restore = be_snapshot_restore;
  be.snapshot_free = be_snapshot_free;
  be.prefill_rows = be_prefill_rows;
  return be;
}

int32_t rg_b200_scheduler_new(rg_session *session, const rg_tokenizer *tokenizer, const rg_serving_options *options,
                              rg_scheduler **out, rg_serving_error *err) {
  if (!session) return fail(err, RG_SERVING_INVALID_ARGUMENT);
  const rg_serving_backend be = session_backend(session);
  return rg_b200_scheduler_new_with_backend(&be, tokenizer, options, out, err);
}

// serving/mod.rs:528-547.  The cached snapshots belong to the session that made them: they are destroyed
// (through the table still in place) before the new table is taken.
int32_t rg_b200_scheduler_rebind_with_backend(rg_scheduler *s, const rg_serving_backend *backend, const rg_tokenizer *tokenizer,
                                              const rg_serving_options *o, int32_t *changed, rg_serving_error *err) {
  if (!s || !backend) return fail(err, RG_SERVING_INVALID_ARGUMENT);
  if (o && o->n_stop_ids && !o->stop_ids) return fail(err, RG_SERVING_INVALID_ARGUMENT);
  if (rg_b200_scheduler_pending(s) != 0) return fail(err, RG_SERVING_ACTIVE_REQUESTS, (int64_t)rg_b200_scheduler_pending(s));
  // the same session: the same object behind the same verbs
  const bool differs = backend->ctx != s->be.ctx || backend->vocab != s->be.vocab || backend->max_context != s->be.max_context ||
                       backend->reset_row != s->be.reset_row || backend->prefill_select != s->be.prefill_select ||
                       backend->decode_rows != s->be.decode_rows || backend->select != s->be.select ||
                       backend->snapshot_create != s->be.snapshot_create || backend->snapshot_restore != s->be.snapshot_restore ||
                       backend->snapshot_free != s->be.snapshot_free || backend->prefill_rows != s->be.prefill_rows;
  if (differs) s->prefixes.invalidate();
  s->be = *backend;
  s->tokenizer = tokenizer;
  if (o) {
    s->stop_ids.clear();
    s->stop_ids.insert(o->stop_ids, o->stop_ids + o->n_stop_ids);
    s->has_bos = o->has_bos != 0;
    s->bos_id = o->bos_id;
  }
  if (changed) *changed = differs ? 1 : 0;
  return RG_SERVING_OK;
}

int32_t rg_b200_scheduler_rebind(rg_scheduler *s, rg_session *session, const rg_tokenizer *tokenizer,
                                 const rg_serving_options *options, int32_t *changed, rg_serving_error *err) {
  if (!session) return fail(err, RG_SERVING_INVALID_ARGUMENT);
  const rg_serving_backend be = session_backend(session);
  return rg_b200_scheduler_rebind_with_backend(s, &be, tokenizer, options, changed, err);
}

void rg_b200_scheduler_free(rg_scheduler *s) {
  if (!s) return;
  for (auto &kv : s->requests) s->release_row(kv.second);
  delete s;  // the prefix entries free their snapshots
}

int32_t rg_b200_scheduler_submit_ids(rg_scheduler *s, const int32_t *prompt, size_t n, size_t max_new,
                                     const rg_serving_sampling *sampling, uint64_t *request_id, rg_serving_error *err) {
  if (!s || (n && !prompt)) return fail(err, RG_SERVING_INVALID_ARGUMENT);
  const int64_t vocab = s->be.vocab, ctx = s->be.max_context;
  if (n == 0) return fail(err, RG_SERVING_EMPTY_PROMPT);
  if (n + max_new > (size_t)ctx) return fail(err, RG_SERVING_CONTEXT_LENGTH, (int64_t)(n + max_new), ctx);
  for (size_t i = 0; i < n; ++i)
    if (prompt[i] < 0 || prompt[i] >= vocab) return fail(err, RG_SERVING_TOKEN_OUT_OF_RANGE, prompt[i], vocab);
  Request r;
  r.greedy = !sampling || sampling->greedy;
  if (!r.greedy) {
    if (!isfinite(sampling->temperature) || sampling->temperature <= 0.0f) return fail(err, RG_SERVING_INVALID_TEMPERATURE);
    const size_t required = max_new * (size_t)vocab;
    const size_t actual = sampling->uniforms ? sampling->n_uniforms : 0;
    if (actual < required) return fail(err, RG_SERVING_UNIFORM_TAPE_LENGTH, (int64_t)required, (int64_t)actual);
    for (size_t i = 0; i < required; ++i) {
      const float u = sampling->uniforms[i];
      if (!isfinite(u) || u < 0.0f || u >= 1.0f) return fail(err, RG_SERVING_INVALID_UNIFORM, (int64_t)i);
    }
    r.temperature = sampling->temperature;
    r.uniforms.assign(sampling->uniforms, sampling->uniforms + required);
  }
  r.id = s->next_id++;
  r.arrival = s->next_arrival++;
  r.prompt.assign(prompt, prompt + n);
  r.max_new = max_new;
  if (max_new == 0) {
    r.status = RG_REQUEST_COMPLETE;
    r.has_result = true;
  }
  if (request_id) *request_id = r.id;
  s->order.push_back(r.id);
  s->requests.emplace(r.id, std::move(r));
  return RG_SERVING_OK;
}

int32_t rg_b200_scheduler_submit_text(rg_scheduler *s, const char *prompt, size_t prompt_len, size_t max_new,
                                      const rg_serving_sampling *sampling, uint64_t *request_id, rg_serving_error *err) {
  if (!s || !s->tokenizer || (prompt_len && !prompt)) return fail(err, RG_SERVING_INVALID_ARGUMENT);
  Key ids;
  if (s->has_bos) ids.push_back(s->bos_id);
  if (int32_t rc = encode_text(s->tokenizer, prompt ? prompt : "", prompt_len, &ids, err)) return rc;
  return rg_b200_scheduler_submit_ids(s, ids.data(), ids.size(), max_new, sampling, request_id, err);
}

int32_t rg_b200_scheduler_submit_chat(rg_scheduler *s, const int32_t *roles, const char *const *contents,
                                      const size_t *content_len, size_t n_messages, size_t max_new,
                                      const rg_serving_sampling *sampling, uint64_t *request_id, rg_serving_error *err) {
  if (!s || !s->tokenizer || (n_messages && (!roles || !contents || !content_len))) return fail(err, RG_SERVING_INVALID_ARGUMENT);
  rg_tok_error terr{};
  size_t bytes = 0;
  int32_t trc = rg_b200_chat_render(s->tokenizer, roles, contents, content_len, n_messages, 1, nullptr, 0, &bytes, &terr);
  if (trc != RG_TOK_OK && !(trc == RG_TOK_INVALID_ARGUMENT && bytes > 0)) return fail(err, RG_SERVING_TOKENIZER, trc);
  std::string rendered(bytes, '\0');
  if (bytes && (trc = rg_b200_chat_render(s->tokenizer, roles, contents, content_len, n_messages, 1, &rendered[0], bytes, &bytes,
                                          &terr)) != RG_TOK_OK)
    return fail(err, RG_SERVING_TOKENIZER, trc);
  Key ids;
  if (int32_t rc = encode_text(s->tokenizer, rendered.data(), rendered.size(), &ids, err)) return rc;
  return rg_b200_scheduler_submit_ids(s, ids.data(), ids.size(), max_new, sampling, request_id, err);
}

int32_t rg_b200_scheduler_status(const rg_scheduler *s, uint64_t id, int32_t *status) {
  if (!s || !status) return RG_SERVING_INVALID_ARGUMENT;
  auto it = s->requests.find(id);
  if (it == s->requests.end()) return RG_SERVING_UNKNOWN_REQUEST;
  *status = it->second.status;
  return RG_SERVING_OK;
}

int32_t rg_b200_scheduler_result(const rg_scheduler *s, uint64_t id, rg_serving_result *out) {
  if (!s || !out) return RG_SERVING_INVALID_ARGUMENT;
  auto it = s->requests.find(id);
  if (it == s->requests.end()) return RG_SERVING_UNKNOWN_REQUEST;
  const Request &r = it->second;
  if (!r.has_result) return RG_SERVING_NOT_COMPLETE;
  *out = rg_serving_result{r.id, r.prompt.data(), r.prompt.size(), r.generated.data(), r.generated.size(),
                           r.decoded.c_str(), r.decoded.size(), r.stopped ? 1 : 0};
  return RG_SERVING_OK;
}

int32_t rg_b200_scheduler_remove(rg_scheduler *s, uint64_t id) {
  if (!s) return RG_SERVING_INVALID_ARGUMENT;
  auto it = s->requests.find(id);
  if (it == s->requests.end()) return RG_SERVING_UNKNOWN_REQUEST;
  s->release_row(it->second);
  s->requests.erase(it);
  s->order.erase(std::find(s->order.begin(), s->order.end(), id));
  return RG_SERVING_OK;
}

size_t rg_b200_scheduler_pending(const rg_scheduler *s) {
  size_t n = 0;
  if (s)
    for (auto &kv : s->requests) n += kv.second.status != RG_REQUEST_COMPLETE;
  return n;
}

size_t rg_b200_scheduler_completed(const rg_scheduler *s, uint64_t *ids, size_t cap) {
  size_t n = 0;
  if (!s) return 0;
  for (uint64_t id : s->order)
    if (s->requests.at(id).has_result) {
      if (ids && n < cap) ids[n] = id;
      ++n;
    }
  return n;
}

void rg_b200_scheduler_prefix_stats(const rg_scheduler *s, rg_prefix_stats *out) {
  if (!s || !out) return;
  const PrefixCache &c = s->prefixes;
  *out = rg_prefix_stats{(uint64_t)c.entries.size(), c.bytes, c.hits, c.misses, c.stale_rejections, c.evictions, c.generation};
}

void rg_b200_scheduler_invalidate_prefix_cache(rg_scheduler *s) {
  if (s) s->prefixes.invalidate();
}

int32_t rg_b200_scheduler_step(rg_scheduler *s, rg_token_event *events, size_t cap, size_t *n_events, rg_serving_error *err) {
  if (!s || !n_events || (!events && cap)) return fail(err, RG_SERVING_INVALID_ARGUMENT);
  *n_events = 0;
  std::vector<Request *> selected;
  for (uint64_t id : s->order) {
    Request &r = s->requests.at(id);
    if (r.status != RG_REQUEST_COMPLETE) selected.push_back(&r);
    if ((int32_t)selected.size() == s->batch_size) break;
  }
  if (selected.empty()) return RG_SERVING_OK;
  if (cap < selected.size()) return fail(err, RG_SERVING_INVALID_ARGUMENT, (int64_t)selected.size(), (int64_t)cap);
  const size_t vocab = (size_t)s->be.vocab;
  std::map<uint64_t, int32_t> chosen;
  std::vector<Request *> decode_cols, admitted;
  // a failure un-admits what this step admitted, so that the step can be run again as a whole
  auto roll_back = [&](int32_t rc) {
    for (Request *r : admitted) {
      s->release_row(*r);
      r->status = RG_REQUEST_QUEUED;
    }
    return fail(err, RG_SERVING_SESSION, rc);
  };
  std::vector<float> last(vocab);
  // greedy prompts admitted in this step wait here and are prefilled together
  struct Deferred {
    Request *r;
    size_t cached;
  };
  std::vector<Deferred> deferred;
  auto remember_prefix = [&](Request *r, const float *logits) -> int32_t {
    if (!(s->prefixes.max_entries && s->prefixes.max_bytes)) return RG_OK;
    void *handle = nullptr;
    size_t bytes = 0;
    if (int32_t rc = s->be.snapshot_create(s->be.ctx, r->row, (int32_t)r->prompt.size(), &handle, &bytes)) return rc;
    auto snap = std::make_shared<Snapshot>(&s->be, handle, (int32_t)r->prompt.size(), bytes);
    s->prefixes.insert(r->prompt, std::move(snap), logits, vocab);
    return RG_OK;
  };
  auto flush = [&]() -> int32_t {
    if (deferred.empty()) return RG_OK;
    const int32_t n = (int32_t)deferred.size();
    std::vector<int32_t> rows(n), ids, sel(n, -1);
    std::vector<size_t> lens(n);
    for (int32_t i = 0; i < n; ++i) {
      const Deferred &d = deferred[i];
      rows[i] = d.r->row;
      lens[i] = d.r->prompt.size() - d.cached;
      ids.insert(ids.end(), d.r->prompt.begin() + (ptrdiff_t)d.cached, d.r->prompt.end());
    }
    std::vector<float> logits((size_t)n * vocab);
    int32_t rc = RG_OK;
    if (n > 1 && s->be.prefill_rows) {
      rc = s->be.prefill_rows(s->be.ctx, rows.data(), ids.data(), lens.data(), n, logits.data(), sel.data());
    } else {
      size_t off = 0;
      for (int32_t i = 0; i < n && !rc; ++i) {
        rc = s->be.prefill_select(s->be.ctx, rows[i], ids.data() + off, lens[i], 0.0f, nullptr, &logits[(size_t)i * vocab], &sel[i]);
        off += lens[i];
      }
    }
    for (int32_t i = 0; i < n && !rc; ++i) {
      rc = remember_prefix(deferred[i].r, &logits[(size_t)i * vocab]);
      chosen[deferred[i].r->id] = sel[i];
    }
    deferred.clear();
    return rc;
  };
  for (Request *r : selected) {
    if (r->has_pending) {
      decode_cols.push_back(r);
      continue;
    }
    // a waiting prompt this one extends must be in the prefix cache before the lookup below
    if (s->prefixes.max_entries && s->prefixes.max_bytes)
      for (const Deferred &d : deferred)
        if (d.r->prompt.size() <= r->prompt.size() && std::equal(d.r->prompt.begin(), d.r->prompt.end(), r->prompt.begin())) {
          if (int32_t rc = flush()) return roll_back(rc);
          break;
        }
    // a new request: lean on the longest cached prefix, prefill what is left
    r->row = *s->free_rows.begin();
    s->free_rows.erase(s->free_rows.begin());
    r->status = RG_REQUEST_RUNNING;
    admitted.push_back(r);
    size_t cached = 0;
    Entry *hit = nullptr;
    const Key *key = s->prefixes.longest(r->prompt, &hit);
    const float *tape = s->tape_row(*r);
    int32_t token = -1, rc = RG_OK;
    if (key) {
      const Key held = *key;  // the reference taken by longest() is dropped once the row has its own copy
      rc = s->be.snapshot_restore(s->be.ctx, hit->snapshot->handle, r->row);
      cached = (size_t)hit->snapshot->length;
      if (!rc && cached == r->prompt.size()) {
        rc = s->be.select(s->be.ctx, hit->logits.data(), r->temperature, tape, &token);
        s->prefixes.release(held);
        if (rc) return roll_back(rc);
        chosen[r->id] = token;
        continue;
      }
      s->prefixes.release(held);
      if (rc) return roll_back(rc);
    }
    if (r->greedy) {
      deferred.push_back({r, cached});
      continue;
    }
    rc = s->be.prefill_select(s->be.ctx, r->row, r->prompt.data() + cached, r->prompt.size() - cached, r->temperature, tape,
                              last.data(), &token);
    if (rc) return roll_back(rc);
    if ((rc = remember_prefix(r, last.data()))) return roll_back(rc);
    chosen[r->id] = token;
  }
  if (int32_t rc = flush()) return roll_back(rc);
  if (!decode_cols.empty()) {
    const int32_t n = (int32_t)decode_cols.size();
    std::vector<int32_t> rows(n), toks(n), ids(n);
    std::vector<float> temps(n, 0.f), tapes;
    for (int32_t i = 0; i < n; ++i) {
      const Request &r = *decode_cols[i];
      rows[i] = r.row;
      toks[i] = r.pending_token;
      if (!r.greedy) {
        if (tapes.empty()) tapes.assign((size_t)n * vocab, 0.f);
        temps[i] = r.temperature;
        memcpy(&tapes[(size_t)i * vocab], s->tape_row(r), vocab * sizeof(float));
      }
    }
    const int32_t rc = s->be.decode_rows(s->be.ctx, rows.data(), toks.data(), n, temps.data(), tapes.empty() ? nullptr : tapes.data(),
                                         ids.data());
    if (rc) return roll_back(rc);
    for (int32_t i = 0; i < n; ++i) chosen[decode_cols[i]->id] = ids[i];
  }
  // commit
  for (Request *r : selected) {
    const int32_t token = chosen.at(r->id);
    rg_token_event ev{r->id, r->arrival, (int32_t)r->generated.size(), token, 0, 0};
    r->generated.push_back(token);
    r->stopped = s->stop_ids.count(token) != 0;
    const bool complete = r->stopped || r->generated.size() == r->max_new;
    if (complete) {
      r->status = RG_REQUEST_COMPLETE;
      r->has_pending = false;
      s->release_row(*r);
      if (s->tokenizer) {
        std::vector<uint32_t> gen(r->generated.begin(), r->generated.end());
        rg_tok_error terr{};
        size_t bytes = 0;
        rg_b200_tokenizer_decode(s->tokenizer, gen.data(), gen.size(), nullptr, 0, &bytes, &terr);
        r->decoded.resize(bytes);
        if (bytes && rg_b200_tokenizer_decode(s->tokenizer, gen.data(), gen.size(), &r->decoded[0], bytes, &bytes, &terr) != RG_TOK_OK)
          r->decoded.clear();
      }
      r->has_result = true;
    } else {
      r->has_pending = true;
      r->pending_token = token;
    }
    ev.stopped = r->stopped;
    ev.complete = complete;
    events[(*n_events)++] = ev;
  }
  return RG_SERVING_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Fixed-size batch generation (src/models/transformer/batch_generation.rs:58-247) over the same
// table of session verbs.
// ---------------------------------------------------------------------------------------------
struct rg_batch_generator {
  rg_serving_backend be{};
  const rg_tokenizer *tokenizer = nullptr;
  int32_t batch = 0;
  std::set<int32_t> stop_ids;
  bool has_bos = false;
  int32_t bos_id = 0;
  std::vector<size_t> lengths;  // committed
  struct Sequence {
    std::vector<int32_t> prompt, generated;
    std::string decoded;
    bool stopped = false;
  };
  std::vector<Sequence> last;
  bool has_result = false;
};

namespace {

int32_t bfail(rg_batch_error *err, int32_t kind, int32_t row = 0, int64_t value = 0, int64_t value2 = 0) {
  if (err) *err = rg_batch_error{kind, row, value, value2};
  return kind;
}

// validate_sampling (batch_generation.rs:215-247)
int32_t check_batch_sampling(const rg_serving_sampling *sp, size_t steps, size_t batch, size_t vocab, rg_batch_error *err) {
  if (!sp || sp->greedy) return RG_BATCH_OK;
  if (!std::isfinite(sp->temperature) || sp->temperature <= 0.0f) return bfail(err, RG_BATCH_INVALID_TEMPERATURE);
  size_t required = 0;
  if (__builtin_mul_overflow(steps, batch, &required) || __builtin_mul_overflow(required, vocab, &required))
    return bfail(err, RG_BATCH_CONTEXT_OVERFLOW);
  if (sp->n_uniforms < required || (required && !sp->uniforms))
    return bfail(err, RG_BATCH_UNIFORM_TAPE_LENGTH, 0, (int64_t)required, (int64_t)(sp->uniforms ? sp->n_uniforms : 0));
  for (size_t i = 0; i < required; ++i) {
    const float u = sp->uniforms[i];
    if (!std::isfinite(u) || u < 0.0f || u >= 1.0f) return bfail(err, RG_BATCH_INVALID_UNIFORM, 0, (int64_t)i);
  }
  return RG_BATCH_OK;
}

// finish (batch_generation.rs:192-213): the decoded text of every row; a tokenizer failure fails the call
int32_t decode_rows_text(rg_batch_generator *g, std::vector<rg_batch_generator::Sequence> *seqs, rg_batch_error *err) {
  for (auto &q : *seqs) {
    q.decoded.clear();
    if (!g->tokenizer) continue;
    std::vector<uint32_t> gen(q.generated.begin(), q.generated.end());
    rg_tok_error terr{};
    size_t bytes = 0;
    int32_t trc = rg_b200_tokenizer_decode(g->tokenizer, gen.data(), gen.size(), nullptr, 0, &bytes, &terr);
    if (trc != RG_TOK_OK && !(trc == RG_TOK_INVALID_ARGUMENT && bytes > 0)) return bfail(err, RG_BATCH_TOKENIZER, 0, trc);
    q.decoded.resize(bytes);
    if (bytes && (trc = rg_b200_tokenizer_decode(g->tokenizer, gen.data(), gen.size(), &q.decoded[0], bytes, &bytes, &terr)) != RG_TOK_OK)
      return bfail(err, RG_BATCH_TOKENIZER, 0, trc);
  }
  return RG_BATCH_OK;
}

}  // namespace

extern "C" {

int32_t rg_b200_batch_generator_new_with_backend(const rg_serving_backend *backend, const rg_tokenizer *tokenizer, int32_t batch_size,
                                                 const rg_serving_options *o, rg_batch_generator **out, rg_batch_error *err) {
  if (!backend || !out || batch_size < 1) return bfail(err, RG_BATCH_INVALID_ARGUMENT);
  if (o && o->n_stop_ids && !o->stop_ids) return bfail(err, RG_BATCH_INVALID_ARGUMENT);
  auto g = new rg_batch_generator();
  g->be = *backend;
  g->tokenizer = tokenizer;
  g->batch = batch_size;
  if (o) {
    g->stop_ids.insert(o->stop_ids, o->stop_ids + o->n_stop_ids);
    g->has_bos = o->has_bos != 0;
    g->bos_id = o->bos_id;
  }
  g->lengths.assign((size_t)batch_size, 0);
  *out = g;
  return RG_BATCH_OK;
}

int32_t rg_b200_batch_generator_new(rg_session *session, const rg_tokenizer *tokenizer, int32_t batch_size,
                                    const rg_serving_options *options, rg_batch_generator **out, rg_batch_error *err) {
  if (!session) return bfail(err, RG_BATCH_INVALID_ARGUMENT);
  const rg_serving_backend be = session_backend(session);
  return rg_b200_batch_generator_new_with_backend(&be, tokenizer, batch_size, options, out, err);
}

void rg_b200_batch_generator_free(rg_batch_generator *g) { delete g; }

size_t rg_b200_batch_generator_cache_lengths(const rg_batch_generator *g, size_t *lengths, size_t cap) {
  if (!g) return 0;
  for (size_t i = 0; i < g->lengths.size() && i < cap && lengths; ++i) lengths[i] = g->lengths[i];
  return g->lengths.size();
}

void rg_b200_batch_generator_clear(rg_batch_generator *g) {
  if (g) std::fill(g->lengths.begin(), g->lengths.end(), (size_t)0);
}

int32_t rg_b200_batch_generate_ids(rg_batch_generator *g, const int32_t *ids, const size_t *lens, size_t n_prompts,
                                   size_t max_new, const rg_serving_sampling *sampling, rg_batch_error *err) {
  if (!g || (n_prompts && (!lens || !ids))) return bfail(err, RG_BATCH_INVALID_ARGUMENT);
  const size_t batch = (size_t)g->batch, vocab = (size_t)g->be.vocab, ctx = (size_t)g->be.max_context;
  if (n_prompts != batch) return bfail(err, RG_BATCH_BATCH_SIZE, 0, (int64_t)batch, (int64_t)n_prompts);
  for (size_t r = 0; r < batch; ++r) {
    if (lens[r] == 0) return bfail(err, RG_BATCH_EMPTY_PROMPT, (int32_t)r);
    size_t requested = 0;
    if (__builtin_add_overflow(lens[r], max_new, &requested)) return bfail(err, RG_BATCH_CONTEXT_OVERFLOW);
    if (requested > ctx) return bfail(err, RG_BATCH_CONTEXT_LENGTH, (int32_t)r, (int64_t)requested, (int64_t)ctx);
  }
  {
    size_t off = 0;
    for (size_t r = 0; r < batch; ++r)
      for (size_t i = 0; i < lens[r]; ++i, ++off)
        if (ids[off] < 0 || (size_t)ids[off] >= vocab) return bfail(err, RG_BATCH_TOKEN_OUT_OF_RANGE, (int32_t)r, ids[off], (int64_t)vocab);
  }
  int32_t rc = check_batch_sampling(sampling, max_new, batch, vocab, err);
  if (rc) return rc;
  const bool greedy = !sampling || sampling->greedy;
  const float temperature = greedy ? 0.0f : sampling->temperature;

  std::vector<rg_batch_generator::Sequence> seqs(batch);
  {
    size_t off = 0;
    for (size_t r = 0; r < batch; ++r) {
      seqs[r].prompt.assign(ids + off, ids + off + lens[r]);
      off += lens[r];
    }
  }
  auto commit = [&](const std::vector<size_t> &lengths) {
    g->last = std::move(seqs);
    g->has_result = true;
    g->lengths = lengths;
    return RG_BATCH_OK;
  };
  if (max_new == 0) {  // nothing runs and the cache stays as it is
    if ((rc = decode_rows_text(g, &seqs, err))) return rc;
    return commit(g->lengths);
  }

  // ---- staged generation: the rows start empty; nothing is committed before the end
  std::vector<size_t> staged(batch, 0);
  auto session_failed = [&](int32_t status) { return bfail(err, RG_BATCH_SESSION, 0, status); };
  std::vector<int32_t> rows(batch), sel(batch, -1);
  for (size_t r = 0; r < batch; ++r) {
    rows[r] = (int32_t)r;
    if ((rc = g->be.reset_row(g->be.ctx, (int32_t)r))) return session_failed(rc);
  }
  if (greedy && batch > 1 && g->be.prefill_rows) {
    std::vector<float> logits(batch * vocab);
    if ((rc = g->be.prefill_rows(g->be.ctx, rows.data(), ids, lens, (int32_t)batch, logits.data(), sel.data()))) return session_failed(rc);
  } else {
    std::vector<float> logits(vocab);
    size_t off = 0;
    for (size_t r = 0; r < batch; ++r) {
      const float *tape = greedy ? nullptr : sampling->uniforms + r * vocab;  // step 0, row r
      if ((rc = g->be.prefill_select(g->be.ctx, (int32_t)r, ids + off, lens[r], temperature, tape, logits.data(), &sel[r])))
        return session_failed(rc);
      off += lens[r];
    }
  }
  for (size_t r = 0; r < batch; ++r) staged[r] = lens[r];
  for (size_t step = 0; step < max_new; ++step) {
    // the tokens selected for this step; rows that stop here do not feed theirs back
    std::vector<int32_t> active, toks;
    for (size_t r = 0; r < batch; ++r) {
      if (seqs[r].stopped) continue;
      seqs[r].generated.push_back(sel[r]);
      seqs[r].stopped = g->stop_ids.count(sel[r]) != 0;
      if (!seqs[r].stopped) {
        active.push_back((int32_t)r);
        toks.push_back(sel[r]);
      }
    }
    if (step + 1 >= max_new || active.empty()) break;
    const int32_t n = (int32_t)active.size();
    std::vector<float> temps((size_t)n, temperature), tape;
    if (!greedy) {
      tape.resize((size_t)n * vocab);
      for (int32_t i = 0; i < n; ++i)
        memcpy(&tape[(size_t)i * vocab], sampling->uniforms + ((step + 1) * batch + (size_t)active[(size_t)i]) * vocab, vocab * sizeof(float));
    }
    std::vector<int32_t> out((size_t)n, -1);
    if ((rc = g->be.decode_rows(g->be.ctx, active.data(), toks.data(), n, temps.data(), greedy ? nullptr : tape.data(), out.data())))
      return session_failed(rc);
    for (int32_t i = 0; i < n; ++i) {
      sel[(size_t)active[(size_t)i]] = out[(size_t)i];
      staged[(size_t)active[(size_t)i]] += 1;
    }
  }
  if ((rc = decode_rows_text(g, &seqs, err))) return rc;
  return commit(staged);
}

int32_t rg_b200_batch_generate_texts(rg_batch_generator *g, const char *const *texts, const size_t *text_bytes, size_t n_prompts,
                                     size_t max_new, const rg_serving_sampling *sampling, rg_batch_error *err) {
  if (!g || (n_prompts && (!texts || !text_bytes))) return bfail(err, RG_BATCH_INVALID_ARGUMENT);
  if (!g->tokenizer) return bfail(err, RG_BATCH_TOKENIZER, 0, RG_TOK_INVALID_ARGUMENT);
  std::vector<int32_t> flat;
  std::vector<size_t> lens;
  for (size_t r = 0; r < n_prompts; ++r) {
    Key ids;
    if (g->has_bos) ids.push_back(g->bos_id);
    rg_serving_error serr{};
    if (encode_text(g->tokenizer, texts[r], text_bytes[r], &ids, &serr)) return bfail(err, RG_BATCH_TOKENIZER, (int32_t)r, serr.value);
    lens.push_back(ids.size());
    flat.insert(flat.end(), ids.begin(), ids.end());
  }
  return rg_b200_batch_generate_ids(g, flat.data(), lens.data(), n_prompts, max_new, sampling, err);
}

int32_t rg_b200_batch_sequence(const rg_batch_generator *g, size_t row, rg_serving_result *out) {
  if (!g || !out || !g->has_result || row >= g->last.size()) return RG_BATCH_INVALID_ARGUMENT;
  const auto &q = g->last[row];
  out->request_id = row;
  out->prompt_ids = q.prompt.data();
  out->n_prompt_ids = q.prompt.size();
  out->generated_ids = q.generated.data();
  out->n_generated_ids = q.generated.size();
  out->decoded = q.decoded.c_str();
  out->decoded_bytes = q.decoded.size();
  out->stopped = q.stopped ? 1 : 0;
  return RG_BATCH_OK;
}

}  // extern "C"
