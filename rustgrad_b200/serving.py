"""Continuous batching with a prefix cache over one ``LlamaCudaSession``: the scheduler of
rustgrad's ``LlamaServingScheduler`` (src/models/transformer/serving/mod.rs:371-690) with the same
verbs (submit_ids / submit_text / submit_chat / status / result / remove / step / prefix_stats /
invalidate_prefix_cache) and the same policy: requests are served in arrival order, at most
``batch_size`` per step, one token per selected request per step.  (The reference stages a step
and commits it as a whole; here a device call that fails raises, the session reports its typed
status, and the requests that were not reached keep their state.)

What differs, because the caches live in HBM rather than in per-request host tensors:

* a request keeps one cache row of the session from its first step to its last, instead of a
  batch being rebuilt from snapshots at every step;
* a prefix entry is taken when a prompt has been prefilled (and for a prompt extended from an
  entry), as a device-to-device copy of the row's K/V; decode steps do not add entries (the
  reference inserts one per computed step and lets its byte budget evict them);
* decode columns of one step run as ONE launch sequence over all running rows; newly admitted
  prompts are prefilled one after the other in the same step.

All device work goes through the C ABI (``rg_b200_prefill_select``, ``rg_b200_decode_rows``,
``rg_b200_select``, ``rg_b200_kv_snapshot_*``); this module only decides what runs.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from . import _lib
from .session import LlamaCudaSession, check


class ServingError(Exception):
    """LlamaServingError (serving/mod.rs:792-860) by kind."""

    def __init__(self, kind: str, **detail):
        self.kind, self.detail = kind, detail
        super().__init__(f"{kind}: {detail}")


@dataclass
class Sampling:
    """LlamaServingSampling (serving/mod.rs:28-38): greedy, or Gumbel-max with an explicit
    row-major [generation_step, vocabulary] uniform tape."""
    temperature: Optional[float] = None
    uniforms: Optional[np.ndarray] = None

    @property
    def greedy(self) -> bool:
        return self.temperature is None


@dataclass
class GenerationConfig:
    max_new_tokens: int
    sampling: Sampling = field(default_factory=Sampling)


@dataclass
class TokenEvent:
    """LlamaTokenEvent (serving/mod.rs:98-129)."""
    request_id: int
    arrival_order: int
    generation_step: int
    token_id: int
    stopped: bool
    complete: bool


@dataclass
class ServingResult:
    """LlamaServingResult (serving/mod.rs:131-155)."""
    request_id: int
    prompt_ids: list
    generated_ids: list
    decoded: str
    stopped: bool


class _Snapshot:
    """A device K/V copy shared by the cache and by requests that lean on it."""

    def __init__(self, session: LlamaCudaSession, row: int, length: int):
        self._L = _lib.load()
        self._h = C.c_void_p()
        check(self._L.rg_b200_kv_snapshot_create(session._h, row, length, C.byref(self._h)))
        self.length = length
        self.bytes = int(self._L.rg_b200_kv_snapshot_bytes(self._h))

    def restore(self, session: LlamaCudaSession, row: int) -> None:
        check(self._L.rg_b200_kv_snapshot_restore(session._h, self._h, row))

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.rg_b200_kv_snapshot_free(self._h)
            self._h = None


@dataclass
class _Entry:
    generation: int
    snapshot: _Snapshot
    logits: np.ndarray
    bytes: int
    last_used: int
    references: int = 0


class _PrefixCache:
    """PrefixCache (serving/mod.rs:192-352): longest-prefix lookup, LRU eviction of unreferenced
    entries under an entry and a byte budget, generation counter for invalidation."""

    def __init__(self, max_entries: int, max_bytes: int):
        self.max_entries, self.max_bytes = max_entries, max_bytes
        self.generation = self.clock = self.bytes = 0
        self.hits = self.misses = self.stale_rejections = self.evictions = 0
        self.entries: dict[tuple, _Entry] = {}

    def stats(self) -> dict:
        return {"entries": len(self.entries), "bytes": self.bytes, "hits": self.hits, "misses": self.misses,
                "stale_rejections": self.stale_rejections, "evictions": self.evictions, "generation": self.generation}

    def invalidate(self) -> None:
        self.generation += 1
        self.bytes = 0
        self.entries.clear()

    def release(self, key) -> None:
        e = self.entries.get(key)
        if e is not None:
            e.references = max(0, e.references - 1)

    def longest(self, tokens: list):
        for key in [k for k, e in self.entries.items() if e.generation != self.generation]:
            self.bytes -= self.entries.pop(key).bytes
            self.stale_rejections += 1
        best = None
        for key in self.entries:
            if len(key) <= len(tokens) and tuple(tokens[: len(key)]) == key and (best is None or len(key) > len(best)):
                best = key
        if best is None:
            self.misses += 1
            return None
        self.clock += 1
        e = self.entries[best]
        e.last_used = self.clock
        e.references += 1
        self.hits += 1
        return best, e.snapshot, e.logits

    def insert(self, tokens: list, snapshot: _Snapshot, logits: np.ndarray) -> bool:
        if self.max_entries == 0 or self.max_bytes == 0:
            return False
        size = snapshot.bytes + logits.size * 4 + len(tokens) * 4
        if size > self.max_bytes:
            return False
        key = tuple(tokens)
        old = self.entries.pop(key, None)
        if old is not None:
            self.bytes -= old.bytes
        while len(self.entries) >= self.max_entries or self.bytes + size > self.max_bytes:
            free = [(e.last_used, k) for k, e in self.entries.items() if e.references == 0]
            if not free:
                return False
            _, victim = min(free)
            self.bytes -= self.entries.pop(victim).bytes
            self.evictions += 1
        self.clock += 1
        self.bytes += size
        self.entries[key] = _Entry(self.generation, snapshot, logits, size, self.clock)
        return True


@dataclass
class _Request:
    id: int
    arrival: int
    prompt: list
    config: GenerationConfig
    status: str  # "queued" | "running" | "complete"
    generated: list = field(default_factory=list)
    stopped: bool = False
    row: Optional[int] = None
    cached: int = 0  # positions of prompt + generated already in the row
    prefix_reference: Optional[tuple] = None
    pending_token: Optional[int] = None
    result: Optional[ServingResult] = None


class LlamaServingScheduler:
    def __init__(self, session: LlamaCudaSession, tokenizer=None, batch_size: int = 1, prefix_max_entries: int = 0,
                 prefix_max_bytes: int = 0, stop_ids=(), bos_id: Optional[int] = None, max_rows: Optional[int] = None):
        if batch_size == 0:
            raise ServingError("EmptyBatch")
        self.session, self.tokenizer, self.batch_size = session, tokenizer, batch_size
        self.stop_ids, self.bos_id = set(int(t) for t in stop_ids), bos_id
        self._rows = list(range(max_rows if max_rows is not None else batch_size))
        if len(self._rows) < batch_size:
            raise ServingError("EmptyBatch", rows=len(self._rows), batch_size=batch_size)
        self._free_rows = list(self._rows)
        self._next_id = self._next_arrival = 0
        self._order: list[int] = []
        self._requests: dict[int, _Request] = {}
        self._prefixes = _PrefixCache(prefix_max_entries, prefix_max_bytes)
        self._L = _lib.load()

    # ---- admission (serving/mod.rs:408-477, validate_request :726-790) ------------------------
    def submit_ids(self, prompt, config: GenerationConfig) -> int:
        prompt = [int(t) for t in prompt]
        vocab, ctx = self.session.vocab_size(), self.session.max_context()
        if not prompt:
            raise ServingError("EmptyPrompt")
        requested = len(prompt) + config.max_new_tokens
        if requested > ctx:
            raise ServingError("ContextLength", requested=requested, maximum=ctx)
        for t in prompt:
            if t < 0 or t >= vocab:
                raise ServingError("TokenOutOfRange", token=t, vocab=vocab)
        s = config.sampling
        if not s.greedy:
            if not math.isfinite(s.temperature) or s.temperature <= 0.0:
                raise ServingError("InvalidTemperature")
            required = config.max_new_tokens * vocab
            flat = np.zeros(0, np.float32) if s.uniforms is None else np.ascontiguousarray(s.uniforms, dtype=np.float32).ravel()
            if flat.size < required:
                raise ServingError("UniformTapeLength", required=required, actual=int(flat.size))
            u = flat[:required].reshape(config.max_new_tokens, vocab)
            bad = np.flatnonzero(~np.isfinite(u.ravel()) | (u.ravel() < 0.0) | (u.ravel() >= 1.0))
            if bad.size:
                raise ServingError("InvalidUniform", index=int(bad[0]))
            config = GenerationConfig(config.max_new_tokens, Sampling(float(s.temperature), u))
        rid = self._next_id
        self._next_id += 1
        arrival = self._next_arrival
        self._next_arrival += 1
        done = config.max_new_tokens == 0
        req = _Request(rid, arrival, prompt, config, "complete" if done else "queued")
        if done:
            req.result = ServingResult(rid, list(prompt), [], "", False)
        self._requests[rid] = req
        self._order.append(rid)
        return rid

    def submit_text(self, prompt: str, config: GenerationConfig) -> int:
        ids = self.tokenizer.encode(prompt)
        if self.bos_id is not None:
            ids.insert(0, self.bos_id)
        return self.submit_ids(ids, config)

    def submit_chat(self, template, messages, config: GenerationConfig) -> int:
        return self.submit_ids(self.tokenizer.encode(template.render(self.tokenizer, messages, True)), config)

    def status(self, rid: int) -> Optional[str]:
        r = self._requests.get(rid)
        return None if r is None else r.status

    def result(self, rid: int) -> Optional[ServingResult]:
        r = self._requests.get(rid)
        return None if r is None else r.result

    def completed_results(self):
        return [self._requests[i].result for i in self._order if self._requests[i].result is not None]

    def pending(self) -> int:
        return sum(1 for r in self._requests.values() if r.status != "complete")

    def prefix_stats(self) -> dict:
        return self._prefixes.stats()

    def remove(self, rid: int) -> bool:
        r = self._requests.pop(rid, None)
        if r is None:
            return False
        if r.prefix_reference is not None:
            self._prefixes.release(r.prefix_reference)
        self._release_row(r)
        self._order.remove(rid)
        return True

    def invalidate_prefix_cache(self) -> None:
        self._prefixes.invalidate()
        for r in self._requests.values():
            r.prefix_reference = None

    def _release_row(self, r: _Request) -> None:
        if r.row is not None:
            check(self._L.rg_b200_reset_row(self.session._h, r.row))
            self._free_rows.append(r.row)
            self._free_rows.sort()
            r.row = None

    # ---- one step (serving/mod.rs:557-690) ----------------------------------------------------
    def step(self) -> list[TokenEvent]:
        selected = [self._requests[i] for i in self._order if self._requests[i].status != "complete"][: self.batch_size]
        if not selected:
            return []
        vocab = self.session.vocab_size()
        chosen: dict[int, int] = {}
        decode_cols = []
        for r in selected:
            r.status = "running"
            if r.row is None:
                r.row = self._free_rows.pop(0)
            if r.pending_token is not None:
                decode_cols.append(r)
                continue
            # a new request: lean on the longest cached prefix, prefill what is left
            hit = self._prefixes.longest(r.prompt)
            logits = None
            if hit is not None:
                key, snapshot, cached_logits = hit
                r.prefix_reference = key
                snapshot.restore(self.session, r.row)
                r.cached = snapshot.length
                if snapshot.length == len(r.prompt):
                    logits = cached_logits
            temp, tape = self._tape_row(r)
            if logits is not None:
                ids = np.empty(1, dtype=np.int32)
                t = np.array([temp], dtype=np.float32)
                check(self._L.rg_b200_select(self.session._h, _f32(np.ascontiguousarray(logits)), 1, _f32(t),
                                             _f32(tape) if tape is not None else None, _i32(ids)))
                chosen[r.id] = int(ids[0])
                self._prefixes.release(r.prefix_reference)  # the row holds its own copy of the prefix now
                r.prefix_reference = None
            else:
                rest = np.ascontiguousarray(r.prompt[r.cached:], dtype=np.int32)
                last = np.empty(vocab, dtype=np.float32)
                sel = C.c_int32(0)
                check(self._L.rg_b200_prefill_select(self.session._h, r.row, _i32(rest), rest.size, float(temp),
                                                     _f32(tape) if tape is not None else None, _f32(last), C.byref(sel)))
                if r.prefix_reference is not None:
                    self._prefixes.release(r.prefix_reference)
                    r.prefix_reference = None
                r.cached = len(r.prompt)
                if self._prefixes.max_entries and self._prefixes.max_bytes:
                    self._prefixes.insert(list(r.prompt), _Snapshot(self.session, r.row, r.cached), last)
                chosen[r.id] = int(sel.value)
        if decode_cols:
            n = len(decode_cols)
            rows = np.array([r.row for r in decode_cols], dtype=np.int32)
            toks = np.array([r.pending_token for r in decode_cols], dtype=np.int32)
            temps = np.zeros(n, dtype=np.float32)
            tapes = None
            for i, r in enumerate(decode_cols):
                temp, tape = self._tape_row(r)
                if tape is not None:
                    if tapes is None:
                        tapes = np.zeros((n, vocab), dtype=np.float32)
                    temps[i], tapes[i] = temp, tape
            ids = np.empty(n, dtype=np.int32)
            check(self._L.rg_b200_decode_rows(self.session._h, _i32(rows), _i32(toks), n, _f32(temps),
                                              _f32(tapes) if tapes is not None else None, None, _i32(ids)))
            for i, r in enumerate(decode_cols):
                r.cached += 1
                r.pending_token = None
                chosen[r.id] = int(ids[i])
        events = []
        for r in selected:
            token = chosen[r.id]
            step = len(r.generated)
            r.generated.append(token)
            r.stopped = token in self.stop_ids
            complete = r.stopped or len(r.generated) == r.config.max_new_tokens
            if complete:
                if r.prefix_reference is not None:
                    self._prefixes.release(r.prefix_reference)
                    r.prefix_reference = None
                r.status = "complete"
                self._release_row(r)
                decoded = self.tokenizer.decode(r.generated) if self.tokenizer is not None else ""
                r.result = ServingResult(r.id, list(r.prompt), list(r.generated), decoded, r.stopped)
            else:
                r.pending_token = token
            events.append(TokenEvent(r.id, r.arrival, step, token, r.stopped, complete))
        return events

    def _tape_row(self, r: _Request):
        s = r.config.sampling
        if s.greedy:
            return 0.0, None
        return s.temperature, np.ascontiguousarray(s.uniforms[len(r.generated)])


def _f32(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _i32(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))
