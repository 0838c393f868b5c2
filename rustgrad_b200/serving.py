"""Continuous batching with a prefix cache over one ``LlamaCudaSession``: the verbs of rustgrad's
``LlamaServingScheduler`` (src/models/transformer/serving/mod.rs:371-690) -- submit_ids /
submit_text / submit_chat / status / result / remove / step / prefix_stats /
invalidate_prefix_cache / rebind -- bound to the scheduler of ``include/rg_b200_serving.h``.

The policy (arrival order, batch size, cache rows, prefix cache, admission checks) is compiled code
in the library; this module only converts arguments and results.  ``ServingBackend`` lets a test
drive that policy through a table of Python callables instead of a device session.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from . import _lib
from .tokenizer import ROLES

KINDS = ["Ok", "EmptyBatch", "EmptyPrompt", "ContextLength", "TokenOutOfRange", "InvalidTemperature", "UniformTapeLength",
         "InvalidUniform", "UnknownRequest", "Session", "Tokenizer", "InvalidArgument", "NotComplete", "ActiveRequests"]
STATUS = ["queued", "running", "complete"]
f32p, i32p, vp = C.POINTER(C.c_float), C.POINTER(C.c_int32), C.c_void_p


class _Error(C.Structure):
    _fields_ = [("kind", C.c_int32), ("value", C.c_int64), ("value2", C.c_int64)]


class _Options(C.Structure):
    _fields_ = [("batch_size", C.c_int32), ("max_rows", C.c_int32), ("prefix_max_entries", C.c_size_t),
                ("prefix_max_bytes", C.c_size_t), ("stop_ids", i32p), ("n_stop_ids", C.c_size_t), ("has_bos", C.c_int32),
                ("bos_id", C.c_int32)]


class _Sampling(C.Structure):
    _fields_ = [("greedy", C.c_int32), ("temperature", C.c_float), ("uniforms", f32p), ("n_uniforms", C.c_size_t)]


class _Event(C.Structure):
    _fields_ = [("request_id", C.c_uint64), ("arrival_order", C.c_uint64), ("generation_step", C.c_int32),
                ("token_id", C.c_int32), ("stopped", C.c_int32), ("complete", C.c_int32)]


class _Result(C.Structure):
    _fields_ = [("request_id", C.c_uint64), ("prompt_ids", i32p), ("n_prompt_ids", C.c_size_t), ("generated_ids", i32p),
                ("n_generated_ids", C.c_size_t), ("decoded", C.c_char_p), ("decoded_bytes", C.c_size_t), ("stopped", C.c_int32)]


class _BatchError(C.Structure):
    _fields_ = [("kind", C.c_int32), ("row", C.c_int32), ("value", C.c_int64), ("value2", C.c_int64)]


class _Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("entries", "bytes", "hits", "misses", "stale_rejections", "evictions", "generation")]


_RESET = C.CFUNCTYPE(C.c_int32, vp, C.c_int32)
_PREFILL = C.CFUNCTYPE(C.c_int32, vp, C.c_int32, i32p, C.c_size_t, C.c_float, f32p, f32p, i32p)
_DECODE = C.CFUNCTYPE(C.c_int32, vp, i32p, i32p, C.c_int32, f32p, f32p, i32p)
_SELECT = C.CFUNCTYPE(C.c_int32, vp, f32p, C.c_float, f32p, i32p)
_SNAP_CREATE = C.CFUNCTYPE(C.c_int32, vp, C.c_int32, C.c_int32, C.POINTER(vp), C.POINTER(C.c_size_t))
_SNAP_RESTORE = C.CFUNCTYPE(C.c_int32, vp, vp, C.c_int32)
_SNAP_FREE = C.CFUNCTYPE(None, vp, vp)
_PREFILL_ROWS = C.CFUNCTYPE(C.c_int32, vp, i32p, i32p, C.POINTER(C.c_size_t), C.c_int32, f32p, i32p)


class _Backend(C.Structure):
    _fields_ = [("ctx", vp), ("vocab", C.c_int32), ("max_context", C.c_int32), ("reset_row", _RESET),
                ("prefill_select", _PREFILL), ("decode_rows", _DECODE), ("select", _SELECT), ("snapshot_create", _SNAP_CREATE),
                ("snapshot_restore", _SNAP_RESTORE), ("snapshot_free", _SNAP_FREE), ("prefill_rows", _PREFILL_ROWS)]


def _L():
    L = _lib.load()
    if getattr(L, "_serving_bound", False):
        return L
    ep, u64p = C.POINTER(_Error), C.POINTER(C.c_uint64)
    L.rg_b200_scheduler_new.argtypes = [vp, vp, C.POINTER(_Options), C.POINTER(vp), ep]
    L.rg_b200_scheduler_new_with_backend.argtypes = [C.POINTER(_Backend), vp, C.POINTER(_Options), C.POINTER(vp), ep]
    L.rg_b200_scheduler_free.restype = None
    L.rg_b200_scheduler_free.argtypes = [vp]
    L.rg_b200_scheduler_submit_ids.argtypes = [vp, i32p, C.c_size_t, C.c_size_t, C.POINTER(_Sampling), u64p, ep]
    L.rg_b200_scheduler_submit_text.argtypes = [vp, C.c_char_p, C.c_size_t, C.c_size_t, C.POINTER(_Sampling), u64p, ep]
    L.rg_b200_scheduler_submit_chat.argtypes = [vp, i32p, C.POINTER(C.c_char_p), C.POINTER(C.c_size_t), C.c_size_t, C.c_size_t,
                                                C.POINTER(_Sampling), u64p, ep]
    L.rg_b200_scheduler_status.argtypes = [vp, C.c_uint64, i32p]
    L.rg_b200_scheduler_result.argtypes = [vp, C.c_uint64, C.POINTER(_Result)]
    L.rg_b200_scheduler_remove.argtypes = [vp, C.c_uint64]
    L.rg_b200_scheduler_pending.restype = C.c_size_t
    L.rg_b200_scheduler_pending.argtypes = [vp]
    L.rg_b200_scheduler_completed.restype = C.c_size_t
    L.rg_b200_scheduler_completed.argtypes = [vp, u64p, C.c_size_t]
    L.rg_b200_scheduler_prefix_stats.restype = None
    L.rg_b200_scheduler_prefix_stats.argtypes = [vp, C.POINTER(_Stats)]
    L.rg_b200_scheduler_invalidate_prefix_cache.restype = None
    L.rg_b200_scheduler_invalidate_prefix_cache.argtypes = [vp]
    L.rg_b200_scheduler_step.argtypes = [vp, C.POINTER(_Event), C.c_size_t, C.POINTER(C.c_size_t), ep]
    L.rg_b200_scheduler_rebind.argtypes = [vp, vp, vp, C.POINTER(_Options), C.POINTER(C.c_int32), ep]
    L.rg_b200_scheduler_rebind_with_backend.argtypes = [vp, C.POINTER(_Backend), vp, C.POINTER(_Options), C.POINTER(C.c_int32), ep]
    bep = C.POINTER(_BatchError)
    L.rg_b200_batch_generator_new.argtypes = [vp, vp, C.c_int32, C.POINTER(_Options), C.POINTER(vp), bep]
    L.rg_b200_batch_generator_new_with_backend.argtypes = [C.POINTER(_Backend), vp, C.c_int32, C.POINTER(_Options), C.POINTER(vp), bep]
    L.rg_b200_batch_generator_free.restype = None
    L.rg_b200_batch_generator_free.argtypes = [vp]
    L.rg_b200_batch_generator_cache_lengths.restype = C.c_size_t
    L.rg_b200_batch_generator_cache_lengths.argtypes = [vp, C.POINTER(C.c_size_t), C.c_size_t]
    L.rg_b200_batch_generator_clear.restype = None
    L.rg_b200_batch_generator_clear.argtypes = [vp]
    L.rg_b200_batch_generate_ids.argtypes = [vp, i32p, C.POINTER(C.c_size_t), C.c_size_t, C.c_size_t, C.POINTER(_Sampling), bep]
    L.rg_b200_batch_generate_texts.argtypes = [vp, C.POINTER(C.c_char_p), C.POINTER(C.c_size_t), C.c_size_t, C.c_size_t,
                                               C.POINTER(_Sampling), bep]
    L.rg_b200_batch_sequence.argtypes = [vp, C.c_size_t, C.POINTER(_Result)]
    L._serving_bound = True
    return L


class ServingError(Exception):
    """LlamaServingError (serving/mod.rs:792-860) by kind; ``value`` / ``value2`` carry its numbers
    (requested and maximum length, token and vocabulary, required and actual tape length, the
    status of the session verb that failed)."""

    def __init__(self, kind: str, value: int = 0, value2: int = 0, text: str = ""):
        self.kind, self.value, self.value2 = kind, value, value2
        super().__init__(f"{kind}: {value}, {value2}" + (f" ({text})" if text else ""))


def _raise(rc: int, err: _Error):
    text = _lib.load().rg_b200_last_error().decode(errors="replace") if rc == 9 else ""
    raise ServingError(KINDS[rc] if 0 <= rc < len(KINDS) else str(rc), err.value, err.value2, text)


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


class ServingBackend:
    """The session verbs of a step as Python callables, for driving the compiled policy without a
    device.  Subclass and override; every verb returns an ``rg_status`` (0 = ok)."""
    vocab = 0
    max_context = 0

    def reset_row(self, row: int) -> int:
        return 0

    def prefill_select(self, row: int, ids: list, temperature: float, uniforms, last_logits: np.ndarray):
        """Returns (status, selected token); fills last_logits [vocab]."""
        raise NotImplementedError

    def decode_rows(self, rows: list, tokens: list, temperatures: list, uniforms):
        """Returns (status, ids)."""
        raise NotImplementedError

    def select(self, logits: np.ndarray, temperature: float, uniforms):
        """Returns (status, id)."""
        raise NotImplementedError

    def snapshot_create(self, row: int, length: int):
        """Returns (status, handle > 0, bytes)."""
        raise NotImplementedError

    def snapshot_restore(self, handle: int, row: int) -> int:
        raise NotImplementedError

    def snapshot_free(self, handle: int) -> None:
        pass

    prefill_rows = None
    """Optional: ``prefill_rows(rows, prompts, last_logits [n, vocab]) -> (status, ids)`` for several
    greedy prompts in one pass; without it the scheduler prefills them one after the other."""

    def _table(self) -> _Backend:
        # one table per object: the scheduler recognises a session by its verbs (rebind)
        cached = getattr(self, "_table_cache", None)
        if cached is not None:
            return cached
        v = self.vocab

        def tape(p, n):
            return None if not p else np.ctypeslib.as_array(p, shape=(n,)).copy()

        def prefill(_, row, ids, n, temp, uni, last, sel):
            rc, tok = self.prefill_select(row, [ids[i] for i in range(n)], temp, tape(uni, v), np.ctypeslib.as_array(last, shape=(v,)))
            sel[0] = tok
            return rc

        def decode(_, rows, toks, n, temps, uni, out):
            rc, ids = self.decode_rows([rows[i] for i in range(n)], [toks[i] for i in range(n)], [temps[i] for i in range(n)],
                                       None if not uni else tape(uni, n * v).reshape(n, v))
            for i, t in enumerate(ids):
                out[i] = t
            return rc

        def select(_, logits, temp, uni, out):
            rc, tok = self.select(np.ctypeslib.as_array(logits, shape=(v,)).copy(), temp, tape(uni, v))
            out[0] = tok
            return rc

        def snap_create(_, row, length, handle, nbytes):
            rc, h, b = self.snapshot_create(row, length)
            handle[0], nbytes[0] = h, b
            return rc

        def prefill_rows(_, rows, ids, lens, n, last, sel):
            prompts, off = [], 0
            for i in range(n):
                prompts.append([ids[off + j] for j in range(lens[i])])
                off += lens[i]
            rc, out = self.prefill_rows([rows[i] for i in range(n)], prompts, np.ctypeslib.as_array(last, shape=(n, v)))
            for i, t in enumerate(out):
                sel[i] = t
            return rc

        self._keep = [_RESET(lambda _, row: self.reset_row(row)), _PREFILL(prefill), _DECODE(decode), _SELECT(select),
                      _SNAP_CREATE(snap_create), _SNAP_RESTORE(lambda _, h, row: self.snapshot_restore(h, row)),
                      _SNAP_FREE(lambda _, h: self.snapshot_free(h))]
        if self.prefill_rows is not None:
            self._keep.append(_PREFILL_ROWS(prefill_rows))
        self._table_cache = _Backend(None, self.vocab, self.max_context, *self._keep)
        return self._table_cache


class LlamaServingScheduler:
    def __init__(self, session, tokenizer=None, batch_size: int = 1, prefix_max_entries: int = 0, prefix_max_bytes: int = 0,
                 stop_ids=(), bos_id: Optional[int] = None, max_rows: Optional[int] = None):
        self._lib = _L()
        self.session, self.tokenizer = session, tokenizer
        stops = np.array(sorted(int(t) for t in stop_ids), dtype=np.int32)
        opts = _Options(batch_size, 0 if max_rows is None else max_rows, prefix_max_entries, prefix_max_bytes,
                        stops.ctypes.data_as(i32p), stops.size, int(bos_id is not None), bos_id or 0)
        if max_rows is not None and max_rows <= 0:
            raise ServingError("EmptyBatch", max_rows, batch_size)
        self._h, err = vp(), _Error()
        tok = tokenizer._h if tokenizer is not None else None
        if isinstance(session, ServingBackend):
            self._table = session._table()
            rc = self._lib.rg_b200_scheduler_new_with_backend(C.byref(self._table), tok, C.byref(opts), C.byref(self._h), C.byref(err))
        else:
            rc = self._lib.rg_b200_scheduler_new(session._h, tok, C.byref(opts), C.byref(self._h), C.byref(err))
        if rc:
            self._h = None
            _raise(rc, err)
        self.batch_size = batch_size

    def close(self):
        if getattr(self, "_h", None):
            self._lib.rg_b200_scheduler_free(self._h)
            self._h = None

    __del__ = close

    @staticmethod
    def _sampling(config: GenerationConfig):
        s = config.sampling
        if s.greedy:
            return _Sampling(1, 0.0, None, 0), None
        flat = np.zeros(0, np.float32) if s.uniforms is None else np.ascontiguousarray(s.uniforms, dtype=np.float32).ravel()
        return _Sampling(0, float(s.temperature), flat.ctypes.data_as(f32p), flat.size), flat

    # ---- admission (serving/mod.rs:408-477) ----------------------------------------------------
    def submit_ids(self, prompt, config: GenerationConfig) -> int:
        ids = np.ascontiguousarray([int(t) for t in prompt], dtype=np.int32)
        sampling, _keep = self._sampling(config)
        rid, err = C.c_uint64(), _Error()
        rc = self._lib.rg_b200_scheduler_submit_ids(self._h, ids.ctypes.data_as(i32p), ids.size, config.max_new_tokens,
                                                    C.byref(sampling), C.byref(rid), C.byref(err))
        if rc:
            _raise(rc, err)
        return rid.value

    def submit_text(self, prompt: str, config: GenerationConfig) -> int:
        raw = prompt.encode("utf-8")
        sampling, _keep = self._sampling(config)
        rid, err = C.c_uint64(), _Error()
        rc = self._lib.rg_b200_scheduler_submit_text(self._h, raw, len(raw), config.max_new_tokens, C.byref(sampling),
                                                     C.byref(rid), C.byref(err))
        if rc:
            _raise(rc, err)
        return rid.value

    def submit_chat(self, messages, config: GenerationConfig) -> int:
        """(role, content) messages through the one checked chat template, generation prompt added."""
        messages = list(messages)
        n = len(messages)
        roles = (C.c_int32 * max(n, 1))(*[ROLES[r] for r, _ in messages])
        raw = [c.encode("utf-8") for _, c in messages]
        strs = (C.c_char_p * max(n, 1))(*raw)
        lens = (C.c_size_t * max(n, 1))(*[len(r) for r in raw])
        sampling, _keep = self._sampling(config)
        rid, err = C.c_uint64(), _Error()
        rc = self._lib.rg_b200_scheduler_submit_chat(self._h, roles, strs, lens, n, config.max_new_tokens, C.byref(sampling),
                                                     C.byref(rid), C.byref(err))
        if rc:
            _raise(rc, err)
        return rid.value

    def status(self, rid: int) -> Optional[str]:
        st = C.c_int32()
        return None if self._lib.rg_b200_scheduler_status(self._h, rid, C.byref(st)) else STATUS[st.value]

    def result(self, rid: int) -> Optional[ServingResult]:
        r = _Result()
        if self._lib.rg_b200_scheduler_result(self._h, rid, C.byref(r)):
            return None
        return ServingResult(r.request_id, [r.prompt_ids[i] for i in range(r.n_prompt_ids)],
                             [r.generated_ids[i] for i in range(r.n_generated_ids)],
                             C.string_at(r.decoded, r.decoded_bytes).decode("utf-8", "replace"), bool(r.stopped))

    def completed_results(self):
        n = self._lib.rg_b200_scheduler_completed(self._h, None, 0)
        ids = (C.c_uint64 * max(n, 1))()
        self._lib.rg_b200_scheduler_completed(self._h, ids, n)
        return [self.result(ids[i]) for i in range(n)]

    def pending(self) -> int:
        return self._lib.rg_b200_scheduler_pending(self._h)

    def prefix_stats(self) -> dict:
        st = _Stats()
        self._lib.rg_b200_scheduler_prefix_stats(self._h, C.byref(st))
        return {n: getattr(st, n) for n, _ in _Stats._fields_}

    def remove(self, rid: int) -> bool:
        return self._lib.rg_b200_scheduler_remove(self._h, rid) == 0

    def invalidate_prefix_cache(self) -> None:
        self._lib.rg_b200_scheduler_invalidate_prefix_cache(self._h)

    def rebind(self, session, tokenizer=None, stop_ids=None, bos_id: Optional[int] = None) -> bool:
        """LlamaServingScheduler::rebind (serving/mod.rs:528-547): an idle scheduler takes another session
        (or backend table) and tokenizer; True when the session differs, in which case every cached prefix
        was dropped.  ``stop_ids`` (with ``bos_id``) replaces the stop rule when given."""
        opts = None
        if stop_ids is not None:
            stops = np.array(sorted(int(t) for t in stop_ids), dtype=np.int32)
            opts = _Options(self.batch_size, 0, 0, 0, stops.ctypes.data_as(i32p), stops.size, int(bos_id is not None), bos_id or 0)
        changed, err = C.c_int32(), _Error()
        tok = tokenizer._h if tokenizer is not None else None
        if isinstance(session, ServingBackend):
            table = session._table()
            rc = self._lib.rg_b200_scheduler_rebind_with_backend(self._h, C.byref(table), tok, C.byref(opts) if opts else None,
                                                                 C.byref(changed), C.byref(err))
        else:
            table = None
            rc = self._lib.rg_b200_scheduler_rebind(self._h, session._h, tok, C.byref(opts) if opts else None,
                                                    C.byref(changed), C.byref(err))
        if rc:
            _raise(rc, err)
        # the callables of the old table stay alive until here: dropped prefixes were freed through them
        self.session, self.tokenizer, self._table = session, tokenizer, table
        return bool(changed.value)

    # ---- one step (serving/mod.rs:557-690) -----------------------------------------------------
    def step(self) -> list[TokenEvent]:
        events, n, err = (_Event * self.batch_size)(), C.c_size_t(), _Error()
        rc = self._lib.rg_b200_scheduler_step(self._h, events, self.batch_size, C.byref(n), C.byref(err))
        if rc:
            _raise(rc, err)
        return [TokenEvent(e.request_id, e.arrival_order, e.generation_step, e.token_id, bool(e.stopped), bool(e.complete))
                for e in events[: n.value]]


BATCH_KINDS = ["Ok", "Session", "InvalidTemperature", "Tokenizer", "BatchSize", "EmptyPrompt", "ContextOverflow", "ContextLength",
               "UniformTapeLength", "InvalidUniform", "TokenOutOfRange", "InvalidArgument"]


class BatchGenerationError(Exception):
    """LlamaBatchGenerationError (batch_generation.rs:251-279) by kind, with the row and the numbers it carries."""

    def __init__(self, kind, row=0, value=0, value2=0, text=""):
        super().__init__(f"{kind} row={row} value={value} value2={value2} {text}".strip())
        self.kind, self.row, self.value, self.value2, self.text = kind, row, value, value2, text


def _raise_batch(rc: int, err: _BatchError):
    text = _lib.load().rg_b200_last_error().decode(errors="replace") if rc == 1 else ""
    raise BatchGenerationError(BATCH_KINDS[rc] if 0 <= rc < len(BATCH_KINDS) else str(rc), err.row, err.value, err.value2, text)


class LlamaBatchGenerator:
    """LlamaBatchGenerator (src/models/transformer/batch_generation.rs:58-189) over a session (rows
    0 .. batch_size-1) or a ``ServingBackend`` table: every generate starts from empty rows, runs all prompts
    together and commits the row lengths only when everything succeeded.  ``sampling.uniforms`` is the
    row-major [step, batch, vocabulary] tape."""

    def __init__(self, session, tokenizer=None, batch_size: int = 1, stop_ids=(), bos_id: Optional[int] = None):
        self._lib = _L()
        self.session, self.tokenizer, self.batch_size = session, tokenizer, batch_size
        stops = np.array(sorted(int(t) for t in stop_ids), dtype=np.int32)
        opts = _Options(batch_size, 0, 0, 0, stops.ctypes.data_as(i32p), stops.size, int(bos_id is not None), bos_id or 0)
        self._h, err = vp(), _BatchError()
        tok = tokenizer._h if tokenizer is not None else None
        if isinstance(session, ServingBackend):
            self._table = session._table()
            rc = self._lib.rg_b200_batch_generator_new_with_backend(C.byref(self._table), tok, batch_size, C.byref(opts),
                                                                    C.byref(self._h), C.byref(err))
        else:
            rc = self._lib.rg_b200_batch_generator_new(session._h, tok, batch_size, C.byref(opts), C.byref(self._h), C.byref(err))
        if rc:
            self._h = None
            _raise_batch(rc, err)

    def close(self):
        if getattr(self, "_h", None):
            self._lib.rg_b200_batch_generator_free(self._h)
            self._h = None

    __del__ = close

    def cache_lengths(self) -> list:
        out = (C.c_size_t * self.batch_size)()
        n = self._lib.rg_b200_batch_generator_cache_lengths(self._h, out, self.batch_size)
        return [out[i] for i in range(n)]

    def clear(self) -> None:
        self._lib.rg_b200_batch_generator_clear(self._h)

    def _sequences(self):
        out = []
        for row in range(self.batch_size):
            r = _Result()
            if self._lib.rg_b200_batch_sequence(self._h, row, C.byref(r)):
                raise BatchGenerationError("InvalidArgument", row)
            out.append(ServingResult(r.request_id, [r.prompt_ids[i] for i in range(r.n_prompt_ids)],
                                     [r.generated_ids[i] for i in range(r.n_generated_ids)],
                                     C.string_at(r.decoded, r.decoded_bytes).decode("utf-8", "replace"), bool(r.stopped)))
        return out

    def generate_ids(self, prompts, max_new_tokens: int, sampling: Optional[Sampling] = None):
        prompts = [[int(t) for t in p] for p in prompts]
        flat = np.ascontiguousarray([t for p in prompts for t in p], dtype=np.int32)
        lens = (C.c_size_t * max(len(prompts), 1))(*[len(p) for p in prompts])
        sp, _keep = LlamaServingScheduler._sampling(GenerationConfig(max_new_tokens, sampling or Sampling()))
        err = _BatchError()
        rc = self._lib.rg_b200_batch_generate_ids(self._h, flat.ctypes.data_as(i32p), lens, len(prompts), max_new_tokens,
                                                  C.byref(sp), C.byref(err))
        if rc:
            _raise_batch(rc, err)
        return self._sequences()

    def generate_texts(self, prompts, max_new_tokens: int, sampling: Optional[Sampling] = None):
        raw = [p.encode("utf-8") for p in prompts]
        strs = (C.c_char_p * max(len(raw), 1))(*raw)
        lens = (C.c_size_t * max(len(raw), 1))(*[len(r) for r in raw])
        sp, _keep = LlamaServingScheduler._sampling(GenerationConfig(max_new_tokens, sampling or Sampling()))
        err = _BatchError()
        rc = self._lib.rg_b200_batch_generate_texts(self._h, strs, lens, len(raw), max_new_tokens, C.byref(sp), C.byref(err))
        if rc:
            _raise_batch(rc, err)
        return self._sequences()

