"""Prompt-to-tokens facade on the CUDA session (``include/rg_b200_workflow.h``).

Mirrors rustgrad's ``LlamaPromptWorkflow`` (src/models/transformer/workflow.rs:18-147) with the
accelerated session behind it: ``from_gguf_bytes`` / ``from_path`` validate the file, build its
tokenizer and chat template and put the model on the GPU; ``generate`` and ``generate_chat`` take
text and return the rendered prompt, the token ids and the decoded text, greedy, on a fresh
sequence, optionally streaming the text token by token.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Iterable, Optional

import numpy as np

from . import _lib
from .session import CudaSessionTarget, RgError, check
from .tokenizer import ROLES


class _Output(C.Structure):
    _fields_ = [("n_prompt_ids", C.c_size_t), ("n_generated_ids", C.c_size_t), ("decoded_bytes", C.c_size_t),
                ("rendered_bytes", C.c_size_t), ("stopped", C.c_int32), ("tokenizer_status", C.c_int32)]


_CALLBACK = C.CFUNCTYPE(None, C.c_void_p, C.c_int32, C.POINTER(C.c_char), C.c_size_t)


def _L():
    L = _lib.load()
    if not getattr(L, "_workflow_bound", False):
        vp = C.c_void_p
        L.rg_b200_workflow_open.argtypes = [C.POINTER(C.c_uint8), C.c_size_t, C.POINTER(_lib.Options), C.POINTER(vp)]
        L.rg_b200_workflow_close.restype = None
        L.rg_b200_workflow_close.argtypes = [vp]
        L.rg_b200_workflow_session.restype = vp
        L.rg_b200_workflow_session.argtypes = [vp]
        L.rg_b200_workflow_tokenizer.restype = vp
        L.rg_b200_workflow_tokenizer.argtypes = [vp]
        L.rg_b200_workflow_generate_text.argtypes = [vp, C.c_char_p, C.c_size_t, C.c_size_t, _CALLBACK, vp, C.POINTER(_Output)]
        L.rg_b200_workflow_generate_chat.argtypes = [vp, C.POINTER(C.c_int32), C.POINTER(C.c_char_p), C.POINTER(C.c_size_t),
                                                     C.c_size_t, C.c_size_t, _CALLBACK, vp, C.POINTER(_Output)]
        for name in ("rg_b200_workflow_prompt_ids", "rg_b200_workflow_generated_ids"):
            getattr(L, name).restype = C.POINTER(C.c_int32)
            getattr(L, name).argtypes = [vp]
        for name in ("rg_b200_workflow_decoded", "rg_b200_workflow_rendered_prompt"):
            getattr(L, name).restype = C.POINTER(C.c_char)
            getattr(L, name).argtypes = [vp]
        L._workflow_bound = True
    return L


@dataclass
class LlamaGeneration:
    """LlamaGeneration (generation.rs:40-60)."""
    prompt_ids: list
    generated_ids: list
    decoded: str
    stopped: bool


@dataclass
class LlamaPromptOutput:
    """LlamaPromptOutput (workflow.rs:150-170)."""
    rendered_prompt: str
    generation: LlamaGeneration


class TokenizerFailure(RgError):
    """A tokenizer or chat-template failure inside a workflow request; ``tokenizer_status`` is the rg_tok_status."""

    def __init__(self, status: int, detail: str, tokenizer_status: int):
        super().__init__(status, detail)
        self.tokenizer_status = tokenizer_status


class LlamaPromptWorkflow:
    def __init__(self, handle):
        self._h = handle

    @classmethod
    def from_gguf_bytes(cls, data, target: Optional[CudaSessionTarget] = None) -> "LlamaPromptWorkflow":
        buf = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data
        opts = (target or CudaSessionTarget()).options()
        h = C.c_void_p()
        check(_L().rg_b200_workflow_open(buf.ctypes.data_as(C.POINTER(C.c_uint8)), buf.size, C.byref(opts), C.byref(h)))
        return cls(h)

    @classmethod
    def from_path(cls, path, target: Optional[CudaSessionTarget] = None) -> "LlamaPromptWorkflow":
        return cls.from_gguf_bytes(np.fromfile(path, dtype=np.uint8), target)

    def close(self):
        if getattr(self, "_h", None):
            _L().rg_b200_workflow_close(self._h)
            self._h = None

    __del__ = close

    def _finish(self, rc: int, out: _Output) -> LlamaPromptOutput:
        L = _L()
        if rc:
            detail = L.rg_b200_last_error().decode(errors="replace")
            if out.tokenizer_status:
                raise TokenizerFailure(rc, detail, out.tokenizer_status)
            check(rc)
        prompt = [L.rg_b200_workflow_prompt_ids(self._h)[i] for i in range(out.n_prompt_ids)]
        gen = [L.rg_b200_workflow_generated_ids(self._h)[i] for i in range(out.n_generated_ids)]
        decoded = C.string_at(L.rg_b200_workflow_decoded(self._h), out.decoded_bytes).decode("utf-8")
        rendered = C.string_at(L.rg_b200_workflow_rendered_prompt(self._h), out.rendered_bytes).decode("utf-8")
        return LlamaPromptOutput(rendered, LlamaGeneration(prompt, gen, decoded, bool(out.stopped)))

    @staticmethod
    def _callback(on_text: Optional[Callable[[int, str], None]]):
        if on_text is None:
            return _CALLBACK(0)

        def hook(_user, token_id, text, n):
            on_text(int(token_id), C.string_at(text, n).decode("utf-8"))

        return _CALLBACK(hook)

    def generate(self, prompt: str, max_new_tokens: int, on_text: Optional[Callable[[int, str], None]] = None) -> LlamaPromptOutput:
        """LlamaPromptWorkflow::generate: plain text prompt, greedy.  ``on_text(token_id, text)`` streams."""
        raw = prompt.encode("utf-8")
        out = _Output()
        cb = self._callback(on_text)
        rc = _L().rg_b200_workflow_generate_text(self._h, raw, len(raw), max_new_tokens, cb, None, C.byref(out))
        return self._finish(rc, out)

    def generate_chat(self, messages: Iterable[tuple[str, str]], max_new_tokens: int,
                      on_text: Optional[Callable[[int, str], None]] = None) -> LlamaPromptOutput:
        """LlamaPromptWorkflow::generate_chat: (role, content) messages through the checked template."""
        messages = list(messages)
        n = len(messages)
        roles = (C.c_int32 * max(n, 1))(*[ROLES[r] for r, _ in messages])
        raw = [c.encode("utf-8") for _, c in messages]
        strs = (C.c_char_p * max(n, 1))(*raw)
        lens = (C.c_size_t * max(n, 1))(*[len(r) for r in raw])
        out = _Output()
        cb = self._callback(on_text)
        rc = _L().rg_b200_workflow_generate_chat(self._h, roles, strs, lens, n, max_new_tokens, cb, None, C.byref(out))
        return self._finish(rc, out)
