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
_GENERATE_CHAT = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_char_p), C.POINTER(C.c_size_t), C.c_size_t,
                             C.c_size_t, _CALLBACK, C.c_void_p, C.POINTER(_Output))
_DECODED = C.CFUNCTYPE(C.c_void_p, C.c_void_p)


class _ChatBackend(C.Structure):
    _fields_ = [("ctx", C.c_void_p), ("generate_chat", _GENERATE_CHAT), ("decoded", _DECODED)]


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
        L.rg_b200_conversation_new.argtypes = [vp, C.POINTER(vp)]
        L.rg_b200_conversation_new_with_backend.argtypes = [C.POINTER(_ChatBackend), C.POINTER(vp)]
        L.rg_b200_conversation_free.restype = None
        L.rg_b200_conversation_free.argtypes = [vp]
        L.rg_b200_conversation_history_len.restype = C.c_size_t
        L.rg_b200_conversation_history_len.argtypes = [vp]
        L.rg_b200_conversation_message.argtypes = [vp, C.c_size_t, C.POINTER(C.c_int32), C.POINTER(C.POINTER(C.c_char)),
                                                   C.POINTER(C.c_size_t)]
        L.rg_b200_conversation_cache_len.restype = C.c_size_t
        L.rg_b200_conversation_cache_len.argtypes = [vp]
        L.rg_b200_conversation_reset.restype = None
        L.rg_b200_conversation_reset.argtypes = [vp]
        L.rg_b200_conversation_send.argtypes = [vp, C.c_char_p, C.c_size_t, C.c_size_t, _CALLBACK, vp, C.POINTER(_Output),
                                                C.POINTER(C.c_int32)]
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

    def conversation(self) -> "LlamaConversation":
        """LlamaPromptWorkflow::conversation (workflow.rs:136-139): a stateful transcript over this workflow."""
        return LlamaConversation(self)

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


ROLE_NAMES = {v: k for k, v in ROLES.items()}
CONVERSATION_KINDS = ["Ok", "EmptyInput", "Chat", "Generation", "InvalidArgument"]


class ConversationError(Exception):
    """LlamaConversationError (conversation.rs:86-91): ``EmptyInput``, ``Chat`` (detail = tokenizer status)
    or ``Generation`` (detail = session status)."""

    def __init__(self, kind: str, detail: int = 0, text: str = ""):
        super().__init__(f"{kind}: {detail}" + (f" ({text})" if text else ""))
        self.kind, self.detail, self.text = kind, detail, text


@dataclass
class LlamaConversationTurn:
    """LlamaConversationTurn (conversation.rs:9-27)."""
    user: tuple
    assistant: tuple
    generation: LlamaGeneration


class ChatBackend:
    """The workflow verbs of a turn as Python callables, for driving the compiled transcript logic without a
    device.  ``generate_chat(messages, max_new_tokens)`` returns ``(status, tokenizer_status, n_prompt_ids,
    generated_ids, decoded, stopped)``."""

    def generate_chat(self, messages, max_new_tokens):
        raise NotImplementedError

    def _table(self) -> _ChatBackend:
        def generate(_ctx, roles, contents, lens, n, max_new, _cb, _user, out):
            msgs = [(ROLE_NAMES[roles[i]], C.string_at(contents[i], lens[i]).decode("utf-8")) for i in range(n)]
            rc, tok, n_prompt, generated, decoded, stopped = self.generate_chat(msgs, max_new)
            self._last = decoded.encode("utf-8")
            self._generated = list(generated)
            out[0] = _Output(n_prompt, len(generated), len(self._last), 0, int(stopped), tok)
            return rc

        def decoded(_ctx):
            self._buf = C.create_string_buffer(self._last)
            return C.addressof(self._buf)

        self._keep = (_GENERATE_CHAT(generate), _DECODED(decoded))
        return _ChatBackend(None, *self._keep)


class LlamaConversation:
    """LlamaConversation (conversation.rs:29-85): the transcript lives in the library; ``send`` renders the
    committed history plus the new user message, generates greedily and commits both messages on success."""

    def __init__(self, workflow):
        self._workflow = workflow
        self._h = C.c_void_p()
        if isinstance(workflow, ChatBackend):
            self._table = workflow._table()
            rc = _L().rg_b200_conversation_new_with_backend(C.byref(self._table), C.byref(self._h))
        else:
            rc = _L().rg_b200_conversation_new(workflow._h, C.byref(self._h))
        if rc:
            self._h = None
            raise ConversationError(CONVERSATION_KINDS[rc])

    def close(self):
        if getattr(self, "_h", None):
            _L().rg_b200_conversation_free(self._h)
            self._h = None

    __del__ = close

    def history(self) -> list:
        L, out = _L(), []
        for i in range(L.rg_b200_conversation_history_len(self._h)):
            role, text, n = C.c_int32(), C.POINTER(C.c_char)(), C.c_size_t()
            L.rg_b200_conversation_message(self._h, i, C.byref(role), C.byref(text), C.byref(n))
            out.append((ROLE_NAMES[role.value], C.string_at(text, n.value).decode("utf-8")))
        return out

    def cache_len(self) -> int:
        return _L().rg_b200_conversation_cache_len(self._h)

    def reset(self) -> None:
        _L().rg_b200_conversation_reset(self._h)

    def send(self, content: str, max_new_tokens: int, on_text: Optional[Callable[[int, str], None]] = None) -> LlamaConversationTurn:
        raw = content.encode("utf-8")
        out, detail = _Output(), C.c_int32()
        cb = LlamaPromptWorkflow._callback(on_text)
        rc = _L().rg_b200_conversation_send(self._h, raw, len(raw), max_new_tokens, cb, None, C.byref(out), C.byref(detail))
        if rc:
            text = _L().rg_b200_last_error().decode(errors="replace") if rc in (2, 3) else ""
            raise ConversationError(CONVERSATION_KINDS[rc] if rc < len(CONVERSATION_KINDS) else str(rc), detail.value, text)
        user, assistant = self.history()[-2:]
        if isinstance(self._workflow, ChatBackend):
            gen = LlamaGeneration([], list(self._workflow._generated), assistant[1], bool(out.stopped))
        else:
            gen = self._workflow._finish(0, out).generation
        return LlamaConversationTurn(user, assistant, gen)

