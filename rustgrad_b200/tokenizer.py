"""Python mirror of rustgrad's ``SimpleTokenizer`` (src/tokenizer/mod.rs) over the C ABI of
``include/rg_b200_tokenizer.h``: same method names, same typed failures.  Host-side only.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Iterable, Optional

from . import _lib

PRESETS = ["llama3", "llama-v3", "llama-bpe", "qwen2", "olmo", "kimi-k2", "tekken", "glm4"]
# TokenizerErrorKind (src/tokenizer/mod.rs:103-139), indexed by rg_tok_status
KINDS = [
    "Ok", "InvalidArgument", "UnsupportedPreset", "MissingMetadata", "MalformedMetadata", "MetadataLengthMismatch",
    "TokenIdOutOfRange", "ConfiguredTokenIdOutOfRange", "InvalidNormalTokenCharacter", "EmptySpecialToken",
    "TokenNotFound", "UnknownTokenId",
    # LlamaChatError (src/models/transformer/chat.rs:163-174)
    "TemplateTooLong", "UnsupportedJinja", "UnsupportedTemplate", "ChatUnsupportedPreset", "MessageTooLong", "ChatTooLong",
    "ChatOverflow",
]


class _Config(C.Structure):
    _fields_ = [("preset", C.c_int32), ("has_bos", C.c_int32), ("bos_id", C.c_uint32), ("eos_id", C.c_uint32),
                ("has_eot", C.c_int32), ("eot_id", C.c_uint32)]


class _Error(C.Structure):
    _fields_ = [("status", C.c_int32), ("value", C.c_uint64), ("value2", C.c_uint64), ("text_len", C.c_size_t),
                ("text", C.c_char * 128)]


class TokenizerError(Exception):
    """A tokenizer failure whose kind can be matched without parsing text (mod.rs:141-156)."""

    def __init__(self, status: int, err: _Error | None = None):
        self.kind = KINDS[status] if 0 <= status < len(KINDS) else f"Status{status}"
        self.value = int(err.value) if err is not None else 0
        self.value2 = int(err.value2) if err is not None else 0
        self.text = bytes(err.text[: err.text_len]) if err is not None else b""
        super().__init__(f"tokenizer error: {self.kind} value={self.value} value2={self.value2} text={self.text!r}")


@dataclass
class TokenizerConfig:
    """TokenizerConfig (mod.rs:82-101)."""
    preset: str = "llama3"
    bos_id: Optional[int] = None
    eos_id: int = 0
    eot_id: Optional[int] = None


_bound = False


def _L():
    global _bound
    L = _lib.load()
    if not _bound:
        vp, sp = C.c_void_p, C.POINTER(C.c_size_t)
        strs, u32p = C.POINTER(C.c_char_p), C.POINTER(C.c_uint32)
        L.rg_b200_tokenizer_new.argtypes = [strs, sp, u32p, C.c_size_t, strs, sp, u32p, C.c_size_t, C.POINTER(_Config),
                                            C.POINTER(vp), C.POINTER(_Error)]
        L.rg_b200_tokenizer_from_gguf.argtypes = [vp, C.POINTER(vp), C.POINTER(_Error)]
        L.rg_b200_tokenizer_free.restype = None
        L.rg_b200_tokenizer_free.argtypes = [vp]
        L.rg_b200_tokenizer_config.restype = None
        L.rg_b200_tokenizer_config.argtypes = [vp, C.POINTER(_Config)]
        L.rg_b200_tokenizer_is_end.argtypes = [vp, C.c_uint32]
        L.rg_b200_tokenizer_parse_preset.argtypes = [C.c_char_p, C.c_size_t, C.POINTER(C.c_int32)]
        L.rg_b200_tokenizer_encode.argtypes = [vp, C.c_char_p, C.c_size_t, u32p, C.c_size_t, sp, C.POINTER(_Error)]
        L.rg_b200_tokenizer_decode.argtypes = [vp, u32p, C.c_size_t, C.c_char_p, C.c_size_t, sp, C.POINTER(_Error)]
        L.rg_b200_tok_stream_new.argtypes = [vp, C.POINTER(vp)]
        L.rg_b200_tok_stream_push.argtypes = [vp, C.c_uint32, C.c_char_p, C.c_size_t, sp, C.POINTER(_Error)]
        L.rg_b200_tok_stream_finish.argtypes = [vp, C.c_char_p, C.c_size_t, sp]
        L.rg_b200_tok_stream_free.restype = None
        L.rg_b200_tok_stream_free.argtypes = [vp]
        L.rg_b200_chat_template_from_gguf.argtypes = [vp, C.POINTER(C.c_int32), C.POINTER(_Error)]
        L.rg_b200_chat_template_text.restype = C.c_char_p
        L.rg_b200_chat_render.argtypes = [vp, C.POINTER(C.c_int32), strs, sp, C.c_size_t, C.c_int32, C.c_char_p, C.c_size_t,
                                          sp, C.POINTER(_Error)]
        _bound = True
    return L


def parse_preset(value: str) -> str:
    """TokenizerPreset::parse (mod.rs:64-79): the normalised preset name."""
    raw = value.encode()
    out = C.c_int32()
    rc = _L().rg_b200_tokenizer_parse_preset(raw, len(raw), C.byref(out))
    if rc:
        e = _Error()
        e.status, e.text_len, e.text = rc, min(len(raw), 128), raw[:128]
        raise TokenizerError(rc, e)
    return PRESETS[out.value]


def _pack(items: Iterable[tuple[str, int]]):
    items = [(s.encode("utf-8", "surrogatepass") if isinstance(s, str) else bytes(s), int(i)) for s, i in items]
    n = len(items)
    strs = (C.c_char_p * max(n, 1))(*[s for s, _ in items])
    lens = (C.c_size_t * max(n, 1))(*[len(s) for s, _ in items])
    ids = (C.c_uint32 * max(n, 1))(*[i for _, i in items])
    return strs, lens, ids, n


class SimpleTokenizer:
    """SimpleTokenizer (mod.rs:158-457)."""

    def __init__(self, normal_tokens: Iterable[tuple[str, int]], special_tokens: Iterable[tuple[str, int]] = (),
                 config: TokenizerConfig | None = None):
        config = config or TokenizerConfig()
        c = _Config(PRESETS.index(parse_preset(config.preset)), int(config.bos_id is not None), config.bos_id or 0,
                    config.eos_id, int(config.eot_id is not None), config.eot_id or 0)
        ns, nl, ni, nn = _pack(normal_tokens)
        ss, sl, si, sn = _pack(special_tokens)
        self._h = C.c_void_p()
        err = _Error()
        rc = _L().rg_b200_tokenizer_new(ns, nl, ni, nn, ss, sl, si, sn, C.byref(c), C.byref(self._h), C.byref(err))
        if rc:
            raise TokenizerError(rc, err)

    @classmethod
    def from_gguf(cls, file) -> "SimpleTokenizer":
        """from_gguf (mod.rs:233-308); ``file`` is a ``session.GgufFile``."""
        self = cls.__new__(cls)
        self._h = C.c_void_p()
        err = _Error()
        rc = _L().rg_b200_tokenizer_from_gguf(file._h, C.byref(self._h), C.byref(err))
        if rc:
            raise TokenizerError(rc, err)
        return self

    def close(self):
        if getattr(self, "_h", None):
            _L().rg_b200_tokenizer_free(self._h)
            self._h = None

    __del__ = close

    def _config(self) -> _Config:
        c = _Config()
        _L().rg_b200_tokenizer_config(self._h, C.byref(c))
        return c

    def preset(self) -> str:
        return PRESETS[self._config().preset]

    def bos_id(self) -> Optional[int]:
        c = self._config()
        return c.bos_id if c.has_bos else None

    def eos_id(self) -> int:
        return self._config().eos_id

    def eot_id(self) -> Optional[int]:
        c = self._config()
        return c.eot_id if c.has_eot else None

    def is_end(self, token_id: int) -> bool:
        return bool(_L().rg_b200_tokenizer_is_end(self._h, token_id))

    def encode(self, text: str) -> list[int]:
        raw = text.encode("utf-8")
        n, err = C.c_size_t(), _Error()
        cap = max(16, len(raw))
        while True:
            buf = (C.c_uint32 * cap)()
            rc = _L().rg_b200_tokenizer_encode(self._h, raw, len(raw), buf, cap, C.byref(n), C.byref(err))
            if rc == 1 and n.value > cap:
                cap = n.value
                continue
            if rc:
                raise TokenizerError(rc, err)
            return list(buf[: n.value])

    def decode(self, ids: Iterable[int]) -> str:
        ids = list(ids)
        arr = (C.c_uint32 * max(len(ids), 1))(*ids)
        n, err = C.c_size_t(), _Error()
        cap = 64
        while True:
            buf = C.create_string_buffer(cap)
            rc = _L().rg_b200_tokenizer_decode(self._h, arr, len(ids), buf, cap, C.byref(n), C.byref(err))
            if rc == 1 and n.value > cap:
                cap = n.value
                continue
            if rc:
                raise TokenizerError(rc, err)
            return buf.raw[: n.value].decode("utf-8")

    def stream_decoder(self) -> "StreamingDecoder":
        return StreamingDecoder(self)


class StreamingDecoder:
    """StreamingDecoder (mod.rs:459-470)."""

    def __init__(self, tokenizer: SimpleTokenizer):
        self._tok = tokenizer  # keeps the tokenizer alive
        self._h = C.c_void_p()
        rc = _L().rg_b200_tok_stream_new(tokenizer._h, C.byref(self._h))
        if rc:
            raise TokenizerError(rc)

    def push(self, token_id: int) -> str:
        n, err = C.c_size_t(), _Error()
        cap = 64
        while True:
            buf = C.create_string_buffer(cap)
            rc = _L().rg_b200_tok_stream_push(self._h, token_id, buf, cap, C.byref(n), C.byref(err))
            if rc == 1 and n.value > cap:
                cap = n.value
                continue
            if rc:
                raise TokenizerError(rc, err)
            return buf.raw[: n.value].decode("utf-8")

    def finish(self) -> str:
        n = C.c_size_t()
        buf = C.create_string_buffer(16)
        rc = _L().rg_b200_tok_stream_finish(self._h, buf, 16, C.byref(n))
        if rc:
            raise TokenizerError(rc)
        return buf.raw[: n.value].decode("utf-8")

    def close(self):
        if getattr(self, "_h", None):
            _L().rg_b200_tok_stream_free(self._h)
            self._h = None

    __del__ = close


def byte_alphabet() -> dict[int, str]:
    """byte -> character of the GPT-2 byte alphabet (inverse of byte_decoder, mod.rs:505-528)."""
    direct = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    table = {b: chr(b) for b in direct}
    extra = 0
    for b in range(256):
        if b not in table:
            table[b] = chr(256 + extra)
            extra += 1
    return table


def encoded_bytes(data: bytes) -> str:
    table = byte_alphabet()
    return "".join(table[b] for b in data)


ROLES = {"system": 0, "user": 1, "assistant": 2}


def llama_simple_chat_template() -> str:
    """LLAMA_SIMPLE_CHAT_TEMPLATE (src/models/transformer/chat.rs:16)."""
    return _L().rg_b200_chat_template_text().decode()


class LlamaChatTemplate:
    """LlamaChatTemplate (chat.rs:62-161): absent metadata or exactly the supported template."""

    def __init__(self, metadata_present: bool = False):
        self._present = metadata_present

    @classmethod
    def from_gguf(cls, file) -> "LlamaChatTemplate":
        present, err = C.c_int32(), _Error()
        rc = _L().rg_b200_chat_template_from_gguf(file._h, C.byref(present), C.byref(err))
        if rc:
            raise TokenizerError(rc, err)
        return cls(bool(present.value))

    def metadata_present(self) -> bool:
        return self._present

    def render(self, tokenizer: SimpleTokenizer, messages: Iterable[tuple[str, str]], add_generation_prompt: bool) -> str:
        """messages: (role, content) with role in system / user / assistant."""
        messages = list(messages)
        roles = (C.c_int32 * max(len(messages), 1))(*[ROLES[r] for r, _ in messages])
        strs, lens, _, n = _pack([(c, 0) for _, c in messages])
        size, err = C.c_size_t(), _Error()
        cap = 256
        while True:
            buf = C.create_string_buffer(cap)
            rc = _L().rg_b200_chat_render(tokenizer._h, roles, strs, lens, n, int(add_generation_prompt), buf, cap,
                                          C.byref(size), C.byref(err))
            if rc == 1 and size.value > cap:
                cap = size.value
                continue
            if rc:
                raise TokenizerError(rc, err)
            return buf.raw[: size.value].decode("utf-8")
