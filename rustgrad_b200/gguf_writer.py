"""Minimal GGUF v3 writer for synthetic Llama models.

Produces files that rustgrad's bounded parser accepts (src/gguf/reader.rs:8-301): magic, version 3,
lower-case dotted keys, tensor dims innermost first, offsets aligned to ``general.alignment``
(32), zero padding between tensors and no trailing bytes.  The metadata set is the one the Llama
binder demands (src/models/transformer/model.rs:126-298, src/tokenizer/mod.rs:242-308).
"""
from __future__ import annotations

import struct
from typing import BinaryIO

import numpy as np

from . import quant

ALIGNMENT = 32
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)


def _s(text: str) -> bytes:
    raw = text.encode("utf-8")
    return struct.pack("<Q", len(raw)) + raw


def _kv(key: str, vtype: int, payload: bytes) -> bytes:
    return _s(key) + struct.pack("<I", vtype) + payload


def kv_u32(key: str, v: int) -> bytes:
    return _kv(key, T_U32, struct.pack("<I", v))


def kv_f32(key: str, v: float) -> bytes:
    return _kv(key, T_F32, struct.pack("<f", v))


def kv_bool(key: str, v: bool) -> bytes:
    return _kv(key, T_BOOL, struct.pack("<B", int(v)))


def kv_str(key: str, v: str) -> bytes:
    return _kv(key, T_STR, _s(v))


def kv_str_array(key: str, items) -> bytes:
    body = b"".join(_s(i) for i in items)
    return _kv(key, T_ARR, struct.pack("<IQ", T_STR, len(items)) + body)


def kv_i32_array(key: str, items) -> bytes:
    arr = np.asarray(items, dtype="<i4")
    return _kv(key, T_ARR, struct.pack("<IQ", T_I32, arr.size) + arr.tobytes())


def synthetic_token_table(vocab: int):
    """Distinct printable-ASCII token strings (GPT-2 byte alphabet, no spaces) plus type 1 = normal."""
    alphabet = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789"
    tokens = []
    for i in range(vocab):
        n, chars = i, []
        while True:
            chars.append(alphabet[n % len(alphabet)])
            n //= len(alphabet)
            if n == 0:
                break
        tokens.append("t" + "".join(chars))
    return tokens, [1] * vocab


CHAT_SPECIALS = ("<|begin_of_text|>", "<|end_of_text|>", "<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>")


def chat_token_table(vocab: int):
    """A token table text can be encoded with: the 256 characters of the GPT-2 byte alphabet
    (src/tokenizer/mod.rs:505-528) as ids 0..255, a few ranked merges (the id of a merged token is
    its rank), filler tokens, and the Llama-3 control tokens as the last five ids (type 3).
    Returns (tokens, types, ids) with ids = {"bos", "eos", "eot"}."""
    direct = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    table = {b: chr(b) for b in direct}
    extra = 0
    for b in range(256):
        if b not in table:
            table[b] = chr(256 + extra)
            extra += 1
    enc = lambda text: "".join(table[b] for b in text.encode("utf-8"))  # noqa: E731
    tokens = [table[b] for b in range(256)]
    for word in ("he", "ll", "lo", "hell", "hello", " w", "or", "ld", " wor", " world", "th", " th", " the", "in", "er", "\n\n"):
        tokens.append(enc(word))
    if vocab < len(tokens) + len(CHAT_SPECIALS):
        raise ValueError("vocabulary too small for the chat token table")
    alphabet = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789"
    i = 0
    while len(tokens) < vocab - len(CHAT_SPECIALS):
        n, chars = i, []
        while True:
            chars.append(alphabet[n % len(alphabet)])
            n //= len(alphabet)
            if n == 0:
                break
        tokens.append("zz" + "".join(chars) + "q")
        i += 1
    types = [1] * len(tokens) + [3] * len(CHAT_SPECIALS)
    tokens += list(CHAT_SPECIALS)
    base = vocab - len(CHAT_SPECIALS)
    return tokens, types, {"bos": base, "eos": base + 1, "eot": base + 4}


def llama_metadata(cfg: dict, chat_tokens: bool = False) -> list[bytes]:
    if chat_tokens:
        tokens, types, ids = chat_token_table(cfg["vocab"])
    else:
        tokens, types = synthetic_token_table(cfg["vocab"])
        ids = None
    kvs = [
        kv_str("general.architecture", "llama"),
        kv_u32("general.alignment", ALIGNMENT),
        kv_u32("llama.block_count", cfg["n_layers"]),
        kv_u32("llama.embedding_length", cfg["d_model"]),
        kv_u32("llama.feed_forward_length", cfg["ffn_dim"]),
        kv_u32("llama.attention.head_count", cfg["n_heads"]),
        kv_u32("llama.attention.head_count_kv", cfg["n_kv_heads"]),
        kv_u32("llama.context_length", cfg["max_context"]),
        kv_f32("llama.attention.layer_norm_rms_epsilon", cfg["norm_eps"]),
        kv_f32("llama.rope.freq_base", cfg["rope_theta"]),
        kv_str("tokenizer.ggml.model", "gpt2"),
        kv_str("tokenizer.ggml.pre", "llama-bpe"),
        kv_str_array("tokenizer.ggml.tokens", tokens),
        kv_i32_array("tokenizer.ggml.token_type", types),
        kv_bool("tokenizer.ggml.add_bos_token", chat_tokens),
    ]
    if ids is not None:
        kvs += [kv_u32("tokenizer.ggml.bos_token_id", ids["bos"]), kv_u32("tokenizer.ggml.eos_token_id", ids["eos"]),
                kv_u32("tokenizer.ggml.eot_token_id", ids["eot"])]
    if cfg.get("rope_dim", 0) and cfg["rope_dim"] != cfg["head_dim"]:
        kvs.append(kv_u32("llama.rope.dimension_count", cfg["rope_dim"]))
    if cfg["head_dim"] * cfg["n_heads"] != cfg["d_model"]:
        kvs.append(kv_u32("llama.attention.key_length", cfg["head_dim"]))
        kvs.append(kv_u32("llama.attention.value_length", cfg["head_dim"]))
    if ids is None and cfg.get("eos_id", -1) >= 0:
        kvs.append(kv_u32("tokenizer.ggml.eos_token_id", cfg["eos_id"]))
    return kvs


def write_gguf(out: BinaryIO, metadata: list[bytes], tensors: dict) -> None:
    """``tensors``: name -> (ggml_type, rows, cols, uint8 array); rows == 1 writes a rank-1 tensor."""
    infos, offset = [], 0
    for name, (t, rows, cols, data) in tensors.items():
        data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
        if data.size != quant.tensor_nbytes(t, rows * cols):
            raise ValueError(f"{name}: byte length does not match its geometry")
        dims = [cols] if rows == 1 else [cols, rows]  # innermost first
        info = _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        info += struct.pack("<IQ", t, offset)
        infos.append(info)
        offset += (data.size + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT
    header = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(metadata)) + b"".join(metadata) + b"".join(infos)
    header += b"\0" * (-len(header) % ALIGNMENT)
    out.write(header)
    names = list(tensors)
    for i, name in enumerate(names):
        data = np.ascontiguousarray(tensors[name][3], dtype=np.uint8).reshape(-1)
        out.write(data.tobytes())
        if i + 1 < len(names):  # the parser accepts no trailing bytes beyond the final tensor
            out.write(b"\0" * (-data.size % ALIGNMENT))
        else:
            out.write(b"\0" * (-data.size % ALIGNMENT))
