"""TEST INFRASTRUCTURE ONLY: a pure-Python restatement of rustgrad's ``SimpleTokenizer``
(src/tokenizer/mod.rs) used to check the C++ tokenizer.  Nothing in the product imports it.

It follows the reference literally: the two patterns of mod.rs:32-44 are handed to Python's ``re``
engine (leftmost-first alternation, greedy quantifiers, backtracking: the same match as the regex
crate finds for these patterns), with the character classes written out as explicit ranges of
the general categories L*, N*, Z* up to U+323AF from ``unicodedata``.

Pinned by the cases of the reference's own tests (src/tokenizer/tests.rs), transcribed in
tests/test_tokenizer.py.
"""
from __future__ import annotations

import re
import unicodedata

LIMIT = 0x323AF


def _class(prefix: str) -> str:
    out, start = [], None
    for cp in range(LIMIT + 2):
        inside = cp <= LIMIT and unicodedata.category(chr(cp)).startswith(prefix)
        if inside and start is None:
            start = cp
        elif not inside and start is not None:
            out.append((start, cp - 1))
            start = None
    return "".join(f"\\U{lo:08x}-\\U{hi:08x}" if lo != hi else f"\\U{lo:08x}" for lo, hi in out)


LETTER, NUMBER, SEPARATOR = _class("L"), _class("N"), _class("Z")
WS = "\\t\\n\\x0b\\x0c\\r\\x85" + SEPARATOR
# mod.rs:32-39
WORD_PREFIX = re.compile(
    "(?:(?i:'s|'t|'re|'ve|'m|'ll|'d)"
    f"|[^\\r\\n{NUMBER}{LETTER}]?[{LETTER}]+"
    f"|[{NUMBER}]{{1,3}}"
    f"| ?[^{WS}{NUMBER}{LETTER}]+[\\r\\n]*"
    f"|[{WS}]*[\\r\\n]+)")
# mod.rs:41-44
WHITESPACE = re.compile(f"[{WS}]+")


def byte_decoder() -> dict[str, int]:
    """mod.rs:505-528"""
    direct = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    table = {chr(b): b for b in direct}
    extra = 0
    for b in range(256):
        if b not in direct:
            table[chr(256 + extra)] = b
            extra += 1
    return table


class TokenizerError(Exception):
    def __init__(self, kind, *detail):
        self.kind, self.detail = kind, detail
        super().__init__(f"{kind}: {detail}")


class SimpleTokenizer:
    """mod.rs:158-457"""

    def __init__(self, normal_tokens, special_tokens=(), eos_id=0, eot_id=None, bos_id=None):
        dec = byte_decoder()
        self.normal: dict[bytes, int] = {}
        order = []
        for token, token_id in normal_tokens:
            raw = bytearray()
            for ch in token:
                if ch not in dec:
                    raise TokenizerError("InvalidNormalTokenCharacter", token_id, ch)
                raw.append(dec[ch])
            raw = bytes(raw)
            if raw not in self.normal:
                order.append(raw)
            self.normal[raw] = token_id
        self.special: list[list] = []
        position = {}
        for token, token_id in special_tokens:
            if not token:
                raise TokenizerError("EmptySpecialToken", token_id)
            if token in position:
                self.special[position[token]][1] = token_id
            else:
                position[token] = len(self.special)
                self.special.append([token, token_id])
        self.tok2bytes = {}
        for raw in order:
            self.tok2bytes[self.normal[raw]] = raw
        for token, token_id in self.special:
            self.tok2bytes[token_id] = token.encode()
        self.eos_id, self.eot_id, self.bos_id = eos_id, eot_id, bos_id

    def is_end(self, token_id):
        return token_id == self.eos_id or (self.eot_id is not None and token_id == self.eot_id)

    # mod.rs:328-338
    def encode(self, text: str) -> list[int]:
        out, position = [], 0
        while True:
            nxt = self._next_special(text, position)
            if nxt is None:
                break
            start, end, token_id = nxt
            self._encode_sentence(text[position:start], out)
            out.append(token_id)
            position = end
        self._encode_sentence(text[position:], out)
        return out

    # mod.rs:379-391
    def _next_special(self, text, position):
        best = None
        for order, (token, token_id) in enumerate(self.special):
            at = text.find(token, position)
            if at >= 0 and (best is None or (at, order) < best[:2]):
                best = (at, order, len(token), token_id)
        return None if best is None else (best[0], best[0] + best[2], best[3])

    # mod.rs:393-424
    def _encode_sentence(self, sentence, out):
        remaining = sentence
        while remaining:
            m = WORD_PREFIX.match(remaining)
            if m:
                n = m.end()
            else:
                w = WHITESPACE.match(remaining)
                if w:
                    n = w.end() if (w.end() == len(remaining) or w.end() <= 1) else w.end() - 1
                else:
                    n = 1
            self._encode_word(remaining[:n].encode(), out)
            remaining = remaining[n:]

    # mod.rs:426-456
    def _encode_word(self, word: bytes, out):
        if word in self.normal:
            out.append(self.normal[word])
            return
        parts = [bytes([b]) for b in word]
        while True:
            best = None
            for i in range(len(parts) - 1):
                rank = self.normal.get(parts[i] + parts[i + 1])
                if rank is not None and (best is None or (rank, i) < best):
                    best = (rank, i)
            if best is None:
                break
            i = best[1]
            parts[i:i + 2] = [parts[i] + parts[i + 1]]
        for part in parts:
            if part not in self.normal:
                raise TokenizerError("TokenNotFound", part)
            out.append(self.normal[part])

    # mod.rs:340-346 (bytes.decode(errors="replace") is the behaviour the reference names)
    def decode(self, ids) -> str:
        raw = bytearray()
        for token_id in ids:
            if token_id not in self.tok2bytes:
                raise TokenizerError("UnknownTokenId", token_id)
            raw += self.tok2bytes[token_id]
        return bytes(raw).decode("utf-8", errors="replace")


def stop_ids_from_gguf_metadata(tokens, token_types, eos_key=None, eot_key=None):
    """The stop ids a model configuration takes from its tokenizer (mod.rs:284-296, read by
    LlamaModelConfig::from_gguf, model.rs:288-292): eos is the `tokenizer.ggml.eos_token_id` value
    or 0; eot is the `tokenizer.ggml.eot_token_id` value, else the id of the LAST special token
    (type other than 1) spelled <|im_end|>, else none; every configured id must index the
    vocabulary.  Returns (eos, eot or None); raises TokenizerError("ConfiguredTokenIdOutOfRange")."""
    count = len(tokens)
    eos = 0 if eos_key is None else eos_key
    eot = eot_key
    if eot is None:
        for token_id in range(count - 1, -1, -1):
            if token_types[token_id] != 1 and tokens[token_id] == "<|im_end|>":
                eot = token_id
                break
    if eos >= count:
        raise TokenizerError("ConfiguredTokenIdOutOfRange", "eos", eos, count)
    if eot is not None and eot >= count:
        raise TokenizerError("ConfiguredTokenIdOutOfRange", "eot", eot, count)
    return eos, eot
