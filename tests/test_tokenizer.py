"""Host tokenizer (C ABI of include/rg_b200_tokenizer.h) against the cases of rustgrad's own
tokenizer tests (src/tokenizer/tests.rs, cited per test) and against the Python restatement in
oracle/tokenizer_oracle.py on seeded random text.  No GPU is involved."""
import random
import struct

import pytest

from oracle import tokenizer_oracle as oracle  # noqa: E402

from rustgrad_b200 import session  # noqa: E402
from rustgrad_b200.tokenizer import (LlamaChatTemplate, SimpleTokenizer, TokenizerConfig, TokenizerError,  # noqa: E402
                                     encoded_bytes, llama_simple_chat_template, parse_preset)


def byte_fallback_vocab():
    # tests.rs:16-23
    return [(encoded_bytes(bytes([b])), 1000 + b) for b in range(256)]


def tokenizer_with(extra_normal=(), specials=()):
    # tests.rs:25-44
    normal = byte_fallback_vocab() + [(encoded_bytes(raw), i) for raw, i in extra_normal]
    return SimpleTokenizer(normal, list(specials)), oracle.SimpleTokenizer(normal, list(specials))


def both(pair, text):
    ours, ref = pair
    got = ours.encode(text)
    assert got == ref.encode(text)
    return got


def test_exact_word_token_wins_before_ranked_merges():
    # tests.rs:46-57
    assert both(tokenizer_with([(b"ab", 5), (b"bc", 4), (b"abc", 99)]), "abc") == [99]
    assert both(tokenizer_with([(b"ab", 5), (b"bc", 4)]), "abc") == [1000 + ord("a"), 4]


def test_unicode_word_splitting_matches_checked_in_source_cases():
    # tests.rs:59-93
    chunks = [b"hello", b" world", " 한국어".encode(), " 中文".encode(), " текст".encode(), b" ", "١٢٣".encode(), b"123",
              " 😊\n".encode(), b"  ", b"\ttoday", b"\n", "'équivalent".encode(), "²³".encode(), "№".encode()]
    pair = tokenizer_with([(c, i + 1) for i, c in enumerate(chunks)])
    text = "hello world 한국어 中文 текст ١٢٣ 123 😊\n  \ttoday\n'équivalent ²³№ "
    ids = both(pair, text)
    assert ids == [1, 2, 3, 4, 5, 6, 7, 6, 8, 9, 10, 11, 12, 13, 6, 14, 15, 6]
    assert pair[0].decode(ids) == text


def test_trailing_whitespace_lookahead_behavior_is_preserved():
    # tests.rs:95-109
    pair = tokenizer_with([(b"  ", 1), (b" hello", 2), (b"123", 3)])
    assert both(pair, "   hello") == [1, 2]
    assert both(pair, "  1234") == [1000 + 32, 1000 + 32, 3, 1000 + ord("4")]


def test_specials_use_source_order_and_override_normal_sentence_coding():
    # tests.rs:111-124
    pair = tokenizer_with([], [("<x>", 20), ("<x>y", 21)])
    assert both(pair, "a<x>yb") == [1000 + ord("a"), 20, 1000 + ord("y"), 1000 + ord("b")]
    assert pair[0].decode([20]) == "<x>"


def test_byte_fallback_round_trips_unicode_and_streams_incomplete_utf8():
    # tests.rs:126-147
    pair = tokenizer_with()
    text = "a😊실\u0085z"
    assert pair[0].decode(both(pair, text)) == text
    tok = SimpleTokenizer([(encoded_bytes(b" \xf0\x9f\x98"), 25677), (encoded_bytes(b"\x8a"), 138)])
    dec = tok.stream_decoder()
    assert dec.push(25677) == " "
    assert dec.push(138) == "😊"
    assert dec.finish() == ""
    assert dec.push(138) == ""  # nothing after finish (mod.rs:462-464)


def test_stream_decoder_flushes_and_replaces():
    tok = SimpleTokenizer([(encoded_bytes(b"\xe2\x82"), 1), (encoded_bytes(b"\xac"), 2), (encoded_bytes(b"\xff"), 3),
                           (encoded_bytes(b"ok"), 4)])
    dec = tok.stream_decoder()
    assert dec.push(1) == ""
    assert dec.push(2) == "€"
    assert dec.push(3) == "�"  # an invalid byte is replaced at once (error_len is known)
    assert dec.push(1) == ""
    assert dec.push(4) == "�ok"  # the truncated sequence becomes one replacement character
    assert dec.push(1) == ""
    assert dec.finish() == "�"


def test_coding_failures_are_structured():
    # tests.rs:149-168
    tok = SimpleTokenizer([(encoded_bytes(b"a"), 1)])
    with pytest.raises(TokenizerError) as e:
        tok.encode("b")
    assert e.value.kind == "TokenNotFound" and e.value.text == b"b"
    with pytest.raises(TokenizerError) as e:
        tok.decode([99])
    assert e.value.kind == "UnknownTokenId" and e.value.value == 99
    with pytest.raises(TokenizerError) as e:
        SimpleTokenizer([("🙂", 1)])
    assert e.value.kind == "InvalidNormalTokenCharacter" and e.value.value == 1 and e.value.value2 == ord("🙂")
    with pytest.raises(TokenizerError) as e:
        SimpleTokenizer([], [("", 7)])
    assert e.value.kind == "EmptySpecialToken" and e.value.value == 7


def test_duplicate_strings_keep_first_position_and_last_id():
    # mod.rs:173-175,207-216
    a = encoded_bytes(b"a")
    tok = SimpleTokenizer([(a, 1), (a, 2)], [("<p>", 10), ("<q>", 11), ("<p>", 12)])
    assert tok.encode("a<p><q>") == [2, 12, 11]
    assert tok.decode([2, 12]) == "a<p>"
    with pytest.raises(TokenizerError):
        tok.decode([10])


# ---- GGUF construction (tests.rs:170-343) ------------------------------------------------------
TOKENS, TYPES, PRE = "tokenizer.ggml.tokens", "tokenizer.ggml.token_type", "tokenizer.ggml.pre"
BOS, EOS, EOT = "tokenizer.ggml.bos_token_id", "tokenizer.ggml.eos_token_id", "tokenizer.ggml.eot_token_id"
ADD_BOS = "tokenizer.ggml.add_bos_token"


def _s(v: str) -> bytes:
    raw = v.encode()
    return struct.pack("<Q", len(raw)) + raw


def gguf_fixture(entries) -> bytes:
    out = b"GGUF" + struct.pack("<IQQ", 3, 0, len(entries))
    for key, (kind, value) in entries:
        out += _s(key)
        if kind == "string":
            out += struct.pack("<I", 8) + _s(value)
        elif kind == "bool":
            out += struct.pack("<IB", 7, int(value))
        elif kind == "u32":
            out += struct.pack("<II", 4, value)
        elif kind == "strings":
            out += struct.pack("<IIQ", 9, 8, len(value)) + b"".join(_s(v) for v in value)
        elif kind == "i32s":
            out += struct.pack("<IIQ", 9, 5, len(value)) + b"".join(struct.pack("<i", v) for v in value)
    return out


def tokenizer_fixture(tokens, types, preset, extra=()):
    return gguf_fixture([(TOKENS, ("strings", tokens)), (TYPES, ("i32s", types)), (PRE, ("string", preset))] + list(extra))


def from_bytes(data):
    f = session.GgufFile(data)
    return SimpleTokenizer.from_gguf(f)


def test_gguf_constructor_binds_types_special_ids_and_presets():
    # tests.rs:231-250
    hello = encoded_bytes(b"hello")
    tok = from_bytes(tokenizer_fixture(["<s>", "</s>", "<|im_end|>", "<|im_end|>", hello], [3, 3, 3, 3, 1], "qwen35",
                                       [(BOS, ("u32", 0)), (EOS, ("u32", 1))]))
    assert tok.preset() == "qwen2" and tok.bos_id() == 0 and tok.eos_id() == 1 and tok.eot_id() == 3
    assert tok.is_end(1) and tok.is_end(3) and not tok.is_end(0)
    assert tok.encode("hello<|im_end|>") == [4, 3]
    assert tok.decode([0, 4, 1]) == "<s>hello</s>"


def test_disabled_bos_does_not_require_or_read_bos_id():
    # tests.rs:252-270
    tok = from_bytes(tokenizer_fixture([encoded_bytes(b"a")], [1], "tekken",
                                       [(ADD_BOS, ("bool", False)), (BOS, ("string", "not an integer"))]))
    assert tok.bos_id() is None and tok.preset() == "tekken"


def test_malformed_gguf_tokenizer_metadata_fails_before_construction():
    # tests.rs:272-308
    a = encoded_bytes(b"a")
    with pytest.raises(TokenizerError) as e:
        from_bytes(tokenizer_fixture([a], [], "llama3"))
    assert e.value.kind == "MetadataLengthMismatch" and (e.value.value, e.value.value2) == (1, 0)
    with pytest.raises(TokenizerError) as e:
        from_bytes(gguf_fixture([(TOKENS, ("strings", [a])), (TYPES, ("strings", ["1"])), (PRE, ("string", "llama3"))]))
    assert e.value.kind == "MalformedMetadata" and e.value.text == TYPES.encode() and e.value.value == 8
    with pytest.raises(TokenizerError) as e:
        from_bytes(tokenizer_fixture([a], [1], "sentencepiece"))
    assert e.value.kind == "UnsupportedPreset" and e.value.text == b"sentencepiece"
    with pytest.raises(TokenizerError) as e:
        from_bytes(gguf_fixture([(TYPES, ("i32s", [1])), (PRE, ("string", "llama3"))]))
    assert e.value.kind == "MissingMetadata" and e.value.text == TOKENS.encode()


def test_gguf_control_token_ids_must_reference_the_vocabulary():
    # tests.rs:310-343
    tokens, types = ["<s>", "</s>", encoded_bytes(b"a")], [3, 3, 1]
    tok = from_bytes(tokenizer_fixture(tokens, types, "llama3", [(BOS, ("u32", 0)), (EOS, ("u32", 1))]))
    assert tok.decode(tok.encode("a")) == "a"
    for key in (BOS, EOS, EOT):
        with pytest.raises(TokenizerError) as e:
            from_bytes(tokenizer_fixture(tokens, types, "llama3", [(key, ("u32", 3))]))
        assert e.value.kind == "ConfiguredTokenIdOutOfRange"
        assert e.value.text == key.encode() and (e.value.value, e.value.value2) == (3, 3)


def test_presets():
    # mod.rs:64-79
    assert parse_preset("qwen35moe") == "qwen2" and parse_preset("llama-bpe") == "llama-bpe"
    with pytest.raises(TokenizerError):
        parse_preset("gpt2")


# ---- seeded random text against the restatement ------------------------------------------------
ALPHABETS = [
    "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ", "0123456789", " \t\n\r\x0b\x0c\x85   　",
    ".,;:!?'\"()[]{}<>-_+=*/\\|@#$%^&~`", "한국어中文текстéàüßſİıǅ", "١٢٣²³№½Ⅷ〇", "😊🙂🇺🇳‍́️", "'sS'tT'rReE'vV'mM'lL'dDſ",
]


def random_text(rng, n):
    out = []
    for _ in range(n):
        alphabet = rng.choice(ALPHABETS)
        out.append("".join(rng.choice(alphabet) for _ in range(rng.randint(1, 4))))
    return "".join(out)


def test_random_text_matches_the_restatement():
    rng = random.Random(20240607)
    merges = []
    for i in range(400):  # random merge table over printable fragments; ids double as ranks
        frag = random_text(rng, rng.randint(1, 2)).encode()[: rng.randint(2, 6)]
        try:
            frag.decode()
        except UnicodeDecodeError:
            pass
        merges.append((frag, 2000 + i))
    specials = [("<|eot|>", 5000), ("<|", 5001), ("<|eot|>x", 5002), ("\n\n", 5003)]
    pair = tokenizer_with(merges, specials)
    for _ in range(400):
        text = random_text(rng, rng.randint(0, 24))
        if rng.random() < 0.3:
            at = rng.randint(0, len(text))
            text = text[:at] + rng.choice(specials)[0] + text[at:]
        ids = both(pair, text)
        assert pair[0].decode(ids) == pair[1].decode(ids) == text


def test_decode_of_arbitrary_bytes_matches_lossy_utf8():
    rng = random.Random(7)
    pair = tokenizer_with()
    interesting = [0x00, 0x41, 0x7F, 0x80, 0xBF, 0xC0, 0xC1, 0xC2, 0xDF, 0xE0, 0xA0, 0x9F, 0xED, 0xEF, 0xF0, 0x90, 0x8F, 0xF4,
                   0xF5, 0xFF]
    for _ in range(600):
        ids = [1000 + rng.choice(interesting) for _ in range(rng.randint(0, 8))]
        assert pair[0].decode(ids) == pair[1].decode(ids)
        dec = pair[0].stream_decoder()
        streamed = "".join(dec.push(i) for i in ids) + dec.finish()
        assert streamed == pair[0].decode(ids)


# ---- chat prompt (src/models/transformer/batch_tests.rs:190-272) -------------------------------
CHAT = "tokenizer.chat_template"


def test_checked_llama_chat_template_matches_fallback_and_rejects_other_jinja():
    template_text = llama_simple_chat_template()
    assert template_text.startswith("{{ bos_token }}{% for message in messages %}") and "\\n\\n" in template_text
    base = [(TOKENS, ("strings", ["<s>", "</s>", encoded_bytes(b"a")])), (TYPES, ("i32s", [3, 3, 1])),
            (PRE, ("string", "llama3")), (EOS, ("u32", 1)), (ADD_BOS, ("bool", False))]
    f = session.GgufFile(gguf_fixture(base + [(CHAT, ("string", template_text))]))
    tok = SimpleTokenizer.from_gguf(f)
    template = LlamaChatTemplate.from_gguf(f)
    assert template.metadata_present()
    assert template.render(tok, [("system", "a"), ("user", "b")], True) == (
        "<|start_header_id|>system<|end_header_id|>\n\na</s>"
        "<|start_header_id|>user<|end_header_id|>\n\nb</s>"
        "<|start_header_id|>assistant<|end_header_id|>\n\n")
    assert template.render(tok, [("user", "b")], False) == "<|start_header_id|>user<|end_header_id|>\n\nb</s>"
    assert not LlamaChatTemplate.from_gguf(session.GgufFile(gguf_fixture(base))).metadata_present()

    for preset in ("llama-v3", "llama-bpe"):
        alternate = SimpleTokenizer([], [("</s>", 1)], TokenizerConfig(preset=preset, eos_id=1))
        assert template.render(alternate, [("user", "a")], True) == (
            "<|start_header_id|>user<|end_header_id|>\n\na</s><|start_header_id|>assistant<|end_header_id|>\n\n")
    with_bos = SimpleTokenizer([], [("<s>", 0), ("</s>", 1)], TokenizerConfig(bos_id=0, eos_id=1))
    assert template.render(with_bos, [], True) == "<s><|start_header_id|>assistant<|end_header_id|>\n\n"
    qwen = SimpleTokenizer([], [("</s>", 1)], TokenizerConfig(preset="qwen2", eos_id=1))
    with pytest.raises(TokenizerError) as e:
        template.render(qwen, [("user", "a")], True)
    assert e.value.kind == "ChatUnsupportedPreset" and e.value.value == 3

    with pytest.raises(TokenizerError) as e:
        LlamaChatTemplate.from_gguf(session.GgufFile(gguf_fixture(
            base + [(CHAT, ("string", "{% for message in messages %}{{ message }}{% endfor %}"))])))
    assert e.value.kind == "UnsupportedJinja"
    with pytest.raises(TokenizerError) as e:
        LlamaChatTemplate.from_gguf(session.GgufFile(gguf_fixture(base + [(CHAT, ("string", "plain text"))])))
    assert e.value.kind == "UnsupportedTemplate"
    with pytest.raises(TokenizerError) as e:
        LlamaChatTemplate.from_gguf(session.GgufFile(gguf_fixture(base + [(CHAT, ("u32", 7))])))
    assert e.value.kind == "MalformedMetadata" and e.value.text == CHAT.encode()


def test_chat_bounds():
    # chat.rs:8-10,45-55,142-147
    tok = SimpleTokenizer([], [("</s>", 1)], TokenizerConfig(eos_id=1))
    template = LlamaChatTemplate()
    with pytest.raises(TokenizerError) as e:
        template.render(tok, [("user", "x" * (1024 * 1024 + 1))], False)
    assert e.value.kind == "MessageTooLong" and e.value.value2 == 1024 * 1024
    big = "x" * (1024 * 1024)
    with pytest.raises(TokenizerError) as e:
        template.render(tok, [("user", big)] * 4, False)
    assert e.value.kind == "ChatTooLong" and e.value.value2 == 4 * 1024 * 1024
    assert len(template.render(tok, [("user", big)] * 3, True)) > 3 * 1024 * 1024
    missing_eos = SimpleTokenizer([], [("</s>", 1)], TokenizerConfig(eos_id=9))
    with pytest.raises(TokenizerError) as e:
        template.render(missing_eos, [], True)
    assert e.value.kind == "UnknownTokenId" and e.value.value == 9
