"""Host-only checks of the C ABI: the library loads, exports what the header declares, and the
GGUF container reader accepts/rejects what rustgrad's reader does (src/gguf/tests.rs:905-1213,
src/models/transformer/model_tests.rs:471-641).  No compute entry point is called here."""
import io
import re
import struct
from pathlib import Path

import numpy as np
import pytest

from rustgrad_b200 import _lib, gguf_writer, quant, session, synth

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    headers = sorted((ROOT / "include").glob("*.h"))
    assert len(headers) >= 2
    declared = set()
    for h in headers:
        declared |= set(re.findall(r"\b(rg_b200_\w+)\s*\(", h.read_text()))
    assert declared, "header declares nothing"
    L = _lib.load()
    missing = [name for name in sorted(declared) if not hasattr(L, name)]
    assert not missing, missing
    assert declared == set(_lib.EXPORTS)
    assert b"sm_100a" in L.rg_b200_version()
    assert L.rg_b200_status_string(6) == b"CONTEXT_EXHAUSTED"


def tiny_file():
    cfg = synth.scaled(synth.TINY, n_layers=1, vocab=64)
    tensors = synth.build_tensors(cfg, seed=0)
    return cfg, tensors, synth.gguf_bytes(cfg, tensors)


def test_gguf_roundtrip_config_and_tensor_inventory():
    cfg, tensors, data = tiny_file()
    g = session.GgufFile(data)
    got = g.llama_config()
    for key in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "ffn_dim", "vocab", "max_context"):
        assert got[key] == cfg[key], key
    assert abs(got["norm_eps"] - 1e-5) < 1e-12 and got["rope_theta"] == 10000.0
    assert got["eos_id"] == 0 and got["eot_id"] == -1  # no stop keys in the file: eos defaults to 0, no eot
    infos = {name: (t, dims, off, n) for name, t, dims, off, n in g.tensors()}
    assert set(infos) == set(tensors)
    raw = np.frombuffer(data, np.uint8)
    for name, (t, rows, cols, payload) in tensors.items():
        gt, dims, off, n = infos[name]
        assert gt == t and dims == ([cols] if rows == 1 else [rows, cols])
        assert off % 32 == 0 and (raw[off:off + n] == payload.reshape(-1)).all()
    # ffn_down has K = 688: not a multiple of 32, so the writer must have stored it dense
    assert infos["blk.0.ffn_down.weight"][0] == quant.F32


def rejects(data, status):
    with pytest.raises(session.RgError) as e:
        session.GgufFile(data)
    assert e.value.status == status, e.value


def test_malformed_containers_are_rejected_with_typed_status():
    _, _, data = tiny_file()
    bad = 14  # RG_MALFORMED_GGUF
    rejects(b"GGUX" + data[4:], bad)                                   # magic
    rejects(data[:4] + struct.pack("<I", 1) + data[8:], bad)           # version 1
    rejects(data[:4] + struct.pack("<I", 4) + data[8:], bad)           # version 4
    rejects(data[:100], bad)                                           # truncated header
    rejects(data[:-40], bad)                                           # truncated tensor data
    rejects(data + b"\0" * 32, bad)                                    # trailing data beyond the padding
    rejects(data[:8] + struct.pack("<Q", 2_000_000) + data[16:], bad)  # tensor count above the limit


def build(metadata, tensors):
    buf = io.BytesIO()
    gguf_writer.write_gguf(buf, metadata, tensors)
    return buf.getvalue()


def test_metadata_and_layout_rules():
    bad = 14
    t = {"a": (quant.F32, 1, 8, np.zeros(32, np.uint8))}
    ok = build([gguf_writer.kv_u32("general.alignment", 32)], t)
    session.GgufFile(ok).close()
    rejects(build([gguf_writer.kv_u32("General.alignment", 32)], t), bad)       # upper-case key
    rejects(build([gguf_writer.kv_u32("a..b", 1)], t), bad)                     # empty key segment
    rejects(build([gguf_writer.kv_u32("a.b", 1), gguf_writer.kv_u32("a.b", 2)], t), bad)  # duplicate key
    rejects(build([gguf_writer.kv_u32("general.alignment", 12)], t), bad)       # alignment not a multiple of 8
    rejects(build([gguf_writer.kv_f32("general.alignment", 32.0)], t), bad)     # alignment of the wrong type
    # non-zero padding between two tensors
    two = {"a": (quant.F32, 1, 1, np.zeros(4, np.uint8)), "b": (quant.F32, 1, 1, np.zeros(4, np.uint8))}
    data = bytearray(build([], two))
    data[-32 - 20] = 1
    rejects(bytes(data), bad)
    # a packed tensor whose element count is not a whole number of blocks
    name = b"q"
    raw = b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + struct.pack("<Q", 1) + name + struct.pack("<IQIQ", 1, 48, 8, 0)
    raw += b"\0" * (-len(raw) % 32) + b"\0" * 64
    rejects(raw, bad)
    # unknown tensor type
    raw = b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + struct.pack("<Q", 1) + name + struct.pack("<IQIQ", 1, 32, 99, 0)
    raw += b"\0" * (-len(raw) % 32) + b"\0" * 64
    rejects(raw, bad)


def test_llama_config_rejections_are_typed():
    cfg, tensors, _ = tiny_file()
    base = gguf_writer.llama_metadata(cfg)

    def cfg_status(metadata, tensors=tensors):
        g = session.GgufFile(build(metadata, tensors))
        with pytest.raises(session.RgError) as e:
            g.llama_config()
        return e.value.status

    swap = lambda key, new: [new if key.encode() in kv[:80] else kv for kv in base]  # noqa: E731
    assert cfg_status(swap("general.architecture", gguf_writer.kv_str("general.architecture", "qwen2"))) == 17
    assert cfg_status([kv for kv in base if b"llama.block_count" not in kv[:80]]) == 18
    assert cfg_status(base + [gguf_writer.kv_f32("llama.rope.scaling.factor", 8.0)]) == 17
    assert cfg_status(base + [gguf_writer.kv_u32("llama.expert_count", 8)]) == 17
    assert cfg_status(base + [gguf_writer.kv_u32("llama.rope.dimension_count", 33)]) == 17   # odd rotary width
    assert cfg_status(base + [gguf_writer.kv_u32("llama.rope.dimension_count", 128)]) == 17  # wider than the head
    assert cfg_status(base + [gguf_writer.kv_u32("llama.attention.value_length", 32)]) == 17
    with_bias = dict(tensors)
    with_bias["blk.0.attn_q.bias"] = (quant.F32, 1, 256, np.zeros(1024, np.uint8))
    assert cfg_status(base, with_bias) == 17          # one bias of the three: a partial family
    only_q_norm = dict(tensors)
    only_q_norm["blk.0.attn_q_norm.weight"] = (quant.F32, 1, 64, np.zeros(256, np.uint8))
    assert cfg_status(base, only_q_norm) == 17        # a query norm without the key norm
    # complete families and partial rotary lanes are model variants the session runs
    g = session.GgufFile(build(base + [gguf_writer.kv_u32("llama.rope.dimension_count", 32)], tensors))
    assert g.llama_config()["rope_dim"] == 32


def test_stop_ids_follow_the_tokenizer_rule():
    """eos = metadata value or 0; eot = metadata value, else the last special token spelled
    <|im_end|>; ids must index the vocabulary (src/tokenizer/mod.rs:284-296 via model.rs:288-292).
    The library's answer is compared with the checker's restatement of the rule."""
    from oracle import tokenizer_oracle as T
    cfg, tensors, _ = tiny_file()
    base = gguf_writer.llama_metadata(cfg)
    tokens, types = gguf_writer.synthetic_token_table(cfg["vocab"])

    def config_of(tokens, types, eos=None, eot=None):
        md = [kv for kv in base if b"tokenizer.ggml.tokens" not in kv[:60] and b"tokenizer.ggml.token_type" not in kv[:60]]
        md += [gguf_writer.kv_str_array("tokenizer.ggml.tokens", tokens), gguf_writer.kv_i32_array("tokenizer.ggml.token_type", types)]
        if eos is not None:
            md.append(gguf_writer.kv_u32("tokenizer.ggml.eos_token_id", eos))
        if eot is not None:
            md.append(gguf_writer.kv_u32("tokenizer.ggml.eot_token_id", eot))
        g = session.GgufFile(build(md, tensors))
        try:
            return g.llama_config()
        finally:
            g.close()

    def agree(tokens, types, eos=None, eot=None):
        got = config_of(tokens, types, eos, eot)
        want = T.stop_ids_from_gguf_metadata(tokens, types, eos, eot)
        assert (got["eos_id"], got["eot_id"]) == (want[0], -1 if want[1] is None else want[1])
        return got["eos_id"], got["eot_id"]

    assert agree(tokens, types) == (0, -1)
    assert agree(tokens, types, eos=7) == (7, -1)
    chatml_tokens, chatml_types = list(tokens), list(types)
    for i in (9, 40):                      # two specials with the ChatML end marker: the last one counts
        chatml_tokens[i], chatml_types[i] = "<|im_end|>", 3
    assert agree(chatml_tokens, chatml_types) == (0, 40)
    assert agree(chatml_tokens, chatml_types, eos=5, eot=11) == (5, 11)   # an explicit key wins
    normal_named = list(tokens)
    normal_named[12] = "<|im_end|>"        # a NORMAL token of that spelling is not a stop token
    assert agree(normal_named, types) == (0, -1)
    for bad in (dict(eos=cfg["vocab"]), dict(eot=cfg["vocab"] + 3)):
        with pytest.raises(session.RgError) as e:
            config_of(tokens, types, **bad)
        assert e.value.status == 1
        with pytest.raises(T.TokenizerError):
            T.stop_ids_from_gguf_metadata(tokens, types, bad.get("eos"), bad.get("eot"))
    # without the token types there is no tokenizer, hence no model configuration
    md = [kv for kv in base if b"tokenizer.ggml.token_type" not in kv[:60]]
    g = session.GgufFile(build(md, tensors))
    with pytest.raises(session.MissingMetadata):
        g.llama_config()


def test_device_info_is_a_typed_error_without_a_device():
    """No GPU here: the verb must say so (RG_CUDA_ERROR with the driver's words), never invent a device."""
    import torch
    if torch.cuda.is_available():
        info = session.device_info(0)
        assert info["sm_count"] > 0 and info["name"]
        return
    with pytest.raises(session.RgError) as e:
        session.device_info(0)
    assert e.value.status == 9 and "cuda" in str(e.value).lower()
