"""Seeded synthetic Llama models in the shapes the benchmark configurations name.

No real checkpoint, tokenizer or dataset is involved: linear and embedding weights are drawn
N(0, 0.02) from a seed and quantized with the GGML rules of :mod:`rustgrad_b200.quant`, norm
weights are 1.0, prompts are uniform random token ids.
"""
from __future__ import annotations

import io

import numpy as np

from . import gguf_writer, quant
from .quant import F32, Q4_0, Q8_0

TINY = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=4, head_dim=64, ffn_dim=688, vocab=512,
            max_context=64, norm_eps=1e-5, rope_theta=10000.0)
LLAMA_8B = dict(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn_dim=14336, vocab=128256,
                max_context=4096, norm_eps=1e-5, rope_theta=500000.0)
LLAMA_70B = dict(n_layers=80, d_model=8192, n_heads=64, n_kv_heads=8, head_dim=128, ffn_dim=28672, vocab=128256,
                 max_context=4096, norm_eps=1e-5, rope_theta=500000.0)


def scaled(cfg: dict, **over) -> dict:
    out = dict(cfg)
    out.update(over)
    return out


def tensor_inventory(cfg: dict, tied_head: bool):
    """(name, rows, cols, is_norm) in file order: src/models/transformer/model.rs:384-455."""
    d, f = cfg["d_model"], cfg["ffn_dim"]
    qw, kw = cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"]
    inv = [("token_embd.weight", cfg["vocab"], d, False), ("output_norm.weight", 1, d, True)]
    for layer in range(cfg["n_layers"]):
        p = f"blk.{layer}."
        inv += [
            (p + "attn_norm.weight", 1, d, True), (p + "attn_q.weight", qw, d, False),
            (p + "attn_k.weight", kw, d, False), (p + "attn_v.weight", kw, d, False),
            (p + "attn_output.weight", d, qw, False), (p + "ffn_norm.weight", 1, d, True),
            (p + "ffn_gate.weight", f, d, False), (p + "ffn_up.weight", f, d, False),
            (p + "ffn_down.weight", d, f, False),
        ]
        # model variants (src/models/transformer/model.rs:427-449): q / k RMS norm weights, projection biases
        if cfg.get("qk_norm", 0):
            per_head = cfg["qk_norm"] == 1
            inv += [(p + "attn_q_norm.weight", 1, cfg["head_dim"] if per_head else qw, True),
                    (p + "attn_k_norm.weight", 1, cfg["head_dim"] if per_head else kw, True)]
        if cfg.get("qkv_bias", 0):
            inv += [(p + "attn_q.bias", 1, qw, True), (p + "attn_k.bias", 1, kw, True), (p + "attn_v.bias", 1, kw, True)]
    if not tied_head:
        inv.append(("output.weight", cfg["vocab"], d, False))
    return inv


def build_tensors(cfg: dict, seed: int, body_type: int = Q8_0, embed_type: int | None = None,
                  head_type: int | None = None, tied_head: bool = True, std: float = 0.02) -> dict:
    """Host-generated model: name -> (ggml_type, rows, cols, uint8 bytes).

    A projection whose column count is not a multiple of 32 cannot be block-quantized (rustgrad
    rejects it, src/gguf/quantization/data.rs:268-270) and is stored as dense F32 instead.
    """
    rng = np.random.default_rng(seed)
    embed_type = body_type if embed_type is None else embed_type
    head_type = embed_type if head_type is None else head_type
    tensors = {}
    for name, rows, cols, is_norm in tensor_inventory(cfg, tied_head):
        if is_norm:
            if name.endswith(".bias"):  # biases and q / k norm weights are not trivial, or a test could not see them
                vec = (rng.standard_normal(cols, dtype=np.float32) * np.float32(0.05)).astype(np.float32)
            elif "_norm.weight" in name and ("attn_q_norm" in name or "attn_k_norm" in name):
                vec = (np.float32(1.0) + rng.standard_normal(cols, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
            else:
                vec = np.ones(cols, dtype=np.float32)
            tensors[name] = (F32, 1, cols, vec.view(np.uint8))
            continue
        t = embed_type if name == "token_embd.weight" else head_type if name == "output.weight" else body_type
        if cols % 32:
            t = F32
        w = (rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(std)).astype(np.float32)
        tensors[name] = (t, rows, cols, quant.encode(t, w))
    return tensors


def gguf_bytes(cfg: dict, tensors: dict, chat_tokens: bool = False) -> bytes:
    """The model as a GGUF file; ``chat_tokens`` gives it a token table that text can be encoded with
    (byte alphabet, merges, Llama-3 control tokens) instead of opaque token names."""
    buf = io.BytesIO()
    gguf_writer.write_gguf(buf, gguf_writer.llama_metadata(cfg, chat_tokens), tensors)
    return buf.getvalue()


def prompt_ids(cfg: dict, n: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n, dtype=np.int32)


def device_weight(ggml_type: int, n: int, k: int, seed: int, std: float = 0.02, device: int = 0) -> np.ndarray:
    """The block bytes of one [n, k] tensor drawn N(0, std) and quantized on the GPU (the generator
    that fills synthetic models, read back): seconds faster than the host encoder for tensors of
    tens of millions of elements.  k must be a multiple of 64."""
    from . import session
    hd = 128 if k % 128 == 0 else 64
    cfg = dict(n_layers=1, d_model=k, n_heads=k // hd, n_kv_heads=k // hd, head_dim=hd, ffn_dim=n, vocab=32,
               max_context=16, norm_eps=1e-5, rope_theta=10000.0)
    plan = session.LlamaCudaPlan.empty(cfg, session.CudaSessionTarget(device=device))
    try:
        plan.synth_tensor("blk.0.ffn_gate.weight", ggml_type, n, k, seed, std)
        return plan.read_tensor("blk.0.ffn_gate.weight")
    finally:
        plan.close()
