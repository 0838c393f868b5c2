"""Q8_0 / Q4_0 block encoders used to write synthetic GGUF files.

rustgrad only decodes GGML blocks (src/gguf/quantization/blocks.rs:1244-1257,1493-1505); it has no
encoder.  These follow the published GGML rules so that the bytes decode under the reference's
decoders exactly as they would for a llama.cpp-written file:

* Q8_0: ``d = max|x| / 127``; ``q = round_half_away(x / d)``; block = f16(d) + 32 int8.
* Q4_0: ``m`` = the element of largest magnitude (sign kept), ``d = m / -8``;
  ``q = min(15, trunc(x / d + 8.5))``; block = f16(d) + 16 bytes, byte j = q[j] | q[j+16] << 4.

The scale used for the division is the unrounded f32 ``d``; the stored scale is its f16 rounding.
Encoding is an offline writer tool: it never runs on the inference path.
"""
from __future__ import annotations

import numpy as np

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K = 0, 1, 2, 8, 12, 14
BLOCK_BYTES = {F32: 4, F16: 2, Q4_0: 18, Q8_0: 34, Q4_K: 144, Q6_K: 210}
BLOCK_ELEMS = {F32: 1, F16: 1, Q4_0: 32, Q8_0: 32, Q4_K: 256, Q6_K: 256}


def random_k_blocks(ggml_type: int, n_blocks: int, rng, scale: float = 0.02) -> np.ndarray:
    """Valid Q4_K / Q6_K super-blocks with random contents and small finite f16 scales.  There is no
    K-quant encoder here (the reference has none either): tests decode these bytes on both sides."""
    bb = BLOCK_BYTES[ggml_type]
    blocks = rng.integers(0, 256, (n_blocks, bb), dtype=np.uint8)
    if ggml_type == Q4_K:
        d = (rng.random(n_blocks) * scale / 63.0 / 8.0 + 1e-5).astype(np.float16)
        dmin = (rng.random(n_blocks) * scale / 63.0 / 2.0).astype(np.float16)
        blocks[:, 0:2] = d.view(np.uint8).reshape(n_blocks, 2)
        blocks[:, 2:4] = dmin.view(np.uint8).reshape(n_blocks, 2)
    elif ggml_type == Q6_K:
        d = (rng.random(n_blocks) * scale / 32.0 / 64.0 + 1e-6).astype(np.float16)
        blocks[:, 208:210] = d.view(np.uint8).reshape(n_blocks, 2)
    else:
        raise ValueError("not a K-quant type")
    return blocks.reshape(-1)


def tensor_nbytes(ggml_type: int, elements: int) -> int:
    be = BLOCK_ELEMS[ggml_type]
    if elements % be:
        raise ValueError("element count is not a multiple of the block size")
    return elements // be * BLOCK_BYTES[ggml_type]


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 32)
    amax = np.abs(x).max(axis=1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    scaled = x * inv[:, None]
    q = np.where(scaled >= 0, np.floor(scaled + np.float32(0.5)), np.ceil(scaled - np.float32(0.5))).astype(np.int8)
    out = np.empty((x.shape[0], 34), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 32)
    idx = np.abs(x).argmax(axis=1)
    m = x[np.arange(x.shape[0]), idx]
    d = (m / np.float32(-8.0)).astype(np.float32)
    inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    q = np.minimum(15, (x * inv[:, None] + np.float32(8.5)).astype(np.int32)).astype(np.uint8)
    out = np.empty((x.shape[0], 18), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def encode(ggml_type: int, x: np.ndarray) -> np.ndarray:
    """Encodes a float32 array into the byte image of a GGML tensor of the given type."""
    if ggml_type == F32:
        return np.ascontiguousarray(x, dtype=np.float32).reshape(-1).view(np.uint8)
    if ggml_type == F16:
        return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).reshape(-1).view(np.uint8)
    if ggml_type == Q8_0:
        return quantize_q8_0(x)
    if ggml_type == Q4_0:
        return quantize_q4_0(x)
    raise ValueError(f"unsupported ggml type {ggml_type}")
