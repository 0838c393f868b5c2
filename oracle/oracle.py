"""ctypes face of the CPU checker (``librg_oracle.so``).  Test infrastructure only.

Nothing in the shipped package imports this module: it is loaded by the test-suite, by the smoke
entry point and by the benchmark's CPU-baseline leg, and only to check or to time the CPU
restatement of rustgrad's GGUF Llama path (see ``rg_oracle.h`` for the reference citations).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "librg_oracle.so"

F32, F16, Q4_0, Q8_0 = 0, 1, 2, 8
MODE_STRICT, MODE_FAST = 0, 1
OK = 0
ERR_ARG, ERR_TYPE, ERR_NON_FINITE, ERR_TOKEN_RANGE, ERR_CONTEXT, ERR_NON_FINITE_LOGITS, ERR_INDEX = range(1, 8)


def build(force: bool = False) -> Path:
    """Compiles the checker with the committed Makefile when the library is absent or stale."""
    src = HERE / "rg_oracle.c"
    hdr = HERE / "rg_oracle.h"
    stale = (not LIB_PATH.exists()) or LIB_PATH.stat().st_mtime < max(src.stat().st_mtime, hdr.stat().st_mtime)
    if force or stale:
        subprocess.run(["make", "-C", str(HERE), "-B", "librg_oracle.so"], check=True, capture_output=True)
    return LIB_PATH


class Config(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int32), ("d_model", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("ffn_dim", C.c_int32), ("vocab", C.c_int32), ("max_context", C.c_int32),
        ("norm_eps", C.c_float), ("rope_theta", C.c_double), ("eos_id", C.c_int32), ("eot_id", C.c_int32),
        ("rope_dim", C.c_int32), ("qk_norm", C.c_int32), ("qkv_bias", C.c_int32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(LIB_PATH))
        u8p, f32p, i32p = C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.POINTER(C.c_int32)
        L.rgo_f16_to_f32.restype = C.c_float
        L.rgo_f16_to_f32.argtypes = [C.c_uint16]
        L.rgo_f32_to_f16.restype = C.c_uint16
        L.rgo_f32_to_f16.argtypes = [C.c_float]
        L.rgo_block_elements.argtypes = [C.c_int]
        L.rgo_block_bytes.argtypes = [C.c_int]
        L.rgo_decode_q4_0_block.argtypes = [u8p, f32p]
        L.rgo_decode_q8_0_block.argtypes = [u8p, f32p]
        L.rgo_dequantize.argtypes = [C.c_int, u8p, C.c_size_t, f32p]
        L.rgo_row_gather.argtypes = [C.c_int, u8p, C.c_size_t, C.c_size_t, C.POINTER(C.c_int64), C.c_size_t, f32p]
        L.rgo_quantized_matmul.argtypes = [C.c_int, u8p, C.c_size_t, C.c_size_t, f32p, C.c_size_t, f32p]
        L.rgo_dense_matmul_strict.restype = None
        L.rgo_dense_matmul_strict.argtypes = [f32p, C.c_size_t, C.c_size_t, f32p, C.c_size_t, f32p]
        L.rgo_model_create.restype = C.c_void_p
        L.rgo_model_create.argtypes = [C.POINTER(Config)]
        L.rgo_model_destroy.restype = None
        L.rgo_model_destroy.argtypes = [C.c_void_p]
        L.rgo_model_set_tensor.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_size_t, C.c_size_t, u8p]
        L.rgo_model_check.argtypes = [C.c_void_p]
        L.rgo_cache_create.restype = C.c_void_p
        L.rgo_cache_create.argtypes = [C.c_void_p, C.c_int]
        L.rgo_cache_destroy.restype = None
        L.rgo_cache_destroy.argtypes = [C.c_void_p]
        L.rgo_cache_clear.restype = None
        L.rgo_cache_clear.argtypes = [C.c_void_p]
        L.rgo_cache_len.argtypes = [C.c_void_p]
        L.rgo_cache_fill_seeded.argtypes = [C.c_void_p, C.c_int, C.c_uint64]
        L.rgo_forward.argtypes = [C.c_void_p, C.c_void_p, i32p, C.c_int, C.c_int, C.c_int, C.c_int, f32p]
        L.rgo_select_greedy.argtypes = [f32p, C.c_int, i32p]
        L.rgo_select_gumbel.argtypes = [f32p, C.c_int, C.c_float, f32p, i32p]
        L.rgo_generate_greedy.argtypes = [C.c_void_p, C.c_void_p, i32p, C.c_int, C.c_int, C.c_int, C.c_int, i32p,
                                          C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.rgo_attention_decode.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int, f32p]
        L.rgo_forward_f64.argtypes = [C.c_void_p, i32p, C.c_int, C.POINTER(C.c_double)]
        _lib = L
    return _lib


class OracleError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"oracle {what} failed with status {code}")
        self.code = code


def _u8(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_uint8))


def _f32(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _i32(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def f16_to_f32(bits: int) -> float:
    return float(lib().rgo_f16_to_f32(bits))


def f32_to_f16(value: float) -> int:
    return int(lib().rgo_f32_to_f16(value))


def dequantize(ggml_type: int, data: np.ndarray, elements: int) -> np.ndarray:
    data = np.ascontiguousarray(data, dtype=np.uint8)
    out = np.empty(elements, dtype=np.float32)
    rc = lib().rgo_dequantize(ggml_type, _u8(data), elements, _f32(out))
    if rc:
        raise OracleError(rc, "dequantize")
    return out


def row_gather(ggml_type: int, data: np.ndarray, rows: int, cols: int, indices) -> np.ndarray:
    data = np.ascontiguousarray(data, dtype=np.uint8)
    idx = np.ascontiguousarray(indices, dtype=np.int64)
    out = np.empty((idx.size, cols), dtype=np.float32)
    rc = lib().rgo_row_gather(ggml_type, _u8(data), rows, cols, idx.ctypes.data_as(C.POINTER(C.c_int64)), idx.size,
                              _f32(out))
    if rc:
        raise OracleError(rc, "row_gather")
    return out


def quantized_matmul(ggml_type: int, weight: np.ndarray, n: int, k: int, activation: np.ndarray) -> np.ndarray:
    """f64-accumulating blockwise plan: activation [m,k] x packed [n,k] -> [m,n]."""
    weight = np.ascontiguousarray(weight, dtype=np.uint8)
    a = np.ascontiguousarray(activation, dtype=np.float32).reshape(-1, k)
    out = np.empty((a.shape[0], n), dtype=np.float32)
    rc = lib().rgo_quantized_matmul(ggml_type, _u8(weight), n, k, _f32(a), a.shape[0], _f32(out))
    if rc:
        raise OracleError(rc, "quantized_matmul")
    return out


def dense_matmul_strict(weight: np.ndarray, activation: np.ndarray) -> np.ndarray:
    w = np.ascontiguousarray(weight, dtype=np.float32)
    a = np.ascontiguousarray(activation, dtype=np.float32).reshape(-1, w.shape[1])
    out = np.empty((a.shape[0], w.shape[0]), dtype=np.float32)
    lib().rgo_dense_matmul_strict(_f32(w), w.shape[0], w.shape[1], _f32(a), a.shape[0], _f32(out))
    return out


def attention_decode(q: np.ndarray, keys: np.ndarray, values: np.ndarray) -> np.ndarray:
    """q [heads, hd]; keys/values [kv_heads, n_pos, hd] (f32) -> [heads, hd]."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    keys = np.ascontiguousarray(keys, dtype=np.float32)
    values = np.ascontiguousarray(values, dtype=np.float32)
    out = np.empty_like(q)
    rc = lib().rgo_attention_decode(_f32(q), _f32(keys), _f32(values), q.shape[0], keys.shape[0], q.shape[1], keys.shape[1],
                                    _f32(out))
    if rc:
        raise OracleError(rc, "attention_decode")
    return out


def select_greedy(row: np.ndarray) -> int:
    row = np.ascontiguousarray(row, dtype=np.float32)
    tok = C.c_int32(-1)
    rc = lib().rgo_select_greedy(_f32(row), row.size, C.byref(tok))
    if rc:
        raise OracleError(rc, "select_greedy")
    return tok.value


def select_gumbel(row: np.ndarray, temperature: float, uniforms: np.ndarray) -> int:
    """Gumbel-max with an explicit uniform row (generation.rs:260-287)."""
    row = np.ascontiguousarray(row, dtype=np.float32)
    u = np.ascontiguousarray(uniforms, dtype=np.float32)
    assert u.size == row.size
    tok = C.c_int32(-1)
    rc = lib().rgo_select_gumbel(_f32(row), row.size, float(temperature), _f32(u), C.byref(tok))
    if rc:
        raise OracleError(rc, "select_gumbel")
    return tok.value


class OracleModel:
    """Owns one rgo_model plus the numpy byte arrays its tensors borrow.

    ``tensors`` maps GGUF tensor names to ``(ggml_type, rows, cols, uint8 array)``; norm vectors use
    rows == 1.
    """

    def __init__(self, config: dict, tensors: dict, kv_f16: bool = False, threads: int | None = None):
        self.cfg = Config(
            config["n_layers"], config["d_model"], config["n_heads"], config["n_kv_heads"], config["head_dim"],
            config["ffn_dim"], config["vocab"], config["max_context"], config["norm_eps"], config["rope_theta"],
            config.get("eos_id", -1), config.get("eot_id", -1), config.get("rope_dim", 0), config.get("qk_norm", 0),
            config.get("qkv_bias", 0))
        self.vocab = config["vocab"]
        self.threads = threads or (os.cpu_count() or 1)
        self._keep = []
        self.model = lib().rgo_model_create(C.byref(self.cfg))
        if not self.model:
            raise OracleError(ERR_ARG, "model_create")
        for name, (t, rows, cols, data) in tensors.items():
            data = np.ascontiguousarray(data, dtype=np.uint8)
            self._keep.append(data)
            rc = lib().rgo_model_set_tensor(self.model, name.encode(), t, rows, cols, _u8(data))
            if rc:
                raise OracleError(rc, f"set_tensor({name})")
        rc = lib().rgo_model_check(self.model)
        if rc:
            raise OracleError(rc, "model_check")
        self.cache = lib().rgo_cache_create(self.model, int(kv_f16))

    def close(self):
        if getattr(self, "cache", None):
            lib().rgo_cache_destroy(self.cache)
            self.cache = None
        if getattr(self, "model", None):
            lib().rgo_model_destroy(self.model)
            self.model = None

    __del__ = close

    def reset(self):
        lib().rgo_cache_clear(self.cache)

    def fill_cache_seeded(self, n_pos: int, seed: int = 1) -> None:
        """Timing aid: the cache holds ``n_pos`` positions of seeded pseudo-random K / V rows afterwards."""
        rc = lib().rgo_cache_fill_seeded(self.cache, n_pos, seed)
        if rc:
            raise OracleError(rc, "cache_fill_seeded")

    @property
    def position(self) -> int:
        return lib().rgo_cache_len(self.cache)

    def forward(self, tokens, mode: int = MODE_STRICT, all_logits: bool = False) -> np.ndarray:
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.empty((t.size if all_logits else 1, self.vocab), dtype=np.float32)
        rc = lib().rgo_forward(self.model, self.cache, _i32(t), t.size, mode, self.threads, int(all_logits), _f32(out))
        if rc:
            raise OracleError(rc, "forward")
        return out if all_logits else out[0]

    def forward_f64(self, tokens) -> np.ndarray:
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.empty((t.size, self.vocab), dtype=np.float64)
        rc = lib().rgo_forward_f64(self.model, _i32(t), t.size, out.ctypes.data_as(C.POINTER(C.c_double)))
        if rc:
            raise OracleError(rc, "forward_f64")
        return out

    def generate_greedy(self, prompt, max_new: int, mode: int = MODE_STRICT):
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.zeros(max(max_new, 1), dtype=np.int32)
        n_out, stopped = C.c_int(0), C.c_int(0)
        rc = lib().rgo_generate_greedy(self.model, self.cache, _i32(p), p.size, max_new, mode, self.threads, _i32(out),
                                       C.byref(n_out), C.byref(stopped))
        if rc:
            raise OracleError(rc, "generate_greedy")
        return out[: n_out.value].tolist(), bool(stopped.value)
