"""Host-side mirror of rustgrad's accelerated-session facade for the CUDA target.

Names and verbs follow the Metal session that rustgrad ships (src/session/target.rs:13-18,165-213;
src/models/transformer/metal_generation.rs:33-52,276-281,453-500,702-715,837-1207):

    target  = CudaSessionTarget(device=0)
    plan    = LlamaCudaPlan.from_gguf_bytes(data, target)      # LlamaMetalPlan::from_workflow_on
    session = target.prepare(plan)                             # SessionTarget::prepare
    session.generate_ids(prompt_ids, max_new)                  # LlamaMetalSession::generate_ids

Every failure is a typed :class:`RgError` subclass carrying the C ABI status; nothing falls back
to a CPU path.  Tokenisation and chat templates stay in the caller, exactly as the Metal session
keeps them host-side (metal_generation.rs:1209-1215): this facade works on token ids.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from ._lib import LlamaConfig, Options, Report

F32, F16, Q4_0, Q8_0 = 0, 1, 2, 8


class RgError(RuntimeError):
    status = -1

    def __init__(self, status: int, detail: str):
        super().__init__(f"{_lib.load().rg_b200_status_string(status).decode()}: {detail}")
        self.status = status
        self.detail = detail


_NAMES = ["Ok", "InvalidArgument", "UnsupportedType", "ShapeMismatch", "NonFiniteScale", "TokenOutOfRange",
          "ContextExhausted", "NonFiniteLogits", "FreshSessionRequired", "CudaError", "NcclError", "OutOfMemory", "Timeout",
          "Poisoned", "MalformedGguf", "MissingTensor", "UnexpectedTensor", "UnsupportedVariant", "MissingMetadata",
          "EmptyPrompt", "UnsupportedGeometry"]
ERRORS = {i: type(n, (RgError,), {"status": i}) for i, n in enumerate(_NAMES) if i}
globals().update({cls.__name__: cls for cls in ERRORS.values()})


def check(status: int) -> None:
    if status:
        detail = _lib.load().rg_b200_last_error().decode(errors="replace")
        raise ERRORS.get(status, RgError)(status, detail)


def _u8(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_uint8))


def _i32(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def _f32(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def config_struct(cfg: dict) -> LlamaConfig:
    return LlamaConfig(cfg["n_layers"], cfg["d_model"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"],
                       cfg["ffn_dim"], cfg["vocab"], cfg["max_context"], cfg["norm_eps"], cfg["rope_theta"],
                       cfg.get("eos_id", -1), cfg.get("eot_id", -1), cfg.get("rope_dim", 0), cfg.get("qk_norm", 0),
                       cfg.get("qkv_bias", 0))


def config_dict(c: LlamaConfig) -> dict:
    return {name: getattr(c, name) for name, _ in LlamaConfig._fields_}


@dataclass
class CudaSessionTarget:
    """One B200 (one process per GPU), optionally one rank of a tensor-parallel group."""
    device: int = 0
    max_batch: int = 1
    max_context: int = 0
    kv_f32: bool = False
    tp_rank: int = 0
    tp_world: int = 1
    nccl_id: bytes = b""
    disable_graph: bool = False
    disable_pdl: bool = False
    general_path_only: bool = False  # never take the fused small-batch decode path (tests)
    gemm_operands: str = ""  # tensor-core path operands: "" (compensated f16), "bf16", "f16", "f16x3"
    disable_fused_allreduce: bool = False  # tensor-parallel partial sums through NCCL instead of peer memory
    _opts: Options = field(default=None, repr=False)

    def options(self) -> Options:
        o = Options()
        o.device, o.max_batch, o.max_context = self.device, self.max_batch, self.max_context
        o.kv_f32, o.tp_rank, o.tp_world = int(self.kv_f32), self.tp_rank, self.tp_world
        o.disable_graph, o.disable_pdl = int(self.disable_graph), int(self.disable_pdl)
        o.disable_fused_allreduce = int(self.disable_fused_allreduce)
        o.general_path_only = int(self.general_path_only)
        o.gemm_operand_mode = {"": 0, "bf16": 1, "f16": 2, "f16x3": 3}[self.gemm_operands]
        if self.tp_world > 1:
            if len(self.nccl_id) != 128:
                raise InvalidArgument(1, "tensor parallelism needs the 128-byte NCCL id of rank 0")  # noqa: F821
            C.memmove(o.nccl_id, self.nccl_id, 128)
        return o

    def prepare(self, plan: "LlamaCudaPlan") -> "LlamaCudaSession":
        return plan.prepare()


def nccl_unique_id() -> bytes:
    buf = (C.c_uint8 * 128)()
    check(_lib.load().rg_b200_nccl_unique_id(buf))
    return bytes(buf)


class GgufFile:
    """read_gguf (src/gguf/mod.rs:384): parses and validates; keeps the bytes alive."""

    def __init__(self, data: bytes | np.ndarray):
        self._data = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data
        self._h = C.c_void_p()
        check(_lib.load().rg_b200_gguf_open(_u8(self._data), self._data.size, C.byref(self._h)))

    def close(self):
        if getattr(self, "_h", None):
            _lib.load().rg_b200_gguf_close(self._h)
            self._h = None

    __del__ = close

    def llama_config(self) -> dict:
        c = LlamaConfig()
        check(_lib.load().rg_b200_gguf_llama_config(self._h, C.byref(c)))
        return config_dict(c)

    def tensors(self):
        L = _lib.load()
        out = []
        for i in range(L.rg_b200_gguf_tensor_count(self._h)):
            name, t, rank = C.c_char_p(), C.c_int32(), C.c_int32()
            dims = (C.c_uint64 * 4)()
            data, n = C.POINTER(C.c_uint8)(), C.c_size_t()
            check(L.rg_b200_gguf_tensor_info(self._h, i, C.byref(name), C.byref(t), C.byref(rank), dims, C.byref(data),
                                             C.byref(n)))
            offset = C.addressof(data.contents) - self._data.ctypes.data
            out.append((name.value.decode(), t.value, [dims[j] for j in range(rank.value)], offset, n.value))
        return out


class LlamaCudaPlan:
    """Validated model bound to a target; weights uploaded once in their native block bytes."""

    def __init__(self, handle, cfg: dict, target: CudaSessionTarget):
        self._h, self.config, self.target = handle, cfg, target

    @classmethod
    def from_gguf_bytes(cls, data, target: CudaSessionTarget) -> "LlamaCudaPlan":
        g = GgufFile(data)
        try:
            cfg = g.llama_config()
            h = C.c_void_p()
            opts = target.options()
            check(_lib.load().rg_b200_plan_from_gguf(g._h, C.byref(opts), C.byref(h)))
            return cls(h, cfg, target)
        finally:
            g.close()

    @classmethod
    def from_path(cls, path, target: CudaSessionTarget) -> "LlamaCudaPlan":
        return cls.from_gguf_bytes(np.fromfile(path, dtype=np.uint8), target)

    @classmethod
    def from_tensors(cls, cfg: dict, tensors: dict, target: CudaSessionTarget) -> "LlamaCudaPlan":
        """``tensors``: name -> (ggml_type, rows, cols, uint8 bytes) (LlamaModelState::bind on parts)."""
        plan = cls.empty(cfg, target)
        for name, (t, rows, cols, data) in tensors.items():
            plan.add_tensor(name, t, rows, cols, data)
        return plan

    @classmethod
    def empty(cls, cfg: dict, target: CudaSessionTarget) -> "LlamaCudaPlan":
        h = C.c_void_p()
        c, opts = config_struct(cfg), target.options()
        check(_lib.load().rg_b200_plan_create(C.byref(c), C.byref(opts), C.byref(h)))
        return cls(h, dict(cfg), target)

    @classmethod
    def synthetic(cls, cfg: dict, target: CudaSessionTarget, seed: int, body_type: int = Q4_0, embed_type: int = Q8_0,
                  head_type: int | None = Q8_0, std: float = 0.02) -> "LlamaCudaPlan":
        """Seeded N(0, std) model generated and quantized on the device (no host copy of the weights)."""
        from .synth import tensor_inventory
        plan = cls.empty(cfg, target)
        for idx, (name, rows, cols, is_norm) in enumerate(tensor_inventory(cfg, tied_head=head_type is None)):
            t = F32 if is_norm else embed_type if name == "token_embd.weight" else head_type if name == "output.weight" \
                else body_type
            if not is_norm and cols % 32:
                t = F32
            plan.synth_tensor(name, t, rows, cols, seed * 1000003 + idx, std)
        return plan

    def add_tensor(self, name: str, ggml_type: int, rows: int, cols: int, data) -> None:
        data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
        check(_lib.load().rg_b200_plan_add_tensor(self._h, name.encode(), ggml_type, rows, cols, _u8(data), data.size))

    def synth_tensor(self, name: str, ggml_type: int, rows: int, cols: int, seed: int, std: float) -> None:
        check(_lib.load().rg_b200_plan_synth_tensor(self._h, name.encode(), ggml_type, rows, cols, seed, std))

    def read_tensor(self, name: str) -> np.ndarray:
        n = C.c_size_t()
        check(_lib.load().rg_b200_plan_tensor_nbytes(self._h, name.encode(), C.byref(n)))
        out = np.empty(n.value, dtype=np.uint8)
        check(_lib.load().rg_b200_plan_read_tensor(self._h, name.encode(), _u8(out), out.size))
        return out

    def prepare(self) -> "LlamaCudaSession":
        h = C.c_void_p()
        check(_lib.load().rg_b200_session_prepare(self._h, C.byref(h)))
        return LlamaCudaSession(h, self.config)

    def close(self):
        if getattr(self, "_h", None):
            _lib.load().rg_b200_plan_destroy(self._h)
            self._h = None

    __del__ = close


@dataclass
class LlamaCudaGeneration:
    """LlamaGeneration (generation.rs:40-60) without the decoded text."""
    prompt_ids: list
    generated_ids: list
    stopped: bool


class LlamaCudaSession:
    def __init__(self, handle, cfg: dict):
        self._h, self.config = handle, cfg
        self._L = _lib.load()

    def close(self):
        if getattr(self, "_h", None):
            self._L.rg_b200_session_destroy(self._h)
            self._h = None

    __del__ = close

    def position(self, row: int = 0) -> int:
        return self._L.rg_b200_position(self._h, row)

    def max_context(self) -> int:
        return self._L.rg_b200_max_context(self._h)

    def vocab_size(self) -> int:
        return self._L.rg_b200_vocab_size(self._h)

    def is_full(self) -> bool:
        return bool(self._L.rg_b200_is_full(self._h))

    def reset_sequence(self) -> None:
        check(self._L.rg_b200_reset_sequence(self._h))

    def prefill_ids(self, ids, row: int = 0, want_logits: bool = True):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        logits = np.empty(self.vocab_size(), dtype=np.float32) if want_logits else None
        check(self._L.rg_b200_prefill(self._h, row, _i32(ids), ids.size, _f32(logits) if want_logits else None))
        return logits

    def prefill_rows(self, prompts: dict, want_logits: bool = True):
        """Several prompts in one pass: ``prompts`` maps cache row -> token ids.  Returns
        (logits [n, vocab] in the dict's order or None, greedy ids [n])."""
        rows = np.ascontiguousarray(list(prompts.keys()), dtype=np.int32)
        lens = (C.c_size_t * len(rows))(*[len(p) for p in prompts.values()])
        ids = np.ascontiguousarray(np.concatenate([np.asarray(p, dtype=np.int32) for p in prompts.values()]) if len(rows)
                                   else np.zeros(0, np.int32), dtype=np.int32)
        logits = np.empty((len(rows), self.vocab_size()), dtype=np.float32) if want_logits else None
        greedy = np.empty(len(rows), dtype=np.int32)
        check(self._L.rg_b200_prefill_rows(self._h, _i32(rows), _i32(ids), lens, len(rows),
                                           _f32(logits) if want_logits else None, _i32(greedy)))
        return logits, greedy

    def run_token(self, token: int) -> np.ndarray:
        logits, _ = self.decode([token], want_logits=True)
        return logits[0]

    def decode(self, tokens, want_logits: bool = False, temperature: float | None = None, uniforms=None):
        """One step for ``len(tokens)`` rows.  With ``temperature`` and ``uniforms`` ([rows, vocab]) the ids are
        Gumbel-max samples (LlamaSampling::GumbelMax, generation.rs:10-19), otherwise greedy."""
        if not want_logits and uniforms is None and len(tokens) <= 32:
            # greedy ids only: reused ctypes arrays, no array objects per step
            io = self.__dict__.get("_step_io")
            if io is None:
                io = self.__dict__["_step_io"] = ((C.c_int32 * 32)(), (C.c_int32 * 32)())
            tin, tout = io
            b = len(tokens)
            for i in range(b):
                tin[i] = int(tokens[i])
            check(self._L.rg_b200_decode(self._h, tin, b, None, tout))
            return None, np.array(tout[:b], dtype=np.int32)
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        b = tokens.size
        logits = np.empty((b, self.vocab_size()), dtype=np.float32) if want_logits else None
        ids = np.empty(b, dtype=np.int32)
        lp = _f32(logits) if want_logits else None
        if uniforms is None:
            check(self._L.rg_b200_decode(self._h, _i32(tokens), b, lp, _i32(ids)))
        else:
            u = np.ascontiguousarray(uniforms, dtype=np.float32).reshape(b, self.vocab_size())
            check(self._L.rg_b200_decode_sampled(self._h, _i32(tokens), b, float(temperature), _f32(u), lp, _i32(ids)))
        return logits, ids

    def generate_ids(self, prompt_ids, max_new_tokens: int, temperature: float | None = None,
                     uniforms=None) -> LlamaCudaGeneration:
        """LlamaMetalSession::generate_ids; ``uniforms`` ([max_new_tokens, vocab], row-major [step, vocabulary])
        selects Gumbel-max sampling with ``temperature``, otherwise greedy."""
        p = np.ascontiguousarray(prompt_ids, dtype=np.int32)
        out = np.zeros(max(1, max_new_tokens), dtype=np.int32)
        n, stopped = C.c_size_t(0), C.c_int32(0)
        if uniforms is None:
            check(self._L.rg_b200_generate_greedy(self._h, _i32(p), p.size, max_new_tokens, _i32(out), C.byref(n),
                                                  C.byref(stopped)))
        else:
            u = np.ascontiguousarray(uniforms, dtype=np.float32).reshape(max_new_tokens, self.vocab_size())
            check(self._L.rg_b200_generate_sampled(self._h, _i32(p), p.size, max_new_tokens, float(temperature), _f32(u),
                                                   _i32(out), C.byref(n), C.byref(stopped)))
        return LlamaCudaGeneration(p.tolist(), out[: n.value].tolist(), bool(stopped.value))

    def decode_loop(self, first_tokens, steps: int):
        """Device-resident greedy loop; returns (ids [steps, batch], CUDA-event milliseconds)."""
        t = np.ascontiguousarray(first_tokens, dtype=np.int32)
        out = np.empty((steps, t.size), dtype=np.int32)
        ms = C.c_float(0)
        check(self._L.rg_b200_decode_loop(self._h, _i32(t), t.size, steps, _i32(out), C.byref(ms)))
        return out, ms.value

    def decode_profile(self, first_tokens, steps: int, in_step: bool = False) -> dict:
        """CUDA-event time per step of each kernel family replayed alone: serialized launches, or
        (``in_step``) with the dependent-launch edges the real step has between consecutive kernels."""
        t = np.ascontiguousarray(first_tokens, dtype=np.int32)
        ms = (C.c_float * 4)()
        marks = (C.c_uint64 * 4)()
        fn = self._L.rg_b200_decode_profile_in_step if in_step else self._L.rg_b200_decode_profile
        check(fn(self._h, _i32(t), t.size, steps, ms, marks))
        keys = ("gemv", "attention", "other", "total")
        return {k: {"ms_per_step": ms[i], "launches_per_step": marks[i]} for i, k in enumerate(keys)}

    def decode_profile_projections(self, first_tokens, steps: int) -> dict:
        """Milliseconds per step of the GEMV launches of each projection, each set replayed alone."""
        t = np.ascontiguousarray(first_tokens, dtype=np.int32)
        ms = (C.c_float * 5)()
        check(self._L.rg_b200_decode_profile_projections(self._h, _i32(t), t.size, steps, ms))
        return dict(zip(("qkv", "attn_output", "gate_up", "down", "head"), (float(v) for v in ms)))

    def report(self) -> dict:
        r = Report()
        check(self._L.rg_b200_report(self._h, C.byref(r)))
        return {name: getattr(r, name) for name, _ in Report._fields_}

    def stream(self) -> int:
        return int(self._L.rg_b200_session_stream(self._h) or 0)

    def expire_device_wait(self) -> None:
        """Test hook: the next step finds that a bounded device-side wait ran out (nothing faults or hangs)."""
        check(self._L.rg_b200_test_expire_device_wait(self._h))


class _DeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("sm_count", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("total_memory_bytes", C.c_uint64), ("l2_bytes", C.c_uint64), ("shared_memory_per_block", C.c_uint64)]


def device_info(device: int = 0) -> dict:
    """What a session on CUDA ordinal ``device`` would run on (rg_b200_device_info); raises when there is none."""
    L = _lib.load()
    L.rg_b200_device_info.argtypes = [C.c_int32, C.POINTER(_DeviceInfo)]
    info = _DeviceInfo()
    check(L.rg_b200_device_info(device, C.byref(info)))
    return {"name": info.name.decode(errors="replace"), "sm_count": info.sm_count, "compute_capability": (info.cc_major, info.cc_minor),
            "total_memory_bytes": info.total_memory_bytes, "l2_bytes": info.l2_bytes,
            "shared_memory_per_block": info.shared_memory_per_block}


def launch_count(kernel: str) -> int:
    """Launches of a kernel family made by this process so far (see rg_b200_launch_count)."""
    n = _lib.load().rg_b200_launch_count(kernel.encode())
    if n == 0xFFFFFFFFFFFFFFFF:
        raise KeyError(kernel)
    return int(n)


# ---- operator-level calls (host arrays in, host arrays out) --------------------------------

def dequantize(ggml_type: int, data, elements: int, device: int = 0) -> np.ndarray:
    data = np.ascontiguousarray(data, dtype=np.uint8)
    out = np.empty(elements, dtype=np.float32)
    check(_lib.load().rg_b200_dequantize(device, ggml_type, _u8(data), elements, _f32(out)))
    return out


def qmatmul(ggml_type: int, weight, n: int, k: int, activation, device: int = 0) -> np.ndarray:
    w = np.ascontiguousarray(weight, dtype=np.uint8)
    a = np.ascontiguousarray(activation, dtype=np.float32).reshape(-1, k) if k else np.zeros((np.asarray(activation).shape[0], 0), np.float32)
    out = np.empty((a.shape[0], n), dtype=np.float32)
    check(_lib.load().rg_b200_qmatmul(device, ggml_type, _u8(w), n, k, _f32(a), a.shape[0], _f32(out)))
    return out


def row_gather(ggml_type: int, weight, rows: int, cols: int, indices, device: int = 0) -> np.ndarray:
    w = np.ascontiguousarray(weight, dtype=np.uint8)
    idx = np.ascontiguousarray(indices, dtype=np.int64)
    out = np.empty((idx.size, cols), dtype=np.float32)
    check(_lib.load().rg_b200_row_gather(device, ggml_type, _u8(w), rows, cols, idx.ctypes.data_as(C.POINTER(C.c_int64)),
                                         idx.size, _f32(out)))
    return out


def qgemm(ggml_type: int, weight, n: int, k: int, activation, iters: int = 0, device: int = 0, operand_mode: int = 0):
    """Tensor-core GEMM, f32 accumulate; operand_mode 0 = bf16, 1 = f16, 2 = compensated f16 (hi + lo planes).
    Returns (output [m,n], mean kernel ms or 0)."""
    w = np.ascontiguousarray(weight, dtype=np.uint8)
    a = np.ascontiguousarray(activation, dtype=np.float32).reshape(-1, k)
    out = np.empty((a.shape[0], n), dtype=np.float32)
    ms = C.c_float(0)
    check(_lib.load().rg_b200_qgemm(device, ggml_type, _u8(w), n, k, _f32(a), a.shape[0], int(operand_mode), iters,
                                    _f32(out), C.byref(ms)))
    return out, ms.value


def attention_decode(q, keys, values, device: int = 0) -> np.ndarray:
    """q [heads, hd] f32; keys/values [kv_heads, n_pos, hd] as float32 or float16 arrays -> [heads, hd]."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    if keys.dtype != values.dtype or keys.dtype not in (np.float32, np.float16):
        raise TypeError("caches must both be float32 or both float16")
    keys, values = np.ascontiguousarray(keys), np.ascontiguousarray(values)
    out = np.empty_like(q)
    check(_lib.load().rg_b200_attention_decode(device, _f32(q), keys.ctypes.data_as(C.c_void_p),
                                               values.ctypes.data_as(C.c_void_p), q.shape[0], keys.shape[0], q.shape[1],
                                               keys.shape[1], int(keys.dtype == np.float32), _f32(out)))
    return out


def qmatmul_bench(ggml_type: int, weight, n: int, k: int, activation, rotate: int, iters: int, warmup: int = 3,
                  device: int = 0):
    """Returns (output [m,n], mean kernel milliseconds) for weights resident in HBM."""
    w = np.ascontiguousarray(weight, dtype=np.uint8)
    a = np.ascontiguousarray(activation, dtype=np.float32).reshape(-1, k)
    out = np.empty((a.shape[0], n), dtype=np.float32)
    ms = C.c_float(0)
    check(_lib.load().rg_b200_qmatmul_bench(device, ggml_type, _u8(w), n, k, _f32(a), a.shape[0], rotate, iters, warmup,
                                            _f32(out), C.byref(ms)))
    return out, ms.value


class KvSnapshot:
    """Immutable device copy of the first ``length`` cached positions of a row, all layers
    (LlamaNativePrefixSnapshot, src/models/transformer/serving/mod.rs:182-190)."""

    def __init__(self, session: "LlamaCudaSession", row: int, length: int):
        self._L = _lib.load()
        self._h = C.c_void_p()
        check(self._L.rg_b200_kv_snapshot_create(session._h, row, length, C.byref(self._h)))
        self.length = length
        self.bytes = int(self._L.rg_b200_kv_snapshot_bytes(self._h))

    def restore(self, session: "LlamaCudaSession", row: int) -> None:
        check(self._L.rg_b200_kv_snapshot_restore(session._h, self._h, row))

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.rg_b200_kv_snapshot_free(self._h)
            self._h = None
