"""ctypes binding of ``librg_b200.so`` (the C ABI of ``include/rg_b200.h``).

Importing this module fails loudly when the CUDA library is missing: there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

HERE = Path(__file__).resolve().parent
# RG_B200_LIB names another build of the library (a development variant); the default is the in-tree build
LIB_PATH = Path(os.environ["RG_B200_LIB"]) if os.environ.get("RG_B200_LIB") else HERE / "librg_b200.so"


class LlamaConfig(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int32), ("d_model", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("ffn_dim", C.c_int32), ("vocab", C.c_int32), ("max_context", C.c_int32),
        ("norm_eps", C.c_float), ("rope_theta", C.c_double), ("eos_id", C.c_int32), ("eot_id", C.c_int32),
        ("rope_dim", C.c_int32), ("qk_norm", C.c_int32), ("qkv_bias", C.c_int32),
    ]


class Options(C.Structure):
    _fields_ = [
        ("device", C.c_int32), ("max_batch", C.c_int32), ("max_context", C.c_int32), ("kv_f32", C.c_int32),
        ("tp_rank", C.c_int32), ("tp_world", C.c_int32), ("nccl_id", C.c_uint8 * 128), ("disable_graph", C.c_int32),
        ("disable_pdl", C.c_int32), ("disable_fused_allreduce", C.c_int32), ("general_path_only", C.c_int32),
        ("gemm_operand_mode", C.c_int32), ("reserved", C.c_int32 * 6),
    ]


class Report(C.Structure):
    _fields_ = [
        ("kernel_launches", C.c_uint64), ("graph_replays", C.c_uint64), ("h2d_calls", C.c_uint64),
        ("h2d_bytes", C.c_uint64), ("d2h_calls", C.c_uint64), ("d2h_bytes", C.c_uint64), ("weight_bytes", C.c_uint64),
        ("kv_bytes", C.c_uint64), ("fallback_count", C.c_uint64), ("last_prefill_ms", C.c_float),
        ("last_decode_ms", C.c_float), ("peer_reduce_launches", C.c_uint64),
    ]


EXPORTS = [
    "rg_b200_version", "rg_b200_status_string", "rg_b200_last_error", "rg_b200_test_fail_after", "rg_b200_test_expire_device_wait", "rg_b200_debug_read_trace", "rg_b200_launch_count", "rg_b200_gguf_open",
    "rg_b200_gguf_close", "rg_b200_gguf_tensor_count", "rg_b200_gguf_tensor_info", "rg_b200_gguf_llama_config",
    "rg_b200_plan_create", "rg_b200_plan_add_tensor", "rg_b200_plan_from_gguf", "rg_b200_plan_synth_tensor",
    "rg_b200_plan_tensor_nbytes", "rg_b200_plan_read_tensor", "rg_b200_plan_destroy", "rg_b200_session_prepare",
    "rg_b200_session_destroy", "rg_b200_position", "rg_b200_max_context", "rg_b200_vocab_size", "rg_b200_is_full",
    "rg_b200_reset_sequence", "rg_b200_prefill", "rg_b200_prefill_rows", "rg_b200_decode", "rg_b200_generate_greedy", "rg_b200_decode_sampled", "rg_b200_generate_sampled", "rg_b200_decode_loop", "rg_b200_decode_profile", "rg_b200_decode_profile_in_step", "rg_b200_decode_profile_projections",
    "rg_b200_report", "rg_b200_session_stream", "rg_b200_nccl_unique_id", "rg_b200_tp_shard", "rg_b200_dequantize", "rg_b200_qmatmul",
    "rg_b200_row_gather", "rg_b200_qmatmul_bench", "rg_b200_qgemm", "rg_b200_attention_decode", "rg_b200_attention_decode_noalloc",
    "rg_b200_reset_row", "rg_b200_prefill_select", "rg_b200_decode_rows", "rg_b200_select", "rg_b200_kv_snapshot_create",
    "rg_b200_kv_snapshot_length", "rg_b200_kv_snapshot_bytes", "rg_b200_kv_snapshot_restore", "rg_b200_kv_snapshot_free",
    # include/rg_b200_tokenizer.h (bound in tokenizer.py)
    "rg_b200_tokenizer_new", "rg_b200_tokenizer_from_gguf", "rg_b200_tokenizer_free", "rg_b200_tokenizer_config",
    "rg_b200_tokenizer_is_end", "rg_b200_tokenizer_parse_preset", "rg_b200_tokenizer_encode", "rg_b200_tokenizer_decode",
    "rg_b200_tok_stream_new", "rg_b200_tok_stream_push", "rg_b200_tok_stream_finish", "rg_b200_tok_stream_free",
    "rg_b200_chat_template_from_gguf", "rg_b200_chat_template_text", "rg_b200_chat_render",
    # include/rg_b200_workflow.h (bound in workflow.py)
    "rg_b200_workflow_open", "rg_b200_workflow_close", "rg_b200_workflow_session", "rg_b200_workflow_tokenizer",
    "rg_b200_workflow_generate_text", "rg_b200_workflow_generate_chat", "rg_b200_workflow_prompt_ids",
    "rg_b200_workflow_generated_ids", "rg_b200_workflow_decoded", "rg_b200_workflow_rendered_prompt",
    # include/rg_b200_serving.h (bound in serving.py)
    "rg_b200_scheduler_new", "rg_b200_scheduler_new_with_backend", "rg_b200_scheduler_free", "rg_b200_scheduler_submit_ids",
    "rg_b200_scheduler_submit_text", "rg_b200_scheduler_submit_chat", "rg_b200_scheduler_status", "rg_b200_scheduler_result",
    "rg_b200_scheduler_remove", "rg_b200_scheduler_pending", "rg_b200_scheduler_completed", "rg_b200_scheduler_prefix_stats",
    "rg_b200_scheduler_invalidate_prefix_cache", "rg_b200_scheduler_step", "rg_b200_scheduler_rebind",
    "rg_b200_scheduler_rebind_with_backend",
    "rg_b200_batch_generator_new", "rg_b200_batch_generator_new_with_backend", "rg_b200_batch_generator_free",
    "rg_b200_batch_generator_cache_lengths", "rg_b200_batch_generator_clear", "rg_b200_batch_generate_ids",
    "rg_b200_batch_generate_texts", "rg_b200_batch_sequence",
    "rg_b200_conversation_new", "rg_b200_conversation_new_with_backend", "rg_b200_conversation_free",
    "rg_b200_conversation_history_len", "rg_b200_conversation_message", "rg_b200_conversation_cache_len",
    "rg_b200_conversation_reset", "rg_b200_conversation_send", "rg_b200_device_info",
]

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m rustgrad_b200.build` (nvcc, sm_100a). "
            "rustgrad_b200 has no CPU fallback.")
    L = C.CDLL(str(LIB_PATH))
    vp, u8p, f32p, i32p = C.c_void_p, C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.POINTER(C.c_int32)
    L.rg_b200_version.restype = C.c_char_p
    L.rg_b200_status_string.restype = C.c_char_p
    L.rg_b200_status_string.argtypes = [C.c_int32]
    L.rg_b200_last_error.restype = C.c_char_p
    L.rg_b200_test_fail_after.argtypes = [C.c_char_p, C.c_int32]
    L.rg_b200_test_expire_device_wait.argtypes = [vp]
    L.rg_b200_debug_read_trace.argtypes = [vp, C.POINTER(C.c_uint64), C.c_int32]
    L.rg_b200_launch_count.restype = C.c_uint64
    L.rg_b200_launch_count.argtypes = [C.c_char_p]
    L.rg_b200_gguf_open.argtypes = [u8p, C.c_size_t, C.POINTER(vp)]
    L.rg_b200_gguf_close.restype = None
    L.rg_b200_gguf_close.argtypes = [vp]
    L.rg_b200_gguf_tensor_count.restype = C.c_size_t
    L.rg_b200_gguf_tensor_count.argtypes = [vp]
    L.rg_b200_gguf_tensor_info.argtypes = [vp, C.c_size_t, C.POINTER(C.c_char_p), i32p, i32p, C.POINTER(C.c_uint64),
                                           C.POINTER(u8p), C.POINTER(C.c_size_t)]
    L.rg_b200_gguf_llama_config.argtypes = [vp, C.POINTER(LlamaConfig)]
    L.rg_b200_plan_create.argtypes = [C.POINTER(LlamaConfig), C.POINTER(Options), C.POINTER(vp)]
    L.rg_b200_plan_add_tensor.argtypes = [vp, C.c_char_p, C.c_int32, C.c_uint64, C.c_uint64, u8p, C.c_size_t]
    L.rg_b200_plan_from_gguf.argtypes = [vp, C.POINTER(Options), C.POINTER(vp)]
    L.rg_b200_plan_synth_tensor.argtypes = [vp, C.c_char_p, C.c_int32, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float]
    L.rg_b200_plan_tensor_nbytes.argtypes = [vp, C.c_char_p, C.POINTER(C.c_size_t)]
    L.rg_b200_plan_read_tensor.argtypes = [vp, C.c_char_p, u8p, C.c_size_t]
    L.rg_b200_plan_destroy.restype = None
    L.rg_b200_plan_destroy.argtypes = [vp]
    L.rg_b200_session_prepare.argtypes = [vp, C.POINTER(vp)]
    L.rg_b200_session_destroy.restype = None
    L.rg_b200_session_destroy.argtypes = [vp]
    L.rg_b200_position.argtypes = [vp, C.c_int32]
    L.rg_b200_max_context.argtypes = [vp]
    L.rg_b200_vocab_size.argtypes = [vp]
    L.rg_b200_is_full.argtypes = [vp]
    L.rg_b200_reset_sequence.argtypes = [vp]
    L.rg_b200_prefill.argtypes = [vp, C.c_int32, i32p, C.c_size_t, f32p]
    L.rg_b200_prefill_rows.argtypes = [vp, i32p, i32p, C.POINTER(C.c_size_t), C.c_int32, f32p, i32p]
    L.rg_b200_decode.argtypes = [vp, i32p, C.c_int32, f32p, i32p]
    L.rg_b200_generate_greedy.argtypes = [vp, i32p, C.c_size_t, C.c_size_t, i32p, C.POINTER(C.c_size_t), i32p]
    L.rg_b200_decode_sampled.argtypes = [vp, i32p, C.c_int32, C.c_float, f32p, f32p, i32p]
    L.rg_b200_generate_sampled.argtypes = [vp, i32p, C.c_size_t, C.c_size_t, C.c_float, f32p, i32p, C.POINTER(C.c_size_t), i32p]
    L.rg_b200_decode_loop.argtypes = [vp, i32p, C.c_int32, C.c_int32, i32p, f32p]
    L.rg_b200_decode_profile.argtypes = [vp, i32p, C.c_int32, C.c_int32, f32p, C.POINTER(C.c_uint64)]
    L.rg_b200_decode_profile_in_step.argtypes = [vp, i32p, C.c_int32, C.c_int32, f32p, C.POINTER(C.c_uint64)]
    L.rg_b200_decode_profile_projections.argtypes = [vp, i32p, C.c_int32, C.c_int32, f32p]
    L.rg_b200_report.argtypes = [vp, C.POINTER(Report)]
    L.rg_b200_session_stream.restype = vp
    L.rg_b200_session_stream.argtypes = [vp]
    L.rg_b200_nccl_unique_id.argtypes = [u8p]
    L.rg_b200_tp_shard.argtypes = [C.c_char_p, C.c_int32, C.c_uint64, C.c_uint64, C.c_int32, C.c_int32] + [C.POINTER(C.c_uint64)] * 4
    L.rg_b200_dequantize.argtypes = [C.c_int32, C.c_int32, u8p, C.c_size_t, f32p]
    L.rg_b200_qmatmul.argtypes = [C.c_int32, C.c_int32, u8p, C.c_uint64, C.c_uint64, f32p, C.c_uint64, f32p]
    L.rg_b200_row_gather.argtypes = [C.c_int32, C.c_int32, u8p, C.c_uint64, C.c_uint64, C.POINTER(C.c_int64),
                                     C.c_size_t, f32p]
    L.rg_b200_qgemm.argtypes = [C.c_int32, C.c_int32, u8p, C.c_uint64, C.c_uint64, f32p, C.c_uint64, C.c_int32, C.c_int32,
                                f32p, f32p]
    L.rg_b200_reset_row.argtypes = [vp, C.c_int32]
    L.rg_b200_prefill_select.argtypes = [vp, C.c_int32, i32p, C.c_size_t, C.c_float, f32p, f32p, i32p]
    L.rg_b200_decode_rows.argtypes = [vp, i32p, i32p, C.c_int32, f32p, f32p, f32p, i32p]
    L.rg_b200_select.argtypes = [vp, f32p, C.c_int32, f32p, f32p, i32p]
    L.rg_b200_kv_snapshot_create.argtypes = [vp, C.c_int32, C.c_int32, C.POINTER(vp)]
    L.rg_b200_kv_snapshot_length.argtypes = [vp]
    L.rg_b200_kv_snapshot_bytes.restype = C.c_size_t
    L.rg_b200_kv_snapshot_bytes.argtypes = [vp]
    L.rg_b200_kv_snapshot_restore.argtypes = [vp, vp, C.c_int32]
    L.rg_b200_kv_snapshot_free.restype = None
    L.rg_b200_kv_snapshot_free.argtypes = [vp]
    L.rg_b200_attention_decode_noalloc.argtypes = [vp, vp, vp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                   C.c_int32, vp, vp, C.c_int32]
    L.rg_b200_attention_decode.argtypes = [C.c_int32, f32p, vp, vp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                           f32p]
    L.rg_b200_qmatmul_bench.argtypes = [C.c_int32, C.c_int32, u8p, C.c_uint64, C.c_uint64, f32p, C.c_uint64, C.c_int32,
                                        C.c_int32, C.c_int32, f32p, f32p]
    _lib = L
    return L
