//! Raw bindings to `librg_b200.so`, the sm_100a implementation of rustgrad's GGUF-quantized Llama
//! inference path, plus (in [`safe`]) the typed facade a rustgrad fork wires to its `SessionTarget`.
//!
//! Every item mirrors a declaration of `include/rg_b200.h`, `include/rg_b200_tokenizer.h`,
//! `include/rg_b200_workflow.h` or `include/rg_b200_serving.h`; the headers carry the documentation and, for each entry point, the
//! rustgrad interface it stands in for.  All 114 exports are declared here.
#![allow(non_camel_case_types)]

use core::ffi::{c_char, c_void};

pub mod safe;

/// `rg_status`: typed, fail-closed statuses (0 = success).
pub mod status {
    pub const OK: i32 = 0;
    pub const INVALID_ARGUMENT: i32 = 1;
    pub const UNSUPPORTED_TYPE: i32 = 2;
    pub const SHAPE_MISMATCH: i32 = 3;
    pub const NON_FINITE_SCALE: i32 = 4;
    pub const TOKEN_OUT_OF_RANGE: i32 = 5;
    pub const CONTEXT_EXHAUSTED: i32 = 6;
    pub const NON_FINITE_LOGITS: i32 = 7;
    pub const FRESH_SESSION_REQUIRED: i32 = 8;
    pub const CUDA_ERROR: i32 = 9;
    pub const NCCL_ERROR: i32 = 10;
    pub const OUT_OF_MEMORY: i32 = 11;
    pub const TIMEOUT: i32 = 12;
    pub const POISONED: i32 = 13;
    pub const MALFORMED_GGUF: i32 = 14;
    pub const MISSING_TENSOR: i32 = 15;
    pub const UNEXPECTED_TENSOR: i32 = 16;
    pub const UNSUPPORTED_VARIANT: i32 = 17;
    pub const MISSING_METADATA: i32 = 18;
    pub const EMPTY_PROMPT: i32 = 19;
    pub const UNSUPPORTED_GEOMETRY: i32 = 20;
}

/// GGML tensor types on this path (`src/gguf/tensor.rs:33-59`).
pub mod ggml_type {
    pub const F32: i32 = 0;
    pub const F16: i32 = 1;
    pub const Q4_0: i32 = 2;
    pub const Q8_0: i32 = 8;
    pub const Q4_K: i32 = 12;
    pub const Q6_K: i32 = 14;
}

macro_rules! opaque {
    ($($name:ident),*) => { $(#[repr(C)] pub struct $name { _private: [u8; 0] })* };
}
opaque!(rg_gguf, rg_plan, rg_session, rg_kv_snapshot, rg_tokenizer, rg_tok_stream, rg_workflow);

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq)]
pub struct rg_llama_config {
    pub n_layers: i32,
    pub d_model: i32,
    pub n_heads: i32,
    pub n_kv_heads: i32,
    pub head_dim: i32,
    pub ffn_dim: i32,
    pub vocab: i32,
    pub max_context: i32,
    pub norm_eps: f32,
    pub rope_theta: f64,
    /// -1 = none
    pub eos_id: i32,
    /// -1 = none
    pub eot_id: i32,
    /// rotary lanes per head; 0 = head_dim
    pub rope_dim: i32,
    /// 0 none, 1 per head, 2 per projection
    pub qk_norm: i32,
    /// 1: q / k / v projection biases are bound
    pub qkv_bias: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct rg_options {
    pub device: i32,
    pub max_batch: i32,
    pub max_context: i32,
    pub kv_f32: i32,
    pub tp_rank: i32,
    pub tp_world: i32,
    pub nccl_id: [u8; 128],
    pub disable_graph: i32,
    pub disable_pdl: i32,
    pub disable_fused_allreduce: i32,
    pub general_path_only: i32,
    pub gemm_operand_mode: i32,
    pub reserved: [i32; 6],
}

impl Default for rg_options {
    fn default() -> Self {
        // the header's rule: zero-initialise, then set what differs
        Self {
            device: 0,
            max_batch: 0,
            max_context: 0,
            kv_f32: 0,
            tp_rank: 0,
            tp_world: 0,
            nccl_id: [0; 128],
            disable_graph: 0,
            disable_pdl: 0,
            disable_fused_allreduce: 0,
            general_path_only: 0,
            gemm_operand_mode: 0,
            reserved: [0; 6],
        }
    }
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq)]
pub struct rg_report {
    pub kernel_launches: u64,
    pub graph_replays: u64,
    pub h2d_calls: u64,
    pub h2d_bytes: u64,
    pub d2h_calls: u64,
    pub d2h_bytes: u64,
    pub weight_bytes: u64,
    pub kv_bytes: u64,
    pub fallback_count: u64,
    pub last_prefill_ms: f32,
    pub last_decode_ms: f32,
    pub peer_reduce_launches: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct rg_tok_config {
    pub preset: i32,
    pub has_bos: i32,
    pub bos_id: u32,
    pub eos_id: u32,
    pub has_eot: i32,
    pub eot_id: u32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct rg_tok_error {
    pub status: i32,
    pub value: u64,
    pub value2: u64,
    pub text_len: usize,
    pub text: [c_char; 128],
}

impl Default for rg_tok_error {
    fn default() -> Self {
        Self { status: 0, value: 0, value2: 0, text_len: 0, text: [0; 128] }
    }
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct rg_prompt_output {
    pub n_prompt_ids: usize,
    pub n_generated_ids: usize,
    pub decoded_bytes: usize,
    pub rendered_bytes: usize,
    pub stopped: i32,
    pub tokenizer_status: i32,
}

/// `rg_text_callback`: one call per generated token (`token_id = -1` for the final flush).
pub type rg_text_callback = unsafe extern "C" fn(user: *mut c_void, token_id: i32, text: *const c_char, text_len: usize);

/// `rg_device_info`: what a session on a CUDA ordinal would run on.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct rg_device_info {
    pub name: [c_char; 128],
    pub sm_count: i32,
    pub cc_major: i32,
    pub cc_minor: i32,
    pub total_memory_bytes: u64,
    pub l2_bytes: u64,
    pub shared_memory_per_block: u64,
}

/// Opaque conversation handle of `include/rg_b200_workflow.h` (`LlamaConversation`).
#[repr(C)]
pub struct rg_conversation {
    _private: [u8; 0],
}

/// The workflow verbs a conversation turn is made of (`rg_chat_backend`).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct rg_chat_backend {
    pub ctx: *mut c_void,
    pub generate_chat: Option<unsafe extern "C" fn(ctx: *mut c_void, roles: *const i32, contents: *const *const c_char, content_len: *const usize, n_messages: usize, max_new_tokens: usize, on_text: Option<rg_text_callback>, user: *mut c_void, out: *mut rg_prompt_output) -> i32>,
    pub decoded: Option<unsafe extern "C" fn(ctx: *mut c_void) -> *const c_char>,
}

/// `LlamaConversationError` by kind.
pub mod conversation_status {
    pub const OK: i32 = 0;
    pub const EMPTY_INPUT: i32 = 1;
    pub const CHAT: i32 = 2;
    pub const GENERATION: i32 = 3;
    pub const INVALID_ARGUMENT: i32 = 4;
}

/// Opaque scheduler handle of `include/rg_b200_serving.h`.
#[repr(C)]
pub struct rg_scheduler {
    _private: [u8; 0],
}

/// `rg_serving_status`: `LlamaServingError` by kind.
pub mod serving_status {
    pub const OK: i32 = 0;
    pub const EMPTY_BATCH: i32 = 1;
    pub const EMPTY_PROMPT: i32 = 2;
    pub const CONTEXT_LENGTH: i32 = 3;
    pub const TOKEN_OUT_OF_RANGE: i32 = 4;
    pub const INVALID_TEMPERATURE: i32 = 5;
    pub const UNIFORM_TAPE_LENGTH: i32 = 6;
    pub const INVALID_UNIFORM: i32 = 7;
    pub const UNKNOWN_REQUEST: i32 = 8;
    pub const SESSION: i32 = 9;
    pub const TOKENIZER: i32 = 10;
    pub const INVALID_ARGUMENT: i32 = 11;
    pub const NOT_COMPLETE: i32 = 12;
    pub const ACTIVE_REQUESTS: i32 = 13;
}

/// Opaque batch-generator handle of `include/rg_b200_serving.h` (`LlamaBatchGenerator`).
#[repr(C)]
pub struct rg_batch_generator {
    _private: [u8; 0],
}

/// `rg_batch_status`: `LlamaBatchGenerationError` by kind.
pub mod batch_status {
    pub const OK: i32 = 0;
    pub const SESSION: i32 = 1;
    pub const INVALID_TEMPERATURE: i32 = 2;
    pub const TOKENIZER: i32 = 3;
    pub const BATCH_SIZE: i32 = 4;
    pub const EMPTY_PROMPT: i32 = 5;
    pub const CONTEXT_OVERFLOW: i32 = 6;
    pub const CONTEXT_LENGTH: i32 = 7;
    pub const UNIFORM_TAPE_LENGTH: i32 = 8;
    pub const INVALID_UNIFORM: i32 = 9;
    pub const TOKEN_OUT_OF_RANGE: i32 = 10;
    pub const INVALID_ARGUMENT: i32 = 11;
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct rg_batch_error {
    pub kind: i32,
    pub row: i32,
    pub value: i64,
    pub value2: i64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct rg_serving_error {
    pub kind: i32,
    pub value: i64,
    pub value2: i64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct rg_serving_options {
    pub batch_size: i32,
    pub max_rows: i32,
    pub prefix_max_entries: usize,
    pub prefix_max_bytes: usize,
    pub stop_ids: *const i32,
    pub n_stop_ids: usize,
    pub has_bos: i32,
    pub bos_id: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct rg_serving_sampling {
    pub greedy: i32,
    pub temperature: f32,
    pub uniforms: *const f32,
    pub n_uniforms: usize,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct rg_token_event {
    pub request_id: u64,
    pub arrival_order: u64,
    pub generation_step: i32,
    pub token_id: i32,
    pub stopped: i32,
    pub complete: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct rg_serving_result {
    pub request_id: u64,
    pub prompt_ids: *const i32,
    pub n_prompt_ids: usize,
    pub generated_ids: *const i32,
    pub n_generated_ids: usize,
    pub decoded: *const c_char,
    pub decoded_bytes: usize,
    pub stopped: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct rg_prefix_stats {
    pub entries: u64,
    pub bytes: u64,
    pub hits: u64,
    pub misses: u64,
    pub stale_rejections: u64,
    pub evictions: u64,
    pub generation: u64,
}

/// `rg_serving_backend`: the session verbs a step is made of, as a table of C functions.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct rg_serving_backend {
    pub ctx: *mut c_void,
    pub vocab: i32,
    pub max_context: i32,
    pub reset_row: Option<unsafe extern "C" fn(ctx: *mut c_void, row: i32) -> i32>,
    pub prefill_select: Option<unsafe extern "C" fn(ctx: *mut c_void, row: i32, ids: *const i32, n: usize, temperature: f32, uniforms: *const f32, last_logits: *mut f32, selected: *mut i32) -> i32>,
    pub decode_rows: Option<unsafe extern "C" fn(ctx: *mut c_void, rows: *const i32, tokens: *const i32, n: i32, temperatures: *const f32, uniforms: *const f32, ids: *mut i32) -> i32>,
    pub select: Option<unsafe extern "C" fn(ctx: *mut c_void, logits: *const f32, temperature: f32, uniforms: *const f32, id: *mut i32) -> i32>,
    pub snapshot_create: Option<unsafe extern "C" fn(ctx: *mut c_void, row: i32, length: i32, snapshot: *mut *mut c_void, bytes: *mut usize) -> i32>,
    pub snapshot_restore: Option<unsafe extern "C" fn(ctx: *mut c_void, snapshot: *const c_void, row: i32) -> i32>,
    pub snapshot_free: Option<unsafe extern "C" fn(ctx: *mut c_void, snapshot: *mut c_void)>,
    pub prefill_rows: Option<unsafe extern "C" fn(ctx: *mut c_void, rows: *const i32, ids: *const i32, lens: *const usize, n: i32, last_logits: *mut f32, selected: *mut i32) -> i32>,
}

unsafe extern "C" {
    // ---- include/rg_b200.h
    pub fn rg_b200_version() -> *const c_char;
    pub fn rg_b200_status_string(status: i32) -> *const c_char;
    pub fn rg_b200_last_error() -> *const c_char;
    pub fn rg_b200_test_fail_after(what: *const c_char, n: i32) -> i32;
    pub fn rg_b200_launch_count(kernel: *const c_char) -> u64;
    pub fn rg_b200_device_info(device: i32, out: *mut rg_device_info) -> i32;
    pub fn rg_b200_test_expire_device_wait(s: *mut rg_session) -> i32;
    pub fn rg_b200_debug_read_trace(s: *mut rg_session, out: *mut u64, max_launches: i32) -> i32;
    pub fn rg_b200_gguf_open(bytes: *const u8, len: usize, out: *mut *mut rg_gguf) -> i32;
    pub fn rg_b200_gguf_close(g: *mut rg_gguf);
    pub fn rg_b200_gguf_tensor_count(g: *const rg_gguf) -> usize;
    pub fn rg_b200_gguf_tensor_info(g: *const rg_gguf, index: usize, name: *mut *const c_char, ggml_type: *mut i32, rank: *mut i32, dims: *mut u64, data: *mut *const u8, nbytes: *mut usize) -> i32;
    pub fn rg_b200_gguf_llama_config(g: *const rg_gguf, out: *mut rg_llama_config) -> i32;
    pub fn rg_b200_plan_create(config: *const rg_llama_config, options: *const rg_options, out: *mut *mut rg_plan) -> i32;
    pub fn rg_b200_plan_add_tensor(plan: *mut rg_plan, name: *const c_char, ggml_type: i32, rows: u64, cols: u64, bytes: *const u8, nbytes: usize) -> i32;
    pub fn rg_b200_plan_from_gguf(g: *const rg_gguf, options: *const rg_options, out: *mut *mut rg_plan) -> i32;
    pub fn rg_b200_plan_synth_tensor(plan: *mut rg_plan, name: *const c_char, ggml_type: i32, rows: u64, cols: u64, seed: u64, std: f32) -> i32;
    pub fn rg_b200_plan_tensor_nbytes(plan: *const rg_plan, name: *const c_char, nbytes: *mut usize) -> i32;
    pub fn rg_b200_plan_read_tensor(plan: *const rg_plan, name: *const c_char, out: *mut u8, nbytes: usize) -> i32;
    pub fn rg_b200_plan_destroy(plan: *mut rg_plan);
    pub fn rg_b200_session_prepare(plan: *mut rg_plan, out: *mut *mut rg_session) -> i32;
    pub fn rg_b200_session_destroy(s: *mut rg_session);
    pub fn rg_b200_position(s: *const rg_session, row: i32) -> i32;
    pub fn rg_b200_max_context(s: *const rg_session) -> i32;
    pub fn rg_b200_vocab_size(s: *const rg_session) -> i32;
    pub fn rg_b200_is_full(s: *const rg_session) -> i32;
    pub fn rg_b200_reset_sequence(s: *mut rg_session) -> i32;
    pub fn rg_b200_prefill(s: *mut rg_session, row: i32, ids: *const i32, n: usize, last_logits: *mut f32) -> i32;
    pub fn rg_b200_prefill_rows(s: *mut rg_session, rows: *const i32, ids: *const i32, lens: *const usize, n_rows: i32, last_logits: *mut f32, greedy: *mut i32) -> i32;
    pub fn rg_b200_decode(s: *mut rg_session, tokens: *const i32, batch: i32, logits: *mut f32, greedy: *mut i32) -> i32;
    pub fn rg_b200_generate_greedy(s: *mut rg_session, prompt: *const i32, n_prompt: usize, max_new: usize, out: *mut i32, n_out: *mut usize, stopped: *mut i32) -> i32;
    pub fn rg_b200_decode_sampled(s: *mut rg_session, tokens: *const i32, batch: i32, temperature: f32, uniforms: *const f32, logits: *mut f32, ids: *mut i32) -> i32;
    pub fn rg_b200_generate_sampled(s: *mut rg_session, prompt: *const i32, n_prompt: usize, max_new: usize, temperature: f32, uniforms: *const f32, out: *mut i32, n_out: *mut usize, stopped: *mut i32) -> i32;
    pub fn rg_b200_decode_loop(s: *mut rg_session, first_tokens: *const i32, batch: i32, steps: i32, out: *mut i32, gpu_ms: *mut f32) -> i32;
    pub fn rg_b200_decode_profile(s: *mut rg_session, first_tokens: *const i32, batch: i32, steps: i32, out_ms: *mut f32, out_launches: *mut u64) -> i32;
    pub fn rg_b200_decode_profile_in_step(s: *mut rg_session, first_tokens: *const i32, batch: i32, steps: i32, out_ms: *mut f32, out_launches: *mut u64) -> i32;
    pub fn rg_b200_decode_profile_projections(s: *mut rg_session, first_tokens: *const i32, batch: i32, steps: i32, out_ms: *mut f32) -> i32;
    pub fn rg_b200_report(s: *const rg_session, out: *mut rg_report) -> i32;
    pub fn rg_b200_session_stream(s: *const rg_session) -> *mut c_void;
    pub fn rg_b200_nccl_unique_id(out: *mut u8) -> i32;
    pub fn rg_b200_tp_shard(name: *const c_char, ggml_type: i32, rows: u64, cols: u64, rank: i32, world: i32, row0: *mut u64, n_rows: *mut u64, col0: *mut u64, n_cols: *mut u64) -> i32;
    pub fn rg_b200_dequantize(device: i32, ggml_type: i32, bytes: *const u8, elements: usize, out: *mut f32) -> i32;
    pub fn rg_b200_qmatmul(device: i32, ggml_type: i32, weight: *const u8, n: u64, k: u64, activation: *const f32, m: u64, out: *mut f32) -> i32;
    pub fn rg_b200_row_gather(device: i32, ggml_type: i32, weight: *const u8, rows: u64, cols: u64, indices: *const i64, count: usize, out: *mut f32) -> i32;
    pub fn rg_b200_qgemm(device: i32, ggml_type: i32, weight: *const u8, n: u64, k: u64, activation: *const f32, m: u64, operand_mode: i32, iters: i32, out: *mut f32, kernel_ms: *mut f32) -> i32;
    pub fn rg_b200_attention_decode(device: i32, q: *const f32, keys: *const c_void, values: *const c_void, heads: i32, kv_heads: i32, head_dim: i32, n_pos: i32, kv_f32: i32, out: *mut f32) -> i32;
    pub fn rg_b200_attention_decode_noalloc(q_dev: *const f32, keys_dev: *const c_void, values_dev: *const c_void, heads: i32, kv_heads: i32, head_dim: i32, ctx: i32, n_pos: i32, kv_f32: i32, out_dev: *mut f32, stream: *mut c_void, wait: i32) -> i32;
    pub fn rg_b200_reset_row(s: *mut rg_session, row: i32) -> i32;
    pub fn rg_b200_prefill_select(s: *mut rg_session, row: i32, ids: *const i32, n: usize, temperature: f32, uniforms: *const f32, last_logits: *mut f32, selected: *mut i32) -> i32;
    pub fn rg_b200_decode_rows(s: *mut rg_session, rows: *const i32, tokens: *const i32, n: i32, temperatures: *const f32, uniforms: *const f32, logits: *mut f32, ids: *mut i32) -> i32;
    pub fn rg_b200_select(s: *mut rg_session, logits: *const f32, n: i32, temperatures: *const f32, uniforms: *const f32, ids: *mut i32) -> i32;
    pub fn rg_b200_kv_snapshot_create(s: *mut rg_session, row: i32, length: i32, out: *mut *mut rg_kv_snapshot) -> i32;
    pub fn rg_b200_kv_snapshot_length(k: *const rg_kv_snapshot) -> i32;
    pub fn rg_b200_kv_snapshot_bytes(k: *const rg_kv_snapshot) -> usize;
    pub fn rg_b200_kv_snapshot_restore(s: *mut rg_session, k: *const rg_kv_snapshot, row: i32) -> i32;
    pub fn rg_b200_kv_snapshot_free(k: *mut rg_kv_snapshot);
    pub fn rg_b200_qmatmul_bench(device: i32, ggml_type: i32, weight: *const u8, n: u64, k: u64, activation: *const f32, m: u64, rotate: i32, iters: i32, warmup: i32, out: *mut f32, kernel_ms: *mut f32) -> i32;

    // ---- include/rg_b200_tokenizer.h
    pub fn rg_b200_tokenizer_new(normal: *const *const c_char, normal_len: *const usize, normal_ids: *const u32, n_normal: usize, special: *const *const c_char, special_len: *const usize, special_ids: *const u32, n_special: usize, cfg: *const rg_tok_config, out: *mut *mut rg_tokenizer, err: *mut rg_tok_error) -> i32;
    pub fn rg_b200_tokenizer_from_gguf(gguf: *const rg_gguf, out: *mut *mut rg_tokenizer, err: *mut rg_tok_error) -> i32;
    pub fn rg_b200_tokenizer_free(t: *mut rg_tokenizer);
    pub fn rg_b200_tokenizer_config(t: *const rg_tokenizer, out: *mut rg_tok_config);
    pub fn rg_b200_tokenizer_is_end(t: *const rg_tokenizer, token_id: u32) -> i32;
    pub fn rg_b200_tokenizer_parse_preset(value: *const c_char, len: usize, preset: *mut i32) -> i32;
    pub fn rg_b200_tokenizer_encode(t: *const rg_tokenizer, text: *const c_char, len: usize, ids: *mut u32, capacity: usize, n_ids: *mut usize, err: *mut rg_tok_error) -> i32;
    pub fn rg_b200_tokenizer_decode(t: *const rg_tokenizer, ids: *const u32, n_ids: usize, text: *mut c_char, capacity: usize, n_bytes: *mut usize, err: *mut rg_tok_error) -> i32;
    pub fn rg_b200_tok_stream_new(t: *const rg_tokenizer, out: *mut *mut rg_tok_stream) -> i32;
    pub fn rg_b200_tok_stream_push(s: *mut rg_tok_stream, token_id: u32, text: *mut c_char, capacity: usize, n_bytes: *mut usize, err: *mut rg_tok_error) -> i32;
    pub fn rg_b200_tok_stream_finish(s: *mut rg_tok_stream, text: *mut c_char, capacity: usize, n_bytes: *mut usize) -> i32;
    pub fn rg_b200_tok_stream_free(s: *mut rg_tok_stream);
    pub fn rg_b200_chat_template_from_gguf(gguf: *const rg_gguf, metadata_present: *mut i32, err: *mut rg_tok_error) -> i32;
    pub fn rg_b200_chat_template_text() -> *const c_char;
    pub fn rg_b200_chat_render(t: *const rg_tokenizer, roles: *const i32, contents: *const *const c_char, content_len: *const usize, n_messages: usize, add_generation_prompt: i32, text: *mut c_char, capacity: usize, n_bytes: *mut usize, err: *mut rg_tok_error) -> i32;

    // ---- include/rg_b200_workflow.h
    pub fn rg_b200_workflow_open(gguf_bytes: *const u8, len: usize, options: *const rg_options, out: *mut *mut rg_workflow) -> i32;
    pub fn rg_b200_workflow_close(w: *mut rg_workflow);
    pub fn rg_b200_workflow_session(w: *mut rg_workflow) -> *mut rg_session;
    pub fn rg_b200_workflow_tokenizer(w: *const rg_workflow) -> *const rg_tokenizer;
    pub fn rg_b200_workflow_generate_text(w: *mut rg_workflow, prompt: *const c_char, prompt_len: usize, max_new_tokens: usize, on_text: Option<rg_text_callback>, user: *mut c_void, out: *mut rg_prompt_output) -> i32;
    pub fn rg_b200_workflow_generate_chat(w: *mut rg_workflow, roles: *const i32, contents: *const *const c_char, content_len: *const usize, n_messages: usize, max_new_tokens: usize, on_text: Option<rg_text_callback>, user: *mut c_void, out: *mut rg_prompt_output) -> i32;
    pub fn rg_b200_workflow_prompt_ids(w: *const rg_workflow) -> *const i32;
    pub fn rg_b200_workflow_generated_ids(w: *const rg_workflow) -> *const i32;
    pub fn rg_b200_workflow_decoded(w: *const rg_workflow) -> *const c_char;
    pub fn rg_b200_workflow_rendered_prompt(w: *const rg_workflow) -> *const c_char;
    pub fn rg_b200_conversation_new(w: *mut rg_workflow, out: *mut *mut rg_conversation) -> i32;
    pub fn rg_b200_conversation_new_with_backend(backend: *const rg_chat_backend, out: *mut *mut rg_conversation) -> i32;
    pub fn rg_b200_conversation_free(c: *mut rg_conversation);
    pub fn rg_b200_conversation_history_len(c: *const rg_conversation) -> usize;
    pub fn rg_b200_conversation_message(c: *const rg_conversation, index: usize, role: *mut i32, content: *mut *const c_char, content_len: *mut usize) -> i32;
    pub fn rg_b200_conversation_cache_len(c: *const rg_conversation) -> usize;
    pub fn rg_b200_conversation_reset(c: *mut rg_conversation);
    pub fn rg_b200_conversation_send(c: *mut rg_conversation, content: *const c_char, content_len: usize, max_new_tokens: usize, on_text: Option<rg_text_callback>, user: *mut c_void, out: *mut rg_prompt_output, detail: *mut i32) -> i32;

    // ---- include/rg_b200_serving.h
    pub fn rg_b200_scheduler_new(session: *mut rg_session, tokenizer: *const rg_tokenizer, options: *const rg_serving_options, out: *mut *mut rg_scheduler, err: *mut rg_serving_error) -> i32;
    pub fn rg_b200_scheduler_new_with_backend(backend: *const rg_serving_backend, tokenizer: *const rg_tokenizer, options: *const rg_serving_options, out: *mut *mut rg_scheduler, err: *mut rg_serving_error) -> i32;
    pub fn rg_b200_scheduler_free(s: *mut rg_scheduler);
    pub fn rg_b200_scheduler_submit_ids(s: *mut rg_scheduler, prompt: *const i32, n: usize, max_new_tokens: usize, sampling: *const rg_serving_sampling, request_id: *mut u64, err: *mut rg_serving_error) -> i32;
    pub fn rg_b200_scheduler_submit_text(s: *mut rg_scheduler, prompt: *const c_char, prompt_len: usize, max_new_tokens: usize, sampling: *const rg_serving_sampling, request_id: *mut u64, err: *mut rg_serving_error) -> i32;
    pub fn rg_b200_scheduler_submit_chat(s: *mut rg_scheduler, roles: *const i32, contents: *const *const c_char, content_len: *const usize, n_messages: usize, max_new_tokens: usize, sampling: *const rg_serving_sampling, request_id: *mut u64, err: *mut rg_serving_error) -> i32;
    pub fn rg_b200_scheduler_status(s: *const rg_scheduler, request_id: u64, status: *mut i32) -> i32;
    pub fn rg_b200_scheduler_result(s: *const rg_scheduler, request_id: u64, out: *mut rg_serving_result) -> i32;
    pub fn rg_b200_scheduler_remove(s: *mut rg_scheduler, request_id: u64) -> i32;
    pub fn rg_b200_scheduler_pending(s: *const rg_scheduler) -> usize;
    pub fn rg_b200_scheduler_completed(s: *const rg_scheduler, ids: *mut u64, cap: usize) -> usize;
    pub fn rg_b200_scheduler_prefix_stats(s: *const rg_scheduler, out: *mut rg_prefix_stats);
    pub fn rg_b200_scheduler_invalidate_prefix_cache(s: *mut rg_scheduler);
    pub fn rg_b200_scheduler_step(s: *mut rg_scheduler, events: *mut rg_token_event, cap: usize, n_events: *mut usize, err: *mut rg_serving_error) -> i32;
    pub fn rg_b200_scheduler_rebind(s: *mut rg_scheduler, session: *mut rg_session, tokenizer: *const rg_tokenizer, options: *const rg_serving_options, changed: *mut i32, err: *mut rg_serving_error) -> i32;
    pub fn rg_b200_scheduler_rebind_with_backend(s: *mut rg_scheduler, backend: *const rg_serving_backend, tokenizer: *const rg_tokenizer, options: *const rg_serving_options, changed: *mut i32, err: *mut rg_serving_error) -> i32;
    pub fn rg_b200_batch_generator_new(session: *mut rg_session, tokenizer: *const rg_tokenizer, batch_size: i32, options: *const rg_serving_options, out: *mut *mut rg_batch_generator, err: *mut rg_batch_error) -> i32;
    pub fn rg_b200_batch_generator_new_with_backend(backend: *const rg_serving_backend, tokenizer: *const rg_tokenizer, batch_size: i32, options: *const rg_serving_options, out: *mut *mut rg_batch_generator, err: *mut rg_batch_error) -> i32;
    pub fn rg_b200_batch_generator_free(g: *mut rg_batch_generator);
    pub fn rg_b200_batch_generator_cache_lengths(g: *const rg_batch_generator, lengths: *mut usize, cap: usize) -> usize;
    pub fn rg_b200_batch_generator_clear(g: *mut rg_batch_generator);
    pub fn rg_b200_batch_generate_ids(g: *mut rg_batch_generator, ids: *const i32, lens: *const usize, n_prompts: usize, max_new_tokens: usize, sampling: *const rg_serving_sampling, err: *mut rg_batch_error) -> i32;
    pub fn rg_b200_batch_generate_texts(g: *mut rg_batch_generator, texts: *const *const c_char, text_bytes: *const usize, n_prompts: usize, max_new_tokens: usize, sampling: *const rg_serving_sampling, err: *mut rg_batch_error) -> i32;
    pub fn rg_b200_batch_sequence(g: *const rg_batch_generator, row: usize, out: *mut rg_serving_result) -> i32;
}
