//! Typed facade over the raw bindings, shaped like rustgrad's accelerated Llama session
//! (`src/models/transformer/metal_generation.rs:33-52,276-281,702-715,837-1207`): a resource-free
//! [`LlamaCudaPlan`] bound to a [`CudaSessionTarget`], prepared into a [`LlamaCudaSession`] whose
//! verbs return typed errors and never fall back to another path.
//!
//! The crate does not depend on rustgrad, so the `SessionTarget` implementation itself lives in
//! `integration/cuda_generation.rs`, the file a rustgrad fork adds next to `metal_generation.rs`.

use crate::*;
use core::ffi::CStr;
use std::ffi::CString;
use std::fmt;

/// A failed call: the `rg_status` code and the library's detail text (CUDA / NCCL code, call site).
#[derive(Clone, Debug, Eq, PartialEq)]
pub struct CudaCallError {
    pub status: i32,
    pub detail: String,
}

impl fmt::Display for CudaCallError {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        let name = unsafe { CStr::from_ptr(rg_b200_status_string(self.status)) }.to_string_lossy();
        write!(f, "{name}: {}", self.detail)
    }
}

impl std::error::Error for CudaCallError {}

fn check(status: i32) -> Result<(), CudaCallError> {
    if status == status::OK {
        return Ok(());
    }
    let detail = unsafe { CStr::from_ptr(rg_b200_last_error()) }.to_string_lossy().into_owned();
    Err(CudaCallError { status, detail })
}

/// Token-execution phase recorded by a partial failure (`LlamaMetalGenerationStage`).
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub enum LlamaCudaGenerationStage {
    Prompt,
    Decode,
}

/// Durable successful prefix accompanying a failure after device work began
/// (`LlamaMetalProgress`, metal_generation.rs:179-187).
#[derive(Clone, Debug, Default, Eq, PartialEq)]
pub struct LlamaCudaProgress {
    pub prompt_ids: Vec<u32>,
    pub generated_ids: Vec<u32>,
    pub start_position: usize,
    pub committed_position: usize,
}

/// Typed planning, preflight or execution failure (`LlamaMetalGenerationError`,
/// metal_generation.rs:196-233).
#[derive(Clone, Debug, PartialEq)]
pub enum LlamaCudaGenerationError {
    /// A call failed before any step of this request ran.
    Call(CudaCallError),
    /// The session is not at position 0 (`FreshSessionRequired`).
    FreshSessionRequired { position: usize },
    /// A step failed after earlier steps of the request had been committed.
    Execution {
        progress: Box<LlamaCudaProgress>,
        stage: LlamaCudaGenerationStage,
        token_offset: usize,
        token: u32,
        source: CudaCallError,
    },
}

impl fmt::Display for LlamaCudaGenerationError {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        write!(f, "Llama CUDA generation error: {self:?}")
    }
}

impl std::error::Error for LlamaCudaGenerationError {}

impl From<CudaCallError> for LlamaCudaGenerationError {
    fn from(e: CudaCallError) -> Self {
        if e.status == status::FRESH_SESSION_REQUIRED {
            return Self::FreshSessionRequired { position: 0 };
        }
        Self::Call(e)
    }
}

/// One B200 (one process per GPU), optionally one rank of a tensor-parallel group.
#[derive(Clone, Debug, Default)]
pub struct CudaSessionTarget {
    pub options: rg_options,
}

impl CudaSessionTarget {
    pub fn new(device: u32) -> Self {
        let mut options = rg_options::default();
        options.device = device as i32;
        Self { options }
    }

    /// Rank `rank` of `world` ranks sharing the 128-byte NCCL id of rank 0 (`rg_b200_nccl_unique_id`).
    pub fn tensor_parallel(mut self, rank: u32, world: u32, nccl_id: [u8; 128]) -> Self {
        self.options.tp_rank = rank as i32;
        self.options.tp_world = world as i32;
        self.options.nccl_id = nccl_id;
        self
    }

    pub fn max_batch(mut self, rows: u32) -> Self {
        self.options.max_batch = rows as i32;
        self
    }

    pub fn max_context(mut self, positions: u32) -> Self {
        self.options.max_context = positions as i32;
        self
    }

    /// Prepares a plan (`SessionTarget::prepare`).
    pub fn prepare(&self, plan: LlamaCudaPlan) -> Result<LlamaCudaSession, LlamaCudaGenerationError> {
        plan.prepare()
    }
}

/// The id a rank-0 process broadcasts to its peers before preparing a tensor-parallel session.
pub fn nccl_unique_id() -> Result<[u8; 128], CudaCallError> {
    let mut id = [0u8; 128];
    check(unsafe { rg_b200_nccl_unique_id(id.as_mut_ptr()) })?;
    Ok(id)
}

/// A parsed and validated GGUF container (`read_gguf`, src/gguf/mod.rs:384); borrows the bytes.
pub struct GgufFile<'a> {
    raw: *mut rg_gguf,
    _bytes: core::marker::PhantomData<&'a [u8]>,
}

impl<'a> GgufFile<'a> {
    pub fn parse(bytes: &'a [u8]) -> Result<Self, CudaCallError> {
        let mut raw = core::ptr::null_mut();
        check(unsafe { rg_b200_gguf_open(bytes.as_ptr(), bytes.len(), &mut raw) })?;
        Ok(Self { raw, _bytes: core::marker::PhantomData })
    }

    /// `LlamaModelConfig::from_gguf` (model.rs:126-298), stop ids from the file's tokenizer included.
    pub fn llama_config(&self) -> Result<rg_llama_config, CudaCallError> {
        let mut cfg = rg_llama_config::default();
        check(unsafe { rg_b200_gguf_llama_config(self.raw, &mut cfg) })?;
        Ok(cfg)
    }
}

impl Drop for GgufFile<'_> {
    fn drop(&mut self) {
        unsafe { rg_b200_gguf_close(self.raw) }
    }
}

/// Validated model bound to a target: weights uploaded once in their native block bytes.
pub struct LlamaCudaPlan {
    raw: *mut rg_plan,
    config: rg_llama_config,
}

impl LlamaCudaPlan {
    /// `LlamaMetalPlan::from_workflow_on` for a whole file: configuration, exact tensor inventory, upload.
    pub fn from_gguf(file: &GgufFile<'_>, target: &CudaSessionTarget) -> Result<Self, CudaCallError> {
        let config = file.llama_config()?;
        let mut raw = core::ptr::null_mut();
        check(unsafe { rg_b200_plan_from_gguf(file.raw, &target.options, &mut raw) })?;
        Ok(Self { raw, config })
    }

    /// An empty plan for a caller that binds tensors itself (`LlamaModelState::bind` on parts): the
    /// route from rustgrad's own `LlamaModelState::{embedding_weight, linear_weights, tensors}`.
    pub fn empty(config: rg_llama_config, target: &CudaSessionTarget) -> Result<Self, CudaCallError> {
        let mut raw = core::ptr::null_mut();
        check(unsafe { rg_b200_plan_create(&config, &target.options, &mut raw) })?;
        Ok(Self { raw, config })
    }

    /// One tensor in its unmodified GGUF bytes (`QuantizedTensorData::bytes`, data.rs:296-302);
    /// borrowed for the call.  `rows == 1` for norm vectors.
    pub fn add_tensor(&mut self, name: &str, ggml_type: i32, rows: u64, cols: u64, bytes: &[u8]) -> Result<(), CudaCallError> {
        let name = CString::new(name).map_err(|_| CudaCallError { status: status::INVALID_ARGUMENT, detail: "tensor name holds a NUL".into() })?;
        check(unsafe { rg_b200_plan_add_tensor(self.raw, name.as_ptr(), ggml_type, rows, cols, bytes.as_ptr(), bytes.len()) })
    }

    pub fn config(&self) -> &rg_llama_config {
        &self.config
    }

    pub fn prepare(self) -> Result<LlamaCudaSession, LlamaCudaGenerationError> {
        let mut raw = core::ptr::null_mut();
        check(unsafe { rg_b200_session_prepare(self.raw, &mut raw) })?;
        Ok(LlamaCudaSession { raw, config: self.config })
        // `self` drops here: the plan handle is released, the session owns the device tensors
    }
}

impl Drop for LlamaCudaPlan {
    fn drop(&mut self) {
        unsafe { rg_b200_plan_destroy(self.raw) }
    }
}

/// `LlamaGeneration` (generation.rs:40-60) without the decoded text, which the caller's tokenizer adds.
#[derive(Clone, Debug, Eq, PartialEq)]
pub struct LlamaCudaGeneration {
    pub prompt_ids: Vec<u32>,
    pub generated_ids: Vec<u32>,
    pub stopped: bool,
}

/// A prepared session on one GPU: KV state on the device, `&mut self` verbs, one driving thread.
pub struct LlamaCudaSession {
    raw: *mut rg_session,
    config: rg_llama_config,
}

impl LlamaCudaSession {
    pub fn position(&self) -> usize {
        unsafe { rg_b200_position(self.raw, 0) }.max(0) as usize
    }

    pub fn max_context(&self) -> usize {
        unsafe { rg_b200_max_context(self.raw) }.max(0) as usize
    }

    pub fn vocab_size(&self) -> usize {
        unsafe { rg_b200_vocab_size(self.raw) }.max(0) as usize
    }

    pub fn is_full(&self) -> bool {
        unsafe { rg_b200_is_full(self.raw) } == 1
    }

    pub fn reset_sequence(&mut self) -> Result<(), CudaCallError> {
        check(unsafe { rg_b200_reset_sequence(self.raw) })
    }

    fn ids(tokens: &[u32]) -> Vec<i32> {
        tokens.iter().map(|&t| t as i32).collect()
    }

    /// `run_token`: one decode step, logits `[vocab]`.
    pub fn run_token(&mut self, token: u32) -> Result<Vec<f32>, CudaCallError> {
        let mut logits = vec![0.0f32; self.vocab_size()];
        let t = token as i32;
        check(unsafe { rg_b200_decode(self.raw, &t, 1, logits.as_mut_ptr(), core::ptr::null_mut()) })?;
        Ok(logits)
    }

    /// `prefill_ids`: the prompt in chunks on the tensor cores, logits of its last token.
    pub fn prefill_ids(&mut self, ids: &[u32]) -> Result<Vec<f32>, CudaCallError> {
        let mut logits = vec![0.0f32; self.vocab_size()];
        let ids = Self::ids(ids);
        check(unsafe { rg_b200_prefill(self.raw, 0, ids.as_ptr(), ids.len(), logits.as_mut_ptr()) })?;
        Ok(logits)
    }

    /// `generate_ids` with greedy selection on a fresh sequence.  A failure after the prompt has been
    /// committed carries the tokens generated so far.
    pub fn generate_ids(&mut self, prompt_ids: &[u32], max_new_tokens: usize) -> Result<LlamaCudaGeneration, LlamaCudaGenerationError> {
        if self.position() != 0 {
            return Err(LlamaCudaGenerationError::FreshSessionRequired { position: self.position() });
        }
        let prompt = Self::ids(prompt_ids);
        let mut out = vec![0i32; max_new_tokens.max(1)];
        let (mut n_out, mut stopped) = (0usize, 0i32);
        let rc = unsafe {
            rg_b200_generate_greedy(self.raw, prompt.as_ptr(), prompt.len(), max_new_tokens, out.as_mut_ptr(), &mut n_out, &mut stopped)
        };
        let generated: Vec<u32> = out[..n_out].iter().map(|&t| t as u32).collect();
        if let Err(source) = check(rc) {
            let committed = self.position();
            if committed == 0 {
                return Err(source.into());
            }
            let stage = if generated.is_empty() { LlamaCudaGenerationStage::Prompt } else { LlamaCudaGenerationStage::Decode };
            return Err(LlamaCudaGenerationError::Execution {
                token_offset: generated.len(),
                token: generated.last().copied().unwrap_or(0),
                progress: Box::new(LlamaCudaProgress {
                    prompt_ids: prompt_ids.to_vec(),
                    generated_ids: generated,
                    start_position: 0,
                    committed_position: committed,
                }),
                stage,
                source,
            });
        }
        Ok(LlamaCudaGeneration { prompt_ids: prompt_ids.to_vec(), generated_ids: generated, stopped: stopped != 0 })
    }

    /// Evidence of the run in the vocabulary of `MetalDeviceRunReport`.
    pub fn report(&self) -> Result<rg_report, CudaCallError> {
        let mut r = rg_report::default();
        check(unsafe { rg_b200_report(self.raw, &mut r) })?;
        Ok(r)
    }

    pub fn config(&self) -> &rg_llama_config {
        &self.config
    }

    /// The raw handle, for the entry points this facade does not wrap (batch rows, sampling, snapshots).
    pub fn as_raw(&mut self) -> *mut rg_session {
        self.raw
    }
}

impl Drop for LlamaCudaSession {
    fn drop(&mut self) {
        unsafe { rg_b200_session_destroy(self.raw) }
    }
}

/// Text in, ids and text out (`LlamaPromptWorkflow`, workflow.rs:18-147) on the GPU.
pub struct LlamaCudaPromptWorkflow {
    raw: *mut rg_workflow,
}

/// `LlamaPromptOutput` (workflow.rs:150-170).
#[derive(Clone, Debug, Eq, PartialEq)]
pub struct LlamaCudaPromptOutput {
    pub rendered_prompt: String,
    pub prompt_ids: Vec<u32>,
    pub generated_ids: Vec<u32>,
    pub decoded: String,
    pub stopped: bool,
}

/// Chat roles of the checked template (`LlamaChatRole`).
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub enum LlamaChatRole {
    System = 0,
    User = 1,
    Assistant = 2,
}

impl LlamaCudaPromptWorkflow {
    pub fn from_gguf_bytes(bytes: &[u8], target: &CudaSessionTarget) -> Result<Self, CudaCallError> {
        let mut raw = core::ptr::null_mut();
        check(unsafe { rg_b200_workflow_open(bytes.as_ptr(), bytes.len(), &target.options, &mut raw) })?;
        Ok(Self { raw })
    }

    pub fn from_path(path: impl AsRef<std::path::Path>, target: &CudaSessionTarget) -> Result<Self, Box<dyn std::error::Error>> {
        let bytes = std::fs::read(path)?;
        Ok(Self::from_gguf_bytes(&bytes, target)?)
    }

    fn collect(&self, rc: i32, out: &rg_prompt_output) -> Result<LlamaCudaPromptOutput, CudaCallError> {
        check(rc)?;
        let slice = |p: *const i32, n: usize| -> Vec<u32> {
            if n == 0 { Vec::new() } else { unsafe { core::slice::from_raw_parts(p, n) }.iter().map(|&t| t as u32).collect() }
        };
        let text = |p: *const c_char, n: usize| -> String {
            String::from_utf8_lossy(unsafe { core::slice::from_raw_parts(p as *const u8, n) }).into_owned()
        };
        Ok(LlamaCudaPromptOutput {
            rendered_prompt: text(unsafe { rg_b200_workflow_rendered_prompt(self.raw) }, out.rendered_bytes),
            prompt_ids: slice(unsafe { rg_b200_workflow_prompt_ids(self.raw) }, out.n_prompt_ids),
            generated_ids: slice(unsafe { rg_b200_workflow_generated_ids(self.raw) }, out.n_generated_ids),
            decoded: text(unsafe { rg_b200_workflow_decoded(self.raw) }, out.decoded_bytes),
            stopped: out.stopped != 0,
        })
    }

    /// `LlamaPromptWorkflow::generate`.
    pub fn generate(&mut self, prompt: &str, max_new_tokens: usize) -> Result<LlamaCudaPromptOutput, CudaCallError> {
        let mut out = rg_prompt_output::default();
        let rc = unsafe {
            rg_b200_workflow_generate_text(self.raw, prompt.as_ptr() as *const c_char, prompt.len(), max_new_tokens, None, core::ptr::null_mut(), &mut out)
        };
        self.collect(rc, &out)
    }

    /// `LlamaPromptWorkflow::generate_chat`.
    pub fn generate_chat(&mut self, messages: &[(LlamaChatRole, &str)], max_new_tokens: usize) -> Result<LlamaCudaPromptOutput, CudaCallError> {
        let roles: Vec<i32> = messages.iter().map(|(r, _)| *r as i32).collect();
        let ptrs: Vec<*const c_char> = messages.iter().map(|(_, c)| c.as_ptr() as *const c_char).collect();
        let lens: Vec<usize> = messages.iter().map(|(_, c)| c.len()).collect();
        let mut out = rg_prompt_output::default();
        let rc = unsafe {
            rg_b200_workflow_generate_chat(self.raw, roles.as_ptr(), ptrs.as_ptr(), lens.as_ptr(), messages.len(), max_new_tokens, None, core::ptr::null_mut(), &mut out)
        };
        self.collect(rc, &out)
    }
}

impl Drop for LlamaCudaPromptWorkflow {
    fn drop(&mut self) {
        unsafe { rg_b200_workflow_close(self.raw) }
    }
}

/// `LlamaServingError` (serving/mod.rs:792-860): the kind (`serving_status::*`) with its numbers.
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub struct LlamaCudaServingError {
    pub kind: i32,
    pub value: i64,
    pub value2: i64,
}

impl fmt::Display for LlamaCudaServingError {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        write!(f, "serving status {} ({}, {})", self.kind, self.value, self.value2)
    }
}

impl std::error::Error for LlamaCudaServingError {}

/// `LlamaServingSampling` (serving/mod.rs:28-38).
pub enum LlamaCudaServingSampling<'a> {
    Greedy,
    GumbelMax { temperature: f32, uniforms: &'a [f32] },
}

/// `LlamaTokenEvent` (serving/mod.rs:98-129).
pub type LlamaCudaTokenEvent = rg_token_event;

/// `LlamaServingResult` (serving/mod.rs:131-155), copied out of the scheduler.
#[derive(Clone, Debug, Eq, PartialEq)]
pub struct LlamaCudaServingResult {
    pub request_id: u64,
    pub prompt_ids: Vec<u32>,
    pub generated_ids: Vec<u32>,
    pub decoded: String,
    pub stopped: bool,
}

/// Continuous batching with a prefix cache over one session (`LlamaServingScheduler`,
/// serving/mod.rs:371-690).  The session must outlive the scheduler.
pub struct LlamaCudaServingScheduler<'s> {
    raw: *mut rg_scheduler,
    batch_size: usize,
    _session: core::marker::PhantomData<&'s mut LlamaCudaSession>,
}

impl<'s> LlamaCudaServingScheduler<'s> {
    pub fn new(session: &'s mut LlamaCudaSession, batch_size: usize, prefix_max_entries: usize, prefix_max_bytes: usize,
               stop_ids: &[i32]) -> Result<Self, LlamaCudaServingError> {
        let options = rg_serving_options {
            batch_size: batch_size as i32,
            max_rows: 0,
            prefix_max_entries,
            prefix_max_bytes,
            stop_ids: stop_ids.as_ptr(),
            n_stop_ids: stop_ids.len(),
            has_bos: 0,
            bos_id: 0,
        };
        let mut raw = core::ptr::null_mut();
        let mut err = rg_serving_error::default();
        let rc = unsafe { rg_b200_scheduler_new(session.as_raw(), core::ptr::null(), &options, &mut raw, &mut err) };
        if rc != 0 {
            return Err(LlamaCudaServingError { kind: rc, value: err.value, value2: err.value2 });
        }
        Ok(Self { raw, batch_size, _session: core::marker::PhantomData })
    }

    /// `submit_ids` (serving/mod.rs:408-477): validated as a whole before it gets an id.
    pub fn submit_ids(&mut self, prompt: &[i32], max_new_tokens: usize, sampling: LlamaCudaServingSampling<'_>) -> Result<u64, LlamaCudaServingError> {
        let s = match sampling {
            LlamaCudaServingSampling::Greedy => rg_serving_sampling { greedy: 1, temperature: 0.0, uniforms: core::ptr::null(), n_uniforms: 0 },
            LlamaCudaServingSampling::GumbelMax { temperature, uniforms } => {
                rg_serving_sampling { greedy: 0, temperature, uniforms: uniforms.as_ptr(), n_uniforms: uniforms.len() }
            }
        };
        let (mut id, mut err) = (0u64, rg_serving_error::default());
        let rc = unsafe { rg_b200_scheduler_submit_ids(self.raw, prompt.as_ptr(), prompt.len(), max_new_tokens, &s, &mut id, &mut err) };
        if rc != 0 {
            return Err(LlamaCudaServingError { kind: rc, value: err.value, value2: err.value2 });
        }
        Ok(id)
    }

    /// `step` (serving/mod.rs:557-690): one token for each of up to `batch_size` requests in arrival order.
    pub fn step(&mut self) -> Result<Vec<LlamaCudaTokenEvent>, LlamaCudaServingError> {
        let mut events = vec![rg_token_event::default(); self.batch_size];
        let (mut n, mut err) = (0usize, rg_serving_error::default());
        let rc = unsafe { rg_b200_scheduler_step(self.raw, events.as_mut_ptr(), events.len(), &mut n, &mut err) };
        if rc != 0 {
            return Err(LlamaCudaServingError { kind: rc, value: err.value, value2: err.value2 });
        }
        events.truncate(n);
        Ok(events)
    }

    pub fn pending(&self) -> usize {
        unsafe { rg_b200_scheduler_pending(self.raw) }
    }

    pub fn result(&self, request_id: u64) -> Option<LlamaCudaServingResult> {
        let mut r = core::mem::MaybeUninit::<rg_serving_result>::zeroed();
        if unsafe { rg_b200_scheduler_result(self.raw, request_id, r.as_mut_ptr()) } != 0 {
            return None;
        }
        let r = unsafe { r.assume_init() };
        let ids = |p: *const i32, n: usize| -> Vec<u32> {
            if n == 0 { Vec::new() } else { unsafe { core::slice::from_raw_parts(p, n) }.iter().map(|&t| t as u32).collect() }
        };
        let decoded = if r.decoded_bytes == 0 {
            String::new()
        } else {
            String::from_utf8_lossy(unsafe { core::slice::from_raw_parts(r.decoded as *const u8, r.decoded_bytes) }).into_owned()
        };
        Some(LlamaCudaServingResult {
            request_id: r.request_id,
            prompt_ids: ids(r.prompt_ids, r.n_prompt_ids),
            generated_ids: ids(r.generated_ids, r.n_generated_ids),
            decoded,
            stopped: r.stopped != 0,
        })
    }

    pub fn remove(&mut self, request_id: u64) -> bool {
        unsafe { rg_b200_scheduler_remove(self.raw, request_id) == 0 }
    }

    pub fn prefix_stats(&self) -> rg_prefix_stats {
        let mut st = rg_prefix_stats::default();
        unsafe { rg_b200_scheduler_prefix_stats(self.raw, &mut st) };
        st
    }

    pub fn invalidate_prefix_cache(&mut self) {
        unsafe { rg_b200_scheduler_invalidate_prefix_cache(self.raw) }
    }

    /// `rebind` (serving/mod.rs:528-547): an idle scheduler takes another session; `Ok(true)` when it differs
    /// from the bound one, in which case every cached prefix was dropped.  Kind 13 (`ActiveRequests`) while
    /// requests are unfinished.  `stop_ids`, when given, replace the stop rule.
    pub fn rebind<'n>(self, session: &'n mut LlamaCudaSession, stop_ids: Option<&[i32]>) -> Result<(LlamaCudaServingScheduler<'n>, bool), LlamaCudaServingError> {
        let options = stop_ids.map(|ids| rg_serving_options {
            batch_size: self.batch_size as i32,
            max_rows: 0,
            prefix_max_entries: 0,
            prefix_max_bytes: 0,
            stop_ids: ids.as_ptr(),
            n_stop_ids: ids.len(),
            has_bos: 0,
            bos_id: 0,
        });
        let mut changed = 0i32;
        let mut err = rg_serving_error::default();
        let rc = unsafe {
            rg_b200_scheduler_rebind(self.raw, session.as_raw(), core::ptr::null(),
                                     options.as_ref().map_or(core::ptr::null(), |o| o as *const _), &mut changed, &mut err)
        };
        if rc != 0 {
            return Err(LlamaCudaServingError { kind: rc, value: err.value, value2: err.value2 });
        }
        let rebound = LlamaCudaServingScheduler { raw: self.raw, batch_size: self.batch_size, _session: core::marker::PhantomData };
        core::mem::forget(self);  // the handle lives on in `rebound`
        Ok((rebound, changed != 0))
    }
}

/// `LlamaBatchGenerator` (batch_generation.rs:58-189) over rows `0 .. batch_size` of one session.
pub struct LlamaCudaBatchGenerator<'s> {
    raw: *mut rg_batch_generator,
    batch_size: usize,
    _session: core::marker::PhantomData<&'s mut LlamaCudaSession>,
}

/// `LlamaBatchGenerationError` by kind (`batch_status`), with the row and the numbers it carries.
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub struct LlamaCudaBatchGenerationError {
    pub kind: i32,
    pub row: i32,
    pub value: i64,
    pub value2: i64,
}

impl<'s> LlamaCudaBatchGenerator<'s> {
    pub fn new(session: &'s mut LlamaCudaSession, batch_size: usize, stop_ids: &[i32]) -> Result<Self, LlamaCudaBatchGenerationError> {
        let options = rg_serving_options {
            batch_size: batch_size as i32,
            max_rows: 0,
            prefix_max_entries: 0,
            prefix_max_bytes: 0,
            stop_ids: stop_ids.as_ptr(),
            n_stop_ids: stop_ids.len(),
            has_bos: 0,
            bos_id: 0,
        };
        let mut raw = core::ptr::null_mut();
        let mut err = rg_batch_error::default();
        let rc = unsafe { rg_b200_batch_generator_new(session.as_raw(), core::ptr::null(), batch_size as i32, &options, &mut raw, &mut err) };
        if rc != 0 {
            return Err(LlamaCudaBatchGenerationError { kind: rc, row: err.row, value: err.value, value2: err.value2 });
        }
        Ok(Self { raw, batch_size, _session: core::marker::PhantomData })
    }

    pub fn cache_lengths(&self) -> Vec<usize> {
        let mut out = vec![0usize; self.batch_size];
        unsafe { rg_b200_batch_generator_cache_lengths(self.raw, out.as_mut_ptr(), out.len()) };
        out
    }

    pub fn clear(&mut self) {
        unsafe { rg_b200_batch_generator_clear(self.raw) }
    }

    /// `generate_ids` (batch_generation.rs:104-189); the Gumbel-max tape is `[step, batch, vocabulary]`.
    pub fn generate_ids(&mut self, prompts: &[Vec<i32>], max_new_tokens: usize, sampling: LlamaCudaServingSampling<'_>)
                        -> Result<Vec<LlamaCudaServingResult>, LlamaCudaBatchGenerationError> {
        let flat: Vec<i32> = prompts.iter().flatten().copied().collect();
        let lens: Vec<usize> = prompts.iter().map(|p| p.len()).collect();
        let s = match sampling {
            LlamaCudaServingSampling::Greedy => rg_serving_sampling { greedy: 1, temperature: 0.0, uniforms: core::ptr::null(), n_uniforms: 0 },
            LlamaCudaServingSampling::GumbelMax { temperature, uniforms } => {
                rg_serving_sampling { greedy: 0, temperature, uniforms: uniforms.as_ptr(), n_uniforms: uniforms.len() }
            }
        };
        let mut err = rg_batch_error::default();
        let rc = unsafe { rg_b200_batch_generate_ids(self.raw, flat.as_ptr(), lens.as_ptr(), prompts.len(), max_new_tokens, &s, &mut err) };
        if rc != 0 {
            return Err(LlamaCudaBatchGenerationError { kind: rc, row: err.row, value: err.value, value2: err.value2 });
        }
        let mut out = Vec::with_capacity(self.batch_size);
        for row in 0..self.batch_size {
            let mut r: rg_serving_result = unsafe { core::mem::zeroed() };
            if unsafe { rg_b200_batch_sequence(self.raw, row, &mut r) } != 0 {
                return Err(LlamaCudaBatchGenerationError { kind: batch_status::INVALID_ARGUMENT, row: row as i32, value: 0, value2: 0 });
            }
            let prompt = unsafe { core::slice::from_raw_parts(r.prompt_ids, r.n_prompt_ids) };
            let generated = unsafe { core::slice::from_raw_parts(r.generated_ids, r.n_generated_ids) };
            let text = unsafe { core::slice::from_raw_parts(r.decoded as *const u8, r.decoded_bytes) };
            out.push(LlamaCudaServingResult {
                request_id: r.request_id,
                prompt_ids: prompt.iter().map(|&t| t as u32).collect(),
                generated_ids: generated.iter().map(|&t| t as u32).collect(),
                decoded: String::from_utf8_lossy(text).into_owned(),
                stopped: r.stopped != 0,
            });
        }
        Ok(out)
    }
}

impl Drop for LlamaCudaBatchGenerator<'_> {
    fn drop(&mut self) {
        unsafe { rg_b200_batch_generator_free(self.raw) }
    }
}

impl Drop for LlamaCudaServingScheduler<'_> {
    fn drop(&mut self) {
        unsafe { rg_b200_scheduler_free(self.raw) }
    }
}
