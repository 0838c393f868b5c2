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
