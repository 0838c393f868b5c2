//! The file a rustgrad fork adds as `src/models/transformer/cuda_generation.rs`, beside
//! `metal_generation.rs`: it implements the crate's own `SessionTarget` for the CUDA target, so the
//! CUDA session drops in next to the CPU and Metal ones without another dispatcher branch
//! (`src/session/target.rs:10-18`; the Metal counterpart is `metal_generation.rs:702-715`).
//!
//! It builds the plan from rustgrad's own public model API, handing every tensor over in its
//! unmodified GGUF bytes: `LlamaModelState::{config, embedding_weight, linear_weights, tensors}`
//! (`model.rs:532-555`), `LlamaLinearWeight::{Dense, Quantized}` (`model.rs:62-68`),
//! `QuantizedTensorData::{bytes, descriptor}` (`data.rs:296-302`).

use crate::models::transformer::{LlamaLinearWeight, LlamaModel};
use crate::session::SessionTarget;
use rustgrad_b200_sys::safe::{CudaCallError, CudaSessionTarget, LlamaCudaGenerationError, LlamaCudaPlan, LlamaCudaSession};
use rustgrad_b200_sys::{ggml_type, rg_llama_config};

/// Resource-free plan: the validated model, not yet on any device.
pub struct LlamaCudaModelPlan {
    model: LlamaModel,
}

impl LlamaCudaModelPlan {
    /// `LlamaMetalPlan::from_workflow_on` for the CUDA target.
    pub fn from_model(model: LlamaModel) -> Self {
        Self { model }
    }

    fn config(&self) -> rg_llama_config {
        let c = self.model.config();
        let s = c.schema();
        rg_llama_config {
            n_layers: c.layer_count() as i32,
            d_model: s.embedding_dim as i32,
            n_heads: s.query_heads as i32,
            n_kv_heads: s.kv_heads as i32,
            head_dim: s.head_dim as i32,
            ffn_dim: s.hidden_dim as i32,
            vocab: s.vocab_size as i32,
            max_context: c.max_context() as i32,
            norm_eps: c.norm_eps(),
            rope_theta: c.rope_theta(),
            eos_id: c.token_ids().eos() as i32,
            eot_id: c.token_ids().eot().map_or(-1, |t| t as i32),
            rope_dim: s.rope_dim() as i32,
            qk_norm: match c.qk_norm() {
                crate::models::transformer::LlamaQkNorm::None => 0,
                crate::models::transformer::LlamaQkNorm::PerHead => 1,
                crate::models::transformer::LlamaQkNorm::PerProjection => 2,
            },
            qkv_bias: c.qkv_bias() as i32,
        }
    }

    fn bind(&self, target: &CudaSessionTarget) -> Result<LlamaCudaPlan, CudaCallError> {
        let mut plan = LlamaCudaPlan::empty(self.config(), target)?;
        let state = self.model.state();
        for (name, weight) in state.linear_weights() {
            match weight {
                LlamaLinearWeight::Quantized(q) => {
                    let d = q.descriptor();
                    plan.add_tensor(name, d.ggml_type().id() as i32, d.rows() as u64, d.columns() as u64, q.bytes())?;
                }
                LlamaLinearWeight::Dense(t) => {
                    let dims = t.shape().dims();
                    plan.add_tensor(name, ggml_type::F32, dims[0] as u64, dims[1] as u64, t.as_f32_bytes())?;
                }
            }
        }
        for (name, t) in state.tensors() {
            // norm vectors (and a dense embedding): rank-1 tensors travel as one row
            let dims = t.shape().dims();
            let (rows, cols) = if dims.len() == 1 { (1, dims[0]) } else { (dims[0], dims[1]) };
            plan.add_tensor(name, ggml_type::F32, rows as u64, cols as u64, t.as_f32_bytes())?;
        }
        Ok(plan)
    }
}

impl SessionTarget<LlamaCudaModelPlan> for CudaSessionTarget {
    type Session = LlamaCudaSession;
    type Error = LlamaCudaGenerationError;

    fn prepare(&self, plan: LlamaCudaModelPlan) -> Result<Self::Session, Self::Error> {
        plan.bind(self)?.prepare()
    }
}
