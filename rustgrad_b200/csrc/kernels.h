// Host-callable launchers of the sm_100a kernels.  Internal to the library (not part of the C ABI).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace rg {

struct LaunchCfg {
  cudaStream_t stream = nullptr;
  bool pdl = false;    // launch with programmatic stream serialization
  int sm_count = 148;
  int *status = nullptr;  // device status word (see rg_device.cuh)
  // Development trace (nullable): 16 u64 slots of this launch; the first and the last CTA of the
  // integer GEMV and of the one-launch attention stamp %globaltimer at their phase boundaries.
  unsigned long long *trace = nullptr;
};

// cudaFuncSetAttribute applies to the current device only: a launcher keeps one flag per device
// ordinal so that a process driving sessions on several GPUs prepares its kernels on each of them.
struct DeviceOnce {
  bool done[64] = {};
  bool *slot() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;  // unknown device: set every time
    return &done[dev];
  }
};

// Launch counters per kernel family (process-wide), so a test can prove which kernel served a call.
enum LaunchCounter {
  LC_QGEMV_I8 = 0, LC_QGEMV, LC_QGEMM_TC, LC_QGEMM_TC_WIDE, LC_ATTN_FUSED, LC_ATTN_PREFILL, LC_ATTN_SPLIT, LC_TP_EXCHANGE,
  LC_KQUANT_GEMV, LC_DENSE_GEMV, LC_ATTN_PREFILL_TC, LC_QGEMV_ROWS, LC_ATTN_DECODE_TC, LC_COUNT
};
void count_launch(int which);

enum GemvEpilogue { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2 };

// y = x . W^T for packed W given as up to three row segments that share K (virtual rows are the
// concatenation).  EPI_SWIGLU pairs row r of segment 0 (gate) with row r of segment 1 (up) and
// writes silu(gate) * up straight into the packed-activation buffer of the next GEMV.
struct GemvArgs {
  int type = 0;  // RG_TYPE_Q4_0 or RG_TYPE_Q8_0
  const uint8_t *w[3] = {nullptr, nullptr, nullptr};
  int seg_rows[3] = {0, 0, 0};
  int nseg = 1;
  int k = 0;               // multiple of 256
  const void *xpack = nullptr;
  int batch = 1;           // 1..16
  int epi = EPI_STORE;
  float *y = nullptr;      // EPI_STORE: y[b*ldy + row] = v;  EPI_RESIDUAL: y[b*ldy + row] += v
  int ldy = 0;
  void *ypack = nullptr;   // EPI_SWIGLU: packed output with K' = seg_rows[0]
  // Deferred RMSNorm between the GEMVs of a batch step (qgemv.cu only; the reference's rms_norm,
  // src/models/transformer/layer.rs:423-443, with the scalar 1 / rms moved behind the linear map):
  //  * producer side (EPI_RESIDUAL): besides y += v, the new rows times `pack_w` (the next norm's weight) are
  //    left packed in `pack_next`, and every CTA leaves the sum of squares of its new rows per batch column in
  //    ssq_out[cta * 16 + b];
  //  * consumer side: the input `xpack` holds such un-normalised rows; the outputs are multiplied by
  //    1 / sqrt(sum over the first ssq_n CTAs' sums / k + norm_eps) of their batch column.
  void *pack_next = nullptr;
  const float *pack_w = nullptr;
  float *ssq_out = nullptr;
  const float *ssq_in = nullptr;
  int ssq_n = 0;
  float norm_eps = 0.0f;
  // Workspace of the K-split form of qgemv_rows.cu (optional; without it matrices with few rows run unsplit):
  // partial tiles, and QGEMV_ROWS_MAX_TILES counters that are zero between launches.
  float *split_scratch = nullptr;
  size_t split_scratch_floats = 0;
  unsigned *split_counters = nullptr;
};
constexpr int QGEMV_ROWS_MAX_TILES = 256;
cudaError_t launch_qgemv(const GemvArgs &a, const LaunchCfg &cfg);
int qgemv_grid(int n_rows, int sm_count);  // CTAs launch_qgemv's own kernel uses for a matrix of n_rows rows
// A second form for 3..16 batch rows on Q4_0 (qgemv_rows.cu: tall row tiles that share one copy of the
// activations, K split over CTAs for matrices with few rows), behind RG_B200_ROWS_GEMV=1; launch_qgemv checks
// the arguments and dispatches.
bool qgemv_rows_enabled();
bool qgemv_rows_applies(const GemvArgs &a);
cudaError_t launch_qgemv_rows(const GemvArgs &a, const LaunchCfg &cfg);
size_t xpack_bytes(int k, int batch);  // K rounded up to a whole 32-element block

// Integer tensor-core GEMV for batch 1..2 with the activations packed (and optionally
// RMS-normalised) by the kernel's own prologue from plain f32 input.  Same segment / epilogue
// conventions as GemvArgs, except that EPI_SWIGLU writes plain f32 to y.
struct GemvI8Args {
  int type = 0;  // RG_TYPE_Q4_0 or RG_TYPE_Q8_0
  const uint8_t *w[3] = {nullptr, nullptr, nullptr};
  int seg_rows[3] = {0, 0, 0};
  int nseg = 1;
  int k = 0;
  const float *x = nullptr;  // [batch][ldx]
  int ldx = 0;
  const int32_t *col_map = nullptr;  // device array: source row of each batch column (nullable)
  const float *norm_w = nullptr;     // RMSNorm weight [k]; nullptr = no normalisation
  float eps = 0.0f;
  int batch = 1;
  int epi = EPI_STORE;
  float *y = nullptr;
  int ldy = 0;
  // Batch 1 only.  xq: the input vector already packed by the kernel that produced it
  // (qgemv_i8_xq_bytes(k) bytes, 128-byte aligned); x, col_map and norm_w are then unused, and with
  // xq_norm the results are scaled by 1 / sqrt(mean(x^2) + eps) taken from the vector's block sums
  // (the producer folded the norm weight into the packed values).
  const uint8_t *xq = nullptr;
  bool xq_norm = false;
  // blocks of xq that its producer left unpacked (device array of block indices): the prologue packs
  // them from x.  A SwiGLU producer leaves the blocks that straddle two of its CTAs.
  const int32_t *xq_fix = nullptr;
  int xq_nfix = 0;
  // EPI_RESIDUAL or EPI_SWIGLU, batch 1, rows a multiple of 32: besides y, write the new rows packed
  // as the input of the next GEMV, whose block type is pack_type, with pack_w (nullable; residual
  // only) folded in.  The residual form packs every block; the SwiGLU form those inside one CTA.
  uint8_t *pack_out = nullptr;
  const float *pack_w = nullptr;
  int pack_type = 0;
  // Weights the NEXT kernel of the step will stream (up to three tensors, 16-byte aligned): once this
  // launch has issued its own loads its producer warps ask L2 for them, so that the next kernel's
  // first stages are L2 hits instead of a cold start of the HBM stream.
  const uint8_t *next_w[3] = {nullptr, nullptr, nullptr};
  size_t next_bytes[3] = {0, 0, 0};
};
bool qgemv_i8_supported(int k, int batch);
size_t qgemv_i8_xq_bytes(int k);
// Output rows per CTA of a launch over n_rows rows (EPI_SWIGLU: rows of the gate matrix).
int qgemv_i8_rows_per_cta(int n_rows, int sm_count, bool whole_blocks);
cudaError_t launch_qgemv_i8(const GemvI8Args &a, const LaunchCfg &cfg);

// tcgen05 GEMM for many tokens: out[m][n] = x[m][k] (16-bit) . W[n][k]^T with W in Q4_0 / Q8_0 blocks
// dequantised to 16-bit tiles; f32 accumulation in TMEM.  Operand modes: bf16; IEEE half (more
// mantissa, saturating activations); compensated half, where activations come as two planes
// (hi = f16(x), lo = f16(x - hi)), the weights are split the same way in the kernel and three
// products per K step give f32-grade accuracy.  splits > 1 divides K over blockIdx.z and writes one
// partial result per split (split_stride floats apart) for a later reduction.
enum QGemmMode { QGEMM_BF16 = 0, QGEMM_F16 = 1, QGEMM_F16X3 = 2 };
struct QGemmArgs {
  int type = 0;
  const uint8_t *w = nullptr;
  int n = 0, k = 0;
  const void *x16 = nullptr;     // [m][ldx] bf16 or f16, 16-byte aligned rows
  const void *x16_lo = nullptr;  // QGEMM_F16X3: the low plane, same shape
  int mode = QGEMM_BF16;
  int ldx = 0;
  int m = 0;
  float *out = nullptr;
  int ldc = 0;
  int splits = 1;
  size_t split_stride = 0;
  bool accumulate = false;  // out += x . W^T (a projection whose result is added to the residual stream); splits must be 1
};
cudaError_t launch_qgemm_tc(const QGemmArgs &a, const LaunchCfg &cfg);
// 128 x 512 tiles with the A operand in shared memory (qgemm_tc_wide.cu): single-operand modes, Q4_0, m > 256
bool qgemm_tc_wide_applies(const QGemmArgs &a);
cudaError_t launch_qgemm_tc_wide(const QGemmArgs &a, const LaunchCfg &cfg);
int qgemm_effective_splits(int k, int splits);
int qgemm_rows_per_cta(int mode);
// out[r][i] = sum over s < splits of part[s * stride + r * n + i]
cudaError_t launch_reduce_splits(const float *part, int splits, size_t stride, int n, int rows, float *out, int ldo,
                                 const LaunchCfg &cfg);
// Destination of the f32 -> operand conversions: lo is written only for f16 operands and may be null.
struct Operand16 {
  void *hi = nullptr, *lo = nullptr;
  int ld = 0;
  bool f16 = false;
};
cudaError_t launch_to16(const float *x, int ldx, int k, int rows, const Operand16 &y, const LaunchCfg &cfg);
// RMSNorm of `rows` token rows to the 16-bit GEMM operand; SwiGLU of (gate, up) rows likewise.
cudaError_t launch_rmsnorm16(const float *x, int ldx, const float *w, int d, float eps, int rows, const Operand16 &y,
                             const LaunchCfg &cfg);
cudaError_t launch_swiglu16(const float *g, const float *u, int n, int ld, int rows, const Operand16 &y, const LaunchCfg &cfg);

// ---- Tensor-parallel partial sum + residual add over peer memory (tp_fused.cu) -----------------
constexpr int TP_FUSED_CTAS = 16;
constexpr int TP_FUSED_MAX_WORLD = 8;
// Words of flag storage every rank provides: [2 buffers][TP_FUSED_CTAS][TP_FUSED_MAX_WORLD].
constexpr int TP_FUSED_FLAG_WORDS = 2 * TP_FUSED_CTAS * TP_FUSED_MAX_WORLD;
struct TpFusedArgs {
  float *x = nullptr;  // residual rows [cols][ldx], local
  int ldx = 0, n = 0, cols = 0;
  const float *const *peer_partial = nullptr;  // device array [world]: this buffer on every rank (own rank included)
  int ldp = 0;
  unsigned *const *peer_flags = nullptr;  // device array [world]: flag storage of every rank
  unsigned *epochs = nullptr;             // local, [2][TP_FUSED_CTAS], zero at start
  int rank = 0, world = 1, buffer = 0;
  unsigned poll_limit = 1u << 22;  // polls of a flag word before the wait gives up with DEV_TIMEOUT
  // One column, n a multiple of 32: besides x, write the new residual row packed as the input of the
  // integer GEMV that reads it next (block type pack_type, norm weight pack_w folded in, per-block
  // sums of squares for the deferred RMSNorm): that GEMV's prologue is then a single bulk copy.
  uint8_t *pack_out = nullptr;
  const float *pack_w = nullptr;
  int pack_type = 0;
  // Push form (nullable: then every rank pulls the others' partials after a flag hand-shake): device
  // array [world] of every rank's receive area, [2 buffers][world source ranks][TP_PUSH_COLS][ldp]
  // 8-byte words {value, epoch}.  A thread stores its elements of the local partial into every peer's
  // area (slot = own rank) and then polls its OWN area for the other ranks' words of this epoch: no
  // flags, no fences, no load from a peer; one NVLink store latency per exchange.
  float *const *peer_recv = nullptr;
};
constexpr int TP_PUSH_COLS = 32;  // columns an exchange in push form can carry
cudaError_t launch_tp_allreduce_add(const TpFusedArgs &a, const LaunchCfg &cfg);

// Dense (F32/F16) weight GEMV for tensors the block formats cannot hold (K % 32 != 0) or that a
// file stores dense.  x is plain f32 [batch, ldx]; same epilogues (EPI_SWIGLU unsupported).
struct DenseGemvArgs {
  int type = 0;  // RG_TYPE_F32, RG_TYPE_F16, or a block type without a tuned kernel (RG_TYPE_Q4_K, RG_TYPE_Q6_K)
  const uint8_t *w = nullptr;
  int rows = 0, k = 0;
  const float *x = nullptr;
  int ldx = 0;
  int batch = 1;
  int epi = EPI_STORE;
  float *y = nullptr;
  int ldy = 0;
};
cudaError_t launch_dense_gemv(const DenseGemvArgs &a, const LaunchCfg &cfg);

// f32 [batch, ldx] -> packed activations of K columns.
cudaError_t launch_pack(const float *x, int ldx, int k, int batch, void *xpack, const LaunchCfg &cfg);
// Packed activations -> f32 (used where a dense-weight GEMV follows a packed producer).
cudaError_t launch_unpack(const void *xpack, int k, int batch, float *x, int ldx, const LaunchCfg &cfg);

// Bit-exact block decode (src/gguf/quantization/blocks.rs:1244-1257,1493-1505).  status receives
// DEV_NON_FINITE when a scale or a decoded value is not finite.
cudaError_t launch_dequantize(int type, const uint8_t *bytes, size_t elements, float *out, const LaunchCfg &cfg);
// Embedding row gather: out[c, :] = decode(row ids[c]); ids validated on the host beforehand.
cudaError_t launch_row_gather(int type, const uint8_t *bytes, int cols, const int32_t *ids, int count, float *out, int ldo,
                              const LaunchCfg &cfg);

// RMSNorm of x[col, :d] with weight w, result written as packed activations (column c of
// `cols`; col_map (nullable) selects source columns) and optionally as plain f32 (y, nullable).
cudaError_t launch_rmsnorm_pack(const float *x, int ldx, const float *w, int d, float eps, int cols, const int32_t *col_map,
                                void *xpack, float *y, int ldy, const LaunchCfg &cfg);

// De-interleave + RoPE of q and k, KV-cache append.  qkv: [cols, qw + 2*kw] raw projections.
// q_out: [cols, heads, hd] rotated.  Caches: [seqs, kv_heads, ctx, hd] (half or float).
struct RopeArgs {
  const float *qkv = nullptr;
  int cols = 0, heads = 0, kv_heads = 0, hd = 0, ctx = 0;
  const int32_t *col_seq = nullptr;  // sequence of each column
  const int32_t *col_pos = nullptr;  // absolute position of each column
  const float *cos_t = nullptr;      // [ctx, hd/2]
  const float *sin_t = nullptr;
  float *q_out = nullptr;
  void *k_cache = nullptr, *v_cache = nullptr;
  bool kv_f32 = false;
  // Model variants (layer.rs:274-346,481-571); the defaults are the plain layer.  rope_dim rotary
  // lanes per head (tables [ctx, rope_dim / 2]); the query is de-interleaved over its last rope_dim
  // lanes, the key over the whole head; biases are added after the permutation; qk_norm 1 is an RMS
  // norm inside every head (weights [hd]), 2 over the whole projection (weights [width]).
  int rope_dim = 0;  // 0 = hd
  int qk_norm = 0;
  float eps = 0.0f;
  const float *q_norm = nullptr, *k_norm = nullptr, *q_bias = nullptr, *k_bias = nullptr, *v_bias = nullptr;
};
cudaError_t launch_rope_append(const RopeArgs &a, const LaunchCfg &cfg);

// Split-context GQA attention for one new token per column, then the combine that writes the
// packed activations of the output projection.  scratch: see attn_scratch_floats().
struct AttnArgs {
  const float *q = nullptr;  // [cols, heads, hd]
  const void *k_cache = nullptr, *v_cache = nullptr;
  bool kv_f32 = false;
  int cols = 0, heads = 0, kv_heads = 0, hd = 0, ctx = 0;
  const int32_t *col_seq = nullptr, *col_pos = nullptr;
  float *scratch = nullptr;
  void *out_pack = nullptr;  // packed [K = heads*hd], batch = cols
  float *out_f32 = nullptr;  // optional plain copy [cols, heads*hd]
};
constexpr int ATTN_SPAN = 128;  // context positions per CTA of the split kernel
bool attention_supported(int heads, int kv_heads, int hd);  // hd in {64,128}, heads/kv_heads in {1,2,4,8}
size_t attn_scratch_floats(int cols, int heads, int hd, int ctx);
cudaError_t launch_attention(const AttnArgs &a, const LaunchCfg &cfg);
// The same for f16 caches and head dimension 128 on the tensor cores, built for batches of rows
// (attn_decode_tc.cu): per-warp cp.async rings keep the K / V stream going.  Two launches (spans, merge).
bool attention_decode_tc_supported(const AttnArgs &a);
size_t attention_decode_tc_scratch_floats(int sm_count, int heads, int kv_heads, int cols, int ctx);
cudaError_t launch_attention_decode_tc(const AttnArgs &a, const LaunchCfg &cfg);

// RoPE + KV append + split-context attention + combine in one launch (attn_fused.cu).  qkv rows are
// the raw projections [cols, qw + 2*kw]; out is [cols, heads*hd] f32.  scratch holds
// cols * heads * max_splits * (hd + 2) floats; counters (cols * kv_heads words) must be zero before
// the first launch and are left zero by every launch.
struct FusedAttnArgs {
  const float *qkv = nullptr;
  int cols = 0, heads = 0, kv_heads = 0, hd = 0, ctx = 0;
  const int32_t *col_seq = nullptr, *col_pos = nullptr;
  const float *cos_t = nullptr, *sin_t = nullptr;
  void *k_cache = nullptr, *v_cache = nullptr;
  bool kv_f32 = false;
  float *scratch = nullptr;
  int max_splits = 0;
  unsigned *counters = nullptr;
  float *out = nullptr;
  // the launch may read positions, rotation tables and cached rows before its grid dependency
  // resolves: only when an earlier attention launch of the same step separates it from their writers
  bool early = false;
  // cols == 1: also leave the output packed as the input of the integer GEMV of the output
  // projection (qgemv_i8_xq_bytes(heads * hd) bytes; pack_type = that projection's block type)
  uint8_t *pack_out = nullptr;
  int pack_type = 0;
  // any cols: also leave the output as the packed activations (hi / lo f16 columns) of the f16-MMA GEMV
  void *xpack_out = nullptr;
};
bool fused_attention_supported(int heads, int kv_heads, int hd);
int fused_attn_per_head(int sm_count, int kv_heads, int cols);
int fused_attn_max_splits(int ctx, int hd, bool kv_f32, int sm_count, int kv_heads);
int fused_attn_split_cap();
cudaError_t launch_attention_fused(const FusedAttnArgs &a, const LaunchCfg &cfg);

// Causal attention for a chunk of consecutive prompt tokens of one sequence (attn_prefill.cu): q is
// the rotated queries [cols][heads][hd] f32, the caches already hold the chunk's K / V rows, out is
// [cols][heads*hd] f32.  Token i of the chunk sits at position pos0 + i.
struct PrefillAttnArgs {
  const float *q = nullptr;
  const void *k_cache = nullptr, *v_cache = nullptr;
  bool kv_f32 = false;
  int cols = 0, heads = 0, kv_heads = 0, ctx = 0, seq = 0, pos0 = 0;
  float *out = nullptr;
  // Tensor-core form only: when out16_hi is set the result goes straight to the 16-bit operand planes of
  // the output projection (row stride out16_ld elements; lo only with f16 operands, may be null) and
  // `out` is not written.
  void *out16_hi = nullptr, *out16_lo = nullptr;
  int out16_ld = 0;
  bool out16_f16 = false;
};
// True when launch_attention_prefill will take the tensor-core form for these arguments.
bool prefill_attention_uses_tc(const PrefillAttnArgs &a);
bool prefill_attention_supported(int heads, int kv_heads, int hd);
cudaError_t launch_attention_prefill(const PrefillAttnArgs &a, const LaunchCfg &cfg);
// Tensor-core form for f16 caches (attn_prefill_tc.cu); launch_attention_prefill dispatches to it.
cudaError_t launch_attention_prefill_tc(const PrefillAttnArgs &a, const LaunchCfg &cfg);

// Greedy selection per column with the reference's rules (generation.rs:260-287): lowest id wins
// ties, any non-finite logit yields -1.  Also advances: next_tokens[c] = id, pos[c] += 1 when
// advance is set.
cudaError_t launch_argmax(const float *logits, int ld, int vocab, int cols, int32_t *out_ids, const LaunchCfg &cfg);
// Same with the Gumbel-max score transform when `uniforms` ([cols][vocab], device) is given (generation.rs:10-19,273-278).
// `temps` (device, nullable): one temperature per column; columns with a non-positive one are greedy.
cudaError_t launch_select(const float *logits, int ld, int vocab, int cols, const float *uniforms, float temperature,
                          int32_t *out_ids, const LaunchCfg &cfg, const float *temps = nullptr);
cudaError_t launch_advance(const int32_t *ids, int32_t *tokens, int32_t *pos, int32_t *history, int32_t *step_counter,
                           int cols, const LaunchCfg &cfg);

// Synthetic tensors: counter-based N(0, std) then GGML quantization, all on the device.
// row0/rows and col0/cols select the shard of the full [full_rows, full_cols] tensor.
cudaError_t launch_synth(int type, uint8_t *out, uint64_t seed, float std, uint64_t full_cols, uint64_t row0, uint64_t rows,
                         uint64_t col0, uint64_t cols, const LaunchCfg &cfg);
cudaError_t launch_fill_f32(float *out, size_t n, float v, const LaunchCfg &cfg);
// h = silu(g) * u for dense-weight gate/up projections (packed and/or plain output).
cudaError_t launch_swiglu(const float *g, const float *u, int n, int ld, int batch, void *pack, float *out, int ldo,
                          const LaunchCfg &cfg);
// x[b, :n] += p[b, :n]
cudaError_t launch_add_rows(float *x, int ldx, const float *p, int ldp, int n, int batch, const LaunchCfg &cfg);

}  // namespace rg
