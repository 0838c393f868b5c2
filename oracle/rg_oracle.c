/*
 * CPU restatement of rustgrad's GGUF-quantized Llama path.  TEST INFRASTRUCTURE ONLY: the
 * shipped CUDA library never links, loads or calls this file (see rg_oracle.h).
 *
 * Arithmetic rule of the reference's CPU backend: every primitive is evaluated in f64 from f32
 * operands and committed to f32 (src/backend/cpu.rs:1449-1491,1620-1694,
 * src/tensor/dtype.rs:347-353).  For +, -, *, / and sqrt an f64 evaluation followed by one f32
 * rounding equals the IEEE f32 operation, so plain `float` arithmetic compiled with
 * -ffp-contract=off reproduces it; transcendental calls go through double explicitly.
 *
 * Build with: gcc -O2 -ffp-contract=off -fopenmp (see Makefile).
 */
#include "rg_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ scalars */

/* src/tensor/scalar.rs:110-135 */
float rgo_f16_to_f32(uint16_t bits) {
  uint32_t sign = ((uint32_t)(bits & 0x8000u)) << 16;
  uint32_t exp = (bits >> 10) & 0x1fu;
  uint32_t mant = bits & 0x03ffu;
  uint32_t out;
  if (exp == 0) {
    if (mant == 0) {
      out = sign;
    } else {
      int exponent = -14;
      while ((mant & 0x0400u) == 0) {
        mant <<= 1;
        exponent -= 1;
      }
      out = sign | ((uint32_t)(exponent + 127) << 23) | ((mant & 0x03ffu) << 13);
    }
  } else if (exp == 31) {
    out = sign | 0x7f800000u | (mant << 13);
  } else {
    out = sign | ((exp + 112u) << 23) | (mant << 13);
  }
  float value;
  memcpy(&value, &out, 4);
  return value;
}

static uint32_t round_shift_right_ties_even(uint32_t value, uint32_t shift) {
  uint32_t truncated = value >> shift;
  uint32_t remainder = value & ((1u << shift) - 1u);
  uint32_t halfway = 1u << (shift - 1);
  return truncated + ((remainder > halfway || (remainder == halfway && (truncated & 1u))) ? 1u : 0u);
}

/* src/tensor/scalar.rs:137-174 (round to nearest even, subnormals kept, overflow to inf) */
uint16_t rgo_f32_to_f16(float value) {
  uint32_t bits;
  memcpy(&bits, &value, 4);
  uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
  uint32_t raw_exponent = (bits >> 23) & 0xffu;
  uint32_t mantissa = bits & 0x7fffffu;
  if (raw_exponent == 0xff) {
    return (uint16_t)(sign | 0x7c00u | (mantissa == 0 ? 0u : ((mantissa >> 13) | 1u)));
  }
  int exponent = (int)raw_exponent - 127 + 15;
  if (exponent <= 0) {
    if (exponent < -10) return sign;
    uint32_t shift = (uint32_t)(14 - exponent);
    return (uint16_t)(sign | round_shift_right_ties_even(mantissa | 0x800000u, shift));
  }
  if (exponent >= 31) return (uint16_t)(sign | 0x7c00u);
  uint32_t rounded = round_shift_right_ties_even(mantissa, 13);
  if (rounded == 0x400u) {
    if (exponent == 30) return (uint16_t)(sign | 0x7c00u);
    return (uint16_t)(sign | ((uint32_t)(exponent + 1) << 10));
  }
  return (uint16_t)(sign | ((uint32_t)exponent << 10) | rounded);
}

/* ------------------------------------------------------------------ blocks */

/* src/gguf/tensor.rs:88-155 */
int rgo_block_elements(int t) {
  switch (t) {
    case RGO_F32: case RGO_F16: return 1;
    case RGO_Q4_0: case RGO_Q8_0: return 32;
    case RGO_Q4_K: case RGO_Q6_K: return 256;
    default: return 0;
  }
}
int rgo_block_bytes(int t) {
  switch (t) {
    case RGO_F32: return 4;
    case RGO_F16: return 2;
    case RGO_Q4_0: return 18;
    case RGO_Q8_0: return 34;
    case RGO_Q4_K: return 144;
    case RGO_Q6_K: return 210;
    default: return 0;
  }
}

static float half_le(const uint8_t *p) { return rgo_f16_to_f32((uint16_t)(p[0] | (p[1] << 8))); }

static int all_finite32(const float *v) {
  for (int i = 0; i < 32; ++i)
    if (!isfinite(v[i])) return 0;
  return 1;
}

/* src/gguf/quantization/blocks.rs:1244-1257: byte j carries element j (low nibble) and
 * element 16+j (high nibble); value = (nibble - 8) * d. */
int rgo_decode_q4_0_block(const uint8_t *block, float out[32]) {
  float d = half_le(block);
  if (!isfinite(d)) return RGO_ERR_NON_FINITE;
  for (int lane = 0; lane < 16; ++lane) {
    uint8_t packed = block[2 + lane];
    out[lane] = ((float)(packed & 0x0f) - 8.0f) * d;
    out[16 + lane] = ((float)(packed >> 4) - 8.0f) * d;
  }
  return all_finite32(out) ? RGO_OK : RGO_ERR_NON_FINITE;
}

/* src/gguf/quantization/blocks.rs:1493-1505 */
int rgo_decode_q8_0_block(const uint8_t *block, float out[32]) {
  float d = half_le(block);
  if (!isfinite(d)) return RGO_ERR_NON_FINITE;
  for (int lane = 0; lane < 32; ++lane) out[lane] = (float)(int8_t)block[2 + lane] * d;
  return all_finite32(out) ? RGO_OK : RGO_ERR_NON_FINITE;
}

/* src/gguf/quantization/blocks.rs:1511-1522: eight 6-bit (scale, min) pairs packed in 12 bytes. */
static void unpack_k_scales_mins(const uint8_t *packed, uint8_t scales[8], uint8_t mins[8]) {
  for (int lane = 0; lane < 4; ++lane) {
    scales[lane] = packed[lane] & 0x3f;
    mins[lane] = packed[4 + lane] & 0x3f;
    scales[4 + lane] = (uint8_t)((packed[8 + lane] & 0x0f) | ((packed[lane] >> 6) << 4));
    mins[4 + lane] = (uint8_t)((packed[8 + lane] >> 4) | ((packed[4 + lane] >> 6) << 4));
  }
}

/* src/gguf/quantization/blocks.rs:1164-1187: d, dmin (f16), 12 bytes of scales / mins, eight groups
 * of 32 four-bit values; value = d * f32(scale) * f32(q) - dmin * f32(min), each step rounded to f32. */
int rgo_decode_q4_k_block(const uint8_t *block, float out[256]) {
  float d = half_le(block), dmin = half_le(block + 2);
  if (!isfinite(d) || !isfinite(dmin)) return RGO_ERR_NON_FINITE;
  uint8_t scales[8], mins[8];
  unpack_k_scales_mins(block + 4, scales, mins);
  const uint8_t *quants = block + 16;
  for (int group = 0; group < 8; ++group) {
    int source_group = group / 2, shift = (group % 2) * 4;
    for (int lane = 0; lane < 32; ++lane) {
      uint8_t q = (uint8_t)((quants[source_group * 32 + lane] >> shift) & 0x0f);
      float a = d * (float)scales[group];
      a = a * (float)q;
      float b = dmin * (float)mins[group];
      out[group * 32 + lane] = a - b;
    }
  }
  for (int i = 0; i < 256; ++i)
    if (!isfinite(out[i])) return RGO_ERR_NON_FINITE;
  return RGO_OK;
}

/* src/gguf/quantization/blocks.rs:1219-1240: 128 bytes of low nibbles, 64 bytes of 2-bit highs, 16
 * signed scales, trailing f16 d; value = d * f32((q - 32) * scale). */
int rgo_decode_q6_k_block(const uint8_t *block, float out[256]) {
  float d = half_le(block + 208);
  if (!isfinite(d)) return RGO_ERR_NON_FINITE;
  for (int index = 0; index < 256; ++index) {
    int half_index = index / 128, within_half = index % 128;
    int low_shift = (within_half / 64) * 4;
    int low = (block[half_index * 64 + within_half % 64] >> low_shift) & 0x0f;
    int high_shift = (within_half / 32) * 2;
    int high = ((block[128 + half_index * 32 + within_half % 32] >> high_shift) & 0x03) << 4;
    int quant = (low | high) - 32;
    int scale = (int)(int8_t)block[192 + index / 16];
    out[index] = d * (float)(quant * scale);
  }
  for (int i = 0; i < 256; ++i)
    if (!isfinite(out[i])) return RGO_ERR_NON_FINITE;
  return RGO_OK;
}

/* Decodes `count` consecutive elements starting at element `first` (both multiples of the block
 * size for packed types).  src/gguf/quantization/data.rs:415-428. */
static int decode_span(int t, const uint8_t *bytes, size_t first, size_t count, float *out) {
  switch (t) {
    case RGO_F32:
      memcpy(out, bytes + first * 4, count * 4);
      return RGO_OK;
    case RGO_F16:
      for (size_t i = 0; i < count; ++i) out[i] = half_le(bytes + (first + i) * 2);
      return RGO_OK;
    case RGO_Q4_0:
    case RGO_Q8_0: {
      if (first % 32 || count % 32) return RGO_ERR_ARG;
      size_t bb = (size_t)rgo_block_bytes(t);
      const uint8_t *p = bytes + (first / 32) * bb;
      for (size_t b = 0; b < count / 32; ++b) {
        int rc = (t == RGO_Q4_0) ? rgo_decode_q4_0_block(p + b * bb, out + b * 32)
                                 : rgo_decode_q8_0_block(p + b * bb, out + b * 32);
        if (rc) return rc;
      }
      return RGO_OK;
    }
    case RGO_Q4_K:
    case RGO_Q6_K: {
      if (first % 256 || count % 256) return RGO_ERR_ARG;
      size_t bb = (size_t)rgo_block_bytes(t);
      const uint8_t *p = bytes + (first / 256) * bb;
      for (size_t b = 0; b < count / 256; ++b) {
        int rc = (t == RGO_Q4_K) ? rgo_decode_q4_k_block(p + b * bb, out + b * 256)
                                 : rgo_decode_q6_k_block(p + b * bb, out + b * 256);
        if (rc) return rc;
      }
      return RGO_OK;
    }
    default:
      return RGO_ERR_TYPE;
  }
}

int rgo_dequantize(int t, const uint8_t *bytes, size_t elements, float *out) {
  if (!rgo_block_elements(t)) return RGO_ERR_TYPE;
  return decode_span(t, bytes, 0, elements, out);
}

/* src/gguf/quantization/row_gather.rs:149-226 */
int rgo_row_gather(int t, const uint8_t *bytes, size_t rows, size_t cols, const int64_t *indices,
                   size_t count, float *out) {
  if (!rgo_block_elements(t)) return RGO_ERR_TYPE;
  if (cols % (size_t)rgo_block_elements(t)) return RGO_ERR_ARG;
  for (size_t i = 0; i < count; ++i)
    if (indices[i] < 0 || (uint64_t)indices[i] >= rows) return RGO_ERR_INDEX;
  for (size_t i = 0; i < count; ++i) {
    int rc = decode_span(t, bytes, (size_t)indices[i] * cols, cols, out + i * cols);
    if (rc) return rc;
  }
  return RGO_OK;
}

/* src/matmul/quantized.rs:126-182 */
int rgo_quantized_matmul(int t, const uint8_t *weight, size_t n, size_t k, const float *a, size_t m,
                         float *out) {
  if (t != RGO_Q4_0 && t != RGO_Q8_0) return RGO_ERR_TYPE;
  if (k % 32) return RGO_ERR_ARG;
  size_t bb = (size_t)rgo_block_bytes(t);
  size_t bpr = k / 32;
  float decoded[32];
  for (size_t row = 0; row < m; ++row) {
    for (size_t col = 0; col < n; ++col) {
      double acc = 0.0;
      for (size_t b = 0; b < bpr; ++b) {
        const uint8_t *blk = weight + (col * bpr + b) * bb;
        int rc = (t == RGO_Q4_0) ? rgo_decode_q4_0_block(blk, decoded) : rgo_decode_q8_0_block(blk, decoded);
        if (rc) return rc;
        const float *x = a + row * k + b * 32;
        for (int lane = 0; lane < 32; ++lane) acc += (double)x[lane] * (double)decoded[lane];
      }
      out[row * n + col] = (float)acc;
    }
  }
  return RGO_OK;
}

/* src/backend/cpu.rs:3506-3529 */
static float dot_strict(const float *x, const float *w, size_t k) {
  float acc = 0.0f;
  for (size_t i = 0; i < k; ++i) {
    float p = x[i] * w[i];
    acc = acc + p;
  }
  return acc;
}

void rgo_dense_matmul_strict(const float *weight, size_t n, size_t k, const float *a, size_t m, float *out) {
  for (size_t row = 0; row < m; ++row)
    for (size_t col = 0; col < n; ++col) out[row * n + col] = dot_strict(a + row * k, weight + col * k, k);
}

/* ------------------------------------------------------------------ model */

typedef struct {
  int type; /* -1 = absent */
  size_t rows, cols;
  const uint8_t *bytes;
} rgo_tensor;

#define RGO_LAYER_TENSORS 14
typedef struct {
  rgo_tensor attn_norm, attn_q, attn_k, attn_v, attn_output, ffn_norm, ffn_gate, ffn_up, ffn_down;
  rgo_tensor q_norm, k_norm, q_bias, k_bias, v_bias; /* variants only */
} rgo_layer;

struct rgo_model {
  rgo_config cfg;
  rgo_tensor token_embd, output_norm, output;
  rgo_layer *layers;
};

struct rgo_cache {
  const rgo_model *model;
  int kv_f16;
  int len;
  float **keys;   /* per layer [kv_heads][max_context][head_dim] */
  float **values; /* same */
};

rgo_model *rgo_model_create(const rgo_config *c) {
  if (!c || c->n_layers <= 0 || c->d_model <= 0 || c->n_heads <= 0 || c->n_kv_heads <= 0 ||
      c->head_dim <= 0 || c->ffn_dim <= 0 || c->vocab <= 0 || c->max_context <= 0 ||
      c->n_heads % c->n_kv_heads || (c->head_dim & 1))
    return NULL;
  if (c->rope_dim < 0 || c->rope_dim > c->head_dim || (c->rope_dim & 1) || c->qk_norm < 0 || c->qk_norm > 2) return NULL;
  if (c->qk_norm == 2 && c->n_heads != c->n_kv_heads) return NULL; /* model.rs:262-268: equal widths only */
  rgo_model *m = (rgo_model *)calloc(1, sizeof(*m));
  m->cfg = *c;
  m->layers = (rgo_layer *)calloc((size_t)c->n_layers, sizeof(rgo_layer));
  m->token_embd.type = m->output_norm.type = m->output.type = -1;
  for (int l = 0; l < c->n_layers; ++l) {
    rgo_tensor *t = (rgo_tensor *)&m->layers[l];
    for (int i = 0; i < RGO_LAYER_TENSORS; ++i) t[i].type = -1;
  }
  return m;
}

void rgo_model_destroy(rgo_model *m) {
  if (!m) return;
  free(m->layers);
  free(m);
}

static rgo_tensor *find_tensor(rgo_model *m, const char *name, size_t *rows, size_t *cols, int *is_norm) {
  const rgo_config *c = &m->cfg;
  size_t qw = (size_t)c->n_heads * c->head_dim, kw = (size_t)c->n_kv_heads * c->head_dim;
  size_t d = (size_t)c->d_model, f = (size_t)c->ffn_dim;
  *is_norm = 0;
  if (!strcmp(name, "token_embd.weight")) { *rows = (size_t)c->vocab; *cols = d; return &m->token_embd; }
  if (!strcmp(name, "output.weight")) { *rows = (size_t)c->vocab; *cols = d; return &m->output; }
  if (!strcmp(name, "output_norm.weight")) { *rows = 1; *cols = d; *is_norm = 1; return &m->output_norm; }
  int layer = -1, consumed = 0;
  if (sscanf(name, "blk.%d.%n", &layer, &consumed) != 1 || layer < 0 || layer >= c->n_layers) return NULL;
  const char *s = name + consumed;
  rgo_layer *L = &m->layers[layer];
  if (!strcmp(s, "attn_norm.weight")) { *rows = 1; *cols = d; *is_norm = 1; return &L->attn_norm; }
  if (!strcmp(s, "ffn_norm.weight")) { *rows = 1; *cols = d; *is_norm = 1; return &L->ffn_norm; }
  if (!strcmp(s, "attn_q.weight")) { *rows = qw; *cols = d; return &L->attn_q; }
  if (!strcmp(s, "attn_k.weight")) { *rows = kw; *cols = d; return &L->attn_k; }
  if (!strcmp(s, "attn_v.weight")) { *rows = kw; *cols = d; return &L->attn_v; }
  if (!strcmp(s, "attn_output.weight")) { *rows = d; *cols = qw; return &L->attn_output; }
  if (!strcmp(s, "ffn_gate.weight")) { *rows = f; *cols = d; return &L->ffn_gate; }
  if (!strcmp(s, "ffn_up.weight")) { *rows = f; *cols = d; return &L->ffn_up; }
  if (!strcmp(s, "ffn_down.weight")) { *rows = d; *cols = f; return &L->ffn_down; }
  /* model.rs:427-449: present only for the variant the configuration names */
  size_t hd = (size_t)c->head_dim;
  if (c->qk_norm && !strcmp(s, "attn_q_norm.weight")) { *rows = 1; *cols = c->qk_norm == 1 ? hd : qw; *is_norm = 1; return &L->q_norm; }
  if (c->qk_norm && !strcmp(s, "attn_k_norm.weight")) { *rows = 1; *cols = c->qk_norm == 1 ? hd : kw; *is_norm = 1; return &L->k_norm; }
  if (c->qkv_bias && !strcmp(s, "attn_q.bias")) { *rows = 1; *cols = qw; *is_norm = 1; return &L->q_bias; }
  if (c->qkv_bias && !strcmp(s, "attn_k.bias")) { *rows = 1; *cols = kw; *is_norm = 1; return &L->k_bias; }
  if (c->qkv_bias && !strcmp(s, "attn_v.bias")) { *rows = 1; *cols = kw; *is_norm = 1; return &L->v_bias; }
  return NULL;
}

/* src/models/transformer/model.rs:384-510: exact names and shapes; norms must be dense; packed
 * tensors need cols % 32 == 0 (src/gguf/quantization/data.rs:268-270). */
int rgo_model_set_tensor(rgo_model *m, const char *name, int type, size_t rows, size_t cols, const uint8_t *bytes) {
  size_t er, ec;
  int is_norm;
  rgo_tensor *t = find_tensor(m, name, &er, &ec, &is_norm);
  if (!t || !bytes) return RGO_ERR_ARG;
  if (!rgo_block_elements(type)) return RGO_ERR_TYPE;
  if (rows != er || cols != ec) return RGO_ERR_ARG;
  if (is_norm && type != RGO_F32 && type != RGO_F16) return RGO_ERR_TYPE;
  if (cols % (size_t)rgo_block_elements(type)) return RGO_ERR_ARG;
  t->type = type;
  t->rows = rows;
  t->cols = cols;
  t->bytes = bytes;
  return RGO_OK;
}

int rgo_model_check(const rgo_model *m) {
  if (m->token_embd.type < 0 || m->output_norm.type < 0) return RGO_ERR_ARG;
  for (int l = 0; l < m->cfg.n_layers; ++l) {
    const rgo_tensor *t = (const rgo_tensor *)&m->layers[l];
    for (int i = 0; i < 9; ++i)
      if (t[i].type < 0) return RGO_ERR_ARG;
    const rgo_layer *L = &m->layers[l];
    if (m->cfg.qk_norm && (L->q_norm.type < 0 || L->k_norm.type < 0)) return RGO_ERR_ARG;
    if (m->cfg.qkv_bias && (L->q_bias.type < 0 || L->k_bias.type < 0 || L->v_bias.type < 0)) return RGO_ERR_ARG;
  }
  return RGO_OK;
}

rgo_cache *rgo_cache_create(const rgo_model *m, int kv_f16) {
  rgo_cache *c = (rgo_cache *)calloc(1, sizeof(*c));
  c->model = m;
  c->kv_f16 = kv_f16;
  int L = m->cfg.n_layers;
  size_t per = (size_t)m->cfg.n_kv_heads * m->cfg.max_context * m->cfg.head_dim;
  c->keys = (float **)calloc((size_t)L, sizeof(float *));
  c->values = (float **)calloc((size_t)L, sizeof(float *));
  for (int l = 0; l < L; ++l) {
    c->keys[l] = (float *)calloc(per, sizeof(float));
    c->values[l] = (float *)calloc(per, sizeof(float));
  }
  return c;
}
void rgo_cache_destroy(rgo_cache *c) {
  if (!c) return;
  for (int l = 0; l < c->model->cfg.n_layers; ++l) {
    free(c->keys[l]);
    free(c->values[l]);
  }
  free(c->keys);
  free(c->values);
  free(c);
}
void rgo_cache_clear(rgo_cache *c) { c->len = 0; }
/* Timing aid (no counterpart in the reference): makes the cache hold `n_pos` positions of seeded
 * pseudo-random K / V rows, uniform in [-1, 1), so that a decode step can be timed at a long context
 * without running the prompt through the CPU path first. */
int rgo_cache_fill_seeded(rgo_cache *c, int n_pos, uint64_t seed) {
  const rgo_config *cfg = &c->model->cfg;
  if (n_pos < 0 || n_pos > cfg->max_context) return RGO_ERR_CONTEXT;
  uint64_t z = seed * 0x9E3779B97F4A7C15ull + 0xD1342543DE82EF95ull;
  for (int l = 0; l < cfg->n_layers; ++l)
    for (int h = 0; h < cfg->n_kv_heads; ++h)
      for (int p = 0; p < n_pos; ++p) {
        size_t base = ((size_t)h * cfg->max_context + (size_t)p) * cfg->head_dim;
        for (int i = 0; i < cfg->head_dim; ++i) {
          z ^= z << 13, z ^= z >> 7, z ^= z << 17; /* xorshift64 */
          float k = (float)((double)(z >> 40) / 8388608.0 - 1.0);
          z ^= z << 13, z ^= z >> 7, z ^= z << 17;
          float v = (float)((double)(z >> 40) / 8388608.0 - 1.0);
          if (c->kv_f16) k = rgo_f16_to_f32(rgo_f32_to_f16(k)), v = rgo_f16_to_f32(rgo_f32_to_f16(v));
          c->keys[l][base + i] = k;
          c->values[l][base + i] = v;
        }
      }
  c->len = n_pos;
  return RGO_OK;
}
int rgo_cache_len(const rgo_cache *c) { return c->len; }

/* ---- primitives of the forward ---- */

/* src/models/transformer/layer.rs:423-443; Mean = f32 running sum then an f32 division by
 * f32(count) (src/reduction_native.rs:245-272,299-314); rsqrt = reciprocal(sqrt)
 * (src/ir/elementwise.rs:5890-5919). */
static void rms_norm_strict(const float *x, const float *w, int d, float eps, float *y) {
  float sum = 0.0f;
  for (int i = 0; i < d; ++i) {
    float sq = x[i] * x[i];
    sum = sum + sq;
  }
  float mean = sum / (float)d;
  float t = mean + eps;
  float r = sqrtf(t);
  float inv = 1.0f / r;
  for (int i = 0; i < d; ++i) {
    float n = x[i] * inv;
    y[i] = n * w[i];
  }
}

static void norm_weight(const rgo_tensor *t, float *out) { decode_span(t->type, t->bytes, 0, t->cols, out); }

static float dot_fast(const float *x, const float *w, size_t k) {
  float p[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  size_t i = 0;
  for (; i + 8 <= k; i += 8)
    for (int j = 0; j < 8; ++j) p[j] += x[i + j] * w[i + j];
  float acc = ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));
  for (; i < k; ++i) acc += x[i] * w[i];
  return acc;
}

/* y[s][n] = x[s][:] . W[n][:].  Packed weights are decoded row by row to f32 first
 * (src/models/transformer/model.rs:982-995) and multiplied by the dense rule
 * (src/backend/cpu.rs:3506-3529).  `head_f64` selects the blockwise f64-accumulating plan that
 * the reference uses for a packed logits head only (model.rs:1036-1064, matmul/quantized.rs:157-177). */
static int linear(const rgo_tensor *w, const float *x, int S, float *y, int mode, int threads, int head_f64) {
  size_t N = w->rows, K = w->cols;
  int packed = (w->type == RGO_Q4_0 || w->type == RGO_Q8_0 || w->type == RGO_Q4_K || w->type == RGO_Q6_K);
  int failed = 0;
#pragma omp parallel num_threads(threads) if (mode == RGO_MODE_FAST && threads > 1)
  {
    float *row = (float *)malloc(K * sizeof(float));
#pragma omp for schedule(static)
    for (long long n = 0; n < (long long)N; ++n) {
      if (decode_span(w->type, w->bytes, (size_t)n * K, K, row)) {
        failed = 1;
        continue;
      }
      for (int s = 0; s < S; ++s) {
        const float *xs = x + (size_t)s * K;
        float v;
        if (packed && head_f64) {
          if (mode == RGO_MODE_STRICT) {
            double acc = 0.0;
            for (size_t k = 0; k < K; ++k) acc += (double)xs[k] * (double)row[k];
            v = (float)acc;
          } else {
            double p0 = 0, p1 = 0, p2 = 0, p3 = 0;
            for (size_t k = 0; k + 4 <= K; k += 4) {
              p0 += (double)xs[k] * (double)row[k];
              p1 += (double)xs[k + 1] * (double)row[k + 1];
              p2 += (double)xs[k + 2] * (double)row[k + 2];
              p3 += (double)xs[k + 3] * (double)row[k + 3];
            }
            v = (float)((p0 + p1) + (p2 + p3));
          }
        } else {
          v = (mode == RGO_MODE_STRICT) ? dot_strict(xs, row, K) : dot_fast(xs, row, K);
        }
        y[(size_t)s * N + (size_t)n] = v;
      }
    }
    free(row);
  }
  return failed ? RGO_ERR_NON_FINITE : RGO_OK;
}

/* permute_rope_projection (src/models/transformer/layer.rs:481-525): inside every head the last
 * `permuted` lanes are de-interleaved, out[prefix + j] = in[prefix + 2j],
 * out[prefix + permuted/2 + j] = in[prefix + 2j + 1], and the first prefix = hd - permuted lanes
 * stay.  The query is permuted over its last rope_dim lanes (preserve_prefix), the key over the
 * whole head (layer.rs:274-293). */
static void deinterleave_heads(float *v, int heads, int hd, int permuted, float *tmp) {
  int half = permuted / 2, prefix = hd - permuted;
  for (int h = 0; h < heads; ++h) {
    float *p = v + (size_t)h * hd + prefix;
    for (int j = 0; j < half; ++j) {
      tmp[j] = p[2 * j];
      tmp[half + j] = p[2 * j + 1];
    }
    memcpy(p, tmp, (size_t)permuted * sizeof(float));
  }
}

/* apply_rope (src/models/transformer/layer.rs:528-571): lanes [0, rope_dim) of every head rotate as
 * the halves [0, rope_dim/2) and [rope_dim/2, rope_dim) with frequency 1 / theta^(2i / rope_dim);
 * lanes [rope_dim, hd) pass through. */
static void rope_heads(float *v, int heads, int hd, int rope_dim, int position, double theta) {
  int half = rope_dim / 2;
  for (int i = 0; i < half; ++i) {
    double frequency = 1.0 / pow(theta, (double)(2 * i) / (double)rope_dim);
    double angle = (double)position * frequency;
    float c = (float)cos(angle), s = (float)sin(angle);
    for (int h = 0; h < heads; ++h) {
      float *p = v + (size_t)h * hd;
      float x1 = p[i], x2 = p[half + i];
      float a = x1 * c, b = x2 * s;
      float e = x2 * c, f = x1 * s;
      p[i] = a - b;
      p[half + i] = e + f;
    }
  }
}

/* src/ir/elementwise.rs:6772-6830,7046-7050 and layer.rs:398-401 */
static float swiglu_strict(float g, float u) {
  float k = (float)(-1.0 / 0.693147180559945309417232121458);
  float z = g * k;
  float e = (float)exp2((double)z);
  float dn = 1.0f + e;
  float sg = 1.0f / dn;
  float si = g * sg;
  return si * u;
}

/* One query row of src/ir/attention.rs:1157-1207 with the softmax of :495-558.  Keys/values are
 * [T][hd] slices of one kv head.  Masked columns (t > last) contribute exact zeros and are skipped. */
static void attend_row(const float *q, const float *keys, const float *values, int hd, int last,
                       float *scores, float *out) {
  float inv_scale = (float)(1.0 / (1.0 / sqrt((double)hd)));
  float log2e = (float)(1.0 / 0.693147180559945309417232121458);
  float m = -INFINITY;
  for (int t = 0; t <= last; ++t) {
    float s = dot_strict(q, keys + (size_t)t * hd, (size_t)hd);
    s = s / inv_scale;
    scores[t] = s;
    if (s > m) m = s;
  }
  float sum = 0.0f;
  for (int t = 0; t <= last; ++t) {
    float c = scores[t] - m;
    float z = c * log2e;
    float e = (float)exp2((double)z);
    scores[t] = e;
    sum = sum + e;
  }
  float r = 1.0f / sum;
  for (int t = 0; t <= last; ++t) scores[t] = scores[t] * r;
  for (int j = 0; j < hd; ++j) {
    float acc = 0.0f;
    for (int t = 0; t <= last; ++t) {
      float p = scores[t] * values[(size_t)t * hd + j];
      acc = acc + p;
    }
    out[j] = acc;
  }
}

/* One new token's attention over caches laid out [kv_heads][n_pos][hd]; q is [heads][hd], already
 * rotated.  src/ir/attention.rs:1157-1240 (GQA head mapping :1226-1240) via attend_row above. */
int rgo_attention_decode(const float *q, const float *keys, const float *values, int heads, int kv_heads, int hd,
                         int n_pos, float *out) {
  if (!q || !keys || !values || !out || heads <= 0 || kv_heads <= 0 || heads % kv_heads || hd <= 0 || n_pos <= 0)
    return RGO_ERR_ARG;
  float *scores = (float *)malloc((size_t)n_pos * sizeof(float));
  int group = heads / kv_heads;
  for (int h = 0; h < heads; ++h) {
    int kvh = h / group;
    attend_row(q + (size_t)h * hd, keys + (size_t)kvh * n_pos * hd, values + (size_t)kvh * n_pos * hd, hd, n_pos - 1,
               scores, out + (size_t)h * hd);
  }
  free(scores);
  return RGO_OK;
}

static float round_f16(float v) { return rgo_f16_to_f32(rgo_f32_to_f16(v)); }

int rgo_forward(const rgo_model *m, rgo_cache *cache, const int32_t *tokens, int S, int mode, int threads,
                int all_logits, float *logits) {
  const rgo_config *c = &m->cfg;
  if (!tokens || S <= 0 || !logits) return RGO_ERR_ARG;
  if (rgo_model_check(m)) return RGO_ERR_ARG;
  for (int s = 0; s < S; ++s)
    if (tokens[s] < 0 || tokens[s] >= c->vocab) return RGO_ERR_TOKEN_RANGE;
  int past = cache->len;
  if (past + S > c->max_context) return RGO_ERR_CONTEXT;
  if (threads < 1) threads = 1;
  int d = c->d_model, hd = c->head_dim, H = c->n_heads, KV = c->n_kv_heads, F = c->ffn_dim;
  int qw = H * hd, kw = KV * hd, group = H / KV, ctx = c->max_context;
  int rc = RGO_OK;

  float *x = (float *)malloc((size_t)S * d * 4), *nx = (float *)malloc((size_t)S * d * 4);
  float *q = (float *)malloc((size_t)S * qw * 4), *k = (float *)malloc((size_t)S * kw * 4);
  float *v = (float *)malloc((size_t)S * kw * 4), *att = (float *)malloc((size_t)S * qw * 4);
  float *proj = (float *)malloc((size_t)S * d * 4);
  float *gate = (float *)malloc((size_t)S * F * 4), *up = (float *)malloc((size_t)S * F * 4);
  float *wn = (float *)malloc((size_t)d * 4), *tmp = (float *)malloc((size_t)hd * 4);
  float *vec = (float *)malloc((size_t)qw * 4), *vec2 = (float *)malloc((size_t)qw * 4);
  const int rope_dim = c->rope_dim ? c->rope_dim : hd;

  /* embedding: src/gguf/quantization/row_gather.rs:170-181 */
  for (int s = 0; s < S && !rc; ++s)
    rc = decode_span(m->token_embd.type, m->token_embd.bytes, (size_t)tokens[s] * d, (size_t)d, x + (size_t)s * d);

  for (int l = 0; l < c->n_layers && !rc; ++l) {
    const rgo_layer *L = &m->layers[l];
    norm_weight(&L->attn_norm, wn);
    for (int s = 0; s < S; ++s) rms_norm_strict(x + (size_t)s * d, wn, d, c->norm_eps, nx + (size_t)s * d);
    if ((rc = linear(&L->attn_q, nx, S, q, mode, threads, 0))) break;
    if ((rc = linear(&L->attn_k, nx, S, k, mode, threads, 0))) break;
    if ((rc = linear(&L->attn_v, nx, S, v, mode, threads, 0))) break;
    float *K_l = cache->keys[l], *V_l = cache->values[l];
    for (int s = 0; s < S; ++s) {
      float *qs = q + (size_t)s * qw, *ks = k + (size_t)s * kw, *vs = v + (size_t)s * kw;
      deinterleave_heads(qs, H, hd, rope_dim, tmp); /* preserve_prefix: only the rotary lanes */
      deinterleave_heads(ks, KV, hd, hd, tmp);
      if (c->qkv_bias) { /* layer.rs:294-299: after the permutation, lane by lane */
        norm_weight(&L->q_bias, vec);
        for (int i = 0; i < qw; ++i) qs[i] = qs[i] + vec[i];
        norm_weight(&L->k_bias, vec);
        for (int i = 0; i < kw; ++i) ks[i] = ks[i] + vec[i];
        norm_weight(&L->v_bias, vec);
        for (int i = 0; i < kw; ++i) vs[i] = vs[i] + vec[i];
      }
      if (c->qk_norm == 2) { /* layer.rs:300-317: RMSNorm over the whole projection */
        norm_weight(&L->q_norm, vec);
        rms_norm_strict(qs, vec, qw, c->norm_eps, vec2);
        memcpy(qs, vec2, (size_t)qw * 4);
        norm_weight(&L->k_norm, vec);
        rms_norm_strict(ks, vec, kw, c->norm_eps, vec2);
        memcpy(ks, vec2, (size_t)kw * 4);
      } else if (c->qk_norm == 1) { /* layer.rs:321-331: RMSNorm inside every head */
        norm_weight(&L->q_norm, vec);
        for (int h = 0; h < H; ++h) {
          rms_norm_strict(qs + (size_t)h * hd, vec, hd, c->norm_eps, vec2);
          memcpy(qs + (size_t)h * hd, vec2, (size_t)hd * 4);
        }
        norm_weight(&L->k_norm, vec);
        for (int h = 0; h < KV; ++h) {
          rms_norm_strict(ks + (size_t)h * hd, vec, hd, c->norm_eps, vec2);
          memcpy(ks + (size_t)h * hd, vec2, (size_t)hd * 4);
        }
      }
      rope_heads(qs, H, hd, rope_dim, past + s, c->rope_theta);
      rope_heads(ks, KV, hd, rope_dim, past + s, c->rope_theta);
      /* cache append: src/models/transformer/layer.rs:348-373 */
      for (int h = 0; h < KV; ++h)
        for (int j = 0; j < hd; ++j) {
          float kk = ks[h * hd + j], vv = vs[h * hd + j];
          if (cache->kv_f16) {
            kk = round_f16(kk);
            vv = round_f16(vv);
          }
          K_l[((size_t)h * ctx + (size_t)(past + s)) * hd + j] = kk;
          V_l[((size_t)h * ctx + (size_t)(past + s)) * hd + j] = vv;
        }
    }
#pragma omp parallel num_threads(threads) if (mode == RGO_MODE_FAST && threads > 1)
    {
      float *scores = (float *)malloc((size_t)ctx * 4);
#pragma omp for collapse(2) schedule(static)
      for (int s = 0; s < S; ++s)
        for (int h = 0; h < H; ++h) {
          int kvh = h / group; /* src/ir/attention.rs:1226-1240 */
          attend_row(q + (size_t)s * qw + (size_t)h * hd, K_l + (size_t)kvh * ctx * hd, V_l + (size_t)kvh * ctx * hd,
                     hd, past + s, scores, att + (size_t)s * qw + (size_t)h * hd);
        }
      free(scores);
    }
    if ((rc = linear(&L->attn_output, att, S, proj, mode, threads, 0))) break;
    for (size_t i = 0; i < (size_t)S * d; ++i) x[i] = x[i] + proj[i];
    norm_weight(&L->ffn_norm, wn);
    for (int s = 0; s < S; ++s) rms_norm_strict(x + (size_t)s * d, wn, d, c->norm_eps, nx + (size_t)s * d);
    if ((rc = linear(&L->ffn_gate, nx, S, gate, mode, threads, 0))) break;
    if ((rc = linear(&L->ffn_up, nx, S, up, mode, threads, 0))) break;
    for (size_t i = 0; i < (size_t)S * F; ++i) gate[i] = swiglu_strict(gate[i], up[i]);
    if ((rc = linear(&L->ffn_down, gate, S, proj, mode, threads, 0))) break;
    for (size_t i = 0; i < (size_t)S * d; ++i) x[i] = x[i] + proj[i];
  }
  if (!rc) {
    norm_weight(&m->output_norm, wn);
    const rgo_tensor *head = (m->output.type >= 0) ? &m->output : &m->token_embd;
    int first = all_logits ? 0 : S - 1;
    int rows = all_logits ? S : 1;
    for (int s = first; s < S; ++s) rms_norm_strict(x + (size_t)s * d, wn, d, c->norm_eps, nx + (size_t)s * d);
    rc = linear(head, nx + (size_t)first * d, rows, logits, mode, threads, 1);
  }
  if (!rc) cache->len = past + S; /* commit only on success: model.rs:917-920 */
  free(x); free(nx); free(q); free(k); free(v); free(att); free(proj); free(gate); free(up); free(wn); free(tmp);
  free(vec); free(vec2);
  return rc;
}

/* src/models/transformer/generation.rs:260-287 */
int rgo_select_greedy(const float *row, int vocab, int32_t *token) {
  if (vocab <= 0) return RGO_ERR_NON_FINITE_LOGITS;
  int best = -1;
  float best_score = 0.0f;
  for (int t = 0; t < vocab; ++t) {
    if (!isfinite(row[t])) return RGO_ERR_NON_FINITE_LOGITS;
    if (best < 0 || row[t] > best_score) {
      best = t;
      best_score = row[t];
    }
  }
  *token = best;
  return RGO_OK;
}

/* Gumbel-max selection with an explicit uniform tape (src/models/transformer/generation.rs:10-19,
 * 260-287): score = logit / max(T, 1e-12) - ln(-ln(max(u, 1e-12))), every step in f32; strict '>'
 * keeps the lowest id among equal scores; only the logits are checked for finiteness. */
int rgo_select_gumbel(const float *row, int vocab, float temperature, const float *uniforms, int32_t *token) {
  if (vocab <= 0 || !uniforms) return RGO_ERR_NON_FINITE_LOGITS;
  int best = -1;
  float best_score = 0.0f;
  const float t = fmaxf(temperature, 1e-12f);
  for (int i = 0; i < vocab; ++i) {
    if (!isfinite(row[i])) return RGO_ERR_NON_FINITE_LOGITS;
    const float u = fmaxf(uniforms[i], 1e-12f);
    const float score = row[i] / t - logf(-logf(u));
    if (best < 0 || score > best_score) {
      best = i;
      best_score = score;
    }
  }
  *token = best;
  return RGO_OK;
}

/* src/models/transformer/generation.rs:106-160: prefill the whole prompt, then one-token steps;
 * the last generated token is not fed back; stop on EOS/EOT. */
int rgo_generate_greedy(const rgo_model *m, rgo_cache *cache, const int32_t *prompt, int n_prompt, int max_new,
                        int mode, int threads, int32_t *out, int *n_out, int *stopped) {
  const rgo_config *c = &m->cfg;
  *n_out = 0;
  *stopped = 0;
  if (n_prompt <= 0) return RGO_ERR_ARG;
  if (n_prompt + max_new > c->max_context) return RGO_ERR_CONTEXT;
  for (int i = 0; i < n_prompt; ++i)
    if (prompt[i] < 0 || prompt[i] >= c->vocab) return RGO_ERR_TOKEN_RANGE;
  if (max_new == 0) return RGO_OK;
  float *logits = (float *)malloc((size_t)c->vocab * 4);
  rgo_cache_clear(cache);
  int rc = rgo_forward(m, cache, prompt, n_prompt, mode, threads, 0, logits);
  for (int step = 0; step < max_new && !rc; ++step) {
    int32_t token;
    if ((rc = rgo_select_greedy(logits, c->vocab, &token))) break;
    out[(*n_out)++] = token;
    if (token == c->eos_id || token == c->eot_id) {
      *stopped = 1;
      break;
    }
    if (step + 1 < max_new) rc = rgo_forward(m, cache, &token, 1, mode, threads, 0, logits);
  }
  free(logits);
  return rc;
}

/* ------------------------------------------------------------------ independent f64 forward */

static void dequant_row_f64(const rgo_tensor *w, size_t n, double *row, float *tmp) {
  decode_span(w->type, w->bytes, n * w->cols, w->cols, tmp);
  for (size_t i = 0; i < w->cols; ++i) row[i] = (double)tmp[i];
}

static void linear_f64(const rgo_tensor *w, const double *x, int S, double *y) {
  size_t N = w->rows, K = w->cols;
  double *row = (double *)malloc(K * 8);
  float *tmp = (float *)malloc(K * 4);
  for (size_t n = 0; n < N; ++n) {
    dequant_row_f64(w, n, row, tmp);
    for (int s = 0; s < S; ++s) {
      double acc = 0;
      for (size_t k = 0; k < K; ++k) acc += x[(size_t)s * K + k] * row[k];
      y[(size_t)s * N + n] = acc;
    }
  }
  free(row);
  free(tmp);
}

static void rms_f64(const double *x, const rgo_tensor *w, int d, double eps, double *y, float *tmp) {
  decode_span(w->type, w->bytes, 0, (size_t)d, tmp);
  double ss = 0;
  for (int i = 0; i < d; ++i) ss += x[i] * x[i];
  double inv = 1.0 / sqrt(ss / d + eps);
  for (int i = 0; i < d; ++i) y[i] = x[i] * inv * (double)tmp[i];
}

/* Textbook Llama forward in double precision (standard exp-based softmax and sigmoid, the
 * rotary pairing of llama GGUF files written directly on interleaved lanes), structured like the
 * in-test oracle of src/models/transformer/model_tests.rs:827-1083. */
int rgo_forward_f64(const rgo_model *m, const int32_t *tokens, int S, double *logits) {
  const rgo_config *c = &m->cfg;
  if (rgo_model_check(m) || S <= 0 || S > c->max_context) return RGO_ERR_ARG;
  int d = c->d_model, hd = c->head_dim, H = c->n_heads, KV = c->n_kv_heads, F = c->ffn_dim;
  int qw = H * hd, kw = KV * hd, group = H / KV, half = hd / 2;
  const int rope_dim = c->rope_dim ? c->rope_dim : hd;
  const int variant = rope_dim != hd || c->qk_norm || c->qkv_bias;
  double *x = (double *)malloc((size_t)S * d * 8), *nx = (double *)malloc((size_t)S * d * 8);
  double *q = (double *)malloc((size_t)S * qw * 8), *k = (double *)malloc((size_t)S * kw * 8);
  double *v = (double *)malloc((size_t)S * kw * 8), *att = (double *)malloc((size_t)S * qw * 8);
  double *proj = (double *)malloc((size_t)S * d * 8), *gate = (double *)malloc((size_t)S * F * 8);
  double *up = (double *)malloc((size_t)S * F * 8), *sc = (double *)malloc((size_t)S * 8);
  size_t tmpn = (size_t)(d > F ? d : F);
  if ((size_t)qw > tmpn) tmpn = (size_t)qw;
  float *tmp = (float *)malloc(tmpn * 4);
  for (int s = 0; s < S; ++s) {
    if (tokens[s] < 0 || tokens[s] >= c->vocab) return RGO_ERR_TOKEN_RANGE;
    decode_span(m->token_embd.type, m->token_embd.bytes, (size_t)tokens[s] * d, (size_t)d, tmp);
    for (int i = 0; i < d; ++i) x[(size_t)s * d + i] = tmp[i];
  }
  for (int l = 0; l < c->n_layers; ++l) {
    const rgo_layer *L = &m->layers[l];
    for (int s = 0; s < S; ++s) rms_f64(x + (size_t)s * d, &L->attn_norm, d, c->norm_eps, nx + (size_t)s * d, tmp);
    linear_f64(&L->attn_q, nx, S, q);
    linear_f64(&L->attn_k, nx, S, k);
    linear_f64(&L->attn_v, nx, S, v);
    if (variant) {
      /* the variants in double precision, written from the definitions: lane permutation of the
       * rotary part, bias, RMS normalisation of q and k, rotation of the first rope_dim lanes */
      double *pd = (double *)malloc((size_t)hd * 8);
      for (int s = 0; s < S; ++s) {
        for (int h = 0; h < H + KV; ++h) {
          double *p = (h < H) ? q + (size_t)s * qw + (size_t)h * hd : k + (size_t)s * kw + (size_t)(h - H) * hd;
          int permuted = (h < H) ? rope_dim : hd, prefix = hd - permuted;
          for (int j = 0; j < permuted / 2; ++j) {
            pd[j] = p[prefix + 2 * j];
            pd[permuted / 2 + j] = p[prefix + 2 * j + 1];
          }
          for (int j = 0; j < permuted; ++j) p[prefix + j] = pd[j];
        }
        if (c->qkv_bias) {
          decode_span(L->q_bias.type, L->q_bias.bytes, 0, (size_t)qw, tmp);
          for (int i = 0; i < qw; ++i) q[(size_t)s * qw + i] += tmp[i];
          decode_span(L->k_bias.type, L->k_bias.bytes, 0, (size_t)kw, tmp);
          for (int i = 0; i < kw; ++i) k[(size_t)s * kw + i] += tmp[i];
          decode_span(L->v_bias.type, L->v_bias.bytes, 0, (size_t)kw, tmp);
          for (int i = 0; i < kw; ++i) v[(size_t)s * kw + i] += tmp[i];
        }
        if (c->qk_norm == 2) {
          rms_f64(q + (size_t)s * qw, &L->q_norm, qw, c->norm_eps, q + (size_t)s * qw, tmp);
          rms_f64(k + (size_t)s * kw, &L->k_norm, kw, c->norm_eps, k + (size_t)s * kw, tmp);
        } else if (c->qk_norm == 1) {
          for (int h = 0; h < H; ++h) rms_f64(q + (size_t)s * qw + (size_t)h * hd, &L->q_norm, hd, c->norm_eps, q + (size_t)s * qw + (size_t)h * hd, tmp);
          for (int h = 0; h < KV; ++h) rms_f64(k + (size_t)s * kw + (size_t)h * hd, &L->k_norm, hd, c->norm_eps, k + (size_t)s * kw + (size_t)h * hd, tmp);
        }
        for (int i = 0; i < rope_dim / 2; ++i) {
          double ang = (double)s / pow(c->rope_theta, (double)(2 * i) / rope_dim);
          double cs = cos(ang), sn = sin(ang);
          for (int h = 0; h < H + KV; ++h) {
            double *p = (h < H) ? q + (size_t)s * qw + (size_t)h * hd : k + (size_t)s * kw + (size_t)(h - H) * hd;
            double a = p[i], b = p[rope_dim / 2 + i];
            p[i] = a * cs - b * sn;
            p[rope_dim / 2 + i] = b * cs + a * sn;
          }
        }
      }
      free(pd);
    } else
    /* rotate adjacent lane pairs (2i, 2i+1) in place: equivalent to de-interleave + split-half */
    for (int s = 0; s < S; ++s)
      for (int i = 0; i < half; ++i) {
        double ang = (double)s / pow(c->rope_theta, (double)(2 * i) / hd);
        double cs = cos(ang), sn = sin(ang);
        for (int h = 0; h < H + KV; ++h) {
          double *p = (h < H) ? q + (size_t)s * qw + (size_t)h * hd : k + (size_t)s * kw + (size_t)(h - H) * hd;
          double a = p[2 * i], b = p[2 * i + 1];
          p[2 * i] = a * cs - b * sn;
          p[2 * i + 1] = b * cs + a * sn;
        }
      }
    for (int s = 0; s < S; ++s)
      for (int h = 0; h < H; ++h) {
        const double *qs = q + (size_t)s * qw + (size_t)h * hd;
        int kvh = h / group;
        double mx = -INFINITY;
        for (int t = 0; t <= s; ++t) {
          const double *kt = k + (size_t)t * kw + (size_t)kvh * hd;
          double a = 0;
          for (int j = 0; j < hd; ++j) a += qs[j] * kt[j];
          sc[t] = a / sqrt((double)hd);
          if (sc[t] > mx) mx = sc[t];
        }
        double sum = 0;
        for (int t = 0; t <= s; ++t) {
          sc[t] = exp(sc[t] - mx);
          sum += sc[t];
        }
        double *o = att + (size_t)s * qw + (size_t)h * hd;
        for (int j = 0; j < hd; ++j) {
          double a = 0;
          for (int t = 0; t <= s; ++t) a += sc[t] / sum * v[(size_t)t * kw + (size_t)kvh * hd + j];
          o[j] = a;
        }
      }
    /* the attention output of the pair-rotated q/k equals that of the de-interleaved layout:
     * the dot product q.k is invariant under the same lane permutation of both operands */
    linear_f64(&L->attn_output, att, S, proj);
    for (size_t i = 0; i < (size_t)S * d; ++i) x[i] += proj[i];
    for (int s = 0; s < S; ++s) rms_f64(x + (size_t)s * d, &L->ffn_norm, d, c->norm_eps, nx + (size_t)s * d, tmp);
    linear_f64(&L->ffn_gate, nx, S, gate);
    linear_f64(&L->ffn_up, nx, S, up);
    for (size_t i = 0; i < (size_t)S * F; ++i) gate[i] = gate[i] / (1.0 + exp(-gate[i])) * up[i];
    linear_f64(&L->ffn_down, gate, S, proj);
    for (size_t i = 0; i < (size_t)S * d; ++i) x[i] += proj[i];
  }
  for (int s = 0; s < S; ++s) rms_f64(x + (size_t)s * d, &m->output_norm, d, c->norm_eps, nx + (size_t)s * d, tmp);
  linear_f64((m->output.type >= 0) ? &m->output : &m->token_embd, nx, S, logits);
  free(x); free(nx); free(q); free(k); free(v); free(att); free(proj); free(gate); free(up); free(sc); free(tmp);
  return RGO_OK;
}
