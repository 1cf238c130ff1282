/*
 * CPU oracle: plain-C restatement of the OrionServe-RS reference CPU forward
 * pass. TEST INFRASTRUCTURE ONLY (see orion_oracle.h). Operation order follows
 * the cited reference lines exactly: sequential f32 dot products, f64 sum of
 * squares in RMSNorm, per-element division in softmax, no FMA contraction.
 */
#include "orion_oracle.h"

#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>

static __thread char g_err[512];
static int g_threads = 1;

static int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
  return code;
}

const char *oracle_last_error(void) { return g_err; }

void oracle_set_threads(int n) { g_threads = n < 1 ? 1 : n; }
int oracle_get_threads(void) { return g_threads; }

/* ------------------------------------------------------------------ */
/* tensor.rs                                                            */
/* ------------------------------------------------------------------ */

/* Shared body of `linear` (tensor.rs:114-128) generalised to sub-ranges so the
 * tensor-parallel restatement can reuse the same inner loop: output features
 * [j0, j1) of a weight whose rows are `w_stride` long, reading input columns
 * [c0, c0+k) of each weight row. With j0=0, j1=out_features, c0=0, k=w_stride
 * this is exactly the reference loop. */
typedef struct {
  const float *x, *w, *bias;
  float *out;
  size_t k, x_stride, w_stride, c0, j0, nj, out_stride;
  size_t begin, end; /* range of flattened (row, feature) indices */
} LinearJob;

static void *linear_worker(void *arg) {
  const LinearJob *job = (const LinearJob *)arg;
  for (size_t idx = job->begin; idx < job->end; ++idx) {
    const size_t i = idx / job->nj;
    const size_t jj = idx % job->nj;
    const size_t j = job->j0 + jj;
    const float *xr = job->x + i * job->x_stride;
    const float *wr = job->w + j * job->w_stride + job->c0;
    float acc = 0.0f; /* tensor.rs:122-125: plain sequential dot, k ascending */
    for (size_t t = 0; t < job->k; ++t) acc += xr[t] * wr[t];
    job->out[i * job->out_stride + jj] = acc + (job->bias ? job->bias[j] : 0.0f); /* :126 */
  }
  return NULL;
}

static void linear_core(const float *x, size_t n, size_t k, size_t x_stride, const float *w,
                        size_t w_stride, size_t c0, size_t j0, size_t j1, const float *bias,
                        float *out, size_t out_stride) {
  const size_t nj = j1 - j0;
  const size_t total = n * nj;
  LinearJob base = {x, w, bias, out, k, x_stride, w_stride, c0, j0, nj, out_stride, 0, total};
  size_t nt = (size_t)g_threads;
  if (nt > 64) nt = 64;
  if (nt <= 1 || total * k < (1u << 16)) {
    linear_worker(&base);
    return;
  }
  if (nt > total) nt = total;
  LinearJob jobs[64];
  pthread_t tid[64];
  int started[64];
  for (size_t t = 0; t < nt; ++t) {
    jobs[t] = base;
    jobs[t].begin = total * t / nt;
    jobs[t].end = total * (t + 1) / nt;
    started[t] = (t + 1 < nt) && pthread_create(&tid[t], NULL, linear_worker, &jobs[t]) == 0;
  }
  for (size_t t = 0; t < nt; ++t)
    if (!started[t]) linear_worker(&jobs[t]); /* last slice, or a thread that failed to start */
  for (size_t t = 0; t < nt; ++t)
    if (started[t]) pthread_join(tid[t], NULL);
}

int oracle_linear(const float *x, size_t n, size_t k, const float *w, size_t out_features,
                  size_t in_features, const float *bias, size_t bias_len, float *out) {
  if (k != in_features) /* tensor.rs:100-104 */
    return fail(ORACLE_ERR_INTERNAL,
                "linear shape mismatch: input has %zu features, weight expects %zu", k,
                in_features);
  if (bias && bias_len != out_features) /* tensor.rs:105-112 */
    return fail(ORACLE_ERR_INTERNAL, "bias has %zu elements, expected %zu", bias_len,
                out_features);
  linear_core(x, n, k, k, w, in_features, 0, 0, out_features, bias, out, out_features);
  return ORACLE_OK;
}

int oracle_rms_norm(float *x, size_t rows, size_t cols, const float *weight, size_t weight_len,
                    float eps) {
  if (weight_len != cols) /* tensor.rs:145-150 */
    return fail(ORACLE_ERR_INTERNAL, "rms_norm weight has %zu elements, expected %zu",
                weight_len, cols);
  for (size_t r = 0; r < rows; ++r) {
    float *row = x + r * cols;
    double sum_sq = 0.0; /* tensor.rs:155 */
    for (size_t c = 0; c < cols; ++c) sum_sq += (double)row[c] * (double)row[c];
    const double rms = sqrt(sum_sq / (double)cols + (double)eps); /* :156 */
    const float scale = (float)(1.0 / rms);                        /* :157 */
    for (size_t c = 0; c < cols; ++c) row[c] = row[c] * scale * weight[c]; /* :159 */
  }
  return ORACLE_OK;
}

float oracle_silu(float x) { return x / (1.0f + expf(-x)); } /* tensor.rs:167-169 */

int oracle_swiglu(float *gate, size_t gate_rows, size_t gate_cols, const float *up,
                  size_t up_rows, size_t up_cols) {
  if (gate_rows != up_rows || gate_cols != up_cols) /* tensor.rs:176-184 */
    return fail(ORACLE_ERR_INTERNAL, "swiglu shape mismatch: gate is %zux%zu, up is %zux%zu",
                gate_rows, gate_cols, up_rows, up_cols);
  const size_t n = gate_rows * gate_cols;
  for (size_t i = 0; i < n; ++i) gate[i] = oracle_silu(gate[i]) * up[i]; /* :185-187 */
  return ORACLE_OK;
}

void oracle_softmax_inplace(float *x, size_t n) {
  /* tensor.rs:193  fold(NEG_INFINITY, f32::max); f32::max ignores NaN like fmaxf. */
  float max = -INFINITY;
  for (size_t i = 0; i < n; ++i) max = fmaxf(max, x[i]);
  if (!isfinite(max)) { /* :194-198 */
    const float uniform = 1.0f / (float)n;
    for (size_t i = 0; i < n; ++i) x[i] = uniform;
    return;
  }
  float sum = 0.0f;
  for (size_t i = 0; i < n; ++i) { /* :199-203 */
    x[i] = expf(x[i] - max);
    sum += x[i];
  }
  if (sum > 0.0f) /* :204-208 */
    for (size_t i = 0; i < n; ++i) x[i] /= sum;
}

int oracle_rope_table(size_t head_dim, size_t max_positions, float theta, float *cos_out,
                      float *sin_out) {
  if (head_dim % 2 != 0) /* tensor.rs:229-233 */
    return fail(ORACLE_ERR_INTERNAL, "RoPE requires an even head_dim, got %zu", head_dim);
  const size_t half = head_dim / 2;
  for (size_t pos = 0; pos < max_positions; ++pos) {
    for (size_t i = 0; i < half; ++i) {
      /* :241  1.0 / theta.powf(2.0 * i as f32 / head_dim as f32) */
      const float inv_freq = 1.0f / powf(theta, 2.0f * (float)i / (float)head_dim);
      const float angle = (float)pos * inv_freq; /* :242 */
      cos_out[pos * half + i] = cosf(angle);
      sin_out[pos * half + i] = sinf(angle);
    }
  }
  return ORACLE_OK;
}

int oracle_apply_rope(float *vec, size_t len, const float *cos_row, const float *sin_row,
                      size_t table_width) {
  const size_t half = len / 2;
  if (table_width != half) /* tensor.rs:285-290 */
    return fail(ORACLE_ERR_INTERNAL, "RoPE table width %zu does not match half of head_dim %zu",
                table_width, half);
  for (size_t i = 0; i < half; ++i) { /* :291-296 */
    const float x0 = vec[i];
    const float x1 = vec[i + half];
    vec[i] = x0 * cos_row[i] - x1 * sin_row[i];
    vec[i + half] = x0 * sin_row[i] + x1 * cos_row[i];
  }
  return ORACLE_OK;
}

/* ------------------------------------------------------------------ */
/* attention.rs                                                         */
/* ------------------------------------------------------------------ */

struct OracleKvStore {
  float *data;
  size_t len;
  size_t num_layers, num_blocks, block_size, num_kv_heads, head_dim;
};

OracleKvStore *oracle_kv_new(size_t num_layers, size_t num_blocks, size_t block_size,
                             size_t num_kv_heads, size_t head_dim) {
  OracleKvStore *s = (OracleKvStore *)calloc(1, sizeof *s);
  if (!s) return NULL;
  s->len = num_layers * num_blocks * 2 * block_size * num_kv_heads * head_dim; /* :53 */
  s->data = (float *)calloc(s->len ? s->len : 1, sizeof(float));               /* :55 zeroed */
  if (!s->data) {
    free(s);
    return NULL;
  }
  s->num_layers = num_layers;
  s->num_blocks = num_blocks;
  s->block_size = block_size;
  s->num_kv_heads = num_kv_heads;
  s->head_dim = head_dim;
  return s;
}

void oracle_kv_free(OracleKvStore *s) {
  if (!s) return;
  free(s->data);
  free(s);
}

size_t oracle_kv_len(const OracleKvStore *s) { return s->len; }
float *oracle_kv_data(OracleKvStore *s) { return s->data; }

/* attention.rs:82-104 */
static size_t kv_slot_offset(const OracleKvStore *s, size_t layer, uint32_t block, int is_value,
                             size_t slot, size_t head) {
  const size_t block_stride = s->block_size * s->num_kv_heads * s->head_dim;
  const size_t per_block = 2 * block_stride;
  const size_t per_layer = s->num_blocks * per_block;
  const size_t region = layer * per_layer + (size_t)block * per_block +
                        (is_value ? block_stride : 0);
  return region + (slot * s->num_kv_heads + head) * s->head_dim;
}

/* attention.rs:136-175 */
static int kv_check(const OracleKvStore *s, size_t layer, uint32_t block, size_t slot,
                    size_t head, size_t vec_len) {
  if (layer >= s->num_layers)
    return fail(ORACLE_ERR_INTERNAL, "layer %zu out of range (have %zu)", layer, s->num_layers);
  if ((size_t)block >= s->num_blocks)
    return fail(ORACLE_ERR_INTERNAL, "block %u out of range (have %zu)", block, s->num_blocks);
  if (slot >= s->block_size)
    return fail(ORACLE_ERR_INTERNAL, "slot %zu out of range (block holds %zu)", slot,
                s->block_size);
  if (head >= s->num_kv_heads)
    return fail(ORACLE_ERR_INTERNAL, "kv head %zu out of range (have %zu)", head,
                s->num_kv_heads);
  if (vec_len != s->head_dim)
    return fail(ORACLE_ERR_INTERNAL, "vector length %zu does not match head_dim %zu", vec_len,
                s->head_dim);
  return ORACLE_OK;
}

int oracle_kv_write(OracleKvStore *s, size_t layer, uint32_t block, size_t slot, size_t head,
                    int is_value, const float *vec, size_t vec_len) {
  int rc = kv_check(s, layer, block, slot, head, vec_len);
  if (rc) return rc;
  memcpy(s->data + kv_slot_offset(s, layer, block, is_value, slot, head), vec,
         s->head_dim * sizeof(float));
  return ORACLE_OK;
}

int oracle_kv_read(const OracleKvStore *s, size_t layer, uint32_t block, size_t slot,
                   size_t head, int is_value, float *out) {
  int rc = kv_check(s, layer, block, slot, head, s->head_dim);
  if (rc) return rc;
  memcpy(out, s->data + kv_slot_offset(s, layer, block, is_value, slot, head),
         s->head_dim * sizeof(float));
  return ORACLE_OK;
}

int oracle_locate(const uint32_t *table, size_t table_len, size_t position, size_t block_size,
                  uint32_t *block, size_t *slot) {
  const size_t logical = position / block_size; /* attention.rs:183 */
  if (logical >= table_len) return 0;           /* :185 */
  *block = table[logical];
  *slot = position % block_size; /* :184 */
  return 1;
}

/* attention.rs:250-293 over query heads [qh0, qh1); the public entry point
 * passes the full range. `query` and `out` are indexed by (qh - qh0). */
static int attention_heads(const OracleKvStore *s, const float *query, const uint32_t *table,
                           size_t table_len, size_t query_position, size_t layer, size_t qh0,
                           size_t qh1, size_t group_size, size_t head_dim, size_t block_size,
                           float *out, float *scores) {
  const float scale = 1.0f / sqrtf((float)head_dim); /* :251 */
  const size_t attend_len = query_position + 1;      /* :253 */
  for (size_t qh = qh0; qh < qh1; ++qh) {
    const size_t kv_head = qh / group_size; /* :258 */
    const float *q = query + (qh - qh0) * head_dim;
    for (size_t pos = 0; pos < attend_len; ++pos) { /* :262-275 */
      uint32_t block;
      size_t slot;
      if (!oracle_locate(table, table_len, pos, block_size, &block, &slot))
        return fail(ORACLE_ERR_INTERNAL,
                    "position %zu is outside the block table of %zu blocks", pos, table_len);
      int rc = kv_check(s, layer, block, slot, kv_head, head_dim);
      if (rc) return rc;
      const float *k = s->data + kv_slot_offset(s, layer, block, 0, slot, kv_head);
      float dot = 0.0f;
      for (size_t d = 0; d < head_dim; ++d) dot += q[d] * k[d];
      scores[pos] = dot * scale;
    }
    oracle_softmax_inplace(scores, attend_len); /* :277 */
    float *o = out + (qh - qh0) * head_dim;
    for (size_t d = 0; d < head_dim; ++d) o[d] = 0.0f; /* :281 */
    for (size_t pos = 0; pos < attend_len; ++pos) {    /* :282-292 */
      const float w = scores[pos];
      if (w == 0.0f) continue;
      uint32_t block;
      size_t slot;
      if (!oracle_locate(table, table_len, pos, block_size, &block, &slot))
        return fail(ORACLE_ERR_INTERNAL, "position %zu unmapped", pos);
      int rc = kv_check(s, layer, block, slot, kv_head, head_dim);
      if (rc) return rc;
      const float *v = s->data + kv_slot_offset(s, layer, block, 1, slot, kv_head);
      for (size_t d = 0; d < head_dim; ++d) o[d] += w * v[d];
    }
  }
  return ORACLE_OK;
}

int oracle_paged_attention(const OracleKvStore *s, const float *query, size_t query_len,
                           const uint32_t *table, size_t table_len, size_t query_position,
                           size_t layer, size_t num_query_heads, size_t num_kv_heads,
                           size_t head_dim, size_t block_size, float *out, size_t out_len) {
  if (query_len != num_query_heads * head_dim || out_len != query_len) /* :236-243 */
    return fail(ORACLE_ERR_INTERNAL, "attention expected %zu query elements, got %zu (out %zu)",
                num_query_heads * head_dim, query_len, out_len);
  if (num_kv_heads == 0 || num_query_heads % num_kv_heads != 0) /* :244-248 */
    return fail(ORACLE_ERR_INTERNAL, "%zu query heads cannot be grouped over %zu kv heads",
                num_query_heads, num_kv_heads);
  float *scores = (float *)malloc((query_position + 1) * sizeof(float)); /* :255 */
  if (!scores) return fail(ORACLE_ERR_ARG, "out of memory");
  int rc = attention_heads(s, query, table, table_len, query_position, layer, 0,
                           num_query_heads, num_query_heads / num_kv_heads, head_dim,
                           block_size, out, scores);
  free(scores);
  return rc;
}

/* ------------------------------------------------------------------ */
/* sampling.rs:196-206                                                  */
/* ------------------------------------------------------------------ */

int64_t oracle_argmax(const float *logits, size_t n) {
  int64_t best = -1;
  float best_val = -INFINITY;
  for (size_t i = 0; i < n; ++i) {
    if (logits[i] > best_val) { /* strict: ties keep the lowest index; NaN never wins */
      best_val = logits[i];
      best = (int64_t)i;
    }
  }
  return best;
}

/* ------------------------------------------------------------------ */
/* loader.rs:74-96  (half crate's exact widening)                       */
/* ------------------------------------------------------------------ */

void oracle_bf16_to_f32(const uint16_t *src, size_t n, float *dst) {
  for (size_t i = 0; i < n; ++i) {
    uint32_t bits = (uint32_t)src[i] << 16;
    memcpy(dst + i, &bits, 4);
  }
}

void oracle_f16_to_f32(const uint16_t *src, size_t n, float *dst) {
  for (size_t i = 0; i < n; ++i) {
    const uint32_t h = src[i];
    const uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
      if (man == 0) {
        bits = sign;
      } else { /* subnormal: renormalise */
        int e = -1;
        do {
          ++e;
          man <<= 1;
        } while ((man & 0x400u) == 0);
        man &= 0x3ffu;
        bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
      }
    } else if (exp == 0x1f) {
      bits = sign | 0x7f800000u | (man << 13);
    } else {
      bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    memcpy(dst + i, &bits, 4);
  }
}

void oracle_f32_to_bf16(const float *src, size_t n, uint16_t *dst) {
  for (size_t i = 0; i < n; ++i) {
    uint32_t bits;
    memcpy(&bits, src + i, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) { /* NaN: keep quiet */
      dst[i] = (uint16_t)((bits >> 16) | 0x0040u);
      continue;
    }
    const uint32_t lsb = (bits >> 16) & 1u;
    bits += 0x7fffu + lsb;
    dst[i] = (uint16_t)(bits >> 16);
  }
}

/* ------------------------------------------------------------------ */
/* transformer.rs                                                       */
/* ------------------------------------------------------------------ */

typedef struct {
  float *input_norm, *q_proj, *k_proj, *v_proj, *o_proj;
  float *q_bias, *k_bias, *v_bias; /* NULL when absent */
  float *post_attn_norm, *gate_proj, *up_proj, *down_proj;
} OracleLayer;

struct OracleModel {
  OracleModelDesc d;
  float *embed_tokens;
  float *final_norm;
  float *lm_head; /* NULL when tied */
  OracleLayer *layers;
  float *rope_cos, *rope_sin;
  OracleKvStore *kv;
};

OracleModel *oracle_model_new(const OracleModelDesc *desc) {
  OracleModel *m = (OracleModel *)calloc(1, sizeof *m);
  if (!m) return NULL;
  m->d = *desc;
  m->layers = (OracleLayer *)calloc(desc->num_layers ? desc->num_layers : 1, sizeof(OracleLayer));
  const size_t half = desc->head_dim / 2;
  const size_t tbl = (size_t)desc->max_position_embeddings * half;
  m->rope_cos = (float *)malloc((tbl ? tbl : 1) * sizeof(float));
  m->rope_sin = (float *)malloc((tbl ? tbl : 1) * sizeof(float));
  m->kv = oracle_kv_new(desc->num_layers, desc->num_blocks, desc->block_size,
                        desc->num_kv_heads, desc->head_dim);
  if (!m->layers || !m->rope_cos || !m->rope_sin || !m->kv ||
      oracle_rope_table(desc->head_dim, desc->max_position_embeddings, desc->rope_theta,
                        m->rope_cos, m->rope_sin) != ORACLE_OK) {
    oracle_model_free(m);
    return NULL;
  }
  return m;
}

void oracle_model_free(OracleModel *m) {
  if (!m) return;
  if (m->layers) {
    for (uint32_t i = 0; i < m->d.num_layers; ++i) {
      OracleLayer *l = &m->layers[i];
      free(l->input_norm), free(l->q_proj), free(l->k_proj), free(l->v_proj), free(l->o_proj);
      free(l->q_bias), free(l->k_bias), free(l->v_bias);
      free(l->post_attn_norm), free(l->gate_proj), free(l->up_proj), free(l->down_proj);
    }
    free(m->layers);
  }
  free(m->embed_tokens), free(m->final_norm), free(m->lm_head);
  free(m->rope_cos), free(m->rope_sin);
  oracle_kv_free(m->kv);
  free(m);
}

OracleKvStore *oracle_model_kv(OracleModel *m) { return m->kv; }

static int store_tensor(float **slot, const float *data, size_t len, size_t expect,
                        const char *name) {
  if (len != expect)
    return fail(ORACLE_ERR_ARG, "tensor `%s` has %zu elements, expected %zu", name, len, expect);
  free(*slot);
  *slot = (float *)malloc((len ? len : 1) * sizeof(float));
  if (!*slot) return fail(ORACLE_ERR_ARG, "out of memory for `%s`", name);
  memcpy(*slot, data, len * sizeof(float));
  return ORACLE_OK;
}

int oracle_model_set_tensor(OracleModel *m, const char *name, const float *data, size_t len) {
  const OracleModelDesc *d = &m->d;
  const size_t H = d->hidden_size, F = d->ffn_dim, V = d->vocab_size;
  const size_t qd = (size_t)d->num_attention_heads * d->head_dim;
  const size_t kvd = (size_t)d->num_kv_heads * d->head_dim;
  if (!strcmp(name, "model.embed_tokens.weight"))
    return store_tensor(&m->embed_tokens, data, len, V * H, name);
  if (!strcmp(name, "model.norm.weight")) return store_tensor(&m->final_norm, data, len, H, name);
  if (!strcmp(name, "lm_head.weight")) {
    if (d->tied_lm_head) return ORACLE_OK; /* transformer.rs:108-110: ignored when tied */
    return store_tensor(&m->lm_head, data, len, V * H, name);
  }
  unsigned layer = 0;
  char rest[96];
  if (sscanf(name, "model.layers.%u.%95s", &layer, rest) == 2 && layer < d->num_layers) {
    OracleLayer *l = &m->layers[layer];
    if (!strcmp(rest, "input_layernorm.weight"))
      return store_tensor(&l->input_norm, data, len, H, name);
    if (!strcmp(rest, "post_attention_layernorm.weight"))
      return store_tensor(&l->post_attn_norm, data, len, H, name);
    if (!strcmp(rest, "self_attn.q_proj.weight"))
      return store_tensor(&l->q_proj, data, len, qd * H, name);
    if (!strcmp(rest, "self_attn.k_proj.weight"))
      return store_tensor(&l->k_proj, data, len, kvd * H, name);
    if (!strcmp(rest, "self_attn.v_proj.weight"))
      return store_tensor(&l->v_proj, data, len, kvd * H, name);
    if (!strcmp(rest, "self_attn.o_proj.weight"))
      return store_tensor(&l->o_proj, data, len, H * qd, name);
    if (!strcmp(rest, "mlp.gate_proj.weight"))
      return store_tensor(&l->gate_proj, data, len, F * H, name);
    if (!strcmp(rest, "mlp.up_proj.weight"))
      return store_tensor(&l->up_proj, data, len, F * H, name);
    if (!strcmp(rest, "mlp.down_proj.weight"))
      return store_tensor(&l->down_proj, data, len, H * F, name);
    if (d->has_qkv_bias) { /* transformer.rs:78-86 */
      if (!strcmp(rest, "self_attn.q_proj.bias"))
        return store_tensor(&l->q_bias, data, len, qd, name);
      if (!strcmp(rest, "self_attn.k_proj.bias"))
        return store_tensor(&l->k_bias, data, len, kvd, name);
      if (!strcmp(rest, "self_attn.v_proj.bias"))
        return store_tensor(&l->v_bias, data, len, kvd, name);
    } else if (strstr(rest, "_proj.bias")) {
      return ORACLE_OK; /* Llama ignores biases (transformer.rs:84-86) */
    }
  }
  return fail(ORACLE_ERR_ARG, "unknown tensor name `%s`", name);
}

static int model_complete(const OracleModel *m) {
  if (!m->embed_tokens || !m->final_norm) return 0;
  if (!m->d.tied_lm_head && !m->lm_head) return 0;
  for (uint32_t i = 0; i < m->d.num_layers; ++i) {
    const OracleLayer *l = &m->layers[i];
    if (!l->input_norm || !l->q_proj || !l->k_proj || !l->v_proj || !l->o_proj ||
        !l->post_attn_norm || !l->gate_proj || !l->up_proj || !l->down_proj)
      return 0;
  }
  return 1;
}

typedef struct {
  size_t q0, q1;   /* query heads owned */
  size_t kv0, kv1; /* kv heads owned */
  size_t f0, f1;   /* ffn slice owned */
  oracle_allreduce_fn allreduce;
  void *ctx;
} Shards;

/* transformer.rs:230-347. With the full shard ranges and no all-reduce this is
 * the reference layer; with a rank's ranges it is the Megatron layout of
 * orion-distributed/src/lib.rs:14-49. */
static int layer_forward(OracleModel *m, size_t layer_idx, float *hidden, size_t n,
                         const uint32_t *positions, const uint32_t *slot_block,
                         const size_t *slot_slot, const size_t *seq_of_row,
                         const uint32_t *tables_flat, const uint64_t *table_offsets,
                         const Shards *sh) {
  const OracleModelDesc *d = &m->d;
  const OracleLayer *w = &m->layers[layer_idx];
  const size_t H = d->hidden_size, hd = d->head_dim, F = d->ffn_dim;
  const size_t Hq = d->num_attention_heads, Hkv = d->num_kv_heads;
  const size_t lq = sh->q1 - sh->q0, lkv = sh->kv1 - sh->kv0, lf = sh->f1 - sh->f0;
  const size_t half = hd / 2;
  int rc = ORACLE_OK;

  float *normed = (float *)malloc(n * H * sizeof(float));
  float *q = (float *)malloc(n * lq * hd * sizeof(float));
  float *k = (float *)malloc(n * lkv * hd * sizeof(float));
  float *v = (float *)malloc(n * lkv * hd * sizeof(float));
  float *attn = (float *)calloc(n * lq * hd, sizeof(float));
  float *proj = (float *)malloc(n * H * sizeof(float));
  float *gate = (float *)malloc(n * lf * sizeof(float));
  float *up = (float *)malloc(n * lf * sizeof(float));
  float *scores = (float *)malloc(((size_t)d->max_position_embeddings + 1) * sizeof(float));
  if (!normed || !q || !k || !v || !attn || !proj || !gate || !up || !scores) {
    rc = fail(ORACLE_ERR_ARG, "out of memory in layer_forward");
    goto done;
  }

  /* :245-250 */
  memcpy(normed, hidden, n * H * sizeof(float));
  rc = oracle_rms_norm(normed, n, H, w->input_norm, H, d->rms_norm_eps);
  if (rc) goto done;
  linear_core(normed, n, H, H, w->q_proj, H, 0, sh->q0 * hd, sh->q1 * hd, w->q_bias, q, lq * hd);
  linear_core(normed, n, H, H, w->k_proj, H, 0, sh->kv0 * hd, sh->kv1 * hd, w->k_bias, k,
              lkv * hd);
  linear_core(normed, n, H, H, w->v_proj, H, 0, sh->kv0 * hd, sh->kv1 * hd, w->v_bias, v,
              lkv * hd);

  /* :255-279 */
  for (size_t row = 0; row < n; ++row) {
    const size_t pos = positions[row];
    if (pos >= d->max_position_embeddings) {
      rc = fail(ORACLE_ERR_INTERNAL, "position %zu exceeds the RoPE table (%u entries)", pos,
                d->max_position_embeddings);
      goto done;
    }
    const float *c = m->rope_cos + pos * half, *s = m->rope_sin + pos * half;
    for (size_t h = 0; h < lq; ++h) oracle_apply_rope(q + (row * lq + h) * hd, hd, c, s, half);
    for (size_t h = 0; h < lkv; ++h) oracle_apply_rope(k + (row * lkv + h) * hd, hd, c, s, half);
  }

  /* :283-297 */
  for (size_t row = 0; row < n; ++row) {
    for (size_t h = 0; h < lkv; ++h) {
      rc = oracle_kv_write(m->kv, layer_idx, slot_block[row], slot_slot[row], sh->kv0 + h, 0,
                           k + (row * lkv + h) * hd, hd);
      if (rc) goto done;
      rc = oracle_kv_write(m->kv, layer_idx, slot_block[row], slot_slot[row], sh->kv0 + h, 1,
                           v + (row * lkv + h) * hd, hd);
      if (rc) goto done;
    }
  }

  /* :300-326 */
  if (Hkv == 0 || Hq % Hkv != 0) {
    rc = fail(ORACLE_ERR_INTERNAL, "%zu query heads cannot be grouped over %zu kv heads", Hq,
              Hkv);
    goto done;
  }
  for (size_t row = 0; row < n; ++row) {
    const size_t seq = seq_of_row[row];
    const uint32_t *table = tables_flat + table_offsets[seq];
    const size_t table_len = (size_t)(table_offsets[seq + 1] - table_offsets[seq]);
    rc = attention_heads(m->kv, q + row * lq * hd, table, table_len, positions[row], layer_idx,
                         sh->q0, sh->q1, Hq / Hkv, hd, d->block_size, attn + row * lq * hd,
                         scores);
    if (rc) goto done;
  }

  /* :328-332  (row-parallel under TP: columns [q0*hd, q1*hd) of o_proj) */
  linear_core(attn, n, lq * hd, lq * hd, w->o_proj, Hq * hd, sh->q0 * hd, 0, H, NULL, proj, H);
  if (sh->allreduce) sh->allreduce(proj, n * H, sh->ctx);
  for (size_t i = 0; i < n * H; ++i) hidden[i] += proj[i];

  /* :335-345 */
  memcpy(normed, hidden, n * H * sizeof(float));
  rc = oracle_rms_norm(normed, n, H, w->post_attn_norm, H, d->rms_norm_eps);
  if (rc) goto done;
  linear_core(normed, n, H, H, w->gate_proj, H, 0, sh->f0, sh->f1, NULL, gate, lf);
  linear_core(normed, n, H, H, w->up_proj, H, 0, sh->f0, sh->f1, NULL, up, lf);
  rc = oracle_swiglu(gate, n, lf, up, n, lf);
  if (rc) goto done;
  linear_core(gate, n, lf, lf, w->down_proj, F, sh->f0, 0, H, NULL, proj, H);
  if (sh->allreduce) sh->allreduce(proj, n * H, sh->ctx);
  for (size_t i = 0; i < n * H; ++i) hidden[i] += proj[i];

done:
  free(normed), free(q), free(k), free(v), free(attn), free(proj), free(gate), free(up);
  free(scores);
  return rc;
}

static int forward_impl(OracleModel *m, const Shards *sh, const uint32_t *tokens,
                        const uint32_t *positions, size_t num_tokens,
                        const uint64_t *slot_token_counts, const uint64_t *context_lens,
                        const uint32_t *tables_flat, const uint64_t *table_offsets,
                        size_t num_sequences, float *logits_out) {
  (void)context_lens; /* carried but unused by the reference (attention.rs:233) */
  const OracleModelDesc *d = &m->d;
  const size_t H = d->hidden_size, V = d->vocab_size;
  int rc = ORACLE_OK;
  if (!model_complete(m)) return fail(ORACLE_ERR_ARG, "model has unset tensors");
  if (num_tokens == 0) return ORACLE_OK; /* transformer.rs:361-367 */

  size_t *seq_of_row = (size_t *)malloc(num_tokens * sizeof(size_t));
  uint32_t *slot_block = (uint32_t *)malloc(num_tokens * sizeof(uint32_t));
  size_t *slot_slot = (size_t *)malloc(num_tokens * sizeof(size_t));
  float *hidden = (float *)malloc(num_tokens * H * sizeof(float));
  float *tail = (float *)malloc((num_sequences ? num_sequences : 1) * H * sizeof(float));
  if (!seq_of_row || !slot_block || !slot_slot || !hidden || !tail) {
    rc = fail(ORACLE_ERR_ARG, "out of memory in forward");
    goto done;
  }

  /* :371-377 */
  {
    size_t row = 0;
    for (size_t s = 0; s < num_sequences; ++s)
      for (uint64_t c = 0; c < slot_token_counts[s]; ++c) seq_of_row[row++] = s;
  }
  /* :378-387  every slot is resolved before any compute or KV write */
  for (size_t row = 0; row < num_tokens; ++row) {
    const size_t seq = seq_of_row[row];
    const uint32_t *table = tables_flat + table_offsets[seq];
    const size_t table_len = (size_t)(table_offsets[seq + 1] - table_offsets[seq]);
    if (!oracle_locate(table, table_len, positions[row], d->block_size, &slot_block[row],
                       &slot_slot[row])) {
      rc = fail(ORACLE_ERR_INTERNAL, "position %u has no block in the table for sequence %zu",
                positions[row], seq);
      goto done;
    }
  }
  /* :389, :208-223 */
  for (size_t i = 0; i < num_tokens; ++i) {
    if (tokens[i] >= V) {
      rc = fail(ORACLE_ERR_INTERNAL, "token id %u is outside the vocabulary of %zu", tokens[i],
                V);
      goto done;
    }
    memcpy(hidden + i * H, m->embed_tokens + (size_t)tokens[i] * H, H * sizeof(float));
  }
  /* :390-400 */
  for (size_t layer = 0; layer < d->num_layers; ++layer) {
    rc = layer_forward(m, layer, hidden, num_tokens, positions, slot_block, slot_slot,
                       seq_of_row, tables_flat, table_offsets, sh);
    if (rc) goto done;
  }
  /* :401-405 */
  rc = oracle_rms_norm(hidden, num_tokens, H, m->final_norm, H, d->rms_norm_eps);
  if (rc) goto done;
  /* :410-428 */
  {
    size_t cursor = 0;
    for (size_t s = 0; s < num_sequences; ++s) {
      if (slot_token_counts[s] == 0) {
        rc = fail(ORACLE_ERR_INTERNAL, "a scheduled sequence contributed zero tokens");
        goto done;
      }
      cursor += (size_t)slot_token_counts[s];
      memcpy(tail + s * H, hidden + (cursor - 1) * H, H * sizeof(float));
    }
  }
  /* :430-435 */
  linear_core(tail, num_sequences, H, H, m->lm_head ? m->lm_head : m->embed_tokens, H, 0, 0, V,
              NULL, logits_out, V);
done:
  free(seq_of_row), free(slot_block), free(slot_slot), free(hidden), free(tail);
  return rc;
}

/* core/traits.rs:232-261 */
static int validate_batch(size_t num_tokens, size_t num_positions, size_t num_sequences,
                          size_t num_slot_counts, size_t num_context_lens,
                          size_t num_block_tables, const uint64_t *slot_token_counts) {
  if (num_slot_counts != num_sequences || num_context_lens != num_sequences ||
      num_block_tables != num_sequences)
    return fail(ORACLE_ERR_INTERNAL,
                "ForwardBatch arrays disagree: %zu sequence ids, %zu token counts, %zu context "
                "lens, %zu block tables",
                num_sequences, num_slot_counts, num_context_lens, num_block_tables);
  if (num_positions != num_tokens)
    return fail(ORACLE_ERR_INTERNAL, "ForwardBatch has %zu tokens but %zu positions", num_tokens,
                num_positions);
  uint64_t summed = 0;
  for (size_t s = 0; s < num_sequences; ++s) summed += slot_token_counts[s];
  if (summed != num_tokens)
    return fail(ORACLE_ERR_INTERNAL,
                "ForwardBatch slot token counts sum to %llu but there are %zu tokens",
                (unsigned long long)summed, num_tokens);
  return ORACLE_OK;
}

int oracle_model_forward(OracleModel *m, const uint32_t *tokens, const uint32_t *positions,
                         size_t num_tokens, const uint64_t *slot_token_counts,
                         const uint64_t *context_lens, const uint32_t *block_tables_flat,
                         const uint64_t *block_table_offsets, size_t num_sequences,
                         size_t num_slot_counts, size_t num_context_lens,
                         size_t num_block_tables, size_t num_positions, float *logits_out) {
  int rc = validate_batch(num_tokens, num_positions, num_sequences, num_slot_counts,
                          num_context_lens, num_block_tables, slot_token_counts);
  if (rc) return rc;
  Shards sh = {0, m->d.num_attention_heads, 0, m->d.num_kv_heads, 0, m->d.ffn_dim, NULL, NULL};
  return forward_impl(m, &sh, tokens, positions, num_tokens, slot_token_counts, context_lens,
                      block_tables_flat, block_table_offsets, num_sequences, logits_out);
}

int oracle_model_forward_tp(OracleModel *m, uint32_t tp_rank, uint32_t tp_world,
                            oracle_allreduce_fn allreduce, void *ctx, const uint32_t *tokens,
                            const uint32_t *positions, size_t num_tokens,
                            const uint64_t *slot_token_counts, const uint64_t *context_lens,
                            const uint32_t *block_tables_flat,
                            const uint64_t *block_table_offsets, size_t num_sequences,
                            float *logits_out) {
  const OracleModelDesc *d = &m->d;
  /* orion-distributed/src/lib.rs:74-90, 139-152, 174-208 */
  if (tp_world == 0) return fail(ORACLE_ERR_ARG, "world_size must be at least 1");
  if (tp_rank >= tp_world)
    return fail(ORACLE_ERR_ARG, "rank %u is out of range for world size %u", tp_rank, tp_world);
  if (tp_world > 1 && d->num_kv_heads < tp_world)
    return fail(ORACLE_ERR_ARG, "model has %u KV heads but world size is %u", d->num_kv_heads,
                tp_world);
  if (d->num_attention_heads % tp_world || d->num_kv_heads % tp_world || d->ffn_dim % tp_world)
    return fail(ORACLE_ERR_ARG, "cannot split heads/ffn evenly across %u ranks", tp_world);
  const size_t lq = d->num_attention_heads / tp_world, lkv = d->num_kv_heads / tp_world,
               lf = d->ffn_dim / tp_world;
  Shards sh = {tp_rank * lq, (tp_rank + 1) * lq,   tp_rank * lkv,
               (tp_rank + 1) * lkv, tp_rank * lf, (tp_rank + 1) * lf,
               tp_world > 1 ? allreduce : NULL, ctx};
  int rc = validate_batch(num_tokens, num_tokens, num_sequences, num_sequences, num_sequences,
                          num_sequences, slot_token_counts);
  if (rc) return rc;
  return forward_impl(m, &sh, tokens, positions, num_tokens, slot_token_counts, context_lens,
                      block_tables_flat, block_table_offsets, num_sequences, logits_out);
}
