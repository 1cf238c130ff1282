/*
 * CPU oracle for the OrionServe-RS per-step transformer forward pass.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference's
 * scalar-f32 CPU path. It exists to check the CUDA library and to be timed as
 * the CPU baseline; nothing on the product path may call it.
 *
 * Parity pin: the reference is Rust and cannot be compiled where this oracle
 * is built, so the oracle is pinned against the known-answer values held by the
 * reference's own unit tests (tests/golden/reference_kats.json) and against the
 * invariants those tests state (incremental decode == full prefill, chunked ==
 * single pass, scattered == contiguous block table, batch independence).
 *
 * Every function cites the reference lines whose operation order it follows.
 * Build with -O2 -ffp-contract=off -fno-fast-math: the reference never
 * contracts a*b+c into an FMA and never reassociates a sum.
 */
#ifndef ORION_ORACLE_H
#define ORION_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes shared by every oracle entry point. */
enum {
  ORACLE_OK = 0,
  ORACLE_ERR_INTERNAL = 1, /* the reference's EngineError::Internal */
  ORACLE_ERR_ARG = 2
};

/* Last error text of the calling thread (empty string when none). */
const char *oracle_last_error(void);

/* Worker threads for oracle_linear. Threads split OUTPUT elements only, so
 * every dot product keeps its sequential order and results are bit-identical
 * for any thread count. 1 = the reference's single-threaded behaviour. */
void oracle_set_threads(int n);
int oracle_get_threads(void);

/* ---- crates/orion-models/src/tensor.rs ---- */

/* tensor.rs:96-130  out[i][j] = (sum_k x[i][k]*w[j][k], k ascending, f32) + bias[j]. */
int oracle_linear(const float *x, size_t n, size_t k, const float *w, size_t out_features,
                  size_t in_features, const float *bias, size_t bias_len, float *out);

/* tensor.rs:143-163  f64 sum of squares, scale=(1/sqrt(ss/cols+eps)) as f32, v=(v*scale)*w. */
int oracle_rms_norm(float *x, size_t rows, size_t cols, const float *weight, size_t weight_len,
                    float eps);

/* tensor.rs:167-169 */
float oracle_silu(float x);

/* tensor.rs:175-189  gate = silu(gate) * up */
int oracle_swiglu(float *gate, size_t gate_rows, size_t gate_cols, const float *up,
                  size_t up_rows, size_t up_cols);

/* tensor.rs:192-209 */
void oracle_softmax_inplace(float *x, size_t n);

/* tensor.rs:228-253  cos/sin tables [max_positions][head_dim/2]. */
int oracle_rope_table(size_t head_dim, size_t max_positions, float theta, float *cos_out,
                      float *sin_out);

/* tensor.rs:283-298  rotate-half: pairs i with i+len/2. */
int oracle_apply_rope(float *vec, size_t len, const float *cos_row, const float *sin_row,
                      size_t table_width);

/* ---- crates/orion-models/src/attention.rs ---- */

typedef struct OracleKvStore OracleKvStore;

/* attention.rs:45-62  zero-filled arena [layer][block][k|v][slot][head][dim]. */
OracleKvStore *oracle_kv_new(size_t num_layers, size_t num_blocks, size_t block_size,
                             size_t num_kv_heads, size_t head_dim);
void oracle_kv_free(OracleKvStore *s);
size_t oracle_kv_len(const OracleKvStore *s);
float *oracle_kv_data(OracleKvStore *s);
/* attention.rs:107-120 */
int oracle_kv_write(OracleKvStore *s, size_t layer, uint32_t block, size_t slot, size_t head,
                    int is_value, const float *vec, size_t vec_len);
/* attention.rs:123-134  copies head_dim floats to out. */
int oracle_kv_read(const OracleKvStore *s, size_t layer, uint32_t block, size_t slot,
                   size_t head, int is_value, float *out);

/* attention.rs:182-186  returns 1 and fills (block, slot) or 0 when past the table. */
int oracle_locate(const uint32_t *table, size_t table_len, size_t position, size_t block_size,
                  uint32_t *block, size_t *slot);

/* attention.rs:219-295 */
int oracle_paged_attention(const OracleKvStore *s, const float *query, size_t query_len,
                           const uint32_t *table, size_t table_len, size_t query_position,
                           size_t layer, size_t num_query_heads, size_t num_kv_heads,
                           size_t head_dim, size_t block_size, float *out, size_t out_len);

/* ---- crates/orion-runtime/src/sampling.rs:196-206 ---- */
/* Index of the first strict maximum; -1 when no element exceeds -inf. */
int64_t oracle_argmax(const float *logits, size_t n);

/* ---- crates/orion-models/src/loader.rs:74-96  exact widening ---- */
void oracle_bf16_to_f32(const uint16_t *src, size_t n, float *dst);
void oracle_f16_to_f32(const uint16_t *src, size_t n, float *dst);
/* Round-to-nearest-even narrowing, used by tests to build bf16 checkpoints. */
void oracle_f32_to_bf16(const float *src, size_t n, uint16_t *dst);

/* ---- crates/orion-models/src/transformer.rs ---- */

typedef struct {
  uint32_t hidden_size;
  uint32_t num_layers;
  uint32_t num_attention_heads;
  uint32_t num_kv_heads;
  uint32_t head_dim;
  uint32_t vocab_size;
  uint32_t ffn_dim;
  uint32_t max_position_embeddings;
  float rope_theta;
  float rms_norm_eps;
  uint32_t has_qkv_bias;  /* Qwen2 (transformer.rs:78-86) */
  uint32_t tied_lm_head;  /* transformer.rs:108-112 */
  uint32_t num_blocks;
  uint32_t block_size;
} OracleModelDesc;

typedef struct OracleModel OracleModel;

/* transformer.rs:148-177  builds the RoPE table and the zeroed arena. */
OracleModel *oracle_model_new(const OracleModelDesc *desc);
void oracle_model_free(OracleModel *m);

/* Copies an f32 tensor under its Hugging Face name (transformer.rs:12-18,62-120).
 * Shape is checked against the descriptor. */
int oracle_model_set_tensor(OracleModel *m, const char *name, const float *data, size_t len);

/* Direct access for tests that compare arenas. */
OracleKvStore *oracle_model_kv(OracleModel *m);

/* transformer.rs:359-442. block_tables are flattened with offsets[S+1].
 * logits_out holds num_sequences*vocab_size floats. An empty batch is OK and
 * writes nothing. */
int oracle_model_forward(OracleModel *m, const uint32_t *tokens, const uint32_t *positions,
                         size_t num_tokens, const uint64_t *slot_token_counts,
                         const uint64_t *context_lens, const uint32_t *block_tables_flat,
                         const uint64_t *block_table_offsets, size_t num_sequences,
                         size_t num_slot_counts, size_t num_context_lens,
                         size_t num_block_tables, size_t num_positions, float *logits_out);

/* Tensor-parallel restatement used by the multi-rank host tests: runs the
 * forward with this rank's column/row shards (orion-distributed/src/lib.rs:
 * 174-208) and calls `allreduce(buf, n, ctx)` after the O and down projections. */
typedef void (*oracle_allreduce_fn)(float *buf, size_t n, void *ctx);
int oracle_model_forward_tp(OracleModel *m, uint32_t tp_rank, uint32_t tp_world,
                            oracle_allreduce_fn allreduce, void *ctx, const uint32_t *tokens,
                            const uint32_t *positions, size_t num_tokens,
                            const uint64_t *slot_token_counts, const uint64_t *context_lens,
                            const uint32_t *block_tables_flat,
                            const uint64_t *block_table_offsets, size_t num_sequences,
                            float *logits_out);

#ifdef __cplusplus
}
#endif
#endif
