// Launchers of the device kernels. Every pointer is a device pointer; every
// launcher enqueues on `stream` and returns an OrionStatus. `T` is the storage
// type of weights, activations and the KV arena (float for the correctness
// build, bf16 for the performance build). GEMM results are always f32
// "partials": `splits` slabs of [rows][n] that the consuming kernel sums, which
// fuses the split-K reduction into the next elementwise step.
#pragma once

#include "common.cuh"

namespace orion {

// Shape of the paged KV arena of one rank:
// [layer][block][local kv head][k|v][slot][dim]. Each (block, head) owns one
// contiguous chunk holding its K rows followed by its V rows, so a decode CTA
// fetches a 16-token block of one head with a single bulk copy.
// With `swizzle` set (16-bit storage, head_dim a multiple of 64) the 16-byte
// groups of every row are XOR-permuted by (slot & 7): the linear bulk copy then
// lands in shared memory in a layout ldmatrix reads without bank conflicts.
struct KvLayout {
  uint32_t num_layers, num_blocks, num_kv_heads, block_size, head_dim, swizzle;
  __host__ __device__ size_t chunk_elems() const { return size_t(2) * block_size * head_dim; }
  __host__ __device__ size_t layer_elems() const {
    return size_t(num_blocks) * num_kv_heads * chunk_elems();
  }
  // Start of the row holding (layer, block, head, k|v, slot).
  __host__ __device__ size_t row(uint32_t layer, uint32_t block, uint32_t head, uint32_t is_v,
                                 uint32_t slot) const {
    return layer * layer_elems() + (size_t(block) * num_kv_heads + head) * chunk_elems() +
           (size_t(is_v) * block_size + slot) * head_dim;
  }
  // Position of logical dim `d` inside the row of `slot`.
  __host__ __device__ uint32_t col(uint32_t slot, uint32_t d) const {
    return swizzle ? ((((d >> 3) ^ (slot & 7u)) << 3) | (d & 7u)) : d;
  }
};

// hidden[r] = embed[tokens[r]] (f32); normed[r] = rms_norm(hidden[r]) * w.
// (transformer.rs:208-223 fused with tensor.rs:143-163)
template <typename T>
int launch_embed_rmsnorm(const T *embed, const uint32_t *tokens, const float *norm_w, float eps,
                         float *hidden, T *normed, uint32_t rows, uint32_t hidden_size,
                         cudaStream_t stream);

// hidden[r] += sum_s partial[s][r] (+ nothing else); out[i] = rms_norm(hidden[src(i)]) * w,
// src(i) = row_map ? row_map[i] : i. With row_map the residual is not written
// back (used for the final norm over the last row of each sequence).
// (transformer.rs:330-336, 343-345, 401-428)
template <typename T>
int launch_residual_rmsnorm(const float *partial, uint32_t splits, size_t split_stride,
                            float *hidden, const float *norm_w, float eps, T *out,
                            const uint32_t *row_map, uint32_t out_rows, uint32_t hidden_size,
                            cudaStream_t stream, uint32_t *ready = nullptr);  // ready: every CTA (one per output row) adds 1 when done

// Plain rms_norm of f32 rows into T (tensor.rs:143-163) for the op-level API.
template <typename T>
int launch_rmsnorm_rows(const float *x, const float *norm_w, float eps, T *out, uint32_t rows,
                        uint32_t cols, cudaStream_t stream);

// Sums the QKV partials (+bias), applies RoPE to q and k heads by table lookup
// at positions[r], writes q to `q_out` [rows][q_heads*hd] and k, v into the
// arena at (slot_block[r], slot_slot[r]). (transformer.rs:248-297, tensor.rs:283-298)
template <typename T>
int launch_rope_kvwrite(const float *partial, uint32_t splits, size_t split_stride,
                        const float *bias, const uint32_t *positions, const uint32_t *slot_block,
                        const uint32_t *slot_slot, const float *rope_cos, const float *rope_sin,
                        T *q_out, T *arena, KvLayout kv, uint32_t layer, uint32_t rows,
                        uint32_t q_heads, cudaStream_t stream);

// In-place RoPE over [rows][heads][hd] of T (op-level API; tensor.rs:283-298).
template <typename T>
int launch_rope_rows(T *x, const uint32_t *positions, const float *rope_cos, const float *rope_sin,
                     uint32_t rows, uint32_t heads, uint32_t head_dim, cudaStream_t stream);

// act[r][f] = silu(g) * u with g = sum_s partial[s][r][f], u = sum_s partial[s][r][ffn + f];
// `interleaved`: gate f and up f sit in columns 2f and 2f + 1 instead. (tensor.rs:167-189)
template <typename T>
int launch_swiglu(const float *partial, uint32_t splits, size_t split_stride, T *act, uint32_t rows,
                  uint32_t ffn, cudaStream_t stream, bool interleaved = false);
// dst[r * dst_stride + c] = src[r * cols + c]
template <typename T>
int launch_copy_rows_strided(const T *src, T *dst, size_t rows, size_t cols, size_t dst_stride, cudaStream_t stream);

// out[r][n] = sum_s partial[s][r][n] + bias[n]  (finishes tensor::linear, tensor.rs:126).
int launch_finish_linear(const float *partial, uint32_t splits, size_t split_stride,
                         const float *bias, float *out, uint32_t rows, uint32_t n,
                         cudaStream_t stream);

// First index of the strict row maximum; UINT32_MAX when nothing exceeds -inf.
// (orion-runtime/src/sampling.rs:196-206)
int launch_argmax(const float *logits, uint32_t rows, uint32_t cols, uint32_t *out,
                  cudaStream_t stream);

// Converts between f32 and T on the device (weight upload, arena read-back).
template <typename T>
int launch_convert_from_f32(const float *src, T *dst, size_t n, cudaStream_t stream);
template <typename T>
int launch_convert_to_f32(const T *src, float *dst, size_t n, cudaStream_t stream);
int launch_f16_to_f32(const uint16_t *src, float *dst, size_t n, cudaStream_t stream);
// dst[i][:] = src[row_map[i]][:]
template <typename T>
int launch_gather_rows(const T *src, const uint32_t *row_map, T *dst, uint32_t rows, uint32_t cols,
                       cudaStream_t stream);
// dst[i] = T(src[i] * scale)
template <typename T>
int launch_scale_convert(const float *src, T *dst, size_t n, float scale, cudaStream_t stream);

// Arena -> the reference's logical order [layer][block][k|v][slot][head][dim], f32.
template <typename T>
int launch_arena_to_reference_order(const T *arena, KvLayout kv, float *out, cudaStream_t stream);
// The reverse, for one layer given in reference order (op-level attention API).
template <typename T>
int launch_arena_from_reference_order(const float *ref, KvLayout kv, T *arena, cudaStream_t stream);

// Fills `n` elements with N(0, 1) values from a counter-based generator.
template <typename T>
int launch_fill_normal(T *dst, size_t n, uint64_t seed, cudaStream_t stream);

// ---- attention ---------------------------------------------------------------

struct AttnBatch {
  const uint32_t *query_positions;  // [rows] absolute position of each query row
  const uint32_t *seq_of_row;       // [rows]
  const uint32_t *tables_flat;      // concatenated block tables
  const uint32_t *table_offsets;    // [sequences + 1]
  uint32_t rows;
  uint32_t max_position;            // largest query position in the batch
};

// Any shape, any mix of prefill and decode rows: one CTA per (row, query head),
// causal by absolute position (attention.rs:219-295).
template <typename T>
int launch_paged_attention_generic(const T *q, const T *arena, KvLayout kv, uint32_t layer,
                                   AttnBatch batch, uint32_t q_heads, T *out, cudaStream_t stream);

// Tuned prefill / mixed-batch path (bf16, head_dim 128, block 16): the batch is cut into
// tiles of consecutive rows of one sequence (prefill_tile_positions rows at most); one CTA per
// (kv head, tile) streams the sequence's K/V once for all rows of the tile.
struct PrefillTile {
  uint32_t row_start;     // first batch row of the tile
  uint32_t num_rows;      // rows (query positions) in the tile
  uint32_t seq;           // sequence the rows belong to
  uint32_t max_position;  // largest query position in the tile
};
bool prefill_attention_supported(KvLayout kv, uint32_t q_heads);
uint32_t prefill_tile_positions(uint32_t q_heads, uint32_t kv_heads);
int launch_paged_attention_prefill(const bf16 *q, const bf16 *arena, KvLayout kv, uint32_t layer,
                                   AttnBatch batch, const PrefillTile *tiles, uint32_t num_tiles,
                                   uint32_t q_heads, bf16 *out, cudaStream_t stream);
int prefill_poll_error(uint32_t *code);
// The same computation on tcgen05 / tensor memory (S and O accumulators in tensor memory, K/V tiles by
// tiled TMA straight out of the arena); same tiles, same arguments.
bool prefill_attention_tc_supported(KvLayout kv, uint32_t q_heads, const void *arena);
int launch_paged_attention_prefill_tc(const bf16 *q, const bf16 *arena, KvLayout kv, uint32_t layer,
                                      AttnBatch batch, const PrefillTile *tiles, uint32_t num_tiles,
                                      uint32_t q_heads, bf16 *out, cudaStream_t stream);
int prefill_tc_poll_error(uint32_t *code);

// Tuned decode path (bf16, head_dim 128, block 16, one query row per sequence):
// one CTA per (sequence, kv head, context split); the query heads of a GQA group
// share every K/V tile. `scratch` holds the per-split partial outputs.
struct DecodeScratch {
  float *partial_out;  // [rows][q_heads][max_splits][head_dim]
  float *partial_ml;   // [rows][q_heads][max_splits][2]  (running max, running sum)
  uint32_t max_splits;
  // [rows * kv_heads] arrival counters, zero between launches: the last CTA of a (row, kv head) to
  // finish merges the splits itself, so no separate combine launch follows. Null = combine kernel.
  uint32_t *counters;
  // 0: every row is cut into max_splits pieces; else a row of n blocks is cut into
  // round(n / blocks_per_split) pieces (at least 1, at most max_splits).
  uint32_t blocks_per_split;
};
// A scratch buffer starts with kDecodeCounterWords counter words (which must be zero when the buffer
// is first used and are left zero by every launch), followed by the partial results.
constexpr uint32_t kDecodeCounterWords = 16384;
bool decode_attention_supported(KvLayout kv, uint32_t q_heads);
// Floats a scratch buffer needs, counter words included.
size_t decode_scratch_floats(uint32_t rows, uint32_t q_heads, uint32_t head_dim,
                             uint32_t max_splits);
// Lays the parts of a scratch buffer of at least decode_scratch_floats(...) floats out.
DecodeScratch decode_scratch_at(float *base, uint32_t rows, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                                uint32_t splits, uint32_t blocks_per_split = 0);
// Length-proportional context split for a ragged batch: `splits` = pieces of the longest row (the
// grid's z extent), `blocks_per_split` = blocks a piece should hold. `total_blocks` = sum over the
// rows of their block counts. splits == 1 means no row is cut.
struct DecodePlan {
  uint32_t splits, blocks_per_split;
};
DecodePlan decode_plan(uint32_t rows, uint32_t kv_heads, uint64_t total_blocks, uint32_t max_position,
                       uint32_t block_size, uint32_t max_splits);
uint32_t decode_choose_splits(uint32_t rows, uint32_t kv_heads, uint32_t max_position,
                              uint32_t block_size, uint32_t max_splits);
// With `partial` set the kernel takes the row's q, k and v straight from the QKV projection's
// f32 partial sums: it folds the split-K slabs, adds the bias, applies RoPE at the row's position
// (transformer.rs:248-297), writes k and v into the arena slot and uses them for this step, so no
// separate RoPE / KV-write kernel runs and `q` is not read.
struct FusedQkv {
  const float *partial = nullptr;  // [slabs][rows][(q_heads + 2 kv_heads) * head_dim]
  uint32_t slabs = 0;
  size_t slab_stride = 0;
  const float *bias = nullptr;     // [(q_heads + 2 kv_heads) * head_dim] or null
  const float *rope_cos = nullptr, *rope_sin = nullptr;  // [max_pos][head_dim / 2]
  const uint32_t *slot_block = nullptr;                  // [rows] physical block of the row's position
  bf16 *arena = nullptr;           // writable view of the arena
};
int launch_paged_attention_decode(const bf16 *q, const bf16 *arena, KvLayout kv, uint32_t layer,
                                  AttnBatch batch, uint32_t q_heads, uint32_t splits,
                                  DecodeScratch scratch, bf16 *out, cudaStream_t stream,
                                  FusedQkv fused = {});
// Tuning: ring depth per warp (2..4) and the CTA count the context split aims for (0 keeps it).
void decode_set_tuning(int stages, uint32_t cta_target);
// Device error word of the decode kernel (0 = none); reading clears it.
int decode_poll_error(uint32_t *code);

// ---- tensor-parallel hand-over ---------------------------------------------------

constexpr int kMaxTpWorld = 8;
// Largest batch the fused hand-over takes; larger (prefill-sized) batches are bandwidth-bound
// and go through the library all-reduce.
constexpr uint32_t kTpFusedMaxRows = 256;
// Peer-mapped inboxes of every rank of the tensor-parallel group (index = rank; the entry of
// this rank is its own local pointer). An inbox is [parity 2][sender world][slot_floats] units
// of 8 bytes (one f32 of a partial sum and the epoch of the hand-over that wrote it), followed by
// [parity 2][slot_floats] units for the normalised rows of the two-shot variant.
struct TpPeers {
  uint32_t *inbox[kMaxTpWorld];
  int rank, world;
  uint32_t slot_floats;
  uint64_t wait_limit_ns = 2000000000ull;  // how long a poll for a peer's unit may last before it gives up
};
// All-reduce of the partial sums over ranks and split-K slabs + residual add + RMSNorm for
// `rows` batch rows; every rank ends up with the full residual stream in `hidden` and all
// normalised rows in `out`. The epoch of the call is *epoch_base + epoch_add (epoch_base may be null: epoch_add
// alone); epochs cycle through 1 .. 0xFFFFFFFE, one step per call, and consecutive calls alternate in parity.
// With the base in device memory (advanced by launch_tp_state_bump at the end of a step) a step's launches take
// the same arguments every time, so the step can be replayed as a CUDA graph.
// `two_shot`: reduce-scatter to the owner of each row + all-gather of the normalised rows (only
// the owner of a row then holds its current residual); else every rank reduces every row.
template <typename T>
int launch_tp_allreduce_residual_rmsnorm(const TpPeers &peers, const uint32_t *epoch_base, uint32_t epoch_add, const float *partial, uint32_t splits,
                                         size_t split_stride, float *hidden, const float *norm_w, float eps, T *out,
                                         uint32_t rows, uint32_t hidden_size, bool two_shot, cudaStream_t stream,
                                         uint32_t *ready = nullptr);  // ready: every CTA (one per row) adds 1 when done
// state[0] += epochs (wrapped as described above), state[1] += rows_counted, after the preceding kernel has completed.
int launch_tp_state_bump(uint32_t *state, uint32_t epochs, uint32_t rows_counted, cudaStream_t stream);
int tp_poll_error(uint32_t *code);
// Vocabulary-parallel LM head: `launch_tp_signal` (ranks other than the leader) stores `epoch` into the
// rank's flag in the leader's memory once the preceding kernel of the stream has completed;
// `launch_tp_wait_flags` (leader) holds the stream until the flags of ranks 1 .. world-1 carry `epoch`
// (bounded: after `limit_ns` the hand-over error word gets bit 1 and the stream goes on).
int launch_tp_signal(uint32_t *flag, uint32_t epoch, cudaStream_t stream);
int launch_tp_wait_flags(const uint32_t *flags, uint32_t epoch, int world, uint64_t limit_ns, cudaStream_t stream);
// Launches a kernel whose only thread waits on a barrier that nothing arrives at, with the given
// limit: the bounded wait must give up (timed_out = 1) and the kernel must end normally.
int selftest_bounded_wait(uint64_t limit_us, uint32_t *timed_out, uint32_t *waited_us);
// The same for the peer polls of the tensor-parallel hand-over: one thread polls inbox units that
// nobody writes (both unit formats); each poll must give up after the limit, the device error word
// must be set (and is cleared again), and the kernel must end normally.
int selftest_peer_wait(uint64_t limit_us, uint32_t *timed_out, uint32_t *waited_us);

// ---- GEMM ----------------------------------------------------------------------

// partial[s][r][n] = sum over the k-range of split s of x[r][k] * w[n][k]
// (tensor.rs:114-128 without the bias). x: [rows][k] (row stride ldx),
// w: [n][k] row-major (row stride ldw).
struct GemmPlan {
  uint32_t splits;
  bool tensor_core;     // tcgen05 path (bf16 only)
  bool cluster_reduce;  // the k splits of a tile form a cluster and reduce in shared memory
  uint32_t out_slabs;   // slabs the consumer has to sum: 1 with cluster_reduce, else `splits`
  uint32_t ldc;         // row stride of the output when it is a column block of a wider matrix (0 = n)
};
GemmPlan gemm_plan(bool is_bf16, uint32_t rows, uint32_t n, uint32_t k, uint32_t ldx, uint32_t ldw);
template <typename T>
int launch_gemm(const T *x, uint32_t ldx, const T *w, uint32_t ldw, float *partial, uint32_t rows,
                uint32_t n, uint32_t k, GemmPlan plan, cudaStream_t stream, ReadyWait ready = {});  // `ready`: honoured by the tensor-core path only (GemmPlan::tensor_core)
size_t gemm_partial_floats(bool is_bf16, uint32_t max_rows, uint32_t n, uint32_t k);
// Number of CTAs split-K aims for on small batches (default 296, two per SM).
void gemm_set_target_ctas(uint32_t ctas);
// Ring layout of the decode-batch GEMM: 5 = deep weight ring + short activation ring, 4 = equal rings.
void gemm_set_small_stages(int stages);

// SIMT GEMM: exact k-ascending accumulation per output, no FMA for f32.
template <typename T>
int launch_gemm_simt(const T *x, uint32_t ldx, const T *w, uint32_t ldw, float *out, uint32_t rows,
                     uint32_t n, uint32_t k, cudaStream_t stream);
// tcgen05 / TMEM / TMA GEMM (bf16).
bool gemm_tc_supported(uint32_t rows, uint32_t n, uint32_t k, uint32_t ldx, uint32_t ldw,
                       const void *x, const void *w);
int launch_gemm_tc(const bf16 *x, uint32_t ldx, const bf16 *w, uint32_t ldw, float *partial,
                   uint32_t rows, uint32_t n, uint32_t k, uint32_t splits, cudaStream_t stream,
                   bf16 *act = nullptr, bool cluster_reduce = false, uint32_t ldc = 0,
                   ReadyWait ready = {});
// Gate/up projection with SwiGLU in the epilogue: `w_interleaved` is [2 * ffn][k] with gate row f
// at 2f and up row f at 2f + 1; writes act[r][f] = silu(x.gate_f) * (x.up_f) and no partials.
// One k split only (gemm_plan(...).splits == 1 and .tensor_core).
int launch_gemm_swiglu(const bf16 *x, uint32_t ldx, const bf16 *w_interleaved, uint32_t ldw, bf16 *act, uint32_t rows,
                       uint32_t ffn, uint32_t k, cudaStream_t stream, ReadyWait ready = {});
// Device error word set by kernels whose bounded waits ran out (0 = none).
int gemm_tc_poll_error(uint32_t *code);

}  // namespace orion
