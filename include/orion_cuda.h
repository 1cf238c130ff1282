/*
 * orion_cuda.h — C ABI of the B200 (sm_100a) implementation of OrionServe-RS's
 * per-step transformer forward pass.
 *
 * The reference has no FFI for this path: its boundary is two Rust traits,
 * `Backend` (crates/orion-core/src/traits.rs:159-183) and `LanguageModel`
 * (crates/orion-core/src/traits.rs:297-309), plus the constructor convention of
 * `TransformerModel::{new, from_directory}` (crates/orion-models/src/
 * transformer.rs:148-205). Each entry point below names the trait method or
 * function it stands in for; a Rust `orion-cuda` crate binds them one to one.
 *
 * Conventions: plain pointers and sizes, opaque handles, no exceptions across
 * the boundary. Every function that can fail returns an OrionStatus; the text
 * of the last failure on the calling thread is read with
 * orion_cuda_last_error(). Host pointers unless a parameter is documented as a
 * device pointer. One forward at a time per model handle (the reference's
 * engine loop is a single thread, crates/orion-runtime/src/engine.rs:502-548).
 * There is no CPU fallback: without a usable device every constructor fails.
 */
#ifndef ORION_CUDA_H
#define ORION_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Error classes, mirroring the reference's error enums. */
typedef enum OrionStatus {
  ORION_OK = 0,
  ORION_ERR_INTERNAL = 1,        /* EngineError::Internal (crates/orion-core/src/error.rs:78-135) */
  ORION_ERR_BACKEND = 2,         /* EngineError::Backend{backend:"cuda",stage,reason} (error.rs:119-124) */
  ORION_ERR_INVALID_REQUEST = 3, /* EngineError::InvalidRequest (orion-distributed/src/lib.rs:76-88) */
  ORION_ERR_UNAVAILABLE = 4,     /* CudaUnavailable::{NoDriver,NoDevices,NoSuchDevice} (orion-cuda/src/lib.rs:40-49) */
  ORION_ERR_MODEL = 5,           /* ModelError::{Malformed,MissingTensor,UnsupportedDtype} (transformer.rs:62-120) */
  ORION_ERR_CONTEXT_LENGTH = 6,  /* EngineError::ContextLengthExceeded (error.rs:84-92) */
  ORION_ERR_QUEUE_FULL = 7,      /* EngineError::QueueFull, retryable (error.rs:95-96) */
  ORION_ERR_CACHE_EXHAUSTED = 8  /* EngineError::CacheExhausted, retryable (error.rs:100-101) */
} OrionStatus;

/* DType (crates/orion-core/src/traits.rs:21-29). */
typedef enum OrionDType {
  ORION_DTYPE_F32 = 0,
  ORION_DTYPE_F16 = 1,
  ORION_DTYPE_BF16 = 2,
  ORION_DTYPE_I8 = 3,
  ORION_DTYPE_I4 = 4
} OrionDType;

typedef struct OrionBackend OrionBackend;
typedef struct OrionModel OrionModel;

/* Text of the last error raised on the calling thread ("" when none). */
const char *orion_cuda_last_error(void);

/* ---- orion_cuda::{is_available, device_count}  (orion-cuda/src/lib.rs:78-95) ---- */
int orion_cuda_is_available(void);
int orion_cuda_device_count(void);

/* ---- CudaBackend: Backend  (orion-cuda/src/lib.rs:104-179, traits.rs:159-183) ---- */

/* CudaBackend::new(ordinal) (orion-cuda/src/lib.rs:116-132). */
int orion_cuda_backend_create(int ordinal, OrionBackend **out);
void orion_cuda_backend_destroy(OrionBackend *backend);
/* Backend::name -> "cuda" (traits.rs:161). */
const char *orion_cuda_backend_name(const OrionBackend *backend);
/* Backend::device -> Device::Cuda(ordinal) (traits.rs:164). */
int orion_cuda_backend_ordinal(const OrionBackend *backend);
/* CudaBackend::device_name (orion-cuda/src/lib.rs:138-140). */
const char *orion_cuda_backend_device_name(const OrionBackend *backend);
/* Backend::total_memory / available_memory (traits.rs:167-173). */
int orion_cuda_backend_total_memory(const OrionBackend *backend, uint64_t *bytes);
int orion_cuda_backend_available_memory(const OrionBackend *backend, uint64_t *bytes);
/* Backend::synchronize (traits.rs:179). */
int orion_cuda_backend_synchronize(const OrionBackend *backend);
/* Backend::supports_dtype (traits.rs:182): 1 for F32 and BF16, else 0. */
int orion_cuda_backend_supports_dtype(const OrionBackend *backend, int dtype);

/* ---- CudaTransformerModel: LanguageModel ---- */

#define ORION_NCCL_ID_BYTES 128

/* ModelMetadata numeric fields (traits.rs:95-123) + HfConfig::ffn_dim
 * (orion-models/src/config.rs:238) + Architecture::has_qkv_bias (config.rs:134)
 * + the tied-head rule (transformer.rs:108-112) + the num_blocks / block_size
 * arguments of TransformerModel::new (transformer.rs:148-154) + the tensor-
 * parallel rank (orion-distributed/src/lib.rs:74-90). */
typedef struct OrionModelDesc {
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
  uint32_t has_qkv_bias;
  uint32_t tied_lm_head;
  uint32_t num_blocks;
  uint32_t block_size;
  /* Arithmetic of the build: ORION_DTYPE_F32 (correctness build, f32 storage
   * and arithmetic) or ORION_DTYPE_BF16 (performance build: bf16 weights, KV
   * arena and activations, f32 accumulation and residual stream). */
  uint32_t compute_dtype;
  /* Largest batch one forward may carry; device work buffers are sized from it. */
  uint32_t max_batch_tokens;
  uint32_t max_batch_sequences;
  /* Tensor parallelism: rank index and world size; world 1 = single GPU. */
  uint32_t tp_rank;
  uint32_t tp_world;
  /* ncclUniqueId shared by all ranks (from orion_cuda_tp_unique_id on rank 0);
   * ignored when tp_world == 1. */
  uint8_t nccl_unique_id[ORION_NCCL_ID_BYTES];
} OrionModelDesc;

/* TransformerModel::new (transformer.rs:148-177): allocates the zeroed KV
 * arena for this rank's KV heads, the RoPE tables and the work buffers. */
int orion_cuda_model_create(OrionBackend *backend, const OrionModelDesc *desc, OrionModel **out);
void orion_cuda_model_destroy(OrionModel *model);

/* Failure-detection self-test (no reference counterpart): every device-side wait of this library
 * gives up after a time limit, records an error word and lets its kernel finish, which the host
 * reports as EngineError::Backend. This entry point runs the same bounded wait on a barrier that
 * nothing ever arrives at, with a limit of `limit_us` (1 .. 1 000 000): it must come back with
 * *timed_out = 1 after about that long, and the device must stay usable. */
int orion_cuda_selftest_bounded_wait(OrionBackend *backend, uint64_t limit_us, uint32_t *timed_out,
                                     uint32_t *waited_us);

/* The same self-test for the peer polls of the tensor-parallel hand-over (no reference counterpart):
 * one thread polls inbox units that no peer ever writes, in both unit formats, with a limit of
 * `limit_us` per poll (1 .. 1 000 000). Both polls must give up, *timed_out = 1 reports that the
 * device's hand-over time-out word was set (it is cleared again), *waited_us the time both polls
 * took together, and the device must stay usable. Needs one GPU only. */
int orion_cuda_selftest_peer_wait(OrionBackend *backend, uint64_t limit_us, uint32_t *timed_out,
                                  uint32_t *waited_us);

/* Reads and clears the time-out words of the backend's device (no reference counterpart): bit 0 the
 * projection GEMM, bit 1 decode attention, bit 2 prefill attention, bit 3 the tensor-parallel
 * hand-over. A set bit means a bounded device-side wait of that kernel family gave up since the last
 * read. orion_cuda_model_forward reads the words itself after every step; a caller that launches
 * kernels through the stand-alone entry points (orion_cuda_paged_decode_attention_noalloc) and wants
 * to know whether one of its launches timed out synchronises its stream and calls this. */
int orion_cuda_poll_wait_timeouts(OrionBackend *backend, uint32_t *mask);

/* CheckpointLoader::open + ModelWeights::load for a whole directory
 * (crates/orion-models/src/loader.rs:112-235, transformer.rs:62-120,180-205): every
 * `*.safetensors` file in name order (the first file wins for a duplicated tensor name),
 * memory-mapped; each tensor the model uses goes from the mapping to the device through
 * orion_cuda_model_load_tensor (this rank's slice only), tensors it does not use are ignored;
 * ends with orion_cuda_model_finalize. `tensors_loaded` may be NULL. */
int orion_cuda_model_load_checkpoint(OrionModel *model, const char *directory, uint64_t *tensors_loaded);
/* ModelWeights::load, one tensor at a time (transformer.rs:62-120). `name` is
 * the Hugging Face tensor name (transformer.rs:12-18); `dtype` the stored type
 * (F32, F16 or BF16, widened or narrowed once at load like loader.rs:74-96);
 * `shape` the FULL, unsharded shape. Under tensor parallelism the rank's
 * column or row slice is taken here. */
int orion_cuda_model_load_tensor(OrionModel *model, const char *name, int dtype,
                                 const uint64_t *shape, int ndim, const void *data);
/* Checks that every required tensor arrived (ModelWeights::load fails on the
 * first missing tensor, transformer.rs:73-118) and resolves the tied head. */
int orion_cuda_model_finalize(OrionModel *model);
/* Seeded random initialisation on the device: every matrix N(0, std), every
 * RMSNorm weight 1.0, biases zero; finalizes the model. Stands in for a
 * checkpoint where none can be shipped (benchmarks at the 8B / 70B shapes). */
int orion_cuda_model_init_random(OrionModel *model, uint64_t seed, float std);

/* LanguageModel::forward (traits.rs:305; transformer.rs:359-442).
 * The arguments are the fields of ForwardBatch (traits.rs:193-210) with the
 * per-array lengths passed separately so that ForwardBatch::validate
 * (traits.rs:232-261) can be applied. block_tables are flattened:
 * table s = block_tables_flat[offsets[s] .. offsets[s+1]).
 * On success writes num_sequences * vocab_size f32 logits, row-major
 * (ForwardOutput, traits.rs:271-277). An empty batch succeeds and writes
 * nothing. No KV slot is written when validation fails. */
int orion_cuda_model_forward(OrionModel *model, const uint32_t *tokens, uint64_t num_tokens,
                             const uint32_t *positions, uint64_t num_positions,
                             const uint64_t *slot_token_counts, uint64_t num_slot_token_counts,
                             const uint64_t *context_lens, uint64_t num_context_lens,
                             const uint32_t *block_tables_flat,
                             const uint64_t *block_table_offsets, uint64_t num_block_tables,
                             uint64_t num_sequences, int has_prefill, float *logits_out,
                             uint64_t logits_capacity);

/* forward + greedy argmax on the device (orion-runtime/src/sampling.rs:196-206:
 * first index of the strict maximum). Writes one token id per sequence; a row
 * with no value above -inf yields UINT32_MAX. logits_out may be NULL. */
int orion_cuda_model_forward_greedy(OrionModel *model, const uint32_t *tokens,
                                    uint64_t num_tokens, const uint32_t *positions,
                                    uint64_t num_positions, const uint64_t *slot_token_counts,
                                    uint64_t num_slot_token_counts, const uint64_t *context_lens,
                                    uint64_t num_context_lens, const uint32_t *block_tables_flat,
                                    const uint64_t *block_table_offsets,
                                    uint64_t num_block_tables, uint64_t num_sequences,
                                    int has_prefill, uint32_t *token_ids_out, float *logits_out,
                                    uint64_t logits_capacity);

/* Replays the previous successful forward on the device without any host<->
 * device copy (inputs and block tables stay resident). Used to time the
 * device-resident step; results land in the model's device logits buffer. */
int orion_cuda_model_replay(OrionModel *model, int iterations, float *elapsed_ms);
/* Timing only (no reference counterpart): replays just the kernels of the
 * categories named by `category_mask` (bit 0 projection GEMMs, bit 1 paged
 * attention, bit 2 elementwise, bit 3 tensor-parallel reductions) back to back
 * on the launching stream, as they run inside a step (programmatic dependent
 * launch included) but without the kernels of the other categories between
 * them. The buffers keep the step's shapes; their contents become meaningless
 * until the next forward. Gives the per-kernel duration the roofline of one
 * kernel family is computed from. */
int orion_cuda_model_replay_categories(OrionModel *model, int iterations, uint32_t category_mask,
                                       float *elapsed_ms);
/* Replays the previous batch with an event pair around every kernel launch and
 * sums device time and launch counts per category: [0] projection GEMMs,
 * [1] paged attention, [2] fused elementwise kernels, [3] tensor-parallel
 * reductions. Accumulated over `iterations` steps. */
int orion_cuda_model_profile(OrionModel *model, int iterations, float category_ms[4],
                             uint64_t category_launches[4]);
/* Fills this rank's KV arena with N(0, std) values (synthetic contexts for
 * benchmarks whose prefill would take too long to run). */
int orion_cuda_model_fill_kv_random(OrionModel *model, uint64_t seed, float std);
/* Kernels launched by the most recent forward / replay iteration. */
int orion_cuda_model_last_launch_count(const OrionModel *model, uint64_t *launches);
/* Copies this rank's KV arena to the host in the reference's logical order
 * [layer][block][k|v][slot][local kv head][dim] as f32 (attention.rs:9-22). */
int orion_cuda_model_read_kv(OrionModel *model, float *out, uint64_t capacity);
/* LanguageModel::metadata (traits.rs:299): returns the descriptor in use. */
int orion_cuda_model_desc(const OrionModel *model, OrionModelDesc *out);

/* Page-locked host memory for ForwardOutput buffers: a logits buffer allocated
 * here is written by DMA directly, a pageable one goes through a bounce copy. */
void *orion_cuda_host_alloc(uint64_t bytes);
void orion_cuda_host_free(void *ptr);
/* Tuning knob: launch the kernels of a step with programmatic dependent launch
 * (each kernel's prologue and weight prefetch overlap its predecessor's tail).
 * On by default; 0 gives plain stream-ordered launches. */
int orion_cuda_set_programmatic_launch(int enabled);
/* Tuning knob of the decode attention kernel: shared-memory ring depth per warp
 * (2, 3 or 4; fewer stages = more CTAs per SM) and the number of CTAs the context
 * split aims for (0 keeps the current value). */
int orion_cuda_attention_set_tuning(int stages, uint32_t cta_target);
/* Tuning knob of the projection GEMM: number of CTAs the split-K planner aims
 * for on decode batches (0 restores the default of two per SM) and the ring
 * layout for token tiles of at most 64 (5 = deep weight ring + short activation ring, the
 * default; 4 = two equal rings; 0 keeps it). */
int orion_cuda_gemm_set_tuning(uint32_t ctas, int small_batch_stages);

/* ---- tensor parallelism (orion-distributed/src/lib.rs) ---- */

/* Shard arithmetic of shard_dimension / ParallelLayout::compute
 * (orion-distributed/src/lib.rs:139-152, 174-208). Each out array receives
 * {start, len}. Refuses uneven splits and world > num_kv_heads. */
int orion_cuda_tp_layout(uint32_t num_attention_heads, uint32_t num_kv_heads, uint32_t ffn_dim,
                         uint32_t rank, uint32_t world, uint64_t query_heads[2],
                         uint64_t kv_heads[2], uint64_t ffn[2]);
/* ncclGetUniqueId for the Collective backing (docs/distributed.md:112-120). */
int orion_cuda_tp_unique_id(uint8_t id[ORION_NCCL_ID_BYTES]);
/* Collective (orion-distributed/src/lib.rs:231-254) backed by NCCL over NVLink, one handle per rank
 * and process, created on the backend's device from the id of orion_cuda_tp_unique_id. Buffers are
 * HOST f32 slices like the trait's (the call uploads, runs the collective on the device and brings
 * the result back); world 1 behaves like SingleRank (lib.rs:257-292): every operation is a copy.
 * all_reduce_sum (lib.rs:243): in place. all_gather (lib.rs:247): out holds world * count_per_rank
 * floats in rank order. reduce_scatter_sum (lib.rs:250): input holds world * count_per_rank floats,
 * out receives this rank's count_per_rank summed floats. barrier (lib.rs:253). A peer that does not
 * answer within the limits described at orion_cuda_tp_selftest_failure_handling ends the call with
 * ORION_ERR_BACKEND. The model's own all-reduces run on device-resident data and do not go through
 * these entry points. */
typedef struct OrionCollective OrionCollective;
int orion_cuda_collective_create(OrionBackend *backend, const uint8_t id[ORION_NCCL_ID_BYTES],
                                 uint32_t rank, uint32_t world, OrionCollective **out);
void orion_cuda_collective_destroy(OrionCollective *collective);
int orion_cuda_collective_all_reduce_sum(OrionCollective *collective, float *buffer, uint64_t count);
int orion_cuda_collective_all_gather(OrionCollective *collective, const float *local,
                                     uint64_t count_per_rank, float *out);
int orion_cuda_collective_reduce_scatter_sum(OrionCollective *collective, const float *input,
                                             uint64_t count_per_rank, float *out);
int orion_cuda_collective_barrier(OrionCollective *collective);

/* Failure handling of the NCCL leg, exercised on the host against a stand-in NCCL (no GPU and no
 * NCCL library are touched; no reference counterpart: the reference's engine loop only states that
 * a failed step is logged and the loop goes on, orion-runtime/src/engine.rs:529-535). The library
 * opens its communicator non-blocking, polls ncclCommGetAsyncError under a host time limit and
 * calls ncclCommAbort when a rank never arrives, a peer dies or a step does not end; the failing
 * call returns ORION_ERR_BACKEND and the communicator refuses further work. Scenarios: 0 healthy
 * group (returns ORION_OK), 1 a rank never joins the rendezvous, 2 a remote error appears while a
 * step is running, 3 a step never ends. `limit_ms` is the time limit used for both waits;
 * *aborted reports whether ncclCommAbort ran, *polls how often the state was polled. The real
 * limits are ORION_TP_INIT_TIMEOUT_S (default 300) and ORION_TP_STEP_TIMEOUT_S (default 60). */
int orion_cuda_tp_selftest_failure_handling(int scenario, uint64_t limit_ms, uint32_t *aborted,
                                            uint64_t *polls);

/* ---- op-level entry points (host buffers in, host buffers out) ----
 * The functions of crates/orion-models/src/tensor.rs and attention.rs run
 * through the same kernels the model uses. `dtype` selects the f32 or the
 * bf16 kernels (bf16: operands are rounded to bf16 on upload, results widened
 * to f32 on download). */

/* tensor::linear (tensor.rs:96-130). */
int orion_cuda_linear(OrionBackend *backend, int dtype, const float *x, uint64_t rows,
                      uint64_t in_features, const float *weight, uint64_t out_features,
                      uint64_t weight_in_features, const float *bias, uint64_t bias_len,
                      float *out);
/* Device-resident timing of the bf16 tensor::linear kernel on N(0,1) operands:
 * mean milliseconds per launch over `iterations` back-to-back launches, and the
 * split-K factor the planner chose. */
int orion_cuda_linear_bench(OrionBackend *backend, uint64_t rows, uint64_t in_features,
                            uint64_t out_features, int warmup, int iterations, float *mean_ms,
                            uint32_t *splits_used);
/* tensor::rms_norm (tensor.rs:143-163), in place. */
int orion_cuda_rms_norm(OrionBackend *backend, int dtype, float *x, uint64_t rows, uint64_t cols,
                        const float *weight, uint64_t weight_len, float eps);
/* tensor::swiglu (tensor.rs:175-189): gate = silu(gate) * up. */
int orion_cuda_swiglu(OrionBackend *backend, int dtype, float *gate, uint64_t gate_rows,
                      uint64_t gate_cols, const float *up, uint64_t up_rows, uint64_t up_cols);
/* RopeTable::new + apply_rope over [rows, heads, head_dim] at positions[rows]
 * (tensor.rs:228-298), in place. */
int orion_cuda_rope(OrionBackend *backend, int dtype, float *x, uint64_t rows, uint64_t heads,
                    uint64_t head_dim, const uint32_t *positions, uint64_t max_positions,
                    float theta);
/* attention::paged_attention for a batch of query rows (attention.rs:219-295).
 * `kv` is an arena in the reference's order [block][k|v][slot][head][dim] for
 * ONE layer; row r attends positions 0..=query_positions[r] through table
 * seq_of_row[r]. */
int orion_cuda_paged_attention(OrionBackend *backend, int dtype, const float *kv,
                               uint64_t num_blocks, uint64_t block_size, uint64_t num_kv_heads,
                               uint64_t head_dim, const float *query, uint64_t rows,
                               uint64_t num_query_heads, const uint32_t *query_positions,
                               const uint32_t *seq_of_row, const uint32_t *block_tables_flat,
                               const uint64_t *block_table_offsets, uint64_t num_sequences,
                               float *out);
/* sampling::argmax per row (orion-runtime/src/sampling.rs:196-206). */
int orion_cuda_argmax(OrionBackend *backend, const float *logits, uint64_t rows, uint64_t cols,
                      uint32_t *out);

/* ---- paged decode attention microbenchmark (device-resident) ----
 * Builds a one-layer bf16 arena of `num_blocks` blocks filled with N(0,1)
 * values from a counter-based generator, `batch` sequences whose block tables
 * are consecutive slices of `block_ids` and whose context lengths are
 * `context_lens`, runs `warmup` + `iterations` launches of the decode kernel
 * and reports the mean launch time. When out/q_host/sample rows are given the
 * result and the inputs of the sampled sequences are copied back for parity
 * checks (the K/V rows of sequence s come back in logical order). */
typedef struct OrionAttnBench OrionAttnBench;
int orion_cuda_attn_bench_create(OrionBackend *backend, uint32_t num_query_heads,
                                 uint32_t num_kv_heads, uint32_t head_dim, uint32_t block_size,
                                 uint64_t num_blocks, const uint32_t *block_ids,
                                 const uint64_t *context_lens, uint32_t batch, uint64_t seed,
                                 OrionAttnBench **out);
int orion_cuda_attn_bench_run(OrionAttnBench *bench, int warmup, int iterations,
                              float *mean_ms, uint64_t *algorithmic_bytes);
/* out: [batch][num_query_heads*head_dim] f32. */
int orion_cuda_attn_bench_output(OrionAttnBench *bench, float *out);
/* q: [num_query_heads*head_dim]; k, v: [context_len][num_kv_heads][head_dim] f32. */
int orion_cuda_attn_bench_sequence(OrionAttnBench *bench, uint32_t seq, float *q, float *k,
                                   float *v);
/* DEVICE pointers of the benchmark's inputs (bf16 q [batch][heads*dim], the bf16
 * arena in the library's layout, and the u32 batch arrays), valid until the
 * handle is destroyed. Any output pointer may be NULL. */
int orion_cuda_attn_bench_device_views(OrionAttnBench *bench, const void **q, const void **kv_arena,
                                       const uint32_t **query_positions, const uint32_t **seq_of_row,
                                       const uint32_t **block_tables_flat,
                                       const uint32_t **block_table_offsets, uint32_t *max_position);
void orion_cuda_attn_bench_destroy(OrionAttnBench *bench);

/* ---- decode attention for callers that cannot allocate ----
 * This entry point has no counterpart in the reference. It is the paged GQA
 * decode attention above (bf16, head_dim 128, 16-token blocks, one query row
 * per sequence) for callers that must not allocate device memory when they
 * call: code between cudaStreamBeginCapture and cudaStreamEndCapture, a serving
 * loop whose memory all belongs to somebody else's pool, a plugin that is
 * handed buffers and a stream and nothing more. It never calls cudaMalloc,
 * cudaFree or any allocating routine.
 *
 * All pointers are DEVICE pointers owned by the caller: q and out are bf16
 * [rows][num_query_heads*128]; kv_arena is ONE layer in the library's layout
 * ([block][kv head][k|v][slot][dim], 16-byte groups of a row XOR-permuted by
 * slot & 7); the u32 arrays are as in orion_cuda_paged_attention. `stream` is
 * a cudaStream_t (NULL = the default stream). `splits` is how many pieces each
 * context is cut into (0 = chosen like the allocating path does).
 *
 * The per-split partial results live in a fixed 16 MiB array inside the
 * library (held by every GPU that loads it until the process exits): 16 Ki
 * arrival counters followed by the partials. A call needing more —
 * 16384 + rows * num_query_heads * splits * 130 floats > 4 Mi floats — is
 * rejected with ORION_ERR_INVALID_REQUEST; splits == 1 needs none.
 * The first call on a device looks the array's address up and opts the kernel
 * in to its shared-memory size on that device; make that first call before
 * starting any stream capture. Every call on a device shares the one array:
 * calls whose kernels can overlap on the GPU (different streams without
 * ordering between them) race on it and must be serialised by the caller. The
 * array needs no clearing between calls: each call overwrites every partial
 * slot it later reads, and the counters start at zero when the library is
 * loaded and are put back to zero by the launch that used them.
 *
 * `device` is made current for the duration of the call and the caller's
 * current device is put back before returning. Nothing the pointers refer to is
 * validated: block ids must be below num_blocks, every table must cover
 * query_positions[r] / 16 + 1 entries and max_position must be the largest
 * query position, or the kernel reads outside the arena (the model's forward
 * checks these on the host; this entry point cannot, the arrays are on the
 * device). The call only enqueues work. A bounded wait inside the kernel that
 * gives up is recorded in the device's time-out word, which this call does not
 * read: synchronise the stream and ask orion_cuda_poll_wait_timeouts (bit 1),
 * otherwise the next orion_cuda_model_forward on that device reports it. */
int orion_cuda_paged_decode_attention_noalloc(
    int device, const void *q, const void *kv_arena, uint32_t num_blocks, uint32_t num_kv_heads,
    uint32_t num_query_heads, const uint32_t *query_positions, const uint32_t *seq_of_row,
    const uint32_t *block_tables_flat, const uint32_t *block_table_offsets, uint32_t rows,
    uint32_t max_position, uint32_t splits, void *out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ORION_CUDA_H */
