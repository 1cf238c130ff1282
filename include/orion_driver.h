/* C ABI of the host-side driver: KV-cache manager, continuous-batching scheduler and the
 * engine step that feeds the device forward pass. The reference has no FFI for these (they are
 * Rust types called directly); each entry point names the reference routine it restates, so a
 * Rust maintainer could bind them 1:1 or, more likely, keep the Rust originals and use this
 * library's engine only where the whole step loop moves next to the GPU.
 *
 * Conventions are those of orion_cuda.h: opaque handles, plain pointers and sizes, status codes
 * with the message in orion_cuda_last_error(), no exceptions across the boundary, one caller
 * thread per handle (the reference's manager and scheduler are `&mut self` types owned by the
 * single engine thread: crates/orion-kv-cache/src/manager.rs:9-16). */
#ifndef ORION_DRIVER_H
#define ORION_DRIVER_H

#include <stdint.h>

#include "orion_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct OrionKvManager OrionKvManager;
typedef struct OrionScheduler OrionScheduler;
typedef struct OrionEngine OrionEngine;

/* AllocationOutcome (manager.rs:26-36) */
typedef struct OrionAllocationOutcome {
  uint64_t allocated, reused, cached_tokens;
} OrionAllocationOutcome;

/* CacheStats (manager.rs:46-56) */
typedef struct OrionCacheStats {
  uint64_t total_blocks, used_blocks, free_blocks, block_size, num_sequences, prefix_cache_entries;
  uint64_t prefix_cache_hits, prefix_cache_misses;
} OrionCacheStats;

/* SchedulerConfig (crates/orion-core/src/config.rs:107-156). max_model_len and
 * request_timeout_secs: 0 = None. Defaults of the reference: 256, 8192, None, chunked, 1024,
 * Some(300), decode first.
 * skip_cached_prefix has no reference counterpart (the reference shares cached blocks but
 * recomputes them, manager.rs:449-451): non-zero starts a new sequence's prefill after the tokens
 * whose blocks came from the prefix cache. 0 = the reference's behaviour.
 * logical_decode_positions has none either: non-zero feeds a decode token at position
 * total_len - 1, its logical place, instead of the reference's total_len (scheduler.rs:283), so
 * that no cache slot is skipped and no step is refused. 0 = the reference's behaviour. */
typedef struct OrionSchedulerConfig {
  uint64_t max_num_seqs, max_num_batched_tokens, max_model_len;
  uint32_t enable_chunked_prefill;
  uint64_t max_waiting_requests, request_timeout_secs;
  uint32_t prioritize_decode;
  uint32_t skip_cached_prefix;
  uint32_t logical_decode_positions;
} OrionSchedulerConfig;

/* SamplingParams (crates/orion-core/src/sampling.rs:25-70), the fields the driver reads. */
typedef struct OrionSamplingParams {
  float temperature, top_p, repetition_penalty;
  uint64_t top_k, max_tokens, min_tokens;
  const uint32_t *stop_token_ids;
  uint64_t num_stop_token_ids;
} OrionSamplingParams;

/* ScheduledSequence (crates/orion-scheduler/src/scheduler.rs:36-50) */
typedef struct OrionScheduledSequence {
  uint64_t id, num_tokens, start_position;
  uint32_t is_prefill;
} OrionScheduledSequence;

/* SchedulerStats (scheduler.rs:99-109) */
typedef struct OrionSchedulerStats {
  uint64_t total_steps, total_admitted, total_finished, total_preempted, total_rejected;
  uint64_t total_batched_tokens, total_prefill_tokens, total_decode_tokens;
  uint64_t total_skipped_prefill_tokens; /* only with skip_cached_prefix */
} OrionSchedulerStats;

/* FinishReason (crates/orion-core/src/sequence.rs:73-87) */
enum { ORION_FINISH_NONE = 0, ORION_FINISH_STOP = 1, ORION_FINISH_LENGTH = 2, ORION_FINISH_CANCELLED = 3,
       ORION_FINISH_TIMEOUT = 4, ORION_FINISH_ERROR = 5 };
/* SequenceState (sequence.rs:26-37) */
enum { ORION_SEQ_WAITING = 0, ORION_SEQ_PREFILLING = 1, ORION_SEQ_DECODING = 2, ORION_SEQ_FINISHED = 3 };

/* StreamEvent (crates/orion-runtime/src/engine.rs:60-90); kind 0 = Token, 1 = Done. */
typedef struct OrionEngineEvent {
  uint64_t id;
  uint32_t kind, token;
  uint64_t index;
  uint32_t reason;
  uint64_t prompt_tokens, completion_tokens;
} OrionEngineEvent;

/* hash_block (crates/orion-kv-cache/src/table.rs:105-120) */
uint64_t orion_hash_block(int has_parent, uint64_t parent, const uint32_t *tokens, uint64_t num_tokens);
/* The id the next sequence will get (SequenceId::next, crates/orion-core/src/id.rs:52-55). */
uint64_t orion_sequence_id_peek(void);

/* ---- KvCacheManager (crates/orion-kv-cache/src/manager.rs:85-425) ---- */
OrionKvManager *orion_kv_manager_create(uint64_t num_blocks, uint64_t block_size, int prefix_caching_enabled);
void orion_kv_manager_destroy(OrionKvManager *m);
int orion_kv_manager_allocate(OrionKvManager *m, uint64_t seq, const uint32_t *prompt, uint64_t num_tokens,
                              OrionAllocationOutcome *outcome);                       /* :163-250 */
void orion_kv_manager_commit_prefill(OrionKvManager *m, uint64_t seq, const uint32_t *prompt, uint64_t num_tokens); /* :258-283 */
int orion_kv_manager_append_token(OrionKvManager *m, uint64_t seq);                    /* :290-335 */
void orion_kv_manager_free(OrionKvManager *m, uint64_t seq);                           /* :341-359 */
uint64_t orion_kv_manager_preempt(OrionKvManager *m, uint64_t seq);                    /* :368-376 */
int orion_kv_manager_stats(const OrionKvManager *m, OrionCacheStats *out);             /* :110-121 */
int orion_kv_manager_can_allocate(const OrionKvManager *m, uint64_t num_tokens);       /* :158-160, 1 = yes */
uint64_t orion_kv_manager_blocks_needed_for(const OrionKvManager *m, uint64_t num_tokens); /* :153-155 */
uint64_t orion_kv_manager_evict_cached(OrionKvManager *m, uint64_t count);             /* :397-409 */
void orion_kv_manager_clear_prefix_cache(OrionKvManager *m);                           /* :412-416 */
uint64_t orion_kv_manager_num_evictable(const OrionKvManager *m);                      /* :419-421 */
/* raw_block_table (:379-381). Returns 1 and fills the outputs when `seq` holds a table (at most
 * `capacity` ids are written, `num_blocks` is the full count), 0 otherwise. */
int orion_kv_manager_block_table(const OrionKvManager *m, uint64_t seq, uint32_t *blocks, uint64_t capacity,
                                 uint64_t *num_blocks, uint64_t *num_tokens);
/* Block::{ref_count,num_tokens,hash} (block.rs:23-36). Returns 0 for an unknown id. */
int orion_kv_manager_block_info(const OrionKvManager *m, uint32_t block, uint32_t *ref_count, uint64_t *num_tokens,
                                int *has_hash, uint64_t *hash);
/* FakeCache::fail_next_{append,allocate} (crates/orion-scheduler/src/testing.rs:29-37): host-side
 * fault injection; the next append (which = 0) or allocate (which = 1) fails with CacheExhausted. */
void orion_kv_manager_fail_next(OrionKvManager *m, int which);

/* ---- Scheduler (crates/orion-scheduler/src/scheduler.rs:127-580) ---- */
OrionScheduler *orion_scheduler_create(const OrionSchedulerConfig *config, uint64_t num_blocks, uint64_t block_size,
                                       int prefix_caching_enabled);
void orion_scheduler_destroy(OrionScheduler *s);
/* The scheduler's own cache manager; borrowed, valid while the scheduler lives (never destroy it). */
OrionKvManager *orion_scheduler_cache(OrionScheduler *s);
int orion_scheduler_add_request(OrionScheduler *s, const uint32_t *prompt, uint64_t num_tokens,
                                const OrionSamplingParams *params, uint64_t *id);        /* :174-214 */
int orion_scheduler_cancel(OrionScheduler *s, uint64_t id);                              /* :226-236, 1 = found */
/* schedule (:239-263). Writes at most the given capacities; the counts are the full sizes. */
int orion_scheduler_schedule(OrionScheduler *s, OrionScheduledSequence *scheduled, uint64_t scheduled_capacity,
                             uint64_t *num_scheduled, uint64_t *preempted, uint64_t preempted_capacity,
                             uint64_t *num_preempted);
/* on_token (:476-507): returns the ORION_FINISH_* reason (NONE while the sequence goes on). */
int orion_scheduler_on_token(OrionScheduler *s, uint64_t id, uint32_t token, const uint32_t *eos_ids, uint64_t num_eos);
uint64_t orion_scheduler_reap_finished(OrionScheduler *s, uint64_t *ids, uint64_t capacity); /* :513-520 */
void orion_scheduler_commit_prefill(OrionScheduler *s, uint64_t id);                    /* :557-564 */
uint64_t orion_scheduler_num_waiting(const OrionScheduler *s);
uint64_t orion_scheduler_num_running(const OrionScheduler *s);
int orion_scheduler_stats(const OrionScheduler *s, OrionSchedulerStats *out);
/* running_sequence (:552-554): 1 and the fields of a running sequence, else 0. */
int orion_scheduler_running_sequence(const OrionScheduler *s, uint64_t id, int *state, uint64_t *computed_prefix_len,
                                     uint64_t *output_len);

/* ---- Engine (crates/orion-runtime/src/engine.rs:186-487) ---- */
/* Greedy forward used instead of a device model (tests, other backends): receives the batch
 * exactly as orion_cuda_model_forward_greedy would, plus the sequence ids, and writes one token
 * id per sequence. Returns an OrionStatus. */
typedef int (*OrionForwardFn)(void *user, const uint32_t *tokens, uint64_t num_tokens, const uint32_t *positions,
                              const uint64_t *sequence_ids, const uint64_t *slot_token_counts,
                              const uint64_t *context_lens, const uint32_t *block_tables_flat,
                              const uint64_t *block_table_offsets, uint64_t num_sequences, int has_prefill,
                              uint32_t *token_ids_out);
/* Exactly one of `model` and `forward` is given. With a model every step runs
 * orion_cuda_model_forward_greedy (argmax on the device, 4 bytes per sequence come back). */
OrionEngine *orion_engine_create(OrionModel *model, OrionForwardFn forward, void *user,
                                 const OrionSchedulerConfig *config, uint64_t num_blocks, uint64_t block_size,
                                 int prefix_caching_enabled, const uint32_t *eos_ids, uint64_t num_eos);
void orion_engine_destroy(OrionEngine *e);
OrionScheduler *orion_engine_scheduler(OrionEngine *e); /* borrowed */
int orion_engine_submit(OrionEngine *e, const uint32_t *prompt, uint64_t num_tokens, const OrionSamplingParams *params,
                        uint64_t *id);                                                   /* :235-268 */
void orion_engine_cancel(OrionEngine *e, uint64_t id);                                   /* :271-281 */
int orion_engine_has_work(const OrionEngine *e);                                         /* :284-286 */
/* step (:293-342): `ran` = sequences in the batch. A forward error is returned with the scheduler
 * and cache already advanced; the caller logs it and steps again (engine.rs:531-536). */
int orion_engine_step(OrionEngine *e, uint64_t *ran);
/* Moves up to `capacity` pending events out, oldest first; returns how many were written. */
uint64_t orion_engine_take_events(OrionEngine *e, OrionEngineEvent *events, uint64_t capacity);
uint64_t orion_engine_num_active(const OrionEngine *e);
/* The batch the last step built (build_batch, :429-487). Pointers are borrowed and valid until
 * the next step. */
int orion_engine_last_batch(const OrionEngine *e, const uint32_t **tokens, uint64_t *num_tokens,
                            const uint32_t **positions, const uint64_t **sequence_ids,
                            const uint64_t **slot_token_counts, const uint64_t **context_lens,
                            const uint32_t **block_tables_flat, const uint64_t **block_table_offsets,
                            uint64_t *num_sequences, int *has_prefill);

#ifdef __cplusplus
}
#endif
#endif /* ORION_DRIVER_H */
