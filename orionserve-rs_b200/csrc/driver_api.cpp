// C ABI of the driver (include/orion_driver.h) over the C++ classes of driver.h.
#include <memory>

#include "common.cuh"
#include "driver.h"
#include "model.h"
#include "../../include/orion_driver.h"

using namespace orion;
using namespace orion::driver;

struct OrionKvManager {
  KvCacheManager *p = nullptr;                // the manager spoken to
  std::unique_ptr<KvCacheManager> owned;      // set when this handle created it
};
struct OrionScheduler {
  Scheduler *p = nullptr;
  std::unique_ptr<Scheduler> owned;
  OrionKvManager cache;                       // borrowed view of p->cache()
};
struct OrionEngine {
  std::unique_ptr<Engine> impl;
  OrionScheduler sched;                       // borrowed view of impl->scheduler()
  std::vector<EngineEvent> pending;           // events that did not fit the caller's buffer yet
};

namespace {

SchedulerConfig to_config(const OrionSchedulerConfig *c) {
  SchedulerConfig out;  // the reference's defaults
  if (!c) return out;
  out.max_num_seqs = c->max_num_seqs;
  out.max_num_batched_tokens = c->max_num_batched_tokens;
  out.max_model_len = c->max_model_len ? std::optional<size_t>(c->max_model_len) : std::nullopt;
  out.enable_chunked_prefill = c->enable_chunked_prefill != 0;
  out.max_waiting_requests = c->max_waiting_requests;
  out.request_timeout_secs = c->request_timeout_secs ? std::optional<uint64_t>(c->request_timeout_secs) : std::nullopt;
  out.prioritize_decode = c->prioritize_decode != 0;
  out.skip_cached_prefix = c->skip_cached_prefix != 0;
  out.logical_decode_positions = c->logical_decode_positions != 0;
  return out;
}

SamplingParams to_params(const OrionSamplingParams *p) {
  SamplingParams out;  // the reference's defaults
  if (!p) return out;
  out.temperature = p->temperature;
  out.top_p = p->top_p;
  out.repetition_penalty = p->repetition_penalty;
  out.top_k = p->top_k;
  out.max_tokens = p->max_tokens;
  out.min_tokens = p->min_tokens;
  if (p->stop_token_ids) out.stop_token_ids.assign(p->stop_token_ids, p->stop_token_ids + p->num_stop_token_ids);
  return out;
}

int null_handle() { return set_error(ORION_ERR_INVALID_REQUEST, "null handle"); }

}  // namespace

extern "C" {

uint64_t orion_hash_block(int has_parent, uint64_t parent, const uint32_t *tokens, uint64_t num_tokens) {
  return hash_block(has_parent ? std::optional<BlockHash>(parent) : std::nullopt, tokens, num_tokens);
}
uint64_t orion_sequence_id_peek(void) { return peek_sequence_id(); }

// ---- manager -----------------------------------------------------------------------------------

OrionKvManager *orion_kv_manager_create(uint64_t num_blocks, uint64_t block_size, int prefix_caching_enabled) {
  clear_error();
  if (block_size == 0) {
    set_error(ORION_ERR_INVALID_REQUEST, "block_size must be non-zero");
    return nullptr;
  }
  auto *h = new OrionKvManager;
  h->owned.reset(new KvCacheManager(num_blocks, block_size, prefix_caching_enabled != 0));
  h->p = h->owned.get();
  return h;
}
void orion_kv_manager_destroy(OrionKvManager *m) {
  if (m && m->owned) delete m;  // borrowed views belong to their scheduler
}
int orion_kv_manager_allocate(OrionKvManager *m, uint64_t seq, const uint32_t *prompt, uint64_t num_tokens,
                              OrionAllocationOutcome *outcome) {
  clear_error();
  if (!m) return null_handle();
  AllocationOutcome out;
  ORION_TRY(m->p->allocate(seq, prompt, num_tokens, &out));
  if (outcome) *outcome = OrionAllocationOutcome{out.allocated, out.reused, out.cached_tokens};
  return ORION_OK;
}
void orion_kv_manager_commit_prefill(OrionKvManager *m, uint64_t seq, const uint32_t *prompt, uint64_t num_tokens) {
  if (m) m->p->commit_prefill(seq, prompt, num_tokens);
}
int orion_kv_manager_append_token(OrionKvManager *m, uint64_t seq) {
  clear_error();
  return m ? m->p->append_token(seq) : null_handle();
}
void orion_kv_manager_free(OrionKvManager *m, uint64_t seq) {
  if (m) m->p->free(seq);
}
uint64_t orion_kv_manager_preempt(OrionKvManager *m, uint64_t seq) { return m ? m->p->preempt(seq) : 0; }
int orion_kv_manager_stats(const OrionKvManager *m, OrionCacheStats *out) {
  clear_error();
  if (!m || !out) return null_handle();
  const CacheStats s = m->p->stats();
  *out = OrionCacheStats{s.total_blocks, s.used_blocks, s.free_blocks, s.block_size, s.num_sequences,
                         s.prefix_cache_entries, s.prefix_cache_hits, s.prefix_cache_misses};
  return ORION_OK;
}
int orion_kv_manager_can_allocate(const OrionKvManager *m, uint64_t num_tokens) {
  return m && m->p->can_allocate(num_tokens) ? 1 : 0;
}
uint64_t orion_kv_manager_blocks_needed_for(const OrionKvManager *m, uint64_t num_tokens) {
  return m ? m->p->blocks_needed_for(num_tokens) : 0;
}
uint64_t orion_kv_manager_evict_cached(OrionKvManager *m, uint64_t count) { return m ? m->p->evict_cached(count) : 0; }
void orion_kv_manager_clear_prefix_cache(OrionKvManager *m) {
  if (m) m->p->clear_prefix_cache();
}
uint64_t orion_kv_manager_num_evictable(const OrionKvManager *m) { return m ? m->p->num_evictable() : 0; }
int orion_kv_manager_block_table(const OrionKvManager *m, uint64_t seq, uint32_t *blocks, uint64_t capacity,
                                 uint64_t *num_blocks, uint64_t *num_tokens) {
  if (!m) return 0;
  const BlockTable *t = m->p->block_table(seq);
  if (!t) return 0;
  if (num_blocks) *num_blocks = t->blocks.size();
  if (num_tokens) *num_tokens = t->num_tokens;
  if (blocks)
    for (size_t i = 0; i < t->blocks.size() && i < capacity; ++i) blocks[i] = t->blocks[i];
  return 1;
}
int orion_kv_manager_block_info(const OrionKvManager *m, uint32_t block, uint32_t *ref_count, uint64_t *num_tokens,
                                int *has_hash, uint64_t *hash) {
  if (!m) return 0;
  const Block *b = m->p->pool().get(block);
  if (!b) return 0;
  if (ref_count) *ref_count = b->ref_count;
  if (num_tokens) *num_tokens = b->num_tokens;
  if (has_hash) *has_hash = b->hash.has_value();
  if (hash) *hash = b->hash.value_or(0);
  return 1;
}
void orion_kv_manager_fail_next(OrionKvManager *m, int which) {
  if (!m) return;
  if (which == 0) m->p->fail_next_append();
  else m->p->fail_next_allocate();
}

// ---- scheduler ---------------------------------------------------------------------------------

OrionScheduler *orion_scheduler_create(const OrionSchedulerConfig *config, uint64_t num_blocks, uint64_t block_size,
                                       int prefix_caching_enabled) {
  clear_error();
  if (block_size == 0) {
    set_error(ORION_ERR_INVALID_REQUEST, "block_size must be non-zero");
    return nullptr;
  }
  auto *h = new OrionScheduler;
  h->owned.reset(new Scheduler(to_config(config), KvCacheManager(num_blocks, block_size, prefix_caching_enabled != 0)));
  h->p = h->owned.get();
  h->cache.p = &h->p->cache();
  return h;
}
void orion_scheduler_destroy(OrionScheduler *s) {
  if (s && s->owned) delete s;
}
OrionKvManager *orion_scheduler_cache(OrionScheduler *s) { return s ? &s->cache : nullptr; }
int orion_scheduler_add_request(OrionScheduler *s, const uint32_t *prompt, uint64_t num_tokens,
                                const OrionSamplingParams *params, uint64_t *id) {
  clear_error();
  if (!s) return null_handle();
  SequenceId sid = 0;
  ORION_TRY(s->p->add_request(Sequence(std::vector<TokenId>(prompt, prompt + num_tokens), to_params(params)), &sid));
  if (id) *id = sid;
  return ORION_OK;
}
int orion_scheduler_cancel(OrionScheduler *s, uint64_t id) { return s && s->p->cancel(id) ? 1 : 0; }
int orion_scheduler_schedule(OrionScheduler *s, OrionScheduledSequence *scheduled, uint64_t scheduled_capacity,
                             uint64_t *num_scheduled, uint64_t *preempted, uint64_t preempted_capacity,
                             uint64_t *num_preempted) {
  clear_error();
  if (!s) return null_handle();
  const SchedulerOutput out = s->p->schedule();
  if (num_scheduled) *num_scheduled = out.scheduled.size();
  if (num_preempted) *num_preempted = out.preempted.size();
  if (scheduled)
    for (size_t i = 0; i < out.scheduled.size() && i < scheduled_capacity; ++i) {
      const ScheduledSequence &x = out.scheduled[i];
      scheduled[i] = OrionScheduledSequence{x.id, x.num_tokens, x.start_position, x.is_prefill ? 1u : 0u};
    }
  if (preempted)
    for (size_t i = 0; i < out.preempted.size() && i < preempted_capacity; ++i) preempted[i] = out.preempted[i];
  return ORION_OK;
}
int orion_scheduler_on_token(OrionScheduler *s, uint64_t id, uint32_t token, const uint32_t *eos_ids, uint64_t num_eos) {
  if (!s) return ORION_FINISH_NONE;
  const std::vector<TokenId> eos(eos_ids, eos_ids + (eos_ids ? num_eos : 0));
  return (int)s->p->on_token(id, token, eos);
}
uint64_t orion_scheduler_reap_finished(OrionScheduler *s, uint64_t *ids, uint64_t capacity) {
  if (!s) return 0;
  const std::vector<Sequence> done = s->p->reap_finished();
  if (ids)
    for (size_t i = 0; i < done.size() && i < capacity; ++i) ids[i] = done[i].id();
  return done.size();
}
void orion_scheduler_commit_prefill(OrionScheduler *s, uint64_t id) {
  if (s) s->p->commit_prefill(id);
}
uint64_t orion_scheduler_num_waiting(const OrionScheduler *s) { return s ? s->p->num_waiting() : 0; }
uint64_t orion_scheduler_num_running(const OrionScheduler *s) { return s ? s->p->num_running() : 0; }
int orion_scheduler_stats(const OrionScheduler *s, OrionSchedulerStats *out) {
  clear_error();
  if (!s || !out) return null_handle();
  const SchedulerStats &t = s->p->stats();
  *out = OrionSchedulerStats{t.total_steps,    t.total_admitted,       t.total_finished,       t.total_preempted,
                             t.total_rejected, t.total_batched_tokens, t.total_prefill_tokens, t.total_decode_tokens,
                             t.total_skipped_prefill_tokens};
  return ORION_OK;
}
int orion_scheduler_running_sequence(const OrionScheduler *s, uint64_t id, int *state, uint64_t *computed_prefix_len,
                                     uint64_t *output_len) {
  if (!s) return 0;
  const Sequence *seq = s->p->running_sequence(id);
  if (!seq) return 0;
  if (state) *state = (int)seq->state();
  if (computed_prefix_len) *computed_prefix_len = seq->computed_prefix_len();
  if (output_len) *output_len = seq->output_len();
  return 1;
}

// ---- engine ------------------------------------------------------------------------------------

OrionEngine *orion_engine_create(OrionModel *model, OrionForwardFn forward, void *user,
                                 const OrionSchedulerConfig *config, uint64_t num_blocks, uint64_t block_size,
                                 int prefix_caching_enabled, const uint32_t *eos_ids, uint64_t num_eos) {
  clear_error();
  if ((model != nullptr) == (forward != nullptr)) {
    set_error(ORION_ERR_INVALID_REQUEST, "give the engine either a device model or a forward function");
    return nullptr;
  }
  if (block_size == 0) {
    set_error(ORION_ERR_INVALID_REQUEST, "block_size must be non-zero");
    return nullptr;
  }
  ForwardFn fn;
  if (model) {
    ModelBase *impl = model->impl.get();
    fn = [impl](const HostBatch &b, uint32_t *token_ids) -> int {
      BatchView v{};
      v.tokens = b.tokens.data();
      v.num_tokens = b.tokens.size();
      v.positions = b.positions.data();
      v.num_positions = b.positions.size();
      v.slot_token_counts = b.slot_token_counts.data();
      v.num_slot_token_counts = b.slot_token_counts.size();
      v.context_lens = b.context_lens.data();
      v.num_context_lens = b.context_lens.size();
      v.block_tables_flat = b.block_tables_flat.data();
      v.block_table_offsets = b.block_table_offsets.data();
      v.num_block_tables = b.sequence_ids.size();
      v.num_sequences = b.sequence_ids.size();
      v.has_prefill = b.has_prefill ? 1 : 0;
      return impl->forward(v, nullptr, 0, token_ids);
    };
  } else {
    fn = [forward, user](const HostBatch &b, uint32_t *token_ids) -> int {
      return forward(user, b.tokens.data(), b.tokens.size(), b.positions.data(), b.sequence_ids.data(),
                     b.slot_token_counts.data(), b.context_lens.data(), b.block_tables_flat.data(),
                     b.block_table_offsets.data(), b.sequence_ids.size(), b.has_prefill ? 1 : 0, token_ids);
    };
  }
  auto *h = new OrionEngine;
  h->impl.reset(new Engine(Scheduler(to_config(config), KvCacheManager(num_blocks, block_size, prefix_caching_enabled != 0)),
                           std::move(fn), std::vector<TokenId>(eos_ids, eos_ids + (eos_ids ? num_eos : 0))));
  h->sched.p = &h->impl->scheduler();
  h->sched.cache.p = &h->sched.p->cache();
  return h;
}
void orion_engine_destroy(OrionEngine *e) { delete e; }
OrionScheduler *orion_engine_scheduler(OrionEngine *e) { return e ? &e->sched : nullptr; }
int orion_engine_submit(OrionEngine *e, const uint32_t *prompt, uint64_t num_tokens, const OrionSamplingParams *params,
                        uint64_t *id) {
  clear_error();
  if (!e) return null_handle();
  SequenceId sid = 0;
  ORION_TRY(e->impl->submit(std::vector<TokenId>(prompt, prompt + num_tokens), to_params(params), &sid));
  if (id) *id = sid;
  return ORION_OK;
}
void orion_engine_cancel(OrionEngine *e, uint64_t id) {
  if (e) e->impl->cancel(id);
}
int orion_engine_has_work(const OrionEngine *e) { return e && e->impl->has_work() ? 1 : 0; }
int orion_engine_step(OrionEngine *e, uint64_t *ran) {
  clear_error();
  if (!e) return null_handle();
  size_t n = 0;
  const int rc = e->impl->step(&n);
  if (ran) *ran = n;
  return rc;
}
uint64_t orion_engine_take_events(OrionEngine *e, OrionEngineEvent *events, uint64_t capacity) {
  if (!e || !events) return 0;
  std::vector<EngineEvent> &pending = e->pending;  // events beyond `capacity` wait for the next call
  std::vector<EngineEvent> fresh = e->impl->take_events();
  pending.insert(pending.end(), fresh.begin(), fresh.end());
  const size_t n = std::min<size_t>(pending.size(), capacity);
  for (size_t i = 0; i < n; ++i) {
    const EngineEvent &x = pending[i];
    events[i] = OrionEngineEvent{x.id, x.kind, x.token, x.index, x.reason, x.prompt_tokens, x.completion_tokens};
  }
  pending.erase(pending.begin(), pending.begin() + (ptrdiff_t)n);
  return n;
}
uint64_t orion_engine_num_active(const OrionEngine *e) { return e ? e->impl->num_active() : 0; }
int orion_engine_last_batch(const OrionEngine *e, const uint32_t **tokens, uint64_t *num_tokens,
                            const uint32_t **positions, const uint64_t **sequence_ids,
                            const uint64_t **slot_token_counts, const uint64_t **context_lens,
                            const uint32_t **block_tables_flat, const uint64_t **block_table_offsets,
                            uint64_t *num_sequences, int *has_prefill) {
  clear_error();
  if (!e) return null_handle();
  const HostBatch &b = e->impl->last_batch();
  if (tokens) *tokens = b.tokens.data();
  if (num_tokens) *num_tokens = b.tokens.size();
  if (positions) *positions = b.positions.data();
  if (sequence_ids) *sequence_ids = b.sequence_ids.data();
  if (slot_token_counts) *slot_token_counts = b.slot_token_counts.data();
  if (context_lens) *context_lens = b.context_lens.data();
  if (block_tables_flat) *block_tables_flat = b.block_tables_flat.data();
  if (block_table_offsets) *block_table_offsets = b.block_table_offsets.data();
  if (num_sequences) *num_sequences = b.sequence_ids.size();
  if (has_prefill) *has_prefill = b.has_prefill ? 1 : 0;
  return ORION_OK;
}

}  // extern "C"
