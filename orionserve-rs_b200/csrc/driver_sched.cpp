// Sequences, the continuous-batching scheduler and the engine step of the driver.
#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "driver.h"

namespace orion {
namespace driver {

// ---- SamplingParams / Sequence ---------------------------------------------------------------

int SamplingParams::validate() const {  // sampling.rs:85-134 (the checks on the fields kept here)
  if (!std::isfinite(temperature) || temperature < 0.0f)
    return set_error(ORION_ERR_INVALID_REQUEST, "invalid request: temperature must be a finite value >= 0.0, got %g",
                     (double)temperature);
  if (!std::isfinite(top_p) || top_p <= 0.0f || top_p > 1.0f)
    return set_error(ORION_ERR_INVALID_REQUEST, "invalid request: top_p must be in (0.0, 1.0], got %g", (double)top_p);
  if (!std::isfinite(repetition_penalty) || repetition_penalty <= 0.0f)
    return set_error(ORION_ERR_INVALID_REQUEST,
                     "invalid request: repetition_penalty must be a finite value > 0.0, got %g", (double)repetition_penalty);
  if (max_tokens == 0) return set_error(ORION_ERR_INVALID_REQUEST, "invalid request: max_tokens must be at least 1");
  if (min_tokens > max_tokens)
    return set_error(ORION_ERR_INVALID_REQUEST, "invalid request: min_tokens (%zu) must not exceed max_tokens (%zu)",
                     min_tokens, max_tokens);
  return ORION_OK;
}

Sequence::Sequence(std::vector<TokenId> prompt, SamplingParams params)  // sequence.rs:178-189
    : id_(next_sequence_id()), prompt_(std::move(prompt)), params_(std::move(params)),
      arrived_at_(std::chrono::steady_clock::now()) {}

bool Sequence::can_transition(SequenceState from, SequenceState to) {  // sequence.rs:41-55
  using S = SequenceState;
  switch (from) {
    case S::Waiting: return to == S::Prefilling || to == S::Finished;
    case S::Prefilling: return to == S::Prefilling || to == S::Decoding || to == S::Waiting || to == S::Finished;
    case S::Decoding: return to == S::Decoding || to == S::Waiting || to == S::Finished;
    case S::Finished: return false;
  }
  return false;
}

bool Sequence::transition_to(SequenceState next) {  // sequence.rs:255-264
  if (!can_transition(state_, next)) return false;
  state_ = next;
  return true;
}

void Sequence::advance_prefill(size_t n) {  // sequence.rs:270-272
  computed_prefix_len_ = std::min(computed_prefix_len_ + n, prompt_.size());
}

void Sequence::finish(FinishReason reason) {  // sequence.rs:286-293: the first reason wins
  if (state_ == SequenceState::Finished) return;
  state_ = SequenceState::Finished;
  finish_reason_ = reason;
}

bool Sequence::preempt() {  // sequence.rs:303-310: prefill progress is dropped, generated tokens are kept
  if (!can_transition(state_, SequenceState::Waiting)) return false;
  state_ = SequenceState::Waiting;
  computed_prefix_len_ = 0;
  return true;
}

// ---- Scheduler -------------------------------------------------------------------------------

size_t SchedulerOutput::num_batched_tokens() const {
  size_t n = 0;
  for (const ScheduledSequence &s : scheduled) n += s.num_tokens;
  return n;
}

Scheduler::Scheduler(SchedulerConfig config, KvCacheManager cache) : config_(config), cache_(std::move(cache)) {}

int Scheduler::add_request(Sequence seq, SequenceId *id) {  // scheduler.rs:174-214
  if (waiting_.size() >= config_.max_waiting_requests) {
    stats_.total_rejected += 1;
    return set_error(ORION_ERR_QUEUE_FULL, "server at capacity: %zu requests already waiting (limit %zu)", waiting_.size(),
                     config_.max_waiting_requests);
  }
  const size_t max_len = config_.max_model_len ? *config_.max_model_len : SIZE_MAX;
  const size_t needed = seq.prompt_len() + seq.params().max_tokens;
  if (needed > max_len) {
    stats_.total_rejected += 1;
    return set_error(ORION_ERR_CONTEXT_LENGTH,
                     "prompt of %zu tokens plus %zu requested output exceeds context length %zu", seq.prompt_len(),
                     seq.params().max_tokens, max_len);
  }
  // a prompt larger than the whole cache would block the queue head forever
  const size_t blocks = cache_.blocks_needed_for(seq.prompt_len());
  if (blocks > cache_.total_blocks()) {
    stats_.total_rejected += 1;
    return set_error(ORION_ERR_CACHE_EXHAUSTED, "KV cache exhausted: needed %zu blocks, %zu free", blocks,
                     cache_.total_blocks());
  }
  if (id) *id = seq.id();
  waiting_.push_back(std::move(seq));
  stats_.total_admitted += 1;
  return ORION_OK;
}

Sequence *Scheduler::running_mut(SequenceId id) {
  for (Sequence &s : running_)
    if (s.id() == id) return &s;
  return nullptr;
}

const Sequence *Scheduler::running_sequence(SequenceId id) const {
  for (const Sequence &s : running_)
    if (s.id() == id) return &s;
  return nullptr;
}

bool Scheduler::cancel(SequenceId id) {  // scheduler.rs:226-236
  for (auto it = waiting_.begin(); it != waiting_.end(); ++it)
    if (it->id() == id) {
      waiting_.erase(it);
      return true;
    }
  for (auto it = running_.begin(); it != running_.end(); ++it)
    if (it->id() == id) {
      running_.erase(it);
      cache_.free(id);
      unwritten_prefill_.erase(id);
      return true;
    }
  return false;
}

SchedulerOutput Scheduler::schedule() {  // scheduler.rs:239-263
  SchedulerOutput out;
  const size_t budget = config_.max_num_batched_tokens;
  size_t used = 0;
  if (config_.prioritize_decode) {
    schedule_decodes(out, budget, used);
    schedule_prefills(out, budget, used);
  } else {
    schedule_prefills(out, budget, used);
    schedule_decodes(out, budget, used);
  }
  stats_.total_steps += 1;
  stats_.total_batched_tokens += out.num_batched_tokens();
  for (const ScheduledSequence &s : out.scheduled)
    (s.is_prefill ? stats_.total_prefill_tokens : stats_.total_decode_tokens) += s.num_tokens;
  return out;
}

void Scheduler::schedule_decodes(SchedulerOutput &out, size_t budget, size_t &used) {  // scheduler.rs:267-313
  std::vector<std::pair<SequenceId, size_t>> candidates;  // collected first: the loop below mutates `running`
  const size_t shift = config_.logical_decode_positions ? 1 : 0;
  for (const Sequence &s : running_)
    if (s.state() == SequenceState::Decoding) candidates.emplace_back(s.id(), s.total_len() - std::min(shift, s.total_len()));
  for (const auto &[id, total_len] : candidates) {
    if (used >= budget) break;
    // Room for the token about to be generated. Note the position: total_len counts the token
    // that was just sampled, so the fed token lands one past its logical place (scheduler.rs:283).
    if (cache_.append_token(id) == ORION_OK) {
      out.scheduled.push_back({id, 1, total_len, false});
      used += 1;
    } else {
      // cache full: evict the newest running sequence and retry once; if the victim is this
      // very sequence it simply does not run this step
      if (!preempt_one(out)) break;
      if (cache_.append_token(id) == ORION_OK) {
        out.scheduled.push_back({id, 1, total_len, false});
        used += 1;
      }
    }
  }
}

bool Scheduler::preempt_one(SchedulerOutput &out) {  // scheduler.rs:317-330
  if (running_.empty()) return false;
  Sequence victim = std::move(running_.back());
  running_.pop_back();
  const SequenceId id = victim.id();
  cache_.free(id);
  victim.preempt();
  unwritten_prefill_.erase(id);  // its prefill starts over, every chunk will be computed again
  waiting_.push_front(std::move(victim));
  out.preempted.push_back(id);
  stats_.total_preempted += 1;
  return true;
}

void Scheduler::schedule_partial_prefills(SchedulerOutput &out, size_t budget, size_t &used) {  // scheduler.rs:343-391
  struct Cand { SequenceId id; size_t already, remaining; };
  std::vector<Cand> candidates;
  for (const Sequence &s : running_)
    if (s.state() == SequenceState::Prefilling && !s.is_prefill_complete())
      candidates.push_back({s.id(), s.computed_prefix_len(), s.remaining_prefill()});
  for (const Cand &c : candidates) {
    if (used >= budget) break;
    const size_t room = budget - used;
    size_t chunk;
    if (config_.enable_chunked_prefill) chunk = std::min(c.remaining, room);
    else if (c.remaining <= room) chunk = c.remaining;
    else continue;
    if (chunk == 0) continue;
    Sequence *seq = running_mut(c.id);
    if (!seq) continue;
    seq->advance_prefill(chunk);
    if (seq->is_prefill_complete()) seq->transition_to(SequenceState::Decoding);
    out.scheduled.push_back({c.id, chunk, c.already, true});
    used += chunk;
  }
}

void Scheduler::schedule_prefills(SchedulerOutput &out, size_t budget, size_t &used) {  // scheduler.rs:394-470
  schedule_partial_prefills(out, budget, used);
  for (;;) {
    if (running_.size() >= config_.max_num_seqs || used >= budget) break;
    if (waiting_.empty()) break;
    const Sequence &next = waiting_.front();
    const size_t prompt_len = next.prompt_len();
    const size_t already = next.computed_prefix_len();
    const size_t remaining = prompt_len - already;
    const size_t room = budget - used;
    size_t chunk;
    if (config_.enable_chunked_prefill) chunk = std::min(remaining, room);
    else if (remaining <= room) chunk = remaining;
    else break;  // unchunked: wait for a step with room for the whole prompt
    if (chunk == 0) break;

    const bool is_first_chunk = already == 0;  // only the first chunk allocates
    if (is_first_chunk && !cache_.can_allocate(prompt_len)) {
      if (!preempt_one(out)) break;
      continue;
    }
    Sequence seq = std::move(waiting_.front());
    waiting_.pop_front();
    const SequenceId id = seq.id();
    size_t start_position = already;
    if (is_first_chunk) {
      AllocationOutcome outcome;
      if (cache_.allocate(id, seq.prompt().data(), seq.prompt().size(), &outcome) != ORION_OK) {
        seq.preempt();
        waiting_.push_front(std::move(seq));
        break;
      }
      if (config_.skip_cached_prefix && outcome.cached_tokens > 0) {
        // The adopted blocks already hold the keys and values of these tokens (published only
        // after their prefill ran). At least the last prompt token is still computed: its logits
        // are what the first sampled token comes from.
        const size_t skip = std::min(outcome.cached_tokens, prompt_len - 1);
        seq.advance_prefill(skip);
        stats_.total_skipped_prefill_tokens += skip;
        start_position = skip;
        chunk = std::min(chunk, prompt_len - skip);
      }
    }
    seq.advance_prefill(chunk);  // progress is recorded at schedule time
    if (seq.state() == SequenceState::Waiting) seq.transition_to(SequenceState::Prefilling);
    if (seq.is_prefill_complete()) seq.transition_to(SequenceState::Decoding);
    out.scheduled.push_back({id, chunk, start_position, true});
    used += chunk;
    running_.push_back(std::move(seq));
  }
}

FinishReason Scheduler::on_token(SequenceId id, TokenId token, const std::vector<TokenId> &eos_ids) {  // scheduler.rs:476-507
  Sequence *seq = running_mut(id);
  if (!seq) return FinishReason::None;
  seq->push_token(token);
  const std::vector<TokenId> &stops = seq->params().stop_token_ids;
  const bool is_stop = std::find(eos_ids.begin(), eos_ids.end(), token) != eos_ids.end() ||
                       std::find(stops.begin(), stops.end(), token) != stops.end();
  FinishReason reason = FinishReason::None;
  if (is_stop && seq->may_stop_on_eos()) reason = FinishReason::Stop;
  else if (seq->reached_max_tokens()) reason = FinishReason::Length;
  if (reason != FinishReason::None) seq->finish(reason);
  return reason;
}

std::vector<Sequence> Scheduler::reap_finished() {  // scheduler.rs:513-520, queue.rs:154-165
  std::vector<Sequence> finished;
  for (size_t i = 0; i < running_.size();) {
    if (running_[i].is_finished()) {
      finished.push_back(std::move(running_[i]));
      running_.erase(running_.begin() + (ptrdiff_t)i);
    } else {
      ++i;
    }
  }
  for (const Sequence &s : finished) {
    cache_.free(s.id());
    unwritten_prefill_.erase(s.id());
  }
  stats_.total_finished += finished.size();
  return finished;
}

std::vector<SequenceId> Scheduler::expire_timeouts() {  // scheduler.rs:527-549
  std::vector<SequenceId> expired;
  if (!config_.request_timeout_secs) return expired;
  const auto limit = std::chrono::seconds(*config_.request_timeout_secs);
  const auto now = std::chrono::steady_clock::now();
  for (Sequence &s : running_)
    if (now - s.arrived_at() > limit) {
      s.finish(FinishReason::Timeout);
      expired.push_back(s.id());
    }
  for (auto it = waiting_.begin(); it != waiting_.end();) {
    if (now - it->arrived_at() > limit) {
      expired.push_back(it->id());
      it = waiting_.erase(it);
    } else {
      ++it;
    }
  }
  return expired;
}

void Scheduler::commit_prefill(SequenceId id) {  // scheduler.rs:557-564
  const Sequence *seq = running_sequence(id);
  if (config_.skip_cached_prefix && unwritten_prefill_.count(id)) return;  // some chunk never reached the device
  if (seq && seq->is_prefill_complete()) cache_.commit_prefill(id, seq->prompt().data(), seq->prompt().size());
}

void Scheduler::note_failed_step(const SchedulerOutput &out) {
  if (!config_.skip_cached_prefix) return;
  for (const ScheduledSequence &s : out.scheduled)
    if (s.is_prefill) unwritten_prefill_.insert(s.id);
}

// ---- Engine ----------------------------------------------------------------------------------

void HostBatch::clear() {
  tokens.clear();
  positions.clear();
  sequence_ids.clear();
  slot_token_counts.clear();
  context_lens.clear();
  block_tables_flat.clear();
  block_table_offsets.assign(1, 0);
  has_prefill = false;
}

Engine::Engine(Scheduler scheduler, ForwardFn forward, std::vector<TokenId> eos_ids)
    : scheduler_(std::move(scheduler)), forward_(std::move(forward)), eos_ids_(std::move(eos_ids)) {
  batch_.clear();
}

int Engine::submit(std::vector<TokenId> prompt, const SamplingParams &params, SequenceId *id) {  // engine.rs:235-268
  ORION_TRY(params.validate());
  // The device path samples greedily (argmax on the GPU); the stochastic samplers of the
  // reference (sampling.rs:215-330) are not built.
  if (params.temperature != 0.0f || params.repetition_penalty != 1.0f)
    return set_error(ORION_ERR_INVALID_REQUEST,
                     "invalid request: only greedy sampling (temperature 0, repetition_penalty 1) is built");
  const size_t prompt_len = prompt.size();
  SequenceId sid = 0;
  ORION_TRY(scheduler_.add_request(Sequence(std::move(prompt), params), &sid));
  active_.emplace(sid, prompt_len);
  if (id) *id = sid;
  return ORION_OK;
}

void Engine::cancel(SequenceId id) {  // engine.rs:271-281
  if (!scheduler_.cancel(id)) return;
  auto it = active_.find(id);
  if (it == active_.end()) return;
  events_.push_back({id, EngineEvent::Done, 0, 0, (uint32_t)FinishReason::Cancelled, it->second, 0});
  active_.erase(it);
}

std::vector<EngineEvent> Engine::take_events() {
  std::vector<EngineEvent> out;
  out.swap(events_);
  return out;
}

int Engine::step(size_t *ran) {  // engine.rs:293-342
  if (ran) *ran = 0;
  for (SequenceId id : scheduler_.expire_timeouts()) finish_request(id, FinishReason::Timeout);
  last_output_ = scheduler_.schedule();
  if (last_output_.scheduled.empty()) {
    batch_.clear();
    reap();  // a sequence may have been cancelled or timed out into a finished state
    return ORION_OK;
  }
  ORION_TRY(build_batch(last_output_));
  const size_t S = batch_.sequence_ids.size();
  sampled_.assign(S, 0);
  if (S > 0) {  // on error nothing is sampled, committed or reaped (engine.rs:310)
    const int rc = forward_(batch_, sampled_.data());
    if (rc != ORION_OK) {
      scheduler_.note_failed_step(last_output_);
      return rc;
    }
  }
  for (size_t row = 0; row < S; ++row) {
    const SequenceId seq_id = batch_.sequence_ids[row];
    const Sequence *seq = scheduler_.running_sequence(seq_id);
    if (seq && !seq->is_prefill_complete()) continue;  // mid-prompt logits produce no token
    emit_token_and_stop(seq_id, sampled_[row]);
  }
  for (const ScheduledSequence &s : last_output_.scheduled)
    if (s.is_prefill) scheduler_.commit_prefill(s.id);
  reap();
  if (ran) *ran = S;
  return ORION_OK;
}

void Engine::emit_token_and_stop(SequenceId seq_id, TokenId token) {  // engine.rs:345-386
  const Sequence *seq = scheduler_.running_sequence(seq_id);
  if (!seq) return;  // cancelled between scheduling and now
  auto it = active_.find(seq_id);
  if (it == active_.end()) return;
  const size_t context_len = seq->total_len();
  const uint64_t index = context_len > it->second ? context_len - it->second : 0;
  const FinishReason reason = scheduler_.on_token(seq_id, token, eos_ids_);
  events_.push_back({seq_id, EngineEvent::Token, token, index, 0, 0, 0});
  if (reason != FinishReason::None) finish_request(seq_id, reason);
}

void Engine::finish_request(SequenceId id, FinishReason reason) {  // engine.rs:395-410
  const Sequence *seq = scheduler_.running_sequence(id);
  const uint64_t completion = seq ? seq->output_len() : 0;
  auto it = active_.find(id);
  if (it == active_.end()) return;
  events_.push_back({id, EngineEvent::Done, 0, 0, (uint32_t)reason, it->second, completion});
  active_.erase(it);
}

void Engine::reap() {  // engine.rs:414-426
  for (const Sequence &seq : scheduler_.reap_finished()) {
    auto it = active_.find(seq.id());
    if (it == active_.end()) continue;
    const FinishReason reason = seq.finish_reason() == FinishReason::None ? FinishReason::Stop : seq.finish_reason();
    events_.push_back({seq.id(), EngineEvent::Done, 0, 0, (uint32_t)reason, it->second, seq.output_len()});
    active_.erase(it);
  }
}

int Engine::build_batch(const SchedulerOutput &output) {  // engine.rs:429-487
  batch_.clear();
  for (const ScheduledSequence &sched : output.scheduled) {
    const Sequence *seq = scheduler_.running_sequence(sched.id);
    if (!seq) continue;  // cancelled since scheduling
    const BlockTable *table = scheduler_.cache().block_table(sched.id);
    if (!table)
      return set_error(ORION_ERR_INTERNAL, "seq-%llu was scheduled without a block table", (unsigned long long)sched.id);
    size_t count = 0;
    if (sched.is_prefill) {  // the prompt slice this chunk covers
      const size_t start = sched.start_position;
      const size_t end = std::min(start + sched.num_tokens, seq->prompt_len());
      for (size_t i = start; i < end; ++i) batch_.tokens.push_back(seq->prompt()[i]);
      count = end > start ? end - start : 0;
    } else if (!seq->output().empty()) {  // decode: the most recent token
      batch_.tokens.push_back(seq->output().back());
      count = 1;
    } else if (!seq->prompt().empty()) {  // decode right after prefill with no output yet
      batch_.tokens.push_back(seq->prompt().back());
      count = 1;
    }
    if (count == 0) continue;
    for (size_t p = sched.start_position; p < sched.start_position + count; ++p) batch_.positions.push_back((uint32_t)p);
    batch_.sequence_ids.push_back(sched.id);
    batch_.slot_token_counts.push_back(count);
    batch_.context_lens.push_back(sched.start_position + count);
    batch_.block_tables_flat.insert(batch_.block_tables_flat.end(), table->blocks.begin(), table->blocks.end());
    batch_.block_table_offsets.push_back(batch_.block_tables_flat.size());
    batch_.has_prefill = batch_.has_prefill || sched.is_prefill;
  }
  return ORION_OK;
}

}  // namespace driver
}  // namespace orion
