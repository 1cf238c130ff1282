// Host-side driver of the device forward pass: the bookkeeping that decides, every engine
// step, which tokens of which sequences run and where their keys and values live. It is a
// C++ restatement of the reference's caller side, kept bit-exact in block ids, slot mapping,
// positions and batch order:
//   BlockPool / BlockHash      crates/orion-kv-cache/src/block.rs:20-275
//   BlockTable / hash_block    crates/orion-kv-cache/src/table.rs:13-126
//   PrefixCache                crates/orion-kv-cache/src/prefix.rs:24-150
//   KvCacheManager             crates/orion-kv-cache/src/manager.rs:26-425
//   Sequence / SequenceState   crates/orion-core/src/sequence.rs:26-330
//   WaitingQueue / RunningQueue crates/orion-scheduler/src/queue.rs:23-174
//   Scheduler                  crates/orion-scheduler/src/scheduler.rs:34-580
//   Engine::{submit,cancel,step,build_batch}  crates/orion-runtime/src/engine.rs:210-487
// Pure host code: no device memory is touched here; Engine hands the batch it built to a
// forward function (the device model, or a caller's function in tests).
#pragma once

#include <chrono>
#include <cstdint>
#include <deque>
#include <functional>
#include <optional>
#include <string>
#include <unordered_map>
#include <utility>
#include <unordered_set>
#include <vector>

namespace orion {
namespace driver {

using TokenId = uint32_t;
using SequenceId = uint64_t;
using BlockId = uint32_t;
using BlockHash = uint64_t;

// SequenceId::next (crates/orion-core/src/id.rs:52-55): process-wide, starts at 1.
SequenceId next_sequence_id();
SequenceId peek_sequence_id();

// hash_block (table.rs:105-120): FxHash-style chain over the parent hash, the length and the tokens.
BlockHash hash_block(const std::optional<BlockHash> &parent, const TokenId *tokens, size_t n);

struct Block {  // block.rs:23-36
  uint32_t ref_count = 0;
  size_t num_tokens = 0;
  std::optional<BlockHash> hash;
};

class BlockPool {  // block.rs:93-275
 public:
  BlockPool(size_t num_blocks, size_t block_size);
  size_t block_size() const { return block_size_; }
  size_t total_blocks() const { return blocks_.size(); }
  size_t num_free() const { return free_list_.size(); }
  size_t num_used() const { return blocks_.size() - free_list_.size(); }
  const Block *get(BlockId id) const { return id < blocks_.size() ? &blocks_[id] : nullptr; }
  // Oldest free block, ref_count 1, contents reset; `evicted` = the hash it used to carry.
  int allocate(BlockId *id, std::optional<BlockHash> *evicted);
  int add_ref(BlockId id);
  int release(BlockId id, bool *became_free);
  int set_contents(BlockId id, size_t num_tokens, std::optional<BlockHash> hash);
  bool evict_oldest_cached(BlockId *id, BlockHash *hash);
  size_t num_evictable() const;

 private:
  std::vector<Block> blocks_;
  std::deque<BlockId> free_list_;  // ref_count == 0, oldest first: also the eviction order
  size_t block_size_;
};

struct BlockTable {  // table.rs:13-97
  std::vector<BlockId> blocks;
  size_t num_tokens = 0;
  static size_t blocks_required(size_t num_tokens, size_t block_size) {
    return (num_tokens + block_size - 1) / block_size;
  }
};

class PrefixCache {  // prefix.rs:24-150
 public:
  size_t len() const { return entries_.size(); }
  uint64_t hits() const { return hits_; }
  uint64_t misses() const { return misses_; }
  bool lookup(BlockHash hash, const TokenId *tokens, size_t n, BlockId *block);
  bool peek(BlockHash hash, BlockId *block) const;
  void insert(BlockHash hash, BlockId block, const TokenId *tokens, size_t n);  // first writer wins
  void remove(BlockHash hash, BlockId block);  // only if the entry still names `block`
  void clear() { entries_.clear(); }

 private:
  struct Entry {
    BlockId block;
    std::vector<TokenId> tokens;
  };
  std::unordered_map<BlockHash, Entry> entries_;
  uint64_t hits_ = 0, misses_ = 0;
};

struct AllocationOutcome {  // manager.rs:26-36
  size_t allocated = 0, reused = 0, cached_tokens = 0;
};

struct CacheStats {  // manager.rs:46-56
  size_t total_blocks, used_blocks, free_blocks, block_size, num_sequences, prefix_cache_entries;
  uint64_t prefix_cache_hits, prefix_cache_misses;
};

class KvCacheManager {  // manager.rs:73-425
 public:
  KvCacheManager(size_t num_blocks, size_t block_size, bool prefix_caching_enabled);
  size_t block_size() const { return pool_.block_size(); }
  size_t total_blocks() const { return pool_.total_blocks(); }
  size_t free_blocks() const { return pool_.num_free(); }
  CacheStats stats() const;
  const BlockTable *block_table(SequenceId seq) const;
  bool is_allocated(SequenceId seq) const { return tables_.count(seq) != 0; }
  size_t blocks_needed_for(size_t num_tokens) const { return BlockTable::blocks_required(num_tokens, block_size()); }
  bool can_allocate(size_t num_tokens) const { return blocks_needed_for(num_tokens) <= pool_.num_free(); }
  int allocate(SequenceId seq, const TokenId *prompt, size_t n, AllocationOutcome *outcome);
  void commit_prefill(SequenceId seq, const TokenId *prompt, size_t n);
  int append_token(SequenceId seq);
  void free(SequenceId seq);
  size_t preempt(SequenceId seq);
  size_t evict_cached(size_t count);
  void clear_prefix_cache();
  size_t num_evictable() const { return pool_.num_evictable(); }
  size_t num_sequences() const { return tables_.size(); }
  const BlockPool &pool() const { return pool_; }
  // Host-side fault injection, the counterpart of the reference's FakeCache
  // (crates/orion-scheduler/src/testing.rs:29-37): the next call fails with CacheExhausted.
  void fail_next_append() { fail_next_append_ = true; }
  void fail_next_allocate() { fail_next_allocate_ = true; }

 private:
  BlockPool pool_;
  std::unordered_map<SequenceId, BlockTable> tables_;
  PrefixCache prefix_cache_;
  bool prefix_caching_enabled_;
  std::unordered_map<SequenceId, BlockHash> chain_tips_;
  bool fail_next_append_ = false, fail_next_allocate_ = false;
};

enum class SequenceState { Waiting, Prefilling, Decoding, Finished };  // sequence.rs:26-37
enum class FinishReason { None = 0, Stop = 1, Length = 2, Cancelled = 3, Timeout = 4, Error = 5 };  // sequence.rs:73-87

struct SamplingParams {  // crates/orion-core/src/sampling.rs:25-70 (the fields the driver reads)
  float temperature = 1.0f, top_p = 1.0f, repetition_penalty = 1.0f;
  size_t top_k = 0, max_tokens = 16, min_tokens = 0;
  std::vector<TokenId> stop_token_ids;
  int validate() const;  // sampling.rs:85-134
};

class Sequence {  // sequence.rs:158-330
 public:
  Sequence(std::vector<TokenId> prompt, SamplingParams params);
  SequenceId id() const { return id_; }
  SequenceState state() const { return state_; }
  const SamplingParams &params() const { return params_; }
  const std::vector<TokenId> &prompt() const { return prompt_; }
  const std::vector<TokenId> &output() const { return output_; }
  size_t prompt_len() const { return prompt_.size(); }
  size_t output_len() const { return output_.size(); }
  size_t total_len() const { return prompt_.size() + output_.size(); }
  size_t computed_prefix_len() const { return computed_prefix_len_; }
  size_t remaining_prefill() const { return prompt_.size() > computed_prefix_len_ ? prompt_.size() - computed_prefix_len_ : 0; }
  bool is_prefill_complete() const { return computed_prefix_len_ >= prompt_.size(); }
  bool is_finished() const { return state_ == SequenceState::Finished; }
  FinishReason finish_reason() const { return finish_reason_; }
  std::chrono::steady_clock::time_point arrived_at() const { return arrived_at_; }
  bool transition_to(SequenceState next);
  void advance_prefill(size_t n);
  void push_token(TokenId t) { output_.push_back(t); }
  void finish(FinishReason reason);
  bool preempt();
  bool reached_max_tokens() const { return output_.size() >= params_.max_tokens; }
  bool may_stop_on_eos() const { return output_.size() >= params_.min_tokens; }
  static bool can_transition(SequenceState from, SequenceState to);

 private:
  SequenceId id_;
  std::vector<TokenId> prompt_, output_;
  size_t computed_prefix_len_ = 0;
  SequenceState state_ = SequenceState::Waiting;
  FinishReason finish_reason_ = FinishReason::None;
  SamplingParams params_;
  std::chrono::steady_clock::time_point arrived_at_;
};

struct SchedulerConfig {  // crates/orion-core/src/config.rs:107-156
  size_t max_num_seqs = 256, max_num_batched_tokens = 8192;
  std::optional<size_t> max_model_len;
  bool enable_chunked_prefill = true;
  size_t max_waiting_requests = 1024;
  std::optional<uint64_t> request_timeout_secs = 300;
  bool prioritize_decode = true;
  // Not in the reference (which plumbs AllocationOutcome.cached_tokens nowhere, manager.rs:449-451,
  // and always prefills from position 0): when set, a new sequence starts its prefill after the
  // tokens whose blocks it adopted from the prefix cache. Off = the reference's behaviour.
  bool skip_cached_prefix = false;
  // Not in the reference either: feed a decode token at its logical position total_len - 1
  // instead of total_len (scheduler.rs:283 counts the token that was just sampled), so no cache
  // slot is skipped and no step is refused for a block the table does not hold yet.
  bool logical_decode_positions = false;
};

struct ScheduledSequence {  // scheduler.rs:36-50
  SequenceId id;
  size_t num_tokens, start_position;
  bool is_prefill;
};

struct SchedulerOutput {  // scheduler.rs:53-61
  std::vector<ScheduledSequence> scheduled;
  std::vector<SequenceId> preempted;
  size_t num_batched_tokens() const;
};

struct SchedulerStats {  // scheduler.rs:99-109
  uint64_t total_steps = 0, total_admitted = 0, total_finished = 0, total_preempted = 0, total_rejected = 0,
           total_batched_tokens = 0, total_prefill_tokens = 0, total_decode_tokens = 0;
  uint64_t total_skipped_prefill_tokens = 0;  // only with skip_cached_prefix
};

class Scheduler {  // scheduler.rs:127-580
 public:
  Scheduler(SchedulerConfig config, KvCacheManager cache);
  const SchedulerConfig &config() const { return config_; }
  const SchedulerStats &stats() const { return stats_; }
  KvCacheManager &cache() { return cache_; }
  const KvCacheManager &cache() const { return cache_; }
  size_t num_waiting() const { return waiting_.size(); }
  size_t num_running() const { return running_.size(); }
  bool has_work() const { return !waiting_.empty() || !running_.empty(); }
  int add_request(Sequence seq, SequenceId *id);
  bool cancel(SequenceId id);
  SchedulerOutput schedule();
  FinishReason on_token(SequenceId id, TokenId token, const std::vector<TokenId> &eos_ids);
  std::vector<Sequence> reap_finished();
  std::vector<SequenceId> expire_timeouts();
  const Sequence *running_sequence(SequenceId id) const;
  void commit_prefill(SequenceId id);
  // Only with skip_cached_prefix: the forward of a step failed, so the prefill chunks it carried
  // wrote no keys or values although their progress was recorded at schedule time. The prompts
  // of these sequences are not published to the prefix cache (a later request would adopt blocks
  // that were never written and skip their computation); they stay usable for their own sequence
  // exactly as in the reference.
  void note_failed_step(const SchedulerOutput &out);

 private:
  Sequence *running_mut(SequenceId id);
  void schedule_decodes(SchedulerOutput &out, size_t budget, size_t &used);
  void schedule_prefills(SchedulerOutput &out, size_t budget, size_t &used);
  void schedule_partial_prefills(SchedulerOutput &out, size_t budget, size_t &used);
  bool preempt_one(SchedulerOutput &out);

  SchedulerConfig config_;
  std::deque<Sequence> waiting_;   // strict FIFO; preempted sequences re-enter at the front (queue.rs:23-99)
  std::vector<Sequence> running_;  // admission order; the newest is the preemption victim (queue.rs:103-174)
  KvCacheManager cache_;
  SchedulerStats stats_;
  std::unordered_set<SequenceId> unwritten_prefill_;  // see note_failed_step
};

// The batch handed to the forward function, laid out as the C ABI of the device model takes it
// (crates/orion-core/src/traits.rs:193-210).
struct HostBatch {
  std::vector<TokenId> tokens;
  std::vector<uint32_t> positions;
  std::vector<SequenceId> sequence_ids;
  std::vector<uint64_t> slot_token_counts, context_lens;
  std::vector<uint32_t> block_tables_flat;
  std::vector<uint64_t> block_table_offsets;  // [sequences + 1]
  bool has_prefill = false;
  void clear();
};

struct EngineEvent {  // StreamEvent (crates/orion-runtime/src/engine.rs:60-90), text left to the API layer
  enum Kind : uint32_t { Token = 0, Done = 1 };
  SequenceId id;
  uint32_t kind;
  TokenId token;              // Token
  uint64_t index;             // Token: position in the output
  uint32_t reason;            // Done: FinishReason
  uint64_t prompt_tokens, completion_tokens;  // Done
};

// Greedy forward: fills one token id per sequence of the batch (argmax of its last row,
// crates/orion-runtime/src/sampling.rs:196-206); returns an OrionStatus.
using ForwardFn = std::function<int(const HostBatch &, uint32_t *token_ids)>;

class Engine {  // engine.rs:186-487
 public:
  Engine(Scheduler scheduler, ForwardFn forward, std::vector<TokenId> eos_ids);
  Scheduler &scheduler() { return scheduler_; }
  int submit(std::vector<TokenId> prompt, const SamplingParams &params, SequenceId *id);
  void cancel(SequenceId id);
  bool has_work() const { return scheduler_.has_work(); }
  // One engine step: schedule, build the batch, forward, sample, emit, commit, reap.
  // `ran` = sequences in the batch (0 for an empty step). A forward error returns early with the
  // scheduler and the cache already advanced, exactly like the reference (engine.rs:309-310).
  int step(size_t *ran);
  const HostBatch &last_batch() const { return batch_; }
  const SchedulerOutput &last_schedule() const { return last_output_; }
  std::vector<EngineEvent> take_events();
  size_t num_active() const { return active_.size(); }

 private:
  int build_batch(const SchedulerOutput &output);
  void emit_token_and_stop(SequenceId id, TokenId token);
  void finish_request(SequenceId id, FinishReason reason);
  void reap();

  Scheduler scheduler_;
  ForwardFn forward_;
  std::vector<TokenId> eos_ids_;
  std::unordered_map<SequenceId, size_t> active_;  // id -> prompt length of requests still owed a Done
  HostBatch batch_;
  SchedulerOutput last_output_;
  std::vector<uint32_t> sampled_;
  std::vector<EngineEvent> events_;
};

}  // namespace driver
}  // namespace orion
