// Cache bookkeeping of the driver: block pool, prefix index, per-sequence block tables.
// Every function follows the reference routine named beside it, statement for statement where
// the order of operations decides which block id a sequence gets.
#include "driver.h"

#include <algorithm>
#include <atomic>
#include <cmath>

#include "common.cuh"

namespace orion {
namespace driver {

namespace {
std::atomic<uint64_t> g_next_sequence_id{1};

int cache_exhausted(size_t needed, size_t available) {  // error.rs:100-101
  return set_error(ORION_ERR_CACHE_EXHAUSTED, "KV cache exhausted: needed %zu blocks, %zu free", needed, available);
}

inline uint64_t rotl64(uint64_t v, int s) { return (v << s) | (v >> (64 - s)); }
inline uint64_t mix(uint64_t state, uint64_t value) {  // table.rs:122-126
  return (rotl64(state, 5) ^ value) * 0x517cc1b727220a95ull;
}
}  // namespace

SequenceId next_sequence_id() { return g_next_sequence_id.fetch_add(1, std::memory_order_relaxed); }
SequenceId peek_sequence_id() { return g_next_sequence_id.load(std::memory_order_relaxed); }

BlockHash hash_block(const std::optional<BlockHash> &parent, const TokenId *tokens, size_t n) {  // table.rs:105-120
  uint64_t state = parent ? *parent : 0xcbf29ce484222325ull;
  state = mix(state, (uint64_t)n);
  for (size_t i = 0; i < n; ++i) state = mix(state, (uint64_t)tokens[i]);
  return state;
}

// ---- BlockPool -------------------------------------------------------------------------------

BlockPool::BlockPool(size_t num_blocks, size_t block_size) : blocks_(num_blocks), block_size_(block_size) {
  for (size_t i = 0; i < num_blocks; ++i) free_list_.push_back((BlockId)i);  // block.rs:102-113
}

int BlockPool::allocate(BlockId *id, std::optional<BlockHash> *evicted) {  // block.rs:153-166
  if (free_list_.empty()) return cache_exhausted(1, 0);
  const BlockId b = free_list_.front();
  free_list_.pop_front();
  Block &blk = blocks_[b];
  *evicted = blk.hash;
  blk = Block{};
  blk.ref_count = 1;
  *id = b;
  return ORION_OK;
}

int BlockPool::add_ref(BlockId id) {  // block.rs:172-185
  if (id >= blocks_.size()) return set_error(ORION_ERR_INTERNAL, "add_ref on unknown block blk-%u", id);
  Block &blk = blocks_[id];
  if (blk.ref_count == 0) {  // reviving a cached block: it leaves the free list, contents kept
    auto it = std::find(free_list_.begin(), free_list_.end(), id);
    if (it != free_list_.end()) free_list_.erase(it);
  }
  blk.ref_count += 1;
  return ORION_OK;
}

int BlockPool::release(BlockId id, bool *became_free) {  // block.rs:191-208
  if (id >= blocks_.size()) return set_error(ORION_ERR_INTERNAL, "release of unknown block blk-%u", id);
  Block &blk = blocks_[id];
  if (blk.ref_count == 0)
    return set_error(ORION_ERR_INTERNAL, "double release of blk-%u: ref_count is already 0", id);
  blk.ref_count -= 1;
  const bool freed = blk.ref_count == 0;
  if (freed) free_list_.push_back(id);  // contents and hash stay: the prefix cache may reclaim it
  if (became_free) *became_free = freed;
  return ORION_OK;
}

int BlockPool::set_contents(BlockId id, size_t num_tokens, std::optional<BlockHash> hash) {  // block.rs:211-230
  if (num_tokens > block_size_)
    return set_error(ORION_ERR_INTERNAL, "block blk-%u cannot hold %zu tokens, capacity is %zu", id, num_tokens,
                     block_size_);
  if (id >= blocks_.size()) return set_error(ORION_ERR_INTERNAL, "set_contents on unknown block blk-%u", id);
  blocks_[id].num_tokens = num_tokens;
  blocks_[id].hash = hash;
  return ORION_OK;
}

bool BlockPool::evict_oldest_cached(BlockId *id, BlockHash *hash) {  // block.rs:241-253
  for (BlockId b : free_list_) {
    Block &blk = blocks_[b];
    if (blk.hash) {
      *id = b;
      *hash = *blk.hash;
      blk.hash.reset();
      blk.num_tokens = 0;
      return true;
    }
  }
  return false;
}

size_t BlockPool::num_evictable() const {  // block.rs:257-262
  size_t n = 0;
  for (BlockId b : free_list_) n += blocks_[b].hash.has_value();
  return n;
}

// ---- PrefixCache -----------------------------------------------------------------------------

bool PrefixCache::lookup(BlockHash hash, const TokenId *tokens, size_t n, BlockId *block) {  // prefix.rs:81-98
  auto it = entries_.find(hash);
  if (it != entries_.end() && it->second.tokens.size() == n &&
      std::equal(it->second.tokens.begin(), it->second.tokens.end(), tokens)) {
    hits_ += 1;
    *block = it->second.block;
    return true;
  }
  misses_ += 1;  // absent, or a hash collision between different token runs
  return false;
}

bool PrefixCache::peek(BlockHash hash, BlockId *block) const {
  auto it = entries_.find(hash);
  if (it == entries_.end()) return false;
  *block = it->second.block;
  return true;
}

void PrefixCache::insert(BlockHash hash, BlockId block, const TokenId *tokens, size_t n) {  // prefix.rs:112-116
  entries_.emplace(hash, Entry{block, std::vector<TokenId>(tokens, tokens + n)});
}

void PrefixCache::remove(BlockHash hash, BlockId block) {  // prefix.rs:123-129
  auto it = entries_.find(hash);
  if (it != entries_.end() && it->second.block == block) entries_.erase(it);
}

// ---- KvCacheManager --------------------------------------------------------------------------

KvCacheManager::KvCacheManager(size_t num_blocks, size_t block_size, bool prefix_caching_enabled)
    : pool_(num_blocks, block_size), prefix_caching_enabled_(prefix_caching_enabled) {}

CacheStats KvCacheManager::stats() const {  // manager.rs:110-121
  return CacheStats{pool_.total_blocks(), pool_.num_used(),      pool_.num_free(),      pool_.block_size(),
                    tables_.size(),       prefix_cache_.len(),   prefix_cache_.hits(),  prefix_cache_.misses()};
}

const BlockTable *KvCacheManager::block_table(SequenceId seq) const {
  auto it = tables_.find(seq);
  return it == tables_.end() ? nullptr : &it->second;
}

int KvCacheManager::allocate(SequenceId seq, const TokenId *prompt, size_t n, AllocationOutcome *outcome) {  // manager.rs:163-250
  if (fail_next_allocate_) {
    fail_next_allocate_ = false;
    return cache_exhausted(1, 0);
  }
  if (tables_.count(seq))
    return set_error(ORION_ERR_INTERNAL, "seq-%llu already has a block table", (unsigned long long)seq);
  const size_t bs = pool_.block_size();
  const size_t needed = BlockTable::blocks_required(n, bs);
  if (needed > pool_.num_free()) return cache_exhausted(needed, pool_.num_free());

  BlockTable table;
  AllocationOutcome out;
  std::optional<BlockHash> chain;
  bool still_matching = prefix_caching_enabled_;  // after the first miss every later chained hash is unknown too
  for (size_t start = 0; start < n; start += bs) {
    const TokenId *chunk = prompt + start;
    const size_t len = std::min(bs, n - start);
    const bool is_full = len == bs;
    std::optional<BlockHash> hash;
    if (still_matching && is_full) hash = hash_block(chain, chunk, len);

    bool adopted = false;
    BlockId blk = 0;
    if (hash && prefix_cache_.lookup(*hash, chunk, len, &blk)) adopted = pool_.add_ref(blk) == ORION_OK;

    if (adopted) {
      table.blocks.push_back(blk);
      out.reused += 1;
      out.cached_tokens += len;
      chain = hash;
    } else {
      still_matching = false;
      std::optional<BlockHash> evicted;
      const int rc = pool_.allocate(&blk, &evicted);
      if (rc != ORION_OK) {  // roll back everything this call took
        for (BlockId b : table.blocks) pool_.release(b, nullptr);
        return rc;
      }
      if (evicted) prefix_cache_.remove(*evicted, blk);  // a recycled block must not stay indexed
      table.blocks.push_back(blk);
      out.allocated += 1;
      pool_.set_contents(blk, len, std::nullopt);  // the hash is published by commit_prefill only
      chain.reset();
    }
  }
  table.num_tokens = n;
  tables_.emplace(seq, std::move(table));
  if (outcome) *outcome = out;
  return ORION_OK;
}

void KvCacheManager::commit_prefill(SequenceId seq, const TokenId *prompt, size_t n) {  // manager.rs:258-283
  if (!prefix_caching_enabled_) return;
  auto it = tables_.find(seq);
  if (it == tables_.end()) return;
  const size_t bs = pool_.block_size();
  std::optional<BlockHash> chain;
  size_t i = 0;
  for (size_t start = 0; start < n; start += bs, ++i) {
    const size_t len = std::min(bs, n - start);
    if (len != bs) break;  // partial tail: still written to during decode
    if (i >= it->second.blocks.size()) break;
    const BlockId blk = it->second.blocks[i];
    const BlockHash h = hash_block(chain, prompt + start, len);
    pool_.set_contents(blk, len, h);
    prefix_cache_.insert(h, blk, prompt + start, len);
    chain = h;
  }
  if (chain) chain_tips_[seq] = *chain;
}

int KvCacheManager::append_token(SequenceId seq) {  // manager.rs:290-335
  if (fail_next_append_) {
    fail_next_append_ = false;
    return cache_exhausted(1, 0);
  }
  auto it = tables_.find(seq);
  if (it == tables_.end()) return set_error(ORION_ERR_INTERNAL, "seq-%llu has no block table", (unsigned long long)seq);
  const size_t bs = pool_.block_size();
  BlockTable &table = it->second;
  const size_t new_len = table.num_tokens + 1;
  if (BlockTable::blocks_required(new_len, bs) > table.blocks.size()) {
    BlockId blk = 0;
    std::optional<BlockHash> evicted;
    if (pool_.allocate(&blk, &evicted) != ORION_OK) return cache_exhausted(1, pool_.num_free());  // table untouched
    if (evicted) prefix_cache_.remove(*evicted, blk);
    table.blocks.push_back(blk);
  }
  table.num_tokens = new_len;
  if (table.blocks.empty())
    return set_error(ORION_ERR_INTERNAL, "seq-%llu has an empty block table", (unsigned long long)seq);
  const size_t filled = new_len - (table.blocks.size() - 1) * bs;
  return pool_.set_contents(table.blocks.back(), filled, std::nullopt);
}

void KvCacheManager::free(SequenceId seq) {  // manager.rs:341-359
  chain_tips_.erase(seq);
  auto it = tables_.find(seq);
  if (it == tables_.end()) return;
  BlockTable table = std::move(it->second);
  tables_.erase(it);
  for (BlockId b : table.blocks) pool_.release(b, nullptr);
}

size_t KvCacheManager::preempt(SequenceId seq) {  // manager.rs:368-376
  const BlockTable *t = block_table(seq);
  const size_t n = t ? t->blocks.size() : 0;
  free(seq);
  return n;
}

size_t KvCacheManager::evict_cached(size_t count) {  // manager.rs:397-409
  size_t evicted = 0;
  while (evicted < count) {
    BlockId blk;
    BlockHash hash;
    if (!pool_.evict_oldest_cached(&blk, &hash)) break;
    prefix_cache_.remove(hash, blk);
    evicted += 1;
  }
  return evicted;
}

void KvCacheManager::clear_prefix_cache() {  // manager.rs:412-416
  evict_cached(pool_.num_evictable());
  prefix_cache_.clear();
}

}  // namespace driver
}  // namespace orion
