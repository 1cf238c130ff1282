// Host side of the device model: the C++ counterpart of the reference's
// `CudaBackend` (orion-cuda/src/lib.rs:104-179) and of `TransformerModel`
// (orion-models/src/transformer.rs:137-443) with the arithmetic on the GPU.
#pragma once

#include <memory>
#include <string>
#include <vector>

#include "kernels.h"
#include "tp_nccl.h"

struct OrionBackend {
  int ordinal = 0;
  std::string device_name;
  uint64_t total_memory = 0;
};

namespace orion {

// A ForwardBatch as it crosses the C ABI (orion-core/src/traits.rs:193-210).
struct BatchView {
  const uint32_t *tokens;
  uint64_t num_tokens;
  const uint32_t *positions;
  uint64_t num_positions;
  const uint64_t *slot_token_counts;
  uint64_t num_slot_token_counts;
  const uint64_t *context_lens;
  uint64_t num_context_lens;
  const uint32_t *block_tables_flat;
  const uint64_t *block_table_offsets;
  uint64_t num_block_tables;
  uint64_t num_sequences;
  int has_prefill;
};

// Shard {start, len} (orion-distributed/src/lib.rs:116-130).
struct Shard {
  uint64_t start = 0, len = 0;
};
struct ParallelLayout {
  Shard query_heads, kv_heads, ffn;
};
// shard_dimension + ParallelLayout::compute (orion-distributed/src/lib.rs:139-208).
int compute_layout(uint32_t heads, uint32_t kv_heads, uint32_t ffn, uint32_t rank, uint32_t world,
                   ParallelLayout *out);

// Kernel categories of a profiled step.
enum { kProfGemm = 0, kProfAttention = 1, kProfElementwise = 2, kProfCollective = 3, kProfCategories = 4 };

class ModelBase {
 public:
  virtual ~ModelBase() = default;
  virtual int load_tensor(const char *name, int dtype, const uint64_t *shape, int ndim,
                          const void *data) = 0;
  virtual int init_random(uint64_t seed, float std) = 0;
  virtual int finalize() = 0;
  virtual int forward(const BatchView &b, float *logits_out, uint64_t logits_capacity,
                      uint32_t *token_ids_out) = 0;
  virtual int replay(int iterations, uint32_t category_mask, float *elapsed_ms) = 0;
  virtual int profile(int iterations, float category_ms[kProfCategories],
                      uint64_t category_launches[kProfCategories]) = 0;
  virtual int fill_kv_random(uint64_t seed, float std) = 0;
  virtual int read_kv(float *out, uint64_t capacity) = 0;
  virtual uint64_t last_launch_count() const = 0;
  virtual const OrionModelDesc &desc() const = 0;
};


int create_model(OrionBackend *backend, const OrionModelDesc *desc, ModelBase **out);
// Loads every tensor the model uses from the `*.safetensors` files of a directory and finalizes
// (CheckpointLoader, crates/orion-models/src/loader.rs:112-235).
int load_checkpoint(ModelBase *model, const char *directory, uint64_t *tensors_loaded);

}  // namespace orion

struct OrionModel {
  std::unique_ptr<orion::ModelBase> impl;
};
