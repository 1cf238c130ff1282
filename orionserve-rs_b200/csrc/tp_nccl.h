// NCCL backing of the reference's `Collective` trait
// (crates/orion-distributed/src/lib.rs:231-254; NCCL is the backing it names,
// docs/distributed.md:112-120). libnccl is opened at run time, only when a
// tensor-parallel world larger than one is requested, so that single-GPU users
// need no NCCL at all and a host process that already loaded NCCL shares it.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace orion {

class NcclCollective {
 public:
  ~NcclCollective();
  // ncclGetUniqueId into a 128-byte buffer.
  static int unique_id(uint8_t id[128]);
  // ncclCommInitRank on the current device.
  int init(const uint8_t id[128], int rank, int world);
  // Collective::all_reduce_sum over f32, in place, on `stream`.
  int all_reduce_sum(float *buf, size_t count, cudaStream_t stream);
  // Collective::all_gather / reduce_scatter_sum / barrier, for completeness of the trait.
  int all_gather(const float *local, float *out, size_t count_per_rank, cudaStream_t stream);
  int reduce_scatter_sum(const float *in, float *out, size_t count_per_rank, cudaStream_t stream);
  int barrier(cudaStream_t stream);
  int rank() const { return rank_; }
  int world() const { return world_; }

 private:
  void *comm_ = nullptr;
  float *barrier_word_ = nullptr;
  int rank_ = 0, world_ = 1;
};

}  // namespace orion
