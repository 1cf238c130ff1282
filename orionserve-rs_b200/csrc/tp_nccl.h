// NCCL backing of the reference's `Collective` trait
// (crates/orion-distributed/src/lib.rs:231-254; NCCL is the backing it names,
// docs/distributed.md:112-120). libnccl is opened at run time, only when a
// tensor-parallel world larger than one is requested, so that single-GPU users
// need no NCCL at all and a host process that already loaded NCCL shares it.
//
// Failure handling. The communicator is opened non-blocking and never blocks the
// host inside NCCL: every call that NCCL reports as "in progress" is followed by
// polling ncclCommGetAsyncError under a host time limit, and a step is waited for
// with wait_stream(), which polls the stream and the communicator's asynchronous
// error state instead of a blocking synchronise. A rank that never arrives, a
// peer that died or a step that does not end in time all end the same way:
// ncclCommAbort, the communicator marked dead, and an EngineError::Backend status
// that the engine loop logs before going on (orion-runtime/src/engine.rs:529-535).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace orion {

struct NcclApi;  // the NCCL entry points in use: the real library, or a stand-in for the host self-test

class NcclCollective {
 public:
  NcclCollective();
  explicit NcclCollective(const NcclApi *api) : api_(api) {}
  ~NcclCollective();
  // ncclGetUniqueId into a 128-byte buffer.
  static int unique_id(uint8_t id[128]);
  // ncclCommInitRankConfig (non-blocking) on the current device, waited for under the init limit.
  int init(const uint8_t id[128], int rank, int world);
  // Collective::all_reduce_sum over f32, in place, on `stream`.
  int all_reduce_sum(float *buf, size_t count, cudaStream_t stream);
  // Collective::all_gather / reduce_scatter_sum / barrier, for completeness of the trait.
  int all_gather(const float *local, float *out, size_t count_per_rank, cudaStream_t stream);
  int reduce_scatter_sum(const float *in, float *out, size_t count_per_rank, cudaStream_t stream);
  int barrier(cudaStream_t stream);
  // Waits until everything enqueued on `stream` has finished, watching the communicator: an
  // asynchronous NCCL error or the step limit running out aborts the communicator and returns
  // ORION_ERR_BACKEND; the host never sits in a blocking synchronise behind a dead peer.
  int wait_stream(cudaStream_t stream, const char *stage);
  int rank() const { return rank_; }
  int world() const { return world_; }
  bool aborted() const { return aborted_; }
  // Host time limits in milliseconds (defaults: ORION_TP_INIT_TIMEOUT_S or 300 s for the rendezvous,
  // ORION_TP_STEP_TIMEOUT_S or 60 s for a call or a step).
  void set_limits(uint64_t init_ms, uint64_t step_ms) { init_limit_ms_ = init_ms, step_limit_ms_ = step_ms; }
  uint64_t polls() const { return polls_; }

 private:
  // Turns the result of an NCCL call into a status; "in progress" is polled to its end.
  int settle(int nccl_result, const char *stage, uint64_t limit_ms);
  int abort_with(const char *stage, const char *why);
  int dead(const char *stage) const;

  const NcclApi *api_ = nullptr;
  void *comm_ = nullptr;
  float *barrier_word_ = nullptr;
  int rank_ = 0, world_ = 1;
  bool aborted_ = false;
  uint64_t init_limit_ms_ = 300000, step_limit_ms_ = 60000;
  uint64_t polls_ = 0;
};

// Host-only self-test of the failure handling above against a stand-in NCCL (no GPU, no NCCL
// library): scenario 0 = a healthy group (rendezvous completes after a few polls, an all-reduce
// and a step end normally); 1 = a rank that never arrives (the rendezvous stays "in progress");
// 2 = a peer dies during a step (the asynchronous error state turns to a remote error while the
// stream is still busy); 3 = a step that never ends without any NCCL error. Returns the status of
// the failing call (ORION_OK for scenario 0) and reports whether ncclCommAbort ran and how often
// the state was polled.
int nccl_failure_selftest(int scenario, uint64_t limit_ms, uint32_t *aborted, uint64_t *polls);

}  // namespace orion
