// NCCL backing of the tensor-parallel collectives; see tp_nccl.h.
#include "tp_nccl.h"

#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

#include "common.cuh"

namespace orion {

struct NcclApi {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t,
                                ncclComm_t, cudaStream_t) = nullptr;
  // cudaStreamQuery, replaceable so that the self-test needs no device
  cudaError_t (*StreamQuery)(cudaStream_t) = nullptr;
  bool ok = false;
};

namespace {

NcclApi &real_api() {
  static NcclApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    // A process that already holds NCCL (for instance through its tensor framework) gets that copy
    // back. Otherwise ORION_NCCL_LIBRARY names the file to open, else the loader's libnccl.so.2. The
    // library is opened privately: a different NCCL that the process loads later under the same
    // name must not find this one's symbols in its way.
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!a.handle) {
      const char *path = std::getenv("ORION_NCCL_LIBRARY");
      if (path && *path) a.handle = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    }
    if (!a.handle) a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!a.handle) a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!a.handle) return;
#define ORION_NCCL_SYM(field, name)                                        \
  a.field = reinterpret_cast<decltype(a.field)>(dlsym(a.handle, name));   \
  if (!a.field) return;
    ORION_NCCL_SYM(GetUniqueId, "ncclGetUniqueId")
    ORION_NCCL_SYM(CommInitRankConfig, "ncclCommInitRankConfig")
    ORION_NCCL_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
    ORION_NCCL_SYM(CommAbort, "ncclCommAbort")
    ORION_NCCL_SYM(CommDestroy, "ncclCommDestroy")
    ORION_NCCL_SYM(GetErrorString, "ncclGetErrorString")
    ORION_NCCL_SYM(AllReduce, "ncclAllReduce")
    ORION_NCCL_SYM(AllGather, "ncclAllGather")
    ORION_NCCL_SYM(ReduceScatter, "ncclReduceScatter")
#undef ORION_NCCL_SYM
    a.StreamQuery = cudaStreamQuery;
    a.ok = true;
  });
  return a;
}

uint64_t env_seconds_ms(const char *name, uint64_t fallback_s) {
  const char *v = std::getenv(name);
  const long s = v ? std::atol(v) : 0;
  return (s > 0 ? (uint64_t)s : fallback_s) * 1000ull;
}

using Clock = std::chrono::steady_clock;
uint64_t ms_since(Clock::time_point t0) {
  return (uint64_t)std::chrono::duration_cast<std::chrono::milliseconds>(Clock::now() - t0).count();
}

}  // namespace

NcclCollective::NcclCollective() {  // the library is looked up by init(): a single rank never needs it
  init_limit_ms_ = env_seconds_ms("ORION_TP_INIT_TIMEOUT_S", 300);
  step_limit_ms_ = env_seconds_ms("ORION_TP_STEP_TIMEOUT_S", 60);
}

NcclCollective::~NcclCollective() {
  // An aborted communicator is already gone; a healthy one is destroyed (which may wait for its
  // own outstanding work, all of it long finished by the time a model is torn down).
  if (comm_ && api_ && api_->ok && !aborted_) api_->CommDestroy(static_cast<ncclComm_t>(comm_));
  if (barrier_word_) cudaFree(barrier_word_);
}

int NcclCollective::dead(const char *stage) const {
  return set_error(ORION_ERR_BACKEND, "backend cuda failed at %s: the communicator was aborted after an earlier failure",
                   stage);
}

int NcclCollective::abort_with(const char *stage, const char *why) {
  if (comm_ && !aborted_) api_->CommAbort(static_cast<ncclComm_t>(comm_));
  aborted_ = true;
  comm_ = nullptr;
  return set_error(ORION_ERR_BACKEND, "backend cuda failed at %s: %s; communicator aborted", stage, why);
}

int NcclCollective::settle(int nccl_result, const char *stage, uint64_t limit_ms) {
  ncclResult_t r = static_cast<ncclResult_t>(nccl_result);
  const Clock::time_point t0 = Clock::now();
  while (r == ncclInProgress) {
    ++polls_;
    ncclResult_t state = ncclSuccess;
    const ncclResult_t q = api_->CommGetAsyncError(static_cast<ncclComm_t>(comm_), &state);
    if (q != ncclSuccess) return abort_with(stage, api_->GetErrorString(q));
    r = state;
    if (r != ncclInProgress) break;
    if (ms_since(t0) > limit_ms) return abort_with(stage, "a peer did not answer within the time limit");
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
  if (r != ncclSuccess) return abort_with(stage, api_->GetErrorString(r));
  return ORION_OK;
}

int NcclCollective::unique_id(uint8_t id[128]) {
  NcclApi &a = real_api();
  if (!a.ok) return set_error(ORION_ERR_BACKEND, "backend cuda failed at nccl load: libnccl.so.2 not found");
  ncclUniqueId u;
  const ncclResult_t r = a.GetUniqueId(&u);
  if (r != ncclSuccess) return set_error(ORION_ERR_BACKEND, "backend cuda failed at ncclGetUniqueId: %s", a.GetErrorString(r));
  static_assert(sizeof(u) == 128, "ncclUniqueId is 128 bytes");
  std::memcpy(id, &u, 128);
  return ORION_OK;
}

int NcclCollective::init(const uint8_t id[128], int rank, int world) {
  if (!api_) api_ = &real_api();
  if (!api_->ok)
    return set_error(ORION_ERR_BACKEND, "backend cuda failed at nccl load: libnccl.so.2 not found");
  ncclUniqueId u;
  std::memcpy(&u, id, 128);
  ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
  config.blocking = 0;  // no call into this communicator ever blocks the host inside NCCL
  ncclComm_t c = nullptr;
  const ncclResult_t r = api_->CommInitRankConfig(&c, world, u, rank, &config);
  comm_ = c;
  rank_ = rank;
  world_ = world;
  if (r != ncclSuccess && r != ncclInProgress) {
    comm_ = nullptr;  // nothing to abort: the call failed outright
    return set_error(ORION_ERR_BACKEND, "backend cuda failed at ncclCommInitRank: %s", api_->GetErrorString(r));
  }
  // the rendezvous itself proceeds in the background: "in progress" until every rank has joined
  return settle(ncclInProgress, "ncclCommInitRank", init_limit_ms_);
}

int NcclCollective::all_reduce_sum(float *buf, size_t count, cudaStream_t stream) {
  if (world_ <= 1 || count == 0) return ORION_OK;  // SingleRank: summing one rank is the identity
  if (aborted_) return dead("all_reduce_sum");
  return settle(api_->AllReduce(buf, buf, count, ncclFloat32, ncclSum, static_cast<ncclComm_t>(comm_), stream),
                "all_reduce_sum", step_limit_ms_);
}

int NcclCollective::all_gather(const float *local, float *out, size_t count_per_rank,
                               cudaStream_t stream) {
  if (world_ <= 1) {
    ORION_CUDA_CHECK("all_gather", cudaMemcpyAsync(out, local, count_per_rank * sizeof(float),
                                                   cudaMemcpyDeviceToDevice, stream));
    return ORION_OK;
  }
  if (aborted_) return dead("all_gather");
  return settle(api_->AllGather(local, out, count_per_rank, ncclFloat32, static_cast<ncclComm_t>(comm_), stream),
                "all_gather", step_limit_ms_);
}

int NcclCollective::reduce_scatter_sum(const float *in, float *out, size_t count_per_rank,
                                       cudaStream_t stream) {
  if (world_ <= 1) {
    ORION_CUDA_CHECK("reduce_scatter", cudaMemcpyAsync(out, in, count_per_rank * sizeof(float),
                                                       cudaMemcpyDeviceToDevice, stream));
    return ORION_OK;
  }
  if (aborted_) return dead("reduce_scatter_sum");
  return settle(api_->ReduceScatter(in, out, count_per_rank, ncclFloat32, ncclSum, static_cast<ncclComm_t>(comm_), stream),
                "reduce_scatter_sum", step_limit_ms_);
}

int NcclCollective::barrier(cudaStream_t stream) {
  if (world_ <= 1) return ORION_OK;
  if (aborted_) return dead("barrier");
  if (!barrier_word_) {
    ORION_CUDA_CHECK("nccl barrier word", cudaMalloc(&barrier_word_, sizeof(float)));
    ORION_CUDA_CHECK("nccl barrier word", cudaMemset(barrier_word_, 0, sizeof(float)));
  }
  ORION_TRY(all_reduce_sum(barrier_word_, 1, stream));
  return wait_stream(stream, "barrier");
}

int NcclCollective::wait_stream(cudaStream_t stream, const char *stage) {
  if (world_ <= 1 || !api_) {
    ORION_CUDA_CHECK(stage, cudaStreamSynchronize(stream));
    return ORION_OK;
  }
  const Clock::time_point t0 = Clock::now();
  for (uint64_t spin = 0;; ++spin) {
    const cudaError_t q = api_->StreamQuery(stream);
    if (q == cudaSuccess) return ORION_OK;
    if (q != cudaErrorNotReady)
      return set_error(ORION_ERR_BACKEND, "backend cuda failed at %s: %s", stage, cudaGetErrorString(q));
    // the stream query is cheap and decides the latency of a healthy step; NCCL's state and the
    // clock are looked at every 64th round
    if ((spin & 63u) != 63u) continue;
    if (!aborted_ && comm_) {
      ++polls_;
      ncclResult_t state = ncclSuccess;
      const ncclResult_t g = api_->CommGetAsyncError(static_cast<ncclComm_t>(comm_), &state);
      if (g != ncclSuccess) return abort_with(stage, api_->GetErrorString(g));
      if (state != ncclSuccess && state != ncclInProgress) return abort_with(stage, api_->GetErrorString(state));
    }
    if (ms_since(t0) > step_limit_ms_) return abort_with(stage, "the step did not end within the time limit");
    if (spin > 4096) std::this_thread::yield();
  }
}

// ---- host self-test against a stand-in NCCL ----------------------------------------------------

namespace {
struct FakeState {
  int scenario = 0;
  int init_polls_left = 0;     // rendezvous answers "in progress" this many times
  int stream_polls_left = 0;   // the stream answers "not ready" this many times (-1 = for ever)
  int error_after_polls = -1;  // asynchronous error state turns to a remote error after this many polls
  int async_polls = 0;
  bool aborted = false, destroyed = false;
};
FakeState g_fake;
int g_fake_comm_storage = 0;

ncclResult_t fake_init(ncclComm_t *c, int, ncclUniqueId, int, ncclConfig_t *cfg) {
  *c = reinterpret_cast<ncclComm_t>(&g_fake_comm_storage);
  return cfg && cfg->blocking == 0 ? ncclInProgress : ncclInternalError;  // the caller must ask for non-blocking
}
ncclResult_t fake_async(ncclComm_t, ncclResult_t *state) {
  ++g_fake.async_polls;
  if (g_fake.scenario == 1) {  // a rank never arrives
    *state = ncclInProgress;
  } else if (g_fake.init_polls_left > 0) {
    --g_fake.init_polls_left;
    *state = ncclInProgress;
  } else if (g_fake.error_after_polls >= 0 && g_fake.async_polls > g_fake.error_after_polls) {
    *state = ncclRemoteError;
  } else {
    *state = ncclSuccess;
  }
  return ncclSuccess;
}
ncclResult_t fake_abort(ncclComm_t) {
  g_fake.aborted = true;
  return ncclSuccess;
}
ncclResult_t fake_destroy(ncclComm_t) {
  g_fake.destroyed = true;
  return ncclSuccess;
}
const char *fake_error_string(ncclResult_t r) {
  switch (r) {
    case ncclRemoteError: return "remote process exited or there was a network error";
    case ncclInProgress: return "operation in progress";
    default: return "stand-in nccl error";
  }
}
ncclResult_t fake_allreduce(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) {
  return ncclInProgress;  // settled by polling, like a non-blocking communicator may answer
}
cudaError_t fake_stream_query(cudaStream_t) {
  if (g_fake.stream_polls_left < 0) return cudaErrorNotReady;
  if (g_fake.stream_polls_left == 0) return cudaSuccess;
  --g_fake.stream_polls_left;
  return cudaErrorNotReady;
}
}  // namespace

int nccl_failure_selftest(int scenario, uint64_t limit_ms, uint32_t *aborted, uint64_t *polls) {
  if (scenario < 0 || scenario > 3) return set_error(ORION_ERR_INVALID_REQUEST, "self-test scenario %d outside 0..3", scenario);
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  g_fake = FakeState{};
  g_fake.scenario = scenario;
  g_fake.init_polls_left = 3;
  g_fake.stream_polls_left = (scenario == 2 || scenario == 3) ? -1 : 500;
  g_fake.error_after_polls = scenario == 2 ? 6 : -1;
  NcclApi fake;
  fake.CommInitRankConfig = fake_init;
  fake.CommGetAsyncError = fake_async;
  fake.CommAbort = fake_abort;
  fake.CommDestroy = fake_destroy;
  fake.GetErrorString = fake_error_string;
  fake.AllReduce = fake_allreduce;
  fake.StreamQuery = fake_stream_query;
  fake.ok = true;
  int rc = ORION_OK;
  uint64_t n_polls = 0;
  {
    NcclCollective c(&fake);
    c.set_limits(limit_ms, limit_ms);
    const uint8_t id[128] = {};
    rc = c.init(id, 0, 2);
    float dummy = 0.f;
    if (rc == ORION_OK) rc = c.all_reduce_sum(&dummy, 1, nullptr);  // the stand-in never touches the buffer
    if (rc == ORION_OK) rc = c.wait_stream(nullptr, "all_reduce");
    if (rc != ORION_OK && !c.aborted()) rc = set_error(ORION_ERR_INTERNAL, "self-test: a failed call left the communicator alive");
    if (rc != ORION_OK) {
      // a dead communicator refuses further work instead of touching NCCL again
      const std::string first = orion_cuda_last_error();
      const int again = c.all_reduce_sum(&dummy, 1, nullptr);
      if (again != ORION_ERR_BACKEND) rc = set_error(ORION_ERR_INTERNAL, "self-test: an aborted communicator accepted a call");
      else set_error(rc, "%s", first.c_str());  // report the failure itself, not the refusal that followed
    }
    n_polls = c.polls();
  }
  if (aborted) *aborted = g_fake.aborted ? 1u : 0u;
  if (polls) *polls = n_polls;
  if (rc == ORION_OK && !g_fake.destroyed) return set_error(ORION_ERR_INTERNAL, "self-test: a healthy communicator was not destroyed");
  if (rc != ORION_OK && g_fake.destroyed) return set_error(ORION_ERR_INTERNAL, "self-test: an aborted communicator was destroyed again");
  return rc;
}

}  // namespace orion
