// NCCL backing of the tensor-parallel collectives; see tp_nccl.h.
#include "tp_nccl.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace orion {
namespace {

struct NcclApi {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t,
                                ncclComm_t, cudaStream_t) = nullptr;
  bool ok = false;
};

NcclApi &api() {
  static NcclApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    // A process that already holds NCCL (for instance through its tensor
    // framework) gets that copy back; otherwise the system library is opened.
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!a.handle) a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!a.handle) return;
#define ORION_NCCL_SYM(field, name)                                        \
  a.field = reinterpret_cast<decltype(a.field)>(dlsym(a.handle, name));   \
  if (!a.field) return;
    ORION_NCCL_SYM(GetUniqueId, "ncclGetUniqueId")
    ORION_NCCL_SYM(CommInitRank, "ncclCommInitRank")
    ORION_NCCL_SYM(CommDestroy, "ncclCommDestroy")
    ORION_NCCL_SYM(GetErrorString, "ncclGetErrorString")
    ORION_NCCL_SYM(AllReduce, "ncclAllReduce")
    ORION_NCCL_SYM(AllGather, "ncclAllGather")
    ORION_NCCL_SYM(ReduceScatter, "ncclReduceScatter")
#undef ORION_NCCL_SYM
    a.ok = true;
  });
  return a;
}

int nccl_fail(const char *stage, ncclResult_t r) {
  return set_error(ORION_ERR_BACKEND, "backend cuda failed at %s: %s", stage,
                   api().GetErrorString ? api().GetErrorString(r) : "nccl error");
}

#define ORION_NCCL_CHECK(stage, expr)                       \
  do {                                                      \
    ncclResult_t _r = (expr);                               \
    if (_r != ncclSuccess) return nccl_fail(stage, _r);     \
  } while (0)

int need_api() {
  if (!api().ok)
    return set_error(ORION_ERR_BACKEND, "backend cuda failed at nccl load: libnccl.so.2 not found");
  return ORION_OK;
}

}  // namespace

NcclCollective::~NcclCollective() {
  if (comm_ && api().ok) api().CommDestroy(static_cast<ncclComm_t>(comm_));
  if (barrier_word_) cudaFree(barrier_word_);
}

int NcclCollective::unique_id(uint8_t id[128]) {
  ORION_TRY(need_api());
  ncclUniqueId u;
  ORION_NCCL_CHECK("ncclGetUniqueId", api().GetUniqueId(&u));
  static_assert(sizeof(u) == 128, "ncclUniqueId is 128 bytes");
  std::memcpy(id, &u, 128);
  return ORION_OK;
}

int NcclCollective::init(const uint8_t id[128], int rank, int world) {
  ORION_TRY(need_api());
  ncclUniqueId u;
  std::memcpy(&u, id, 128);
  ncclComm_t c = nullptr;
  ORION_NCCL_CHECK("ncclCommInitRank", api().CommInitRank(&c, world, u, rank));
  comm_ = c;
  rank_ = rank;
  world_ = world;
  ORION_CUDA_CHECK("nccl barrier word", cudaMalloc(&barrier_word_, sizeof(float)));
  ORION_CUDA_CHECK("nccl barrier word", cudaMemset(barrier_word_, 0, sizeof(float)));
  return ORION_OK;
}

int NcclCollective::all_reduce_sum(float *buf, size_t count, cudaStream_t stream) {
  if (world_ <= 1 || count == 0) return ORION_OK;  // SingleRank: summing one rank is the identity
  ORION_NCCL_CHECK("all_reduce_sum", api().AllReduce(buf, buf, count, ncclFloat32, ncclSum,
                                                     static_cast<ncclComm_t>(comm_), stream));
  return ORION_OK;
}

int NcclCollective::all_gather(const float *local, float *out, size_t count_per_rank,
                               cudaStream_t stream) {
  if (world_ <= 1) {
    ORION_CUDA_CHECK("all_gather", cudaMemcpyAsync(out, local, count_per_rank * sizeof(float),
                                                   cudaMemcpyDeviceToDevice, stream));
    return ORION_OK;
  }
  ORION_NCCL_CHECK("all_gather", api().AllGather(local, out, count_per_rank, ncclFloat32,
                                                 static_cast<ncclComm_t>(comm_), stream));
  return ORION_OK;
}

int NcclCollective::reduce_scatter_sum(const float *in, float *out, size_t count_per_rank,
                                       cudaStream_t stream) {
  if (world_ <= 1) {
    ORION_CUDA_CHECK("reduce_scatter", cudaMemcpyAsync(out, in, count_per_rank * sizeof(float),
                                                       cudaMemcpyDeviceToDevice, stream));
    return ORION_OK;
  }
  ORION_NCCL_CHECK("reduce_scatter_sum",
                   api().ReduceScatter(in, out, count_per_rank, ncclFloat32, ncclSum,
                                       static_cast<ncclComm_t>(comm_), stream));
  return ORION_OK;
}

int NcclCollective::barrier(cudaStream_t stream) {
  if (world_ <= 1) return ORION_OK;
  ORION_TRY(all_reduce_sum(barrier_word_, 1, stream));
  ORION_CUDA_CHECK("barrier", cudaStreamSynchronize(stream));
  return ORION_OK;
}

}  // namespace orion
