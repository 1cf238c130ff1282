// Device self-tests of the failure-detection building blocks. Every wait in the kernels of this
// library (mbarrier pipelines of the GEMM and the attention kernels, the peer polls of the
// tensor-parallel hand-over) is bounded by %globaltimer: when the limit passes the waiter gives
// up, records an error word and the kernel runs to its end, so the context stays usable and the
// host reports EngineError::Backend. This file lets a test make such a wait run out on purpose,
// the harmless way: a barrier that nothing ever arrives at, and a short limit.
#include "kernels.h"

namespace orion {
namespace {

__global__ void bounded_wait_probe_kernel(uint64_t limit_ns, uint32_t *result) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint64_t t0 = global_timer_ns();
    const bool completed = mbar_wait(&bar, 0, limit_ns);  // nobody arrives: must return false after the limit
    result[0] = completed ? 0u : 1u;
    const uint64_t waited = global_timer_ns() - t0;
    result[1] = (uint32_t)(waited / 1000);  // microseconds spent waiting
  }
}

}  // namespace

int selftest_bounded_wait(uint64_t limit_us, uint32_t *timed_out, uint32_t *waited_us) {
  if (limit_us == 0 || limit_us > 1000000)
    return set_error(ORION_ERR_INVALID_REQUEST, "the probe takes a limit between 1 us and 1 s");
  uint32_t *d = nullptr;
  ORION_CUDA_CHECK("allocate", cudaMalloc(reinterpret_cast<void **>(&d), 2 * sizeof(uint32_t)));
  cudaMemset(d, 0, 2 * sizeof(uint32_t));
  bounded_wait_probe_kernel<<<1, 32>>>(limit_us * 1000, d);
  uint32_t h[2] = {0, 0};
  cudaError_t e = cudaMemcpy(h, d, sizeof h, cudaMemcpyDeviceToHost);
  cudaFree(d);
  ORION_CUDA_CHECK("bounded wait probe", e);
  if (timed_out) *timed_out = h[0];
  if (waited_us) *waited_us = h[1];
  return ORION_OK;
}

}  // namespace orion
