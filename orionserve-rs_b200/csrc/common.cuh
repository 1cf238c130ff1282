// Shared helpers for the sm_100a kernels and their host launchers: error
// reporting in the reference's error vocabulary, storage-type conversion, and
// thin wrappers over the PTX used by more than one kernel (mbarrier, bulk
// async copies, TMA tensor copies, tcgen05).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/orion_cuda.h"

namespace orion {

// ---- errors ---------------------------------------------------------------

// Records the message for orion_cuda_last_error() and returns `status`.
int set_error(int status, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();

// EngineError::Backend{backend:"cuda", stage, reason} (orion-core/src/error.rs:119-124).
#define ORION_CUDA_CHECK(stage, expr)                                                      \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess)                                                                 \
      return ::orion::set_error(ORION_ERR_BACKEND, "backend cuda failed at %s: %s", stage, \
                                cudaGetErrorString(_e));                                   \
  } while (0)

#define ORION_TRY(expr)        \
  do {                         \
    int _rc = (expr);          \
    if (_rc != ORION_OK) return _rc; \
  } while (0)

// Number of kernels launched through launch accounting since the last reset.
extern thread_local uint64_t g_launch_count;
inline void count_launch() { ++g_launch_count; }

// Launches `kernel` with the programmatic-stream-serialization attribute (see
// pdl_wait / pdl_trigger below). `enabled` false gives a plain launch.
extern bool g_pdl_enabled;
// Counts the calls that change a tuning value; a captured step graph belongs to the value it was captured under.
extern uint32_t g_tuning_generation;
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl_enabled ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
// The same with the grid cut into thread-block clusters of `cluster` CTAs (each dimension of the
// grid must be a multiple of the cluster's).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem,
                                      cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl_enabled ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Opt-in to more than 48 KiB of dynamic shared memory for `kernel`. The attribute belongs to the
// (kernel, device) pair, so it is set once per device ordinal: `done` is the caller's static
// array of kMaxDeviceOrdinals flags for this kernel instantiation.
constexpr int kMaxDeviceOrdinals = 64;
template <typename K>
inline cudaError_t ensure_dynamic_smem(K kernel, int bytes, bool *done) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool tracked = dev >= 0 && dev < kMaxDeviceOrdinals;
  if (tracked && done[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && tracked) done[dev] = true;
  return e;
}

// ---- storage types ----------------------------------------------------------

using bf16 = __nv_bfloat16;

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum of `n` f32 slabs at `p` (slab stride `stride` floats), in slab order, four floats per call.
// The loads of a batch of eight slabs are independent of one another, so a batch costs one memory
// round trip rather than eight.
constexpr int kSlabBatch = 8;
__device__ __forceinline__ float4 sum_slabs4(const float *p, uint32_t n, size_t stride) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (uint32_t j0 = 0; j0 < n; j0 += kSlabBatch) {
    float4 x[kSlabBatch];
#pragma unroll
    for (int j = 0; j < kSlabBatch; ++j) {
      x[j] = (j0 + j < n) ? *reinterpret_cast<const float4 *>(p + (size_t)(j0 + j) * stride)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < kSlabBatch; ++j) {
      acc.x += x[j].x; acc.y += x[j].y; acc.z += x[j].z; acc.w += x[j].w;
    }
  }
  return acc;
}

// ---- PTX wrappers ------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls and reports failure, so that a
// missing arrival turns into an error status instead of a hung kernel.
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity,
                                          uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t start = global_timer_ns();
  for (uint32_t i = 0; i < (1u << 30); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && global_timer_ns() - start > limit_ns) return false;
  }
  return false;
}

// Untiled bulk async copy global -> shared (both 16-byte aligned, size % 16 == 0),
// completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_copy_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes,
                                              uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// 2-D tiled TMA load; c0 is the innermost coordinate (c0 * element size must be
// a multiple of 16 bytes).
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const void *tensor_map, int c0, int c1,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst_smem)),
      "l"(tensor_map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}

// Programmatic dependent launch. Every kernel of the step is launched with the
// programmatic-serialization attribute: it may become resident while its
// predecessor is still running, and must call pdl_wait() before it touches
// anything a kernel of the step writes (before the wait only immutable data —
// weights, norm gains, RoPE tables — may be read). pdl_wait() returns once the
// predecessor grid has completed and its writes are visible. pdl_trigger() lets
// the successor start its own prologue. Both are no-ops in a plain launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A dependency between two kernels of a step carried by a counter in device memory instead of by the
// completion of the earlier kernel. Every CTA of the producer adds 1 when its results are written
// (signal_ready, after a CTA-wide barrier); the consumer, already resident through its programmatic
// launch, polls until the counter has reached `target` and never executes griddepcontrol.wait. The
// counter only grows (the host keeps the running total), compared modulo 2^32. The wait is bounded.
struct ReadyWait {
  const uint32_t *counter = nullptr;  // nullptr: wait for the preceding kernel as usual
  uint32_t target = 0;
  const uint32_t *base = nullptr;     // if set, the target is *base + target (the step's starting count, device state)
};
__device__ __forceinline__ void signal_ready(uint32_t *counter) {
  __threadfence();
  atomicAdd(counter, 1u);
}
__device__ __forceinline__ bool wait_ready(ReadyWait r, uint64_t limit_ns = 2000000000ull) {
  if (r.base) {
    uint32_t b;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(b) : "l"(r.base) : "memory");
    r.target += b;
  }
  uint64_t start = 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(r.counter) : "memory");
    if ((int32_t)(v - r.target) >= 0) return true;
    if ((i & 63u) == 0u) {
      if (start == 0) start = global_timer_ns();
      else if (global_timer_ns() - start > limit_ns) return false;
    }
  }
}
// Orders this thread's generic-proxy accesses (the acquire above) before its later async-proxy ones (TMA loads).
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

}  // namespace orion
