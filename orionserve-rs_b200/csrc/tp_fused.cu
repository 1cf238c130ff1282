// Fused tensor-parallel hand-over after a row-parallel projection (O or down):
//   all-reduce of the per-rank partial sums  +  residual add  +  RMSNorm
// in ONE kernel over peer-mapped memory (orion-distributed/src/lib.rs:317-319 places one
// all-reduce here; transformer.rs:330-336 the residual add and the norm).
//
// One-shot, flag-in-data: every thread folds this rank's split-K slabs for four elements,
// pushes the four sums into every peer's inbox with plain peer stores over NVLink, then
// collects the peers' sums for the same four elements from its own inbox, adds them in rank
// order (identical on every rank, so all ranks hold bit-identical residual streams), updates
// the f32 residual and normalises the row. Each 8-byte unit in an inbox carries one f32 and
// the 32-bit epoch of the hand-over, so a unit validates itself: there is no barrier, no
// fence and no separate flag, and the only latency on the path is one NVLink store.
//
// Inboxes are double-buffered by the parity of the epoch. A rank can enter hand-over k+2
// only after it received every peer's data of hand-over k+1, which a peer sends only after
// it finished reading hand-over k, so a slot is never overwritten while it is being read.
//
// Every wait is bounded: after about two seconds a thread records an error word and goes
// on with what it has; the host turns the word into a backend error after the step.
// One process per GPU; the kernel never waits on another launch on the same GPU.
#include "kernels.h"

#include <algorithm>
#include <cstdlib>
#include <type_traits>

namespace orion {
namespace {

__device__ uint32_t g_tp_error = 0;
#ifdef ORION_TRACE
// Phase trace, compiled in with -DORION_TRACE only and switched on by ORION_TP_TRACE=1: %globaltimer at
// the phase boundaries of CTA 0 of the most recent launches. Stamps: 0 entry, 1 dependency wait over,
// 2 slabs folded and sent, 3 owned groups reduced and published (one-shot: sums received), 4 end,
// 5 the latest end over all CTAs of the launch.
constexpr int kTpTraceLaunches = 80;
__device__ unsigned long long g_tp_trace[kTpTraceLaunches][8];
__device__ uint32_t g_tp_trace_on = 0, g_tp_trace_next = 0, g_tp_trace_slot = 0;
__device__ __forceinline__ void trace(int k) {
  if (g_tp_trace_on && blockIdx.x == 0 && threadIdx.x == 0) {
    if (k == 0) {
      g_tp_trace_slot = g_tp_trace_next++ % kTpTraceLaunches;
      g_tp_trace[g_tp_trace_slot][5] = 0;
    }
    g_tp_trace[g_tp_trace_slot][k] = global_timer_ns();
  }
  // CTA 0 has chosen the slot long before any CTA ends
  if (g_tp_trace_on && k == 4 && threadIdx.x == 0) atomicMax(&g_tp_trace[g_tp_trace_slot][5], global_timer_ns());
}
#else
__device__ __forceinline__ void trace(int) {}
#endif

__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_unit2(uint32_t *dst, float a, float b, uint32_t epoch) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(__float_as_uint(a)), "r"(epoch),
               "r"(__float_as_uint(b)), "r"(epoch)
               : "memory");
}
__device__ __forceinline__ uint4 ld_unit2(const uint32_t *src) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
  return v;
}
// Polls two 16-byte slots (four self-validating units) until all carry `epoch`.
__device__ __forceinline__ float4 receive4(const uint32_t *src, uint32_t epoch, uint64_t limit_ns) {
  uint4 lo = ld_unit2(src), hi = ld_unit2(src + 4);
  if (lo.y != epoch || lo.w != epoch || hi.y != epoch || hi.w != epoch) {
    const uint64_t start = global_timer_ns();
    uint32_t spins = 0;
    do {
      lo = ld_unit2(src);
      hi = ld_unit2(src + 4);
      if ((++spins & 1023u) == 0 && global_timer_ns() - start > limit_ns) {
        atomicOr(&g_tp_error, 1u);
        break;
      }
    } while (lo.y != epoch || lo.w != epoch || hi.y != epoch || hi.w != epoch);
  }
  return make_float4(__uint_as_float(lo.x), __uint_as_float(lo.z), __uint_as_float(hi.x), __uint_as_float(hi.z));
}

// A group of four elements as the two-shot kernel sends it. Wide: four {f32, epoch} units (32 bytes at
// word offset 2 x element). Packed: two {bf16 pair, epoch} units (16 bytes at word offset = element),
// the bf16 payload with f32 accumulation that orion-distributed/src/lib.rs:317-319 has in mind.
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&p);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&u));
}
template <bool Packed>
__device__ __forceinline__ void send_group(uint32_t *base, size_t element, float4 v, uint32_t epoch) {
  if (Packed) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(base + element), "r"(pack_bf16x2(v.x, v.y)),
                 "r"(epoch), "r"(pack_bf16x2(v.z, v.w)), "r"(epoch)
                 : "memory");
  } else {
    st_unit2(base + element * 2, v.x, v.y, epoch);
    st_unit2(base + element * 2 + 4, v.z, v.w, epoch);
  }
}
template <bool Packed>
__device__ __forceinline__ float4 receive_group(const uint32_t *base, size_t element, uint32_t epoch, uint64_t limit_ns) {
  if (!Packed) return receive4(base + element * 2, epoch, limit_ns);
  const uint32_t *src = base + element;
  uint4 u = ld_unit2(src);
  if (u.y != epoch || u.w != epoch) {
    const uint64_t start = global_timer_ns();
    uint32_t spins = 0;
    do {
      u = ld_unit2(src);
      if ((++spins & 1023u) == 0 && global_timer_ns() - start > limit_ns) {
        atomicOr(&g_tp_error, 1u);
        break;
      }
    } while (u.y != epoch || u.w != epoch);
  }
  const float2 lo = unpack_bf16x2(u.x), hi = unpack_bf16x2(u.z);
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

template <typename T>
__device__ __forceinline__ void st_row4(T *dst, float4 v);
template <>
__device__ __forceinline__ void st_row4<float>(float *dst, float4 v) { *reinterpret_cast<float4 *>(dst) = v; }
template <>
__device__ __forceinline__ void st_row4<bf16>(bf16 *dst, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 packed;
  packed.x = *reinterpret_cast<uint32_t *>(&lo);
  packed.y = *reinterpret_cast<uint32_t *>(&hi);
  *reinterpret_cast<uint2 *>(dst) = packed;
}

// One CTA per batch row. Packed: the sums travel as bf16 pairs (half the NVLink bytes); every rank
// then adds the bf16-rounded sums of ALL ranks, its own included, so the residual streams stay
// bit-identical across ranks.
template <typename T, typename Acc, bool Packed>
__global__ void __launch_bounds__(1024)
tp_allreduce_residual_rmsnorm_kernel(TpPeers peers, const uint32_t *epoch_base, uint32_t epoch_add, const float *__restrict__ partial,
                                     uint32_t splits, size_t split_stride, float *__restrict__ hidden,
                                     const float *__restrict__ w, float eps, T *__restrict__ out, uint32_t H,
                                     uint32_t *__restrict__ ready) {
  __shared__ Acc red[32];
  pdl_trigger();
  trace(0);
  pdl_wait();  // this rank's projection has finished
  trace(1);
  // the epoch of this hand-over: the step's first epoch (device state, advanced once per step) + its place in the step
  const uint32_t epoch = (epoch_base ? ld_volatile_u32(epoch_base) : 0u) + epoch_add;
  const uint32_t nvec = H / 4, row = blockIdx.x;
  const size_t slot = (size_t)peers.slot_floats * 2;  // u32 words per (parity, sender) slot
  const size_t parity_base = (size_t)(epoch & 1u) * peers.world * slot;
  float4 v[4];  // H / 4 <= 4 * blockDim.x is guaranteed by the launcher

  // ---- send: fold the local split-K slabs and push the sums to every peer ----
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t idx = threadIdx.x + c * blockDim.x;
    if (idx < nvec) {
      const size_t off = (size_t)row * H + 4 * (size_t)idx;
      v[c] = sum_slabs4(partial + off, splits, split_stride);
      for (int r = 0; r < peers.world; ++r)
        if (r != peers.rank) send_group<Packed>(peers.inbox[r] + parity_base + (size_t)peers.rank * slot, off, v[c], epoch);
      if (Packed) {  // what the peers receive is what this rank adds for itself
        const float2 lo = unpack_bf16x2(pack_bf16x2(v[c].x, v[c].y)), hi = unpack_bf16x2(pack_bf16x2(v[c].z, v[c].w));
        v[c] = make_float4(lo.x, lo.y, hi.x, hi.y);
      }
    }
  }
  trace(2);
  // ---- receive: add the ranks' sums in rank order, update the residual ----
  Acc ss = Acc(0);
  float *h = hidden + (size_t)row * H;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t idx = threadIdx.x + c * blockDim.x;
    if (idx < nvec) {
      const size_t off = (size_t)row * H + 4 * (size_t)idx;
      float4 add = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < peers.world; ++r) {
        const float4 x = r == peers.rank ? v[c]
                                         : receive_group<Packed>(peers.inbox[peers.rank] + parity_base + (size_t)r * slot, off, epoch,
                                                                 peers.wait_limit_ns);
        add.x += x.x; add.y += x.y; add.z += x.z; add.w += x.w;
      }
      const float4 old = *reinterpret_cast<const float4 *>(h + 4 * (size_t)idx);
      v[c] = make_float4(old.x + add.x, old.y + add.y, old.z + add.z, old.w + add.w);
      *reinterpret_cast<float4 *>(h + 4 * (size_t)idx) = v[c];
      ss += (Acc)v[c].x * (Acc)v[c].x + (Acc)v[c].y * (Acc)v[c].y + (Acc)v[c].z * (Acc)v[c].z +
            (Acc)v[c].w * (Acc)v[c].w;
    }
  }
  trace(3);
  // ---- RMSNorm of the row (tensor.rs:143-163) ----
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  Acc total = Acc(0);
  for (uint32_t i = 0; i < (blockDim.x + 31) / 32; ++i) total += red[i];
  const float scale = sizeof(Acc) == 8 ? (float)(1.0 / sqrt((double)total / (double)H + (double)eps))
                                       : rsqrtf((float)total / (float)H + eps);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t idx = threadIdx.x + c * blockDim.x;
    if (idx < nvec) {
      const float4 g = *reinterpret_cast<const float4 *>(w + 4 * (size_t)idx);
      st_row4<T>(out + (size_t)row * H + 4 * (size_t)idx,
                 make_float4(__fmul_rn(__fmul_rn(v[c].x, scale), g.x), __fmul_rn(__fmul_rn(v[c].y, scale), g.y),
                             __fmul_rn(__fmul_rn(v[c].z, scale), g.z), __fmul_rn(__fmul_rn(v[c].w, scale), g.w)));
    }
  }
  trace(4);
  if (ready) {  // the next projection polls this count instead of waiting for the kernel to complete
    __syncthreads();
    if (threadIdx.x == 0) signal_ready(ready);
  }
}

// Two-shot variant for more than two ranks. One CTA per row on every rank; inside a row the
// four-float groups are dealt to the ranks in contiguous slices, and a rank owns its slice of
// EVERY row, so all CTAs of all ranks send and receive the same amount in both phases (with rows
// owned whole, only the owner's few CTAs would publish, and a handful of SMs cannot fill NVLink).
//   reduce-scatter: a thread pushes the folded sums of the groups it does not own to their owners;
//   reduce:         for a group it owns it collects the peers' sums, adds them in rank order and
//   all-gather:     pushes the total to every peer;
//   every thread then has the total of each of its groups (its own or received), adds it to the
//   residual (all ranks add identical totals, so the residual streams stay bit-identical) and the
//   CTA normalises the row.
// Both pushes use the self-validating 8-byte units of the one-shot kernel: no barrier, no fence.
// All pushes of a phase are issued before any poll of the next, so a thread never waits for data
// whose sender waits for this thread. A rank sends rows x H x 8 B x (world-1)/world twice instead
// of world - 1 times. Inbox of a rank: [parity 2][sender world][slot] units for the
// reduce-scatter, then [parity 2][slot] units for the all-gather, both addressed by (row, element).
template <typename T, typename Acc, bool Packed>
__global__ void __launch_bounds__(1024)
tp_twoshot_kernel(TpPeers peers, const uint32_t *epoch_base, uint32_t epoch_add, const float *__restrict__ partial, uint32_t splits,
                  size_t split_stride, float *__restrict__ hidden, const float *__restrict__ w, float eps,
                  T *__restrict__ out, uint32_t rows, uint32_t H, uint32_t *__restrict__ ready) {
  __shared__ Acc red[32];
  pdl_trigger();
  trace(0);
  pdl_wait();  // this rank's projection has finished
  trace(1);
  // the epoch of this hand-over: the step's first epoch (device state, advanced once per step) + its place in the step
  const uint32_t epoch = (epoch_base ? ld_volatile_u32(epoch_base) : 0u) + epoch_add;
  (void)rows;
  const uint32_t nvec = H / 4, row = blockIdx.x;
  const uint32_t per = (nvec + peers.world - 1) / peers.world;  // groups per owner
  const size_t slot = (size_t)peers.slot_floats * 2;            // u32 words per slot
  const size_t scatter = ((size_t)(epoch & 1u) * peers.world) * slot;  // + sender * slot
  const size_t gather = (size_t)2 * peers.world * slot + (size_t)(epoch & 1u) * slot;
  float4 v[4];  // H / 4 <= 4 * blockDim.x is guaranteed by the launcher
  // ---- fold the local split-K slabs; hand the groups of other owners over ----
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t idx = threadIdx.x + c * blockDim.x;
    if (idx < nvec) {
      const size_t off = (size_t)row * H + 4 * (size_t)idx;
      v[c] = sum_slabs4(partial + off, splits, split_stride);
      const int owner = (int)(idx / per);
      if (owner != peers.rank)
        send_group<Packed>(peers.inbox[owner] + scatter + (size_t)peers.rank * slot, off, v[c], epoch);
    }
  }
  trace(2);
  // ---- own groups: collect, add in rank order, publish the totals ----
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t idx = threadIdx.x + c * blockDim.x;
    if (idx < nvec && (int)(idx / per) == peers.rank) {
      const size_t off = (size_t)row * H + 4 * (size_t)idx;
      float4 add = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < peers.world; ++r) {
        const float4 x = r == peers.rank
                             ? v[c]
                             : receive_group<Packed>(peers.inbox[peers.rank] + scatter + (size_t)r * slot, off, epoch, peers.wait_limit_ns);
        add.x += x.x; add.y += x.y; add.z += x.z; add.w += x.w;
      }
      if (Packed) {  // every rank must add exactly what the peers receive
        const float2 lo = unpack_bf16x2(pack_bf16x2(add.x, add.y)), hi = unpack_bf16x2(pack_bf16x2(add.z, add.w));
        add = make_float4(lo.x, lo.y, hi.x, hi.y);
      }
      v[c] = add;
      for (int r = 0; r < peers.world; ++r)
        if (r != peers.rank) send_group<Packed>(peers.inbox[r] + gather, off, add, epoch);
    }
  }
  trace(3);
  // ---- the other groups: receive the totals; residual update on every rank ----
  Acc ss = Acc(0);
  float *h = hidden + (size_t)row * H;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t idx = threadIdx.x + c * blockDim.x;
    if (idx < nvec) {
      const size_t off = (size_t)row * H + 4 * (size_t)idx;
      const float4 add = (int)(idx / per) == peers.rank
                             ? v[c]
                             : receive_group<Packed>(peers.inbox[peers.rank] + gather, off, epoch, peers.wait_limit_ns);
      const float4 old = *reinterpret_cast<const float4 *>(h + 4 * (size_t)idx);
      v[c] = make_float4(old.x + add.x, old.y + add.y, old.z + add.z, old.w + add.w);
      *reinterpret_cast<float4 *>(h + 4 * (size_t)idx) = v[c];
      ss += (Acc)v[c].x * (Acc)v[c].x + (Acc)v[c].y * (Acc)v[c].y + (Acc)v[c].z * (Acc)v[c].z +
            (Acc)v[c].w * (Acc)v[c].w;
    }
  }
  // ---- RMSNorm of the row (tensor.rs:143-163) ----
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  Acc total = Acc(0);
  for (uint32_t i = 0; i < (blockDim.x + 31) / 32; ++i) total += red[i];
  const float scale = sizeof(Acc) == 8 ? (float)(1.0 / sqrt((double)total / (double)H + (double)eps))
                                       : rsqrtf((float)total / (float)H + eps);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t idx = threadIdx.x + c * blockDim.x;
    if (idx < nvec) {
      const float4 g = *reinterpret_cast<const float4 *>(w + 4 * (size_t)idx);
      st_row4<T>(out + (size_t)row * H + 4 * (size_t)idx,
                 make_float4(__fmul_rn(__fmul_rn(v[c].x, scale), g.x), __fmul_rn(__fmul_rn(v[c].y, scale), g.y),
                             __fmul_rn(__fmul_rn(v[c].z, scale), g.z), __fmul_rn(__fmul_rn(v[c].w, scale), g.w)));
    }
  }
  trace(4);
  if (ready) {  // the next projection polls this count instead of waiting for the kernel to complete
    __syncthreads();
    if (threadIdx.x == 0) signal_ready(ready);
  }
}

}  // namespace

template <typename T>
int launch_tp_allreduce_residual_rmsnorm(const TpPeers &peers, const uint32_t *epoch_base, uint32_t epoch_add, const float *partial, uint32_t splits,
                                         size_t split_stride, float *hidden, const float *norm_w, float eps, T *out,
                                         uint32_t rows, uint32_t hidden_size, bool two_shot, cudaStream_t stream,
                                         uint32_t *ready) {
  if (hidden_size % 4 != 0 || hidden_size / 4 > 4096 || split_stride % 4 != 0 ||
      (size_t)rows * hidden_size > peers.slot_floats || (epoch_base == nullptr && (epoch_add == 0 || epoch_add == 0xFFFFFFFFu)))
    return set_error(ORION_ERR_INTERNAL, "fused tensor-parallel hand-over: unsupported shape or epoch");
  if (rows == 0) return ORION_OK;
  const uint32_t nvec = hidden_size / 4;
  uint32_t threads = nvec >= 1024 ? 1024 : ((nvec + 31) / 32) * 32;
  if (threads < 32) threads = 32;
  using Acc = typename std::conditional<sizeof(T) == 4, double, float>::type;
  // What the kernels of the bf16 build send: bf16 pairs (default; half the NVLink bytes, measured
  // 29.2 -> 27.6 ms per batch-128 step of the 70B shape at 2 ranks) or, with ORION_TP_PAYLOAD=f32, f32 values.
  // The f32 build always sends f32.
  static const bool packed = [] {
    const char *e = std::getenv("ORION_TP_PAYLOAD");
    return e == nullptr || e[0] != 'f';
  }();
  if (two_shot && sizeof(T) == 2 && packed)
    ORION_CUDA_CHECK("tp_allreduce_residual_rmsnorm",
                     launch_pdl(tp_twoshot_kernel<T, Acc, true>, dim3(rows), dim3(threads), 0, stream, peers, epoch_base, epoch_add,
                                partial, splits, split_stride, hidden, norm_w, eps, out, rows, hidden_size, ready));
  else if (two_shot)
    ORION_CUDA_CHECK("tp_allreduce_residual_rmsnorm",
                     launch_pdl(tp_twoshot_kernel<T, Acc, false>, dim3(rows), dim3(threads), 0, stream, peers, epoch_base, epoch_add,
                                partial, splits, split_stride, hidden, norm_w, eps, out, rows, hidden_size, ready));
  else if (sizeof(T) == 2 && packed)
    ORION_CUDA_CHECK("tp_allreduce_residual_rmsnorm",
                     launch_pdl(tp_allreduce_residual_rmsnorm_kernel<T, Acc, true>, dim3(rows), dim3(threads), 0, stream, peers,
                                epoch_base, epoch_add, partial, splits, split_stride, hidden, norm_w, eps, out, hidden_size, ready));
  else
    ORION_CUDA_CHECK("tp_allreduce_residual_rmsnorm",
                     launch_pdl(tp_allreduce_residual_rmsnorm_kernel<T, Acc, false>, dim3(rows), dim3(threads), 0, stream, peers,
                                epoch_base, epoch_add, partial, splits, split_stride, hidden, norm_w, eps, out, hidden_size, ready));
  count_launch();
  ORION_CUDA_CHECK("tp_allreduce_residual_rmsnorm", cudaGetLastError());
  return ORION_OK;
}
template int launch_tp_allreduce_residual_rmsnorm<float>(const TpPeers &, const uint32_t *, uint32_t, const float *, uint32_t, size_t,
                                                         float *, const float *, float, float *, uint32_t, uint32_t,
                                                         bool, cudaStream_t, uint32_t *);
template int launch_tp_allreduce_residual_rmsnorm<bf16>(const TpPeers &, const uint32_t *, uint32_t, const float *, uint32_t, size_t,
                                                        float *, const float *, float, bf16 *, uint32_t, uint32_t,
                                                        bool, cudaStream_t, uint32_t *);

namespace {
// Vocabulary-parallel LM head: a rank that has stored its column block of the logits into the
// leader's memory raises its flag there; the leader waits for every flag before it touches the logits.
// Advances the device-resident hand-over state at the end of a step: state[0] = the epoch of the next step's first
// hand-over, state[1] = the count of finished hand-over rows the next step starts from. Epochs stay inside
// 1 .. 0xFFFFFFFE and keep alternating in parity (the parity selects the inbox half).
__global__ void tp_state_bump_kernel(uint32_t *state, uint32_t epochs, uint32_t rows_counted) {
  pdl_trigger();
  pdl_wait();  // every hand-over of the step has read the state
  if (threadIdx.x == 0) {
    uint32_t e = state[0] + epochs;
    if (e > 0xFFFFFF00u) e = (e & 1u) ? 1u : 2u;
    state[0] = e;
    state[1] += rows_counted;
  }
}

__global__ void tp_signal_kernel(uint32_t *flag, uint32_t epoch) {
  pdl_trigger();
  pdl_wait();                // the projection that wrote the block has completed
  __threadfence_system();    // its peer stores are ordered before the flag at system scope
  if (threadIdx.x == 0) {
    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
  }
}
__global__ void tp_wait_flags_kernel(const uint32_t *flags, uint32_t epoch, int world, uint64_t limit_ns) {
  pdl_trigger();
  pdl_wait();
  const int r = (int)threadIdx.x + 1;  // flag of rank r; the leader has none
  if (r < world) {
    const volatile uint32_t *f = flags + r;
    if (*f != epoch) {
      const uint64_t start = global_timer_ns();
      uint32_t spins = 0;
      while (*f != epoch) {
        if ((++spins & 255u) == 0 && global_timer_ns() - start > limit_ns) {
          atomicOr(&g_tp_error, 2u);
          break;
        }
      }
    }
  }
  __threadfence_system();
}
}  // namespace

int launch_tp_state_bump(uint32_t *state, uint32_t epochs, uint32_t rows_counted, cudaStream_t stream) {
  ORION_CUDA_CHECK("tp_state_bump", launch_pdl(tp_state_bump_kernel, dim3(1), dim3(32), 0, stream, state, epochs, rows_counted));
  count_launch();
  ORION_CUDA_CHECK("tp_state_bump", cudaGetLastError());
  return ORION_OK;
}

int launch_tp_signal(uint32_t *flag, uint32_t epoch, cudaStream_t stream) {
  ORION_CUDA_CHECK("tp_signal", launch_pdl(tp_signal_kernel, dim3(1), dim3(32), 0, stream, flag, epoch));
  count_launch();
  return ORION_OK;
}
int launch_tp_wait_flags(const uint32_t *flags, uint32_t epoch, int world, uint64_t limit_ns, cudaStream_t stream) {
  ORION_CUDA_CHECK("tp_wait_flags", launch_pdl(tp_wait_flags_kernel, dim3(1), dim3(32), 0, stream, flags, epoch, world, limit_ns));
  count_launch();
  return ORION_OK;
}

namespace {
// One thread polls inbox units that nobody ever writes, in both unit formats, with the given limit.
__global__ void tp_peer_wait_probe_kernel(const uint32_t *inbox, uint32_t epoch, uint64_t limit_ns, uint32_t *waited_us) {
  if (threadIdx.x != 0) return;
  const uint64_t t0 = global_timer_ns();
  const float4 a = receive4(inbox, epoch, limit_ns);                     // f32 units
  const float4 b = receive_group<true>(inbox + 64, 0, epoch, limit_ns);  // packed bf16 units
  waited_us[0] = (uint32_t)((global_timer_ns() - t0) / 1000);
  waited_us[1] = __float_as_uint(a.x + b.x);  // keeps both polls alive
}
}  // namespace

int selftest_peer_wait(uint64_t limit_us, uint32_t *timed_out, uint32_t *waited_us) {
  if (limit_us == 0 || limit_us > 1000000)
    return set_error(ORION_ERR_INVALID_REQUEST, "the probe takes a limit between 1 us and 1 s");
  uint32_t code = 0;
  ORION_TRY(tp_poll_error(&code));  // start from a clear error word
  uint32_t *d = nullptr;
  ORION_CUDA_CHECK("allocate", cudaMalloc(reinterpret_cast<void **>(&d), 256 * sizeof(uint32_t)));
  cudaMemset(d, 0, 256 * sizeof(uint32_t));  // epoch 0 is never sent, so no unit ever validates
  tp_peer_wait_probe_kernel<<<1, 32>>>(d, 5u, limit_us * 1000, d + 128);
  uint32_t h[2] = {0, 0};
  cudaError_t e = cudaMemcpy(h, d + 128, sizeof h, cudaMemcpyDeviceToHost);
  cudaFree(d);
  ORION_CUDA_CHECK("peer wait probe", e);
  ORION_TRY(tp_poll_error(&code));  // the word the host reads after a step (and clears)
  if (timed_out) *timed_out = code ? 1u : 0u;
  if (waited_us) *waited_us = h[0];
  return ORION_OK;
}

int tp_poll_error(uint32_t *code) {
#ifdef ORION_TRACE
  static const bool tracing = std::getenv("ORION_TP_TRACE") != nullptr &&
                              (std::getenv("LOCAL_RANK") == nullptr || std::atoi(std::getenv("LOCAL_RANK")) == 0);  // one rank prints
  if (tracing) {
    uint32_t on = 1, next = 0;
    static unsigned long long t[kTpTraceLaunches][8];
    cudaMemcpyFromSymbol(t, g_tp_trace, sizeof t);
    cudaMemcpyFromSymbol(&next, g_tp_trace_next, sizeof next);
    cudaMemcpyToSymbol(g_tp_trace_on, &on, sizeof on);
    if (next >= (uint32_t)kTpTraceLaunches) {
      fprintf(stderr, "tp trace of CTA 0 (us): entry(abs mod 1e5) | gap-from-prev-end wait fold+send reduce+publish rest total-after-wait last-CTA-end-after-CTA-0\n");
      unsigned long long prev_end = 0;
      for (int i = 0; i < kTpTraceLaunches; ++i) {
        const unsigned long long *r = t[(next + i) % kTpTraceLaunches];
        fprintf(stderr, "  tp %10.2f | %7.2f %6.2f %6.2f %6.2f %6.2f %6.2f %6.2f\n", (double)(r[0] % 100000000ull) / 1e3,
                prev_end ? ((double)r[0] - (double)prev_end) / 1e3 : 0.0, (r[1] - r[0]) / 1e3, (r[2] - r[1]) / 1e3, (r[3] - r[2]) / 1e3,
                (r[4] - r[3]) / 1e3, (r[4] - r[1]) / 1e3, ((double)r[5] - (double)r[4]) / 1e3);
        prev_end = r[4];
      }
    }
  }
#endif
  uint32_t v = 0;
  ORION_CUDA_CHECK("tp error word", cudaMemcpyFromSymbol(&v, g_tp_error, sizeof v));
  if (v) {
    uint32_t zero = 0;
    ORION_CUDA_CHECK("tp error word", cudaMemcpyToSymbol(g_tp_error, &zero, sizeof zero));
  }
  *code = v;
  return ORION_OK;
}

}  // namespace orion
