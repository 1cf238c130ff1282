// bf16 GEMM on the 5th-generation tensor cores:  partial[s][r][n] = sum_k x[r][k] * w[n][k]
// (tensor.rs:114-128 without the bias), f32 accumulation in tensor memory.
//
// The weight matrix is the M operand of the MMA ("swap A/B"): a CTA owns a tile
// of 128 weight rows x TOKN tokens, so the batch size only changes the N extent
// of the instruction and a decode step (1..256 tokens) streams every weight
// byte exactly once. W [n][k] and x [r][k] are both K-major as stored, so no
// transposition is needed.
//
// Per CTA (256 threads):
//   warp 0   one lane streams the W tile (TMA tensor loads, 128B-swizzled 64-wide k
//            slabs) into the deep weight ring; it never waits for the preceding kernel;
//   warp 2   one lane waits for the preceding kernel (programmatic dependent launch),
//            then keeps the short activation ring full (x tiles come from L2);
//   warp 1   allocates tensor memory, one lane issues tcgen05.mma (128 x TOKN x 16,
//            four per k slab) and commits to the "empty" barriers of both stages;
//   warps 4-7 epilogue: tcgen05.ld the accumulator (lane = weight row, column =
//            token) and store f32 partials, 128 contiguous bytes per warp store.
// Split-K: blockIdx.z owns a contiguous range of k slabs and writes its own slab
// of the partial buffer; the consumer kernel sums the slabs.
// Every CTA loads its own tiles, nothing is multicast. Clusters appear in two optional forms only: CTA pairs
// for batches of 4096 rows and more (PAIR below), and the split-K reduction over distributed shared
// memory (off by default). The activation producer can take its dependency from a counter in device
// memory instead of the preceding kernel's completion (ReadyWait, used after a tensor-parallel hand-over).
// Every wait is bounded; a wait that runs out sets a device error word and the
// CTA still releases its tensor memory before returning.
#include "kernels.h"

#include <cuda.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

namespace orion {
namespace {

constexpr int kTileN = 128;   // weight rows per CTA (M of the MMA)
constexpr int kSlabK = 64;    // k elements per stage: 128 bytes = one swizzle atom
constexpr int kUmmaK = 16;
constexpr int kThreads = 256;

__device__ uint32_t g_gemm_error = 0;
#ifdef ORION_TRACE
// Phase trace, compiled in with -DORION_TRACE only and switched on by ORION_GEMM_TRACE=1:
// %globaltimer stamps of CTA (0,0,0) of the last launches.
constexpr int kTraceLaunches = 160, kTraceStamps = 8;
__device__ unsigned long long g_gemm_trace[kTraceLaunches][kTraceStamps];
__device__ uint32_t g_gemm_trace_on = 0, g_gemm_trace_next = 0;
__device__ __forceinline__ void gtrace(uint32_t slot, int k) {
  if (slot != 0xFFFFFFFFu) g_gemm_trace[slot][k] = global_timer_ns();
}
#define ORION_GTRACE(slot, k) gtrace(slot, k)
#else
#define ORION_GTRACE(slot, k) ((void)0)
#endif

// Two rings per CTA. Weight tiles come from HBM (long latency, the stream that must never
// stall): WST stages of 16 KiB. Activation tiles come from L2 (every CTA re-reads them):
// XST stages of TOKN x 128 B are enough. Measured on decode shapes, weight bandwidth follows
// the weight bytes in flight per SM (160 KiB -> 6.0 TB/s, 128 KiB -> 5.3 TB/s), so shared
// memory goes to the W ring first.
// MT = weight tiles of 128 rows per CTA. Decode batches stream weights (MT = 1, as many CTAs as
// possible); prefill batches are tensor-bound and limited by the shared-memory fill rate, so a
// CTA there takes two weight tiles against one activation tile (MT = 2: 64 KiB of operands per
// 2.1 MFLOP instead of 48 KiB per 1.05), with two accumulators in tensor memory.
// PAIR: two CTAs of a cluster work as one MMA unit (tcgen05 cta_group::2): each loads its own weight
// tiles and HALF of the activation tile, the leader issues 256-row MMAs that read both CTAs' shared
// memory and write both CTAs' tensor memory. Per CTA an activation stage is half as large, so a
// prefill-sized projection moves 48 KiB of operands per 8.4 MFLOP instead of 64 KiB.
template <int TOKN, int WST, int XST, int MT = 1, bool PAIR = false>
struct TcConfig {
  static constexpr int kWBytes = MT * kTileN * kSlabK * 2;
  static constexpr int kXRows = PAIR ? TOKN / 2 : TOKN;  // activation rows this CTA loads per stage
  static constexpr int kXBytes = kXRows * kSlabK * 2;
  static constexpr int kWStages = WST;
  static constexpr int kXStages = XST;
  static constexpr int kXRingOffset = WST * kWBytes;
  static constexpr int kBarrierOffset = kXRingOffset + XST * kXBytes;
  static constexpr int kTmemCols = MT * TOKN < 32 ? 32 : MT * TOKN;
  static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "tensor memory columns: a power of two up to 512");
  static constexpr int kSmemBytes = kBarrierOffset + 1024 /*align*/ + 512 /*barriers*/;
};

__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// ---- cta_group::2 (a pair of CTAs as one MMA unit) ----
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *dst_smem, uint32_t ncols) {  // one warp in EACH CTA of the pair
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrives on the barrier at cluster shared-memory address `bar_cluster_addr` (this CTA's or the
// peer's) once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 2-D tiled TMA load of one CTA of a pair: the data lands in THIS CTA's shared memory, the bytes are
// counted on the barrier at cluster address `bar_cluster_addr` (the leader's). No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void *dst_smem, const void *tensor_map, int c0, int c1,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst_smem)),
      "l"(tensor_map), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in cluster member `rank`.
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes
// with the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride offset),
// the leading offset is unused for swizzled K-major tiles (encoded 1),
// descriptor version 1, layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor: f32 accumulate, bf16 x bf16, both operands K-major,
// N = TOKN (>>3 at bit 17), M = 128 (>>4 at bit 24).
template <int TOKN, int M = kTileN>
__device__ __forceinline__ constexpr uint32_t instr_desc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TOKN >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

template <int TOKN, int WST, int XST, int MT, bool PAIR = false>
__global__ void __launch_bounds__(kThreads)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               float *__restrict__ partial, bf16 *__restrict__ act, uint32_t M, uint32_t N, uint32_t K,
               uint32_t splits, uint32_t cluster_reduce, uint32_t ldc, ReadyWait ready) {
  using Cfg = TcConfig<TOKN, WST, XST, MT, PAIR>;
  extern __shared__ uint8_t raw_smem[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                              ~uintptr_t(1023));
  uint8_t *w_ring = smem, *x_ring = smem + Cfg::kXRingOffset;
  uint64_t *full_w = reinterpret_cast<uint64_t *>(smem + Cfg::kBarrierOffset);
  uint64_t *empty_w = full_w + WST;
  uint64_t *full_x = empty_w + WST;
  uint64_t *empty_x = full_x + XST;
  uint64_t *acc_ready = empty_x + XST;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_ready + 1);

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t n0 = blockIdx.x * (MT * kTileN), t0 = blockIdx.y * TOKN, split = blockIdx.z;
  const uint32_t nkb = (K + kSlabK - 1) / kSlabK;
  const uint32_t kb_begin = (uint32_t)((uint64_t)split * nkb / splits);
  const uint32_t kb_end = (uint32_t)((uint64_t)(split + 1) * nkb / splits);
  const uint32_t my_kb = kb_end - kb_begin;
  // Pair mode: the two CTAs of a cluster sit next to each other in x; the even one leads.
  const uint32_t pair_rank = PAIR ? (blockIdx.x & 1u) : 0u;
  const bool leader = pair_rank == 0;

  pdl_trigger();
#ifdef ORION_TRACE
  __shared__ uint32_t trace_slot_s;
#endif
  if (threadIdx.x == 0) {
#ifdef ORION_TRACE
    uint32_t slot = 0xFFFFFFFFu;
    if (g_gemm_trace_on && blockIdx.x + blockIdx.y + blockIdx.z == 0) {
      slot = atomicAdd(&g_gemm_trace_next, 1u) % kTraceLaunches;
      g_gemm_trace[slot][7] = ((unsigned long long)gridDim.x << 32) | (gridDim.z << 16) | my_kb;
    }
    trace_slot_s = slot;
    gtrace(slot, 0);
#endif
    for (int s = 0; s < WST; ++s) {
      mbar_init(&full_w[s], 1);
      mbar_init(&empty_w[s], 1);
    }
    for (int s = 0; s < XST; ++s) {
      mbar_init(&full_x[s], 1);
      mbar_init(&empty_x[s], 1);
    }
    mbar_init(acc_ready, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, Cfg::kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) {  // the peer's barriers exist before anything of this CTA signals them
    cluster_arrive_release();
    cluster_wait_acquire();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
#ifdef ORION_TRACE
  const uint32_t tslot = trace_slot_s;
#endif
  bool ok = true;

  if (warp == 0) {
    // Weight producer. Weights are immutable, so this stream starts while the kernel that
    // produces the activations is still running and never waits for it.
    if (lane == 0) {
      ORION_GTRACE(tslot, 1);
      for (uint32_t i = 0; i < my_kb; ++i) {
        const uint32_t s = i % WST, use = i / WST;
        if (!mbar_wait(&empty_w[s], (use & 1) ^ 1)) { ok = false; break; }
        if (PAIR) {
          // both CTAs' tiles are counted on the leader's barrier, which expects the bytes of both
          if (leader) mbar_arrive_expect_tx(&full_w[s], 2 * Cfg::kWBytes);
          const uint32_t bar = mapa_u32(smem_u32(&full_w[s]), 0);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            tma_load_2d_pair(w_ring + s * Cfg::kWBytes + mt * (kTileN * kSlabK * 2), &map_w, (int)((kb_begin + i) * kSlabK),
                             (int)(n0 + mt * kTileN), bar);
          continue;
        }
        mbar_arrive_expect_tx(&full_w[s], Cfg::kWBytes);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)  // rows past the matrix read as zeros and still count their bytes
          tma_load_2d(w_ring + s * Cfg::kWBytes + mt * (kTileN * kSlabK * 2), &map_w, (int)((kb_begin + i) * kSlabK),
                      (int)(n0 + mt * kTileN), &full_w[s]);
      }
    }
  } else if (warp == 2) {
    // Activation producer: waits for the preceding kernel, then keeps the short x ring full.
    if (lane == 0) {
      if (ready.counter) {  // the activations' producer counts its finished CTAs: no wait for its completion
        if (!wait_ready(ready)) atomicOr(&g_gemm_error, 2u);
        fence_proxy_async_all();
      } else {
        pdl_wait();
      }
      ORION_GTRACE(tslot, 3);
      for (uint32_t i = 0; i < my_kb; ++i) {
        const uint32_t s = i % XST, use = i / XST;
        if (!mbar_wait(&empty_x[s], (use & 1) ^ 1)) { ok = false; break; }
        if (PAIR) {  // this CTA's half of the token tile; counted on the leader's barrier like the weights
          if (leader) mbar_arrive_expect_tx(&full_x[s], 2 * Cfg::kXBytes);
          tma_load_2d_pair(x_ring + s * Cfg::kXBytes, &map_x, (int)((kb_begin + i) * kSlabK),
                           (int)(t0 + pair_rank * Cfg::kXRows), mapa_u32(smem_u32(&full_x[s]), 0));
          continue;
        }
        mbar_arrive_expect_tx(&full_x[s], Cfg::kXBytes);
        tma_load_2d(x_ring + s * Cfg::kXBytes, &map_x, (int)((kb_begin + i) * kSlabK), (int)t0, &full_x[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {  // in pair mode the leader issues for both CTAs
      constexpr uint32_t idesc = PAIR ? instr_desc<TOKN, 2 * kTileN>() : instr_desc<TOKN>();
      for (uint32_t i = 0; i < my_kb; ++i) {
        const uint32_t sw = i % WST, sx = i % XST;
        if (!mbar_wait(&full_w[sw], (i / WST) & 1)) { ok = false; break; }
        if (i == 0) ORION_GTRACE(tslot, 2);
        if (!mbar_wait(&full_x[sx], (i / XST) & 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t wt = smem_u32(w_ring + sw * Cfg::kWBytes);
        const uint32_t xt = smem_u32(x_ring + sx * Cfg::kXBytes);
#pragma unroll
        for (int k = 0; k < kSlabK / kUmmaK; ++k) {
          // advancing 16 k elements inside the swizzle atom = +32 bytes on the start address
          const uint64_t b = smem_desc_sw128(xt + k * kUmmaK * 2);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {  // one accumulator of TOKN columns per weight tile
            const uint64_t a = smem_desc_sw128(wt + mt * (kTileN * kSlabK * 2) + k * kUmmaK * 2);
            if (PAIR) umma_bf16_pair(tmem_base + (uint32_t)(mt * TOKN), a, b, idesc, (i > 0 || k > 0) ? 1u : 0u);
            else umma_bf16(tmem_base + (uint32_t)(mt * TOKN), a, b, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
        }
        if (PAIR) {  // the same stage of both CTAs is free once these MMAs have read it
#pragma unroll
          for (uint32_t r = 0; r < 2; ++r) {
            umma_commit_pair(mapa_u32(smem_u32(&empty_w[sw]), r));
            umma_commit_pair(mapa_u32(smem_u32(&empty_x[sx]), r));
          }
          continue;
        }
        umma_commit(&empty_w[sw]);  // both stages are free once these MMAs have read them
        umma_commit(&empty_x[sx]);
      }
      if (PAIR) {
        umma_commit_pair(mapa_u32(smem_u32(acc_ready), 0));
        umma_commit_pair(mapa_u32(smem_u32(acc_ready), 1));
      } else
      umma_commit(acc_ready);  // arrives when every MMA above has completed
      ORION_GTRACE(tslot, 4);
    }
  } else if (warp >= 4) {
    // Epilogue warps: warp w may touch tensor-memory lanes 32*(w%4) .. +31.
    const uint32_t lq = warp & 3;
    // The partial buffer may still be read by the kernel before the producer of x: wait for the
    // predecessor here, while the main loop runs, rather than after the accumulator is ready. (With a
    // ready counter the producer has read the buffer before it counted, and the accumulator follows the count.)
    if (!ready.counter) pdl_wait();
    if (my_kb > 0) {
      if (!mbar_wait(acc_ready, 0)) ok = false;
    }
    tc_fence_after();
    if (threadIdx.x == 128) ORION_GTRACE(tslot, 5);
    float *dst = partial + (size_t)split * M * N;
    // Split-K inside a cluster: the tile goes to shared memory as stage[token][128 weight rows]
    // (the rings are idle: every load has landed and every MMA has read its operands).
    float *stage = reinterpret_cast<float *>(smem);
    // Tensor-memory loads are issued for up to four 16-column chunks before the one wait, so the
    // round trips of a batch overlap; stores follow chunk by chunk.
    constexpr int kBatch = TOKN >= 64 ? 4 : TOKN / 16;
#pragma unroll 1
    for (int mb = 0; mb < MT * TOKN; mb += 16 * kBatch) {
      uint32_t rr[kBatch][16];
      if (ok && my_kb > 0) {
#pragma unroll
        for (int b = 0; b < kBatch; ++b) tmem_ld16(tmem_base + ((lq * 32u) << 16) + (uint32_t)(mb + 16 * b), rr[b]);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int b = 0; b < kBatch; ++b)
#pragma unroll
          for (int j = 0; j < 16; ++j) rr[b][j] = 0u;
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
      const int mc = mb + 16 * b;
      const int mt = mc / TOKN, c = mc % TOKN;  // weight tile, first token column of this chunk
      const uint32_t n = n0 + mt * kTileN + lq * 32 + lane;
      if (t0 + c >= M) continue;  // warp-uniform
      uint32_t (&r)[16] = rr[b];
      if (cluster_reduce) {
#pragma unroll
        for (int j = 0; j < 16; ++j) stage[(c + j) * kTileN + lq * 32 + lane] = __uint_as_float(r[j]);
      } else if (act != nullptr) {
        // Fused SwiGLU (tensor.rs:167-189): weight rows are interleaved, lane 2i holds gate_f and
        // lane 2i + 1 holds up_f of the same f for these 16 tokens. Each lane of a pair trades
        // half of its values with the other and finishes one token of every token pair.
        const uint32_t odd = lane & 1u;
        const uint32_t f = n >> 1, F = N >> 1;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const uint32_t send = odd ? r[2 * jj] : r[2 * jj + 1];
          const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 1);
          const float g = __uint_as_float(odd ? recv : r[2 * jj]);
          const float u = __uint_as_float(odd ? r[2 * jj + 1] : recv);
          const uint32_t tok = t0 + c + 2 * jj + odd;
          if (tok < M && n < N) act[(size_t)tok * F + f] = __float2bfloat16_rn(__fmul_rn(g / (1.0f + __expf(-g)), u));
        }
      } else if (n < N) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const uint32_t tok = t0 + c + j;
          if (tok < M) dst[(size_t)tok * ldc + n] = __uint_as_float(r[j]);  // ldc: row stride of the output
        }
      }
      }
    }
  }
  if (cluster_reduce) {
    // The `splits` CTAs of one tile form a cluster (1, 1, splits). Every CTA sums a share of the
    // tile's tokens over all members' staged tiles (distributed shared memory, member order, so
    // the result is the same as summing slabs in order) and writes slab 0 only.
    __syncthreads();
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp >= 4) {
      const uint32_t row = (warp & 3) * 32 + lane, n = n0 + row;
      const uint32_t valid = (M - t0) < (uint32_t)TOKN ? (M - t0) : (uint32_t)TOKN;
      const uint32_t tb = split * valid / splits, te = (split + 1) * valid / splits;
      const uint32_t base = smem_u32(smem) + row * 4;
#pragma unroll 2
      for (uint32_t tok = tb; tok < te; ++tok) {
        float x[8];
#pragma unroll
        for (uint32_t s = 0; s < 8; ++s) x[s] = s < splits ? ld_dsmem_f32(mapa_u32(base + tok * (kTileN * 4), s)) : 0.f;
        float acc = 0.f;
#pragma unroll
        for (uint32_t s = 0; s < 8; ++s)
          if (s < splits) acc += x[s];
        if (n < N) partial[(size_t)(t0 + tok) * N + n] = acc;
      }
    }
    cluster_arrive_release();  // nobody leaves while a peer may still read its staged tile
    cluster_wait_acquire();
  }
  if (threadIdx.x == 128) ORION_GTRACE(tslot, 6);
  if (!ok) atomicOr(&g_gemm_error, 1u);
  tc_fence_before();
  __syncthreads();
  if (PAIR) {
    // Neither CTA leaves, nor frees the tensor memory the pair allocated together, while the other may
    // still be read by an MMA or be reading its accumulator.
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    return;
  }
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// ---- host side -----------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                              const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                              const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return (EncodeFn) nullptr;
    return (EncodeFn)p;
  }();
  return fn;
}

// [rows][k] bf16 matrix with row stride ld; box = 64 k x box_rows, 128-byte swizzle.
int make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t k, uint64_t ld,
             uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (!fn) return set_error(ORION_ERR_BACKEND, "backend cuda failed at tensor map: driver entry point missing");
  const cuuint64_t dims[2] = {k, rows};
  const cuuint64_t strides[1] = {ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kSlabK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(ORION_ERR_BACKEND, "backend cuda failed at tensor map: encode returned %d (rows %llu k %llu ld %llu)",
                     (int)r, (unsigned long long)rows, (unsigned long long)k, (unsigned long long)ld);
  return ORION_OK;
}

struct MapKey {
  const void *base;
  uint64_t rows, k, ld;
  uint32_t box_rows;
  bool operator<(const MapKey &o) const {
    return std::tie(base, rows, k, ld, box_rows) < std::tie(o.base, o.rows, o.k, o.ld, o.box_rows);
  }
};

int cached_map(const void *base, uint64_t rows, uint64_t k, uint64_t ld, uint32_t box_rows,
               const CUtensorMap **out) {
  static std::mutex mu;
  static std::map<MapKey, CUtensorMap> cache;
  std::lock_guard<std::mutex> lock(mu);
  MapKey key{base, rows, k, ld, box_rows};
  auto it = cache.find(key);
  if (it == cache.end()) {
    if (cache.size() > 65536) cache.clear();
    CUtensorMap m;
    ORION_TRY(make_map(&m, base, rows, k, ld, box_rows));
    it = cache.emplace(key, m).first;
  }
  *out = &it->second;
  return ORION_OK;
}

template <int TOKN, int WST, int XST, int MT = 1, bool PAIR = false>
int launch_tc(const bf16 *x, uint32_t ldx, const bf16 *w, uint32_t ldw, float *partial, bf16 *act,
              uint32_t rows, uint32_t n, uint32_t k, uint32_t splits, bool cluster_reduce, uint32_t ldc,
              cudaStream_t stream, ReadyWait ready = {}) {
  if (ldc == 0) ldc = n;
  if (ldc != n && (splits != 1 || act != nullptr))
    return set_error(ORION_ERR_INTERNAL, "a strided GEMM output needs one k split and f32 results");
  using Cfg = TcConfig<TOKN, WST, XST, MT, PAIR>;
  static_assert(Cfg::kSmemBytes <= 232448, "ring exceeds the shared memory of an SM");
  if (MT > 1 && cluster_reduce) return set_error(ORION_ERR_INTERNAL, "cluster split-K is built for one weight tile per CTA");
  static bool attr_set[kMaxDeviceOrdinals] = {};
  ORION_CUDA_CHECK("gemm_tc attr", ensure_dynamic_smem(gemm_tc_kernel<TOKN, WST, XST, MT, PAIR>, Cfg::kSmemBytes, attr_set));
  const CUtensorMap *mw, *mx;
  ORION_TRY(cached_map(w, n, k, ldw, kTileN, &mw));
  ORION_TRY(cached_map(x, rows, k, ldx, Cfg::kXRows, &mx));
  dim3 grid((n + MT * kTileN - 1) / (MT * kTileN), (rows + TOKN - 1) / TOKN, splits);
  if (PAIR) {
    if (cluster_reduce || (grid.x & 1u))
      return set_error(ORION_ERR_INTERNAL, "the paired GEMM needs an even number of weight tile groups and no cluster split-K");
    ORION_CUDA_CHECK("gemm_tc", launch_pdl_cluster(gemm_tc_kernel<TOKN, WST, XST, MT, PAIR>, grid, dim3(kThreads), dim3(2, 1, 1),
                                                   Cfg::kSmemBytes, stream, *mw, *mx, partial, act, rows, n, k, splits,
                                                   0u, ldc, ready));
  } else if (cluster_reduce)
    ORION_CUDA_CHECK("gemm_tc", launch_pdl_cluster(gemm_tc_kernel<TOKN, WST, XST, MT, PAIR>, grid, dim3(kThreads), dim3(1, 1, splits),
                                                   Cfg::kSmemBytes, stream, *mw, *mx, partial, act, rows, n, k, splits,
                                                   1u, ldc, ready));
  else
    ORION_CUDA_CHECK("gemm_tc", launch_pdl(gemm_tc_kernel<TOKN, WST, XST, MT, PAIR>, grid, dim3(kThreads), Cfg::kSmemBytes, stream,
                                           *mw, *mx, partial, act, rows, n, k, splits, 0u, ldc, ready));
  count_launch();
  ORION_CUDA_CHECK("gemm_tc", cudaGetLastError());
  return ORION_OK;
}

// 256-token tiles as CTA pairs (tcgen05 cta_group::2). Measured on the Llama-3-8B shape, projections of
// a step of 512 / 2048 / 8192 tokens: 616 / 869 / 1034 TFLOP/s paired against 630 / 900 / 996 unpaired:
// the pair pays off once a step has many token tiles. 1 (default) = pairs from 4096 rows on, 2 = wherever
// the grid allows (the parity tests run this), 0 = never. ORION_GEMM_PAIR overrides.
int g_gemm_pair = std::getenv("ORION_GEMM_PAIR") ? std::atoi(std::getenv("ORION_GEMM_PAIR")) : 1;
constexpr uint32_t kPairMinRows = 4096;

// Tuning A/B: ORION_GEMM_PREFILL_TILES=1 keeps one weight tile per CTA for prefill-sized batches
// (two tiles measured 3 % faster on the continuous-batching workload, gate/up only: the other
// projections have too few tiles to halve their grid).
int g_prefill_tiles = std::getenv("ORION_GEMM_PREFILL_TILES") ? std::atoi(std::getenv("ORION_GEMM_PREFILL_TILES")) : 2;
// How a prefill-sized projection with fewer than 148 tiles of 256 tokens reaches every SM: 2 = k
// splits (default), 1 = 128-token tiles, 0 = not at all. Measured on the continuous-batching
// workload at the 8B shape: 12.07 / 12.46 / 12.32 s. ORION_GEMM_PREFILL_FILL overrides.
int g_prefill_fill = std::getenv("ORION_GEMM_PREFILL_FILL") ? std::atoi(std::getenv("ORION_GEMM_PREFILL_FILL")) : 2;
// Weight tiles per CTA for a prefill-sized batch: two share one activation tile (less shared-memory
// fill per flop). Mode 2 (default): only where the grid stays full without k splits; mode 3: always
// (measured no better on the continuous-batching workload: 12.19 vs 11.94 s).
// Batches of 129..256 rows stream weights like decode but already feel the fill rate (48 KiB of operands per
// 4.2 MFLOP with one weight tile): ORION_GEMM_MID_MT=2 (default) gives a CTA two weight tiles there too.
int g_mid_mt = std::getenv("ORION_GEMM_MID_MT") ? std::atoi(std::getenv("ORION_GEMM_MID_MT")) : 2;
uint32_t prefill_weight_tiles(uint32_t rows, uint32_t n) {
  if (rows > 128 && rows <= 256) return g_mid_mt >= 2 && n >= 2 * (uint32_t)kTileN ? 2 : 1;
  if (rows <= 256 || g_prefill_tiles < 2) return 1;
  if (g_prefill_tiles >= 3) return 2;
  return ((n + kTileN - 1) / kTileN) * ((rows + 255) / 256) >= 296 ? 2 : 1;
}
int g_small_stages = 5;  // 5: deep weight ring + short activation ring for decode batches; 4: equal rings
// Batches of 65..128 rows: 0 (default) = 4 weight + 2 activation stages, 96 KiB, two CTAs per SM like the
// smaller tiles (the split-K planner counts on two); 1 = 6 + 6 stages, 192 KiB, one CTA per SM, k splits
// sized for one wave of 148; 2 = the same tile with k splits sized for 296 CTAs, also for 129..256 rows
// (two waves of uneven length). ORION_GEMM_MID_TILE overrides (tuning A/B).
int g_mid_tile = std::getenv("ORION_GEMM_MID_TILE") ? std::atoi(std::getenv("ORION_GEMM_MID_TILE")) : 0;

uint32_t token_tile(uint32_t rows) {
  if (rows <= 16) return 16;
  if (rows <= 32) return 32;
  if (rows <= 64) return 64;
  if (rows <= 128) return 128;
  return 256;
}

}  // namespace

bool gemm_tc_supported(uint32_t rows, uint32_t n, uint32_t k, uint32_t ldx, uint32_t ldw,
                       const void *x, const void *w) {
  return rows > 0 && n > 0 && k >= (uint32_t)kSlabK && k % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
         encode_fn() != nullptr;
}

int launch_gemm_tc(const bf16 *x, uint32_t ldx, const bf16 *w, uint32_t ldw, float *partial,
                   uint32_t rows, uint32_t n, uint32_t k, uint32_t splits, cudaStream_t stream,
                   bf16 *act, bool cluster_reduce, uint32_t ldc, ReadyWait ready) {
  const uint32_t nkb = (k + kSlabK - 1) / kSlabK;
  if (cluster_reduce && (splits < 2 || splits > 8 || act != nullptr))
    return set_error(ORION_ERR_INTERNAL, "cluster split-K needs 2..8 splits and f32 output");
  if (act != nullptr && (splits != 1 || n % 2 != 0))
    return set_error(ORION_ERR_INTERNAL, "the fused SwiGLU epilogue needs one k split and an even row count");
  if (splits < 1 || splits > nkb)
    return set_error(ORION_ERR_INTERNAL, "gemm split count %u outside 1..%u", splits, nkb);
  const bool deep = g_small_stages >= 5;
  uint32_t tt = token_tile(rows);
  // prefill batches whose 256-token tiles would leave SMs idle take 128-token tiles instead
  if (rows > 256 && g_prefill_fill == 1 && ((n + kTileN - 1) / kTileN) * ((rows + 255) / 256) < 148) tt = 128;
  switch (tt) {
    case 16:
      return deep ? launch_tc<16, 6, 3>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready)
                  : launch_tc<16, 5, 3>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready);
    case 32:
      return deep ? launch_tc<32, 6, 3>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready)
                  : launch_tc<32, 5, 3>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready);
    case 64:
      return deep ? launch_tc<64, 5, 3>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready)
                  : launch_tc<64, 4, 4>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready);
    case 128:
      return g_mid_tile == 0
                 ? launch_tc<128, 4, 2>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready)
                 : launch_tc<128, 6, 6>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready);
    default: {
      const uint32_t mt = (!cluster_reduce && prefill_weight_tiles(rows, n) == 2) ? 2 : 1;
      // CTA pairs: each CTA loads half of the activation tile, so the rings go a stage deeper
      const bool pair = (g_gemm_pair >= 2 || (g_gemm_pair == 1 && rows >= kPairMinRows)) && !cluster_reduce &&
                        (((n + mt * kTileN - 1) / (mt * kTileN)) & 1u) == 0;
      if (mt == 2)
        return pair ? launch_tc<256, 4, 4, 2, true>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready)
                    : launch_tc<256, 3, 3, 2>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready);
      return pair ? launch_tc<256, 6, 6, 1, true>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready)
                  : launch_tc<256, 4, 4>(x, ldx, w, ldw, partial, act, rows, n, k, splits, cluster_reduce, ldc, stream, ready);
    }
  }
}

int gemm_tc_poll_error(uint32_t *code) {
#ifdef ORION_TRACE
  static const bool tracing = std::getenv("ORION_GEMM_TRACE") != nullptr &&
                              (std::getenv("LOCAL_RANK") == nullptr || std::atoi(std::getenv("LOCAL_RANK")) == 0);  // one rank prints
  if (tracing) {
    static unsigned long long t[kTraceLaunches][kTraceStamps];
    uint32_t next = 0, on = 1;
    cudaMemcpyFromSymbol(t, g_gemm_trace, sizeof t);
    cudaMemcpyFromSymbol(&next, g_gemm_trace_next, sizeof next);
    cudaMemcpyToSymbol(g_gemm_trace_on, &on, sizeof on);
    if (next >= (uint32_t)kTraceLaunches) {
      unsigned long long prev_end = 0;
      fprintf(stderr, "gemm trace of CTA 0 (us): entry(abs mod 1e5) grid.x splits slabs | gap-from-prev-end setup first-W pdl-wait last-mma acc-ready epilogue total\n");
      for (int i = 0; i < kTraceLaunches; ++i) {
        const unsigned long long *r = t[(next + i) % kTraceLaunches];
        fprintf(stderr, "  gemm %10.2f %4u %2u %3u | %7.2f %6.2f %6.2f %6.2f %6.2f %6.2f %6.2f %6.2f\n", (double)(r[0] % 100000000ull) / 1e3, (unsigned)(r[7] >> 32),
                (unsigned)((r[7] >> 16) & 0xFFFF), (unsigned)(r[7] & 0xFFFF), prev_end ? ((double)r[0] - (double)prev_end) / 1e3 : 0.0,
                (r[1] - r[0]) / 1e3, (r[2] - r[0]) / 1e3, (r[3] - r[0]) / 1e3, (r[4] - r[0]) / 1e3, (r[5] - r[0]) / 1e3,
                (r[6] - r[0]) / 1e3, (r[6] - r[0]) / 1e3);
        prev_end = r[6];
      }
    }
  }
#endif
  uint32_t v = 0;
  ORION_CUDA_CHECK("gemm error word", cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof v));
  if (v) {
    uint32_t zero = 0;
    ORION_CUDA_CHECK("gemm error word", cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof zero));
  }
  *code = v;
  return ORION_OK;
}

// ---- planning and dispatch -------------------------------------------------------

namespace {
uint32_t g_target_ctas = 296;  // two CTAs fit on each of the 148 SMs
// Split-K reduction inside a thread-block cluster (distributed shared memory) instead of one f32
// slab per split summed by the consumer. Off by default: measured on the headline step it removes
// 8/9 of the slab traffic but costs more than it saves (5.27 vs 5.01 ms per step): clusters of 8
// CTAs of 105 KiB must be co-scheduled, which delays the dependent-launch overlap, and each GEMM
// gains two cluster barriers. ORION_CLUSTER_SPLITK=1 turns it on (tests cover both).
bool g_cluster_splitk = std::getenv("ORION_CLUSTER_SPLITK") ? std::atoi(std::getenv("ORION_CLUSTER_SPLITK")) != 0 : false;
}

void gemm_set_target_ctas(uint32_t v) { g_target_ctas = v ? v : 296; }
void gemm_set_small_stages(int stages) { g_small_stages = stages >= 5 ? 5 : 4; }

GemmPlan gemm_plan(bool is_bf16, uint32_t rows, uint32_t n, uint32_t k, uint32_t ldx,
                   uint32_t ldw) {
  GemmPlan p{1, false, false, 1, 0};
  if (!is_bf16) return p;
  // alignment of the pointers is checked at launch; shapes decide the plan
  if (!(rows > 0 && n > 0 && k >= (uint32_t)kSlabK && k % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 &&
        encode_fn() != nullptr))
    return p;
  p.tensor_core = true;
  if (rows > 256) {
    // Prefill-sized batches are tensor-bound; the 256-token tiles take a whole SM each (192 KiB of
    // rings), so a projection with few weight tiles (N = 4096: 32) needs k splits to reach all SMs.
    const uint32_t rows_per_cta = kTileN * prefill_weight_tiles(rows, n);
    const uint32_t big = ((n + rows_per_cta - 1) / rows_per_cta) * ((rows + 255) / 256);
    const uint32_t nkb_big = (k + kSlabK - 1) / kSlabK;
    if (big < 148 && g_prefill_fill == 2) {
      uint32_t s = 296 / big;
      const uint32_t cap = nkb_big / 8 ? nkb_big / 8 : 1;  // at least eight k slabs per split
      if (s > cap) s = cap;
      if (s > 4) s = 4;
      p.splits = p.out_slabs = s < 1 ? 1 : s;
    }
    (void)nkb_big;
    return p;
  }
  const uint32_t rows_per_cta = kTileN * (g_cluster_splitk ? 1 : prefill_weight_tiles(rows, n));
  const uint32_t tiles = ((n + rows_per_cta - 1) / rows_per_cta) * ((rows + token_tile(rows) - 1) / token_tile(rows));
  const uint32_t nkb = (k + kSlabK - 1) / kSlabK;
  // the 256-token tile (and the 6 + 6 stage 128-token one) fills an SM by itself: one wave is 148 CTAs
  const bool one_per_sm = g_mid_tile != 2 && (token_tile(rows) == 256 || (token_tile(rows) == 128 && g_mid_tile == 1));
  uint32_t s = (one_per_sm ? g_target_ctas / 2 : g_target_ctas) / (tiles ? tiles : 1);
  const uint32_t cap = nkb / 4 ? nkb / 4 : 1;  // at least four k slabs per split
  if (s > cap) s = cap;
  if (s > 16) s = 16;
  if (g_cluster_splitk && s > 8) s = 8;  // portable cluster size
  p.splits = s < 1 ? 1 : s;
  p.cluster_reduce = g_cluster_splitk && p.splits > 1;
  p.out_slabs = p.cluster_reduce ? 1 : p.splits;
  return p;
}

size_t gemm_partial_floats(bool is_bf16, uint32_t max_rows, uint32_t n, uint32_t k) {
  size_t best = (size_t)max_rows * n;
  if (!is_bf16) return best;
  for (uint32_t r = 1; r <= max_rows; ++r) {
    const GemmPlan p = gemm_plan(true, r, n, k, k, k);
    const size_t need = (size_t)p.splits * r * n;
    if (need > best) best = need;
  }
  return best;
}

int launch_gemm_swiglu(const bf16 *x, uint32_t ldx, const bf16 *w_interleaved, uint32_t ldw, bf16 *act, uint32_t rows,
                       uint32_t ffn, uint32_t k, cudaStream_t stream, ReadyWait ready) {
  if (!gemm_tc_supported(rows, 2 * ffn, k, ldx, ldw, x, w_interleaved))
    return set_error(ORION_ERR_INTERNAL, "tensor-core GEMM planned for an unaligned operand");
  return launch_gemm_tc(x, ldx, w_interleaved, ldw, nullptr, rows, 2 * ffn, k, 1, stream, act, false, 0, ready);
}

template <>
int launch_gemm<float>(const float *x, uint32_t ldx, const float *w, uint32_t ldw, float *partial,
                       uint32_t rows, uint32_t n, uint32_t k, GemmPlan, cudaStream_t stream, ReadyWait) {
  return launch_gemm_simt<float>(x, ldx, w, ldw, partial, rows, n, k, stream);
}

template <>
int launch_gemm<bf16>(const bf16 *x, uint32_t ldx, const bf16 *w, uint32_t ldw, float *partial,
                      uint32_t rows, uint32_t n, uint32_t k, GemmPlan plan, cudaStream_t stream,
                      ReadyWait ready) {
  if (plan.tensor_core) {
    if (!gemm_tc_supported(rows, n, k, ldx, ldw, x, w))
      return set_error(ORION_ERR_INTERNAL, "tensor-core GEMM planned for an unaligned operand");
    return launch_gemm_tc(x, ldx, w, ldw, partial, rows, n, k, plan.splits, stream, nullptr, plan.cluster_reduce,
                          plan.ldc, ready);
  }
  if (plan.ldc != 0 && plan.ldc != n) return set_error(ORION_ERR_INTERNAL, "a strided GEMM output needs the tensor-core path");
  return launch_gemm_simt<bf16>(x, ldx, w, ldw, partial, rows, n, k, stream);
}

}  // namespace orion
