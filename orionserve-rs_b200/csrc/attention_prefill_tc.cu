// Chunked-prefill paged attention on the 5th-generation tensor cores (bf16, head_dim 128, 16-token
// blocks): the same arithmetic as attention_prefill.cu (transformer.rs:281-326, causal by absolute
// position, attention.rs:252-253), with S = Q K^T and O += P V as tcgen05 MMAs whose accumulators
// live in tensor memory.
//
// One CTA per (kv head, tile of query rows of one sequence), two CTAs per SM. The MMA's M dimension
// is (query position, query head of the GQA group), 128 rows; a key tile is 64 keys = four KV blocks.
//   warp 0     one lane fetches K and V of a key tile with tiled TMA copies straight out of the paged
//              arena (one 3-D tensor map over [chunk][k|v x slot][dim]; a 16-slot x 64-dim box lands as
//              sixteen 128-byte rows, and because the arena keeps the 16-byte groups of a row XOR-permuted
//              by slot & 7, those rows ARE the 128-byte-swizzled operand layout the MMA expects);
//   warp 1     allocates tensor memory; one lane issues S = Q K^T (M 128, N 64, K 128) and, once the
//              softmax warps have written P, O (+)= P V (M 128, N 128, K 64; V is the MN-major operand);
//   warps 2-5  one thread per row: read the row of S from tensor memory (lane = row, so max and sum
//              are thread-local), mask by position, exponentiate, write P as bf16 into the shared
//              memory the K tile has just vacated, and at the end scale O by 1 / sum and store it.
// O stays in tensor memory across key tiles. The running maximum a row's exponentials refer to is
// only moved when the true maximum exceeds it by more than 2^8; then the row's O is rescaled in
// tensor memory (load, multiply, store), which is rare after the first tiles.
// Every wait is bounded; a wait that runs out sets the device error word and the CTA still frees its
// tensor memory.
#include "kernels.h"

#include <cuda.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

namespace orion {
namespace {

constexpr int kHd = 128, kBlk = 16;
constexpr int kM = 128;      // (position, head) rows per CTA
constexpr int kKeys = 64;    // keys per tile
constexpr int kStages = 2;
constexpr int kThreads = 192;
constexpr int kQBytes = 2 * kM * 128;        // two 64-dim halves of [128 rows][128 bytes]
constexpr int kKBytes = 2 * kKeys * 128;     // two 64-dim halves of [64 keys][128 bytes]; P reuses it as [128 rows][128 bytes]
constexpr int kStageBytes = 2 * kKBytes;     // K tile, then V tile
constexpr int kBarOffset = kQBytes + kStages * kStageBytes;
constexpr int kSmem = kBarOffset + 256 + 1024;
constexpr uint32_t kTmemCols = 256;          // S: columns 0..63, O: columns 64..191
constexpr uint32_t kTmemO = 64;
constexpr float kRescaleThreshold = 8.0f;    // log2 units

__device__ uint32_t g_prefill_tc_error = 0;

__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 3-D tiled TMA load (no multicast); c0 is the innermost coordinate.
__device__ __forceinline__ void tma_load_3d(void *dst_smem, const void *tensor_map, int c0, int c1, int c2, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst_smem)),
      "l"(tensor_map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}

// K-major operand, rows of 128 bytes with the 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// MN-major operand with the 128-byte swizzle: a 128-byte row holds 64 consecutive MN elements of one k;
// eight k rows (1024 bytes) form an atom; the next eight k follow `sbo` bytes later, the next 64 MN
// elements `lbo` bytes later.
__device__ __forceinline__ uint64_t desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// f32 accumulate, bf16 x bf16; b_mn: the B operand is MN-major.
__device__ __forceinline__ constexpr uint32_t idesc(uint32_t m, uint32_t n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }  // warps 2..5

__global__ void __launch_bounds__(kThreads, 2)
paged_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_kv, const bf16 *__restrict__ q, KvLayout kv, uint32_t layer,
                        AttnBatch batch, const PrefillTile *__restrict__ tiles, uint32_t q_heads, bf16 *__restrict__ out) {
  extern __shared__ uint8_t raw_smem[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  uint8_t *q_smem = smem;                 // [half 2][row 128][128 B]
  uint8_t *ring = smem + kQBytes;         // [stage][K tile 16 KiB | V tile 16 KiB]
  uint64_t *kv_full = reinterpret_cast<uint64_t *>(smem + kBarOffset);
  uint64_t *kv_empty = kv_full + kStages;
  uint64_t *q_ready = kv_empty + kStages;
  uint64_t *s_ready = q_ready + 1;
  uint64_t *p_ready = s_ready + 1;
  uint64_t *o_ready = p_ready + 1;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(o_ready + 1);

  pdl_trigger();
  const uint32_t kvh = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const PrefillTile tile = tiles[blockIdx.y];
  const uint32_t group = q_heads / kv.num_kv_heads;
  const uint32_t *table = batch.tables_flat + batch.table_offsets[tile.seq];
  const uint32_t nblocks = tile.max_position / kBlk + 1;
  const uint32_t ntiles = (nblocks + (kKeys / kBlk) - 1) / (kKeys / kBlk);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(q_ready, 1);
    mbar_init(s_ready, 1);
    mbar_init(p_ready, 1);
    mbar_init(o_ready, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;
  // Once any wait of this CTA has run out, later waits give up at once: every thread still walks
  // through the same barriers, so nobody is left behind at a bar.sync.
  __shared__ volatile uint32_t failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  auto wait = [&](uint64_t *bar, uint32_t parity) -> bool {
    if (failed) return false;
    if (mbar_wait(bar, parity)) return true;
    failed = 1;
    return false;
  };

  if (warp == 0) {
    // ---- K/V producer ----
    if (lane == 0) {
      pdl_wait();  // this step's K/V rows come from the preceding kernel
      const uint32_t chunk0 = layer * kv.num_blocks;
      for (uint32_t j = 0; j < ntiles; ++j) {
        const uint32_t s = j % kStages, use = j / kStages;
        if (!wait(&kv_empty[s], (use & 1) ^ 1)) { ok = false; break; }
        mbar_arrive_expect_tx(&kv_full[s], kStageBytes);
        uint8_t *k_dst = ring + s * kStageBytes, *v_dst = k_dst + kKBytes;
#pragma unroll
        for (uint32_t b = 0; b < kKeys / kBlk; ++b) {
          // a block past the row's context repeats block 0: its keys are masked, its values must be finite
          const uint32_t lb = j * (kKeys / kBlk) + b;
          const uint32_t block = table[lb < nblocks ? lb : 0];
          const int chunk = (int)((chunk0 + block) * kv.num_kv_heads + kvh);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            tma_load_3d(k_dst + h * (kKeys * 128) + b * (kBlk * 128), &map_kv, h * 64, 0, chunk, &kv_full[s]);
            tma_load_3d(v_dst + h * (kKeys * 128) + b * (kBlk * 128), &map_kv, h * 64, kBlk, chunk, &kv_full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue ----
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc(kM, kKeys, false), idesc_o = idesc(kM, kHd, true);
      const uint32_t qa = smem_u32(q_smem);
      if (!wait(q_ready, 0)) ok = false;
      for (uint32_t j = 0; ok && j < ntiles; ++j) {
        const uint32_t s = j % kStages;
        if (!wait(&kv_full[s], (j / kStages) & 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ka = smem_u32(ring + s * kStageBytes), va = ka + kKBytes;
        // S = Q K^T: two 64-dim halves, four 16-dim steps each (+32 bytes inside the swizzle atom)
#pragma unroll
        for (int ks = 0; ks < kHd / 16; ++ks) {
          const uint32_t h = ks >> 2, kk = ks & 3;
          umma_bf16(tmem_base, desc_k_sw128(qa + h * (kM * 128) + kk * 32), desc_k_sw128(ka + h * (kKeys * 128) + kk * 32),
                    idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(s_ready);
        if (!wait(p_ready, j & 1)) { ok = false; break; }
        tc_fence_after();
        // O (+)= P V: P sits where the K tile was, [128 rows][64 keys]; V is [key][dim]: MN-major, 16 keys per step
#pragma unroll
        for (int ks = 0; ks < kKeys / 16; ++ks)
          umma_bf16(tmem_base + kTmemO, desc_k_sw128(ka + ks * 32), desc_mn_sw128(va + ks * (16 * 128), kKeys * 128, 1024),
                    idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit(o_ready);
        umma_commit(&kv_empty[s]);
      }
    }
  } else {
    // ---- softmax: thread = row ----
    const uint32_t quad = warp & 3;  // tensor-memory lanes this warp may touch
    const uint32_t m = quad * 32 + lane;
    const uint32_t pl = m / group;
    const bool valid = pl < tile.num_rows;
    const uint32_t row = tile.row_start + (valid ? pl : 0), head = kvh * group + m % group;
    const uint32_t taddr = tmem_base + ((quad * 32u) << 16);
    pdl_wait();  // q comes from the preceding kernel
    const int pos = valid ? (int)batch.query_positions[row] : -1;
    {
      const uint4 *src = reinterpret_cast<const uint4 *>(q + ((size_t)row * q_heads + head) * kHd);
#pragma unroll
      for (uint32_t c = 0; c < 16; ++c) {
        const uint4 v = valid ? src[c] : make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4 *>(q_smem + (c >> 3) * (kM * 128) + m * 128 + (((c & 7) ^ (m & 7)) << 4)) = v;
      }
    }
    fence_proxy_async_smem();
    softmax_bar();
    if (threadIdx.x == 64) mbar_arrive(q_ready);

    const float sl2 = 1.4426950408889634f / sqrtf((float)kHd);
    float ref = -INFINITY, l = 0.f;
    for (uint32_t j = 0; j < ntiles; ++j) {
      const uint32_t s = j % kStages;
      if (!__all_sync(0xffffffffu, wait(s_ready, j & 1))) ok = false;  // no break: the barriers below stay matched
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld32(taddr, sr[0]);
      tmem_ld32(taddr + 32, sr[1]);
      tmem_ld_wait();
      const int key0 = (int)(j * kKeys);
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < kKeys; ++i) {
        const float v = (key0 + i <= pos) ? __uint_as_float(sr[i >> 5][i & 31]) * sl2 : -INFINITY;
        sr[i >> 5][i & 31] = __float_as_uint(v);
        mx = fmaxf(mx, v);
      }
      // The reference of the exponentials moves only when the maximum runs away from it.
      float corr = 1.0f;
      if (mx > ref + kRescaleThreshold || ref == -INFINITY) {
        const float nref = fmaxf(ref, mx);
        corr = (ref == -INFINITY) ? 1.0f : ex2(ref - nref);  // nothing accumulated yet under a reference of -inf
        ref = nref;
      }
      if (__any_sync(0xffffffffu, corr != 1.0f) && j > 0) {
        // rescale this warp's rows of O in tensor memory (the MMAs of the previous tile have completed:
        // S of this tile was issued after them)
#pragma unroll 1
        for (uint32_t c = 0; c < kHd; c += 32) {
          uint32_t orow[32];
          tmem_ld32(taddr + kTmemO + c, orow);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * corr);
          tmem_st32(taddr + kTmemO + c, orow);
        }
        tmem_st_wait();
      }
      l *= corr;
      const float base = ref == -INFINITY ? 0.f : ref;
      uint8_t *p_row = ring + s * kStageBytes + m * 128;
#pragma unroll
      for (int c = 0; c < kKeys / 8; ++c) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          p[i] = ex2(__uint_as_float(sr[(c * 8 + i) >> 5][(c * 8 + i) & 31]) - base);
          l += p[i];
        }
        *reinterpret_cast<uint4 *>(p_row + ((c ^ (m & 7)) << 4)) =
            make_uint4(pack2(p[0], p[1]), pack2(p[2], p[3]), pack2(p[4], p[5]), pack2(p[6], p[7]));
      }
      tc_fence_before();        // the loads of S (and the rescale of O) precede the next MMAs
      fence_proxy_async_smem();  // P was written through the generic proxy, the MMA reads it through the async proxy
      softmax_bar();
      if (threadIdx.x == 64) mbar_arrive(p_ready);
    }
    // ---- epilogue: O / l ----
    if (!__all_sync(0xffffffffu, ntiles == 0 || wait(o_ready, (ntiles - 1) & 1))) ok = false;
    tc_fence_after();
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    bf16 *dst = out + ((size_t)row * q_heads + head) * kHd;
#pragma unroll 1
    for (uint32_t c = 0; c < kHd; c += 32) {
      uint32_t orow[32];
      tmem_ld32(taddr + kTmemO + c, orow);
      tmem_ld_wait();
      if (valid) {
#pragma unroll
        for (int i = 0; i < 32; i += 8)
          *reinterpret_cast<uint4 *>(dst + c + i) =
              make_uint4(pack2(__uint_as_float(orow[i]) * inv, __uint_as_float(orow[i + 1]) * inv),
                         pack2(__uint_as_float(orow[i + 2]) * inv, __uint_as_float(orow[i + 3]) * inv),
                         pack2(__uint_as_float(orow[i + 4]) * inv, __uint_as_float(orow[i + 5]) * inv),
                         pack2(__uint_as_float(orow[i + 6]) * inv, __uint_as_float(orow[i + 7]) * inv));
      }
    }
  }
  if (!ok && lane == 0) atomicOr(&g_prefill_tc_error, 1u);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ---- host side -----------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                              const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return (EncodeFn) nullptr;
    return (EncodeFn)p;
  }();
  return fn;
}

// The arena as [chunk = (layer, block, kv head)][32 rows: 16 K slots then 16 V slots][128 dims]; a box is 16 rows x
// 64 dims with no swizzle of its own (the rows are stored pre-permuted).
int arena_map(const bf16 *arena, KvLayout kv, const CUtensorMap **out) {
  static std::mutex mu;
  static std::map<std::tuple<const void *, uint64_t>, CUtensorMap> cache;
  EncodeFn fn = encode_fn();
  if (!fn) return set_error(ORION_ERR_BACKEND, "backend cuda failed at tensor map: driver entry point missing");
  const uint64_t chunks = (uint64_t)kv.num_layers * kv.num_blocks * kv.num_kv_heads;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_tuple((const void *)arena, chunks);
  auto it = cache.find(key);
  if (it == cache.end()) {
    if (cache.size() > 4096) cache.clear();
    CUtensorMap m;
    const cuuint64_t dims[3] = {(cuuint64_t)kHd, (cuuint64_t)2 * kBlk, chunks};
    const cuuint64_t strides[2] = {(cuuint64_t)kHd * 2, (cuuint64_t)2 * kBlk * kHd * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)kBlk, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<bf16 *>(arena), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return set_error(ORION_ERR_BACKEND, "backend cuda failed at tensor map: encode returned %d (arena of %llu chunks)", (int)r,
                       (unsigned long long)chunks);
    it = cache.emplace(key, m).first;
  }
  *out = &it->second;
  return ORION_OK;
}

// Tuning A/B and the parity tests of both paths: ORION_PREFILL_TC=0 keeps the mma.sync kernel.
bool g_prefill_tc = std::getenv("ORION_PREFILL_TC") ? std::atoi(std::getenv("ORION_PREFILL_TC")) != 0 : true;

}  // namespace

bool prefill_attention_tc_supported(KvLayout kv, uint32_t q_heads, const void *arena) {
  return g_prefill_tc && prefill_attention_supported(kv, q_heads) && (reinterpret_cast<uintptr_t>(arena) & 15) == 0 &&
         (uint64_t)kv.num_layers * kv.num_blocks * kv.num_kv_heads < (1ull << 31) && encode_fn() != nullptr;
}

int launch_paged_attention_prefill_tc(const bf16 *q, const bf16 *arena, KvLayout kv, uint32_t layer, AttnBatch batch,
                                      const PrefillTile *tiles, uint32_t num_tiles, uint32_t q_heads, bf16 *out,
                                      cudaStream_t stream) {
  if (num_tiles == 0) return ORION_OK;
  if (!prefill_attention_tc_supported(kv, q_heads, arena))
    return set_error(ORION_ERR_INTERNAL, "tensor-core prefill attention does not cover this shape");
  const CUtensorMap *map = nullptr;
  ORION_TRY(arena_map(arena, kv, &map));
  static bool attr_set[kMaxDeviceOrdinals] = {};
  ORION_CUDA_CHECK("paged_prefill_tc attr", ensure_dynamic_smem(paged_prefill_tc_kernel, (int)kSmem, attr_set));
  ORION_CUDA_CHECK("paged_prefill_tc", launch_pdl(paged_prefill_tc_kernel, dim3(kv.num_kv_heads, num_tiles), dim3(kThreads),
                                                  (size_t)kSmem, stream, *map, q, kv, layer, batch, tiles, q_heads, out));
  count_launch();
  ORION_CUDA_CHECK("paged_prefill_tc", cudaGetLastError());
  return ORION_OK;
}

int prefill_tc_poll_error(uint32_t *code) {
  uint32_t v = 0;
  ORION_CUDA_CHECK("prefill error word", cudaMemcpyFromSymbol(&v, g_prefill_tc_error, sizeof v));
  if (v) {
    uint32_t zero = 0;
    ORION_CUDA_CHECK("prefill error word", cudaMemcpyToSymbol(g_prefill_tc_error, &zero, sizeof zero));
  }
  *code = v;
  return ORION_OK;
}

}  // namespace orion
