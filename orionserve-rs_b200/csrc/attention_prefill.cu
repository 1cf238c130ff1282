// Chunked-prefill paged attention (bf16, head_dim 128, 16-token blocks): query rows of a
// sequence attend the cached tokens AND the earlier rows of the same chunk, whose K/V were
// written first (transformer.rs:281-326); causal by absolute position (attention.rs:252-253).
//
// One CTA per (kv head, tile of query rows of one sequence). The M dimension of the MMA is
// (query position, query head of the GQA group): 8 consumer warps x 16 such rows, Q fragments
// in registers. A ninth warp streams the sequence's K/V blocks (one 8 KiB bulk copy per block
// and head, the same chunks the decode kernel reads) through a ring shared by all consumers, so
// every K/V byte is fetched once per 128 rows instead of once per row. S = Q K^T and O += P V
// run on mma.sync m16n8k16 with the accumulator-to-operand register reuse for P; online softmax
// in the log2 domain per row.
#include "kernels.h"

namespace orion {
namespace {

constexpr int kHd = 128, kBlk = 16, kChunkBytes = 2 * kBlk * kHd * 2;
constexpr int kConsumers = 8;                 // warps doing the math
constexpr int kThreads = (kConsumers + 1) * 32;
constexpr int kRows = kConsumers * 16;        // (position, head) rows per CTA
constexpr int kStages = 6;
constexpr uint32_t kSmem = kStages * kChunkBytes + 256;

__device__ uint32_t g_prefill_error = 0;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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

__global__ void __launch_bounds__(kThreads, 1)
paged_prefill_kernel(const bf16 *__restrict__ q, const bf16 *__restrict__ arena, KvLayout kv, uint32_t layer,
                     AttnBatch batch, const PrefillTile *__restrict__ tiles, uint32_t q_heads,
                     bf16 *__restrict__ out) {
  extern __shared__ __align__(1024) uint8_t psmem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(psmem + kStages * kChunkBytes);
  uint64_t *empty = full + kStages;

  pdl_trigger();
  const uint32_t kvh = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const PrefillTile tile = tiles[blockIdx.y];
  const uint32_t group = q_heads / kv.num_kv_heads;
  const uint32_t *table = batch.tables_flat + batch.table_offsets[tile.seq];
  const uint32_t nblocks = tile.max_position / kBlk + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumers);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait();  // q and this step's K/V rows come from the preceding kernel

  if (warp == kConsumers) {
    // Producer: blocks in logical order, one bulk copy each.
    if (lane == 0) {
      const size_t layer_base = (size_t)layer * kv.layer_elems();
      uint32_t next_block = table[0];
      for (uint32_t b = 0; b < nblocks; ++b) {
        const uint32_t s = b % kStages, use = b / kStages;
        const uint32_t block = next_block;
        if (b + 1 < nblocks) next_block = table[b + 1];  // in flight while this thread waits below
        if (!mbar_wait(&empty[s], (use & 1) ^ 1)) {
          atomicOr(&g_prefill_error, 1u);
          break;
        }
        const bf16 *src = arena + layer_base + ((size_t)block * kv.num_kv_heads + kvh) * kv.chunk_elems();
        mbar_arrive_expect_tx(&full[s], kChunkBytes);
        bulk_copy_g2s(psmem + s * kChunkBytes, src, kChunkBytes, &full[s]);
      }
    }
    return;
  }

  // Rows of this warp: r = warp*16 + {lane/4, lane/4 + 8}; row r is (position r / group, head r % group).
  const uint32_t r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const uint32_t pl_lo = r_lo / group, pl_hi = r_hi / group;  // position index inside the tile
  const bool v_lo = pl_lo < tile.num_rows, v_hi = pl_hi < tile.num_rows;
  const uint32_t row_lo = tile.row_start + (v_lo ? pl_lo : 0), row_hi = tile.row_start + (v_hi ? pl_hi : 0);
  const uint32_t head_lo = kvh * group + r_lo % group, head_hi = kvh * group + r_hi % group;
  const int pos_lo = v_lo ? (int)batch.query_positions[row_lo] : -1;
  const int pos_hi = v_hi ? (int)batch.query_positions[row_hi] : -1;

  // Q as the A operand: per 16-dim chunk a0 (row lo, k lo), a1 (row hi, k lo), a2 (lo, k+8), a3 (hi, k+8).
  uint32_t qa[kHd / 16][4];
  {
    const bf16 *ql = q + ((size_t)row_lo * q_heads + head_lo) * kHd + (lane & 3) * 2;
    const bf16 *qh = q + ((size_t)row_hi * q_heads + head_hi) * kHd + (lane & 3) * 2;
#pragma unroll
    for (int c = 0; c < kHd / 16; ++c) {
      qa[c][0] = v_lo ? *reinterpret_cast<const uint32_t *>(ql + c * 16) : 0u;
      qa[c][1] = v_hi ? *reinterpret_cast<const uint32_t *>(qh + c * 16) : 0u;
      qa[c][2] = v_lo ? *reinterpret_cast<const uint32_t *>(ql + c * 16 + 8) : 0u;
      qa[c][3] = v_hi ? *reinterpret_cast<const uint32_t *>(qh + c * 16 + 8) : 0u;
    }
  }
  // Largest position any row of this warp attends: later blocks are skipped by the whole warp.
  int wmax = max(pos_lo, pos_hi);
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) wmax = max(wmax, __shfl_xor_sync(0xffffffffu, wmax, off));

  const float sl2 = 1.4426950408889634f / sqrtf((float)kHd);
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o[kHd / 8][4];
#pragma unroll
  for (int j = 0; j < kHd / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  bool ok = true;
  for (uint32_t b = 0; b < nblocks; ++b) {
    const uint32_t s = b % kStages;
    if (!mbar_wait(&full[s], (b / kStages) & 1)) {
      ok = false;
      break;
    }
    if ((int)(b * kBlk) <= wmax) {
      const uint32_t kbase = smem_u32(psmem + s * kChunkBytes), vbase = kbase + kBlk * kHd * 2;
      // S[row][token] for the 16 tokens of the block: two 8-token n tiles
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      {
        const uint32_t mi = lane >> 3, t = (mi >> 1) * 8 + (lane & 7);
#pragma unroll
        for (int c = 0; c < kHd / 16; ++c) {
          uint32_t kb[4];  // {b0,b1} of tokens 0-7, {b0,b1} of tokens 8-15
          const uint32_t chunk = (uint32_t)c * 2 + (mi & 1);
          ldsm_x4(kb, kbase + t * (kHd * 2) + ((chunk ^ (t & 7)) << 4));
          mma16816(s0, qa[c], kb[0], kb[1]);
          mma16816(s1, qa[c], kb[2], kb[3]);
        }
      }
      // causal mask by absolute position, log2-domain scaling
      const int t0 = (int)(b * kBlk) + (lane & 3) * 2;
      s0[0] = (t0 <= pos_lo) ? s0[0] * sl2 : -INFINITY;
      s0[1] = (t0 + 1 <= pos_lo) ? s0[1] * sl2 : -INFINITY;
      s0[2] = (t0 <= pos_hi) ? s0[2] * sl2 : -INFINITY;
      s0[3] = (t0 + 1 <= pos_hi) ? s0[3] * sl2 : -INFINITY;
      s1[0] = (t0 + 8 <= pos_lo) ? s1[0] * sl2 : -INFINITY;
      s1[1] = (t0 + 9 <= pos_lo) ? s1[1] * sl2 : -INFINITY;
      s1[2] = (t0 + 8 <= pos_hi) ? s1[2] * sl2 : -INFINITY;
      s1[3] = (t0 + 9 <= pos_hi) ? s1[3] * sl2 : -INFINITY;
      float bm_lo = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
      float bm_hi = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
      bm_lo = fmaxf(bm_lo, __shfl_xor_sync(0xffffffffu, bm_lo, 1));
      bm_lo = fmaxf(bm_lo, __shfl_xor_sync(0xffffffffu, bm_lo, 2));
      bm_hi = fmaxf(bm_hi, __shfl_xor_sync(0xffffffffu, bm_hi, 1));
      bm_hi = fmaxf(bm_hi, __shfl_xor_sync(0xffffffffu, bm_hi, 2));
      const float mn_lo = fmaxf(m_lo, bm_lo), mn_hi = fmaxf(m_hi, bm_hi);
      // a row with nothing attended so far keeps m = -inf: use 0 as the reference to avoid inf - inf
      const float ref_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
      const float c_lo = ex2(m_lo - ref_lo), c_hi = ex2(m_hi - ref_hi);
      float p[8];
      p[0] = ex2(s0[0] - ref_lo); p[1] = ex2(s0[1] - ref_lo); p[2] = ex2(s0[2] - ref_hi); p[3] = ex2(s0[3] - ref_hi);
      p[4] = ex2(s1[0] - ref_lo); p[5] = ex2(s1[1] - ref_lo); p[6] = ex2(s1[2] - ref_hi); p[7] = ex2(s1[3] - ref_hi);
      l_lo = l_lo * c_lo + p[0] + p[1] + p[4] + p[5];
      l_hi = l_hi * c_hi + p[2] + p[3] + p[6] + p[7];
      m_lo = mn_lo;
      m_hi = mn_hi;
      // P as the A operand of P.V (k = 16 tokens): a0 (lo, tok 0-7), a1 (hi, tok 0-7), a2 (lo, 8-15), a3 (hi, 8-15)
      uint32_t pa[4] = {pack2(p[0], p[1]), pack2(p[2], p[3]), pack2(p[4], p[5]), pack2(p[6], p[7])};
      {
        const uint32_t mi = lane >> 3, t = (mi & 1) * 8 + (lane & 7);
#pragma unroll
        for (int j = 0; j < kHd / 8; j += 2) {
          uint32_t vb[4];  // {b0,b1} for dims 8j.., {b0,b1} for dims 8(j+1)..
          const uint32_t chunk = (uint32_t)j + (mi >> 1);
          ldsm_x4_t(vb, vbase + t * (kHd * 2) + ((chunk ^ (t & 7)) << 4));
          o[j][0] *= c_lo; o[j][1] *= c_lo; o[j][2] *= c_hi; o[j][3] *= c_hi;
          o[j + 1][0] *= c_lo; o[j + 1][1] *= c_lo; o[j + 1][2] *= c_hi; o[j + 1][3] *= c_hi;
          mma16816(o[j], pa, vb[0], vb[1]);
          mma16816(o[j + 1], pa, vb[2], vb[3]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }
  if (!ok && lane == 0) atomicOr(&g_prefill_error, 1u);

  // row sums live in the 4 lanes of a quad
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
  bf16 *ol = out + ((size_t)row_lo * q_heads + head_lo) * kHd + (lane & 3) * 2;
  bf16 *oh = out + ((size_t)row_hi * q_heads + head_hi) * kHd + (lane & 3) * 2;
#pragma unroll
  for (int j = 0; j < kHd / 8; ++j) {
    if (v_lo) *reinterpret_cast<uint32_t *>(ol + j * 8) = pack2(o[j][0] * inv_lo, o[j][1] * inv_lo);
    if (v_hi) *reinterpret_cast<uint32_t *>(oh + j * 8) = pack2(o[j][2] * inv_hi, o[j][3] * inv_hi);
  }
}

}  // namespace

uint32_t prefill_tile_positions(uint32_t q_heads, uint32_t kv_heads) {
  const uint32_t group = q_heads / kv_heads;
  return group ? kRows / group : 0;
}

bool prefill_attention_supported(KvLayout kv, uint32_t q_heads) {
  return kv.head_dim == kHd && kv.block_size == kBlk && kv.swizzle == 1 && kv.num_kv_heads > 0 &&
         q_heads % kv.num_kv_heads == 0 && q_heads / kv.num_kv_heads <= 16;
}

int launch_paged_attention_prefill(const bf16 *q, const bf16 *arena, KvLayout kv, uint32_t layer, AttnBatch batch,
                                   const PrefillTile *tiles, uint32_t num_tiles, uint32_t q_heads, bf16 *out,
                                   cudaStream_t stream) {
  if (num_tiles == 0) return ORION_OK;
  if (prefill_attention_tc_supported(kv, q_heads, arena))  // tcgen05 / tensor-memory kernel; this file's is the fallback
    return launch_paged_attention_prefill_tc(q, arena, kv, layer, batch, tiles, num_tiles, q_heads, out, stream);
  if (!prefill_attention_supported(kv, q_heads))
    return set_error(ORION_ERR_INTERNAL, "prefill attention kernel does not cover this shape");
  static bool attr_set[kMaxDeviceOrdinals] = {};
  ORION_CUDA_CHECK("paged_prefill attr", ensure_dynamic_smem(paged_prefill_kernel, (int)kSmem, attr_set));
  ORION_CUDA_CHECK("paged_prefill", launch_pdl(paged_prefill_kernel, dim3(kv.num_kv_heads, num_tiles), dim3(kThreads),
                                               (size_t)kSmem, stream, q, arena, kv, layer, batch, tiles, q_heads, out));
  count_launch();
  ORION_CUDA_CHECK("paged_prefill", cudaGetLastError());
  return ORION_OK;
}

int prefill_poll_error(uint32_t *code) {
  uint32_t tc = 0;
  ORION_TRY(prefill_tc_poll_error(&tc));
  uint32_t v = 0;
  ORION_CUDA_CHECK("prefill error word", cudaMemcpyFromSymbol(&v, g_prefill_error, sizeof v));
  if (v) {
    uint32_t zero = 0;
    ORION_CUDA_CHECK("prefill error word", cudaMemcpyToSymbol(g_prefill_error, &zero, sizeof zero));
  }
  v |= tc ? 2u : 0u;
  *code = v;
  return ORION_OK;
}

}  // namespace orion
