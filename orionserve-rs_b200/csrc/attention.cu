// Paged GQA attention over the block-table-indexed KV arena
// (crates/orion-models/src/attention.rs:219-295).
//
//  * paged_attention_generic_kernel: any head_dim / block size / storage type,
//    any mix of prefill and decode rows; one CTA per (row, query head). This is
//    the correctness tier (f32 build) and the fallback for shapes the tuned
//    kernel does not cover.
//  * paged_decode_kernel: bf16, head_dim 128, 16-token blocks, one query row
//    per sequence. One CTA per (kv head, sequence, context split); each warp owns
//    a private multi-stage ring of 8 KiB K/V chunks filled by bulk async copies
//    (one copy per 16-token block of one head), computes Q.K^T and P.V with
//    mma.sync m16n8k16 (tokens on M, the GQA group's query heads on N so the group
//    shares every K/V tile) and keeps an online softmax in registers. Warps are
//    merged in shared memory; context splits are merged by decode_combine_kernel.
#include "kernels.h"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>

namespace orion {
namespace {

// ---------------------------------------------------------------------------
// Generic kernel
// ---------------------------------------------------------------------------

constexpr int kGenThreads = 128;
constexpr int kGenChunk = 512;
constexpr int kGenMaxDimsPerThread = 4;  // head_dim <= 512

template <typename T>
__global__ void __launch_bounds__(kGenThreads)
paged_attention_generic_kernel(const T *__restrict__ q, const T *__restrict__ arena, KvLayout kv,
                               uint32_t layer, AttnBatch batch, uint32_t q_heads,
                               T *__restrict__ out) {
  extern __shared__ float smem[];
  const uint32_t hd = kv.head_dim;
  float *q_s = smem;            // [hd]
  float *scores = smem + hd;    // [kGenChunk]
  __shared__ float red[kGenThreads / 32];
  __shared__ float bcast;
  pdl_trigger();
  pdl_wait();

  const uint32_t row = blockIdx.x, head = blockIdx.y;
  const uint32_t group = q_heads / kv.num_kv_heads;  // attention.rs:250
  const uint32_t kvh = head / group;                 // attention.rs:258
  const uint32_t qpos = batch.query_positions[row];
  const uint32_t seq = batch.seq_of_row[row];
  const uint32_t *table = batch.tables_flat + batch.table_offsets[seq];
  const uint32_t B = kv.block_size;
  const float scale = 1.0f / sqrtf((float)hd);  // attention.rs:251

  for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x)
    q_s[d] = to_f32<T>(q[((size_t)row * q_heads + head) * hd + d]);
  __syncthreads();

  float m = -INFINITY, l = 0.0f;
  float acc[kGenMaxDimsPerThread] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t attend = qpos + 1;  // attention.rs:253: positions 0..=query_position

  for (uint32_t c0 = 0; c0 < attend; c0 += kGenChunk) {
    const uint32_t n = min((uint32_t)kGenChunk, attend - c0);
    float cmax = -INFINITY;
    for (uint32_t p = threadIdx.x; p < n; p += blockDim.x) {
      const uint32_t pos = c0 + p, slot = pos % B;
      const T *k = arena + kv.row(layer, table[pos / B], kvh, 0, slot);
      float dot = 0.0f;  // attention.rs:270-273: sequential, unfused
      for (uint32_t d = 0; d < hd; ++d)
        dot = __fadd_rn(dot, __fmul_rn(q_s[d], to_f32<T>(k[kv.col(slot, d)])));
      const float s = __fmul_rn(dot, scale);
      scores[p] = s;
      cmax = fmaxf(cmax, s);
    }
    cmax = warp_max(cmax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = cmax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float v = red[0];
      for (int w = 1; w < kGenThreads / 32; ++w) v = fmaxf(v, red[w]);
      bcast = v;
    }
    __syncthreads();
    const float m_new = fmaxf(m, bcast);
    float csum = 0.0f;
    for (uint32_t p = threadIdx.x; p < n; p += blockDim.x) {
      const float e = expf(scores[p] - m_new);  // tensor.rs:201
      scores[p] = e;
      csum += e;
    }
    csum = warp_sum(csum);
    __syncthreads();  // everyone has read bcast; scores[] are final
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = csum;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < kGenThreads / 32; ++w) total += red[w];
    const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    l = l * corr + total;
#pragma unroll
    for (int j = 0; j < kGenMaxDimsPerThread; ++j) {
      const uint32_t d = threadIdx.x + j * kGenThreads;
      if (d >= hd) break;
      float a = acc[j] * corr;
      for (uint32_t p = 0; p < n; ++p) {
        const float w = scores[p];
        if (w == 0.0f) continue;  // attention.rs:283-285
        const uint32_t pos = c0 + p, slot = pos % B;
        const T *v = arena + kv.row(layer, table[pos / B], kvh, 1, slot);
        a = __fadd_rn(a, __fmul_rn(w, to_f32<T>(v[kv.col(slot, d)])));
      }
      acc[j] = a;
    }
    m = m_new;
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < kGenMaxDimsPerThread; ++j) {
    const uint32_t d = threadIdx.x + j * kGenThreads;
    if (d >= hd) break;
    out[((size_t)row * q_heads + head) * hd + d] = from_f32<T>(l > 0.0f ? acc[j] / l : acc[j]);
  }
}

// ---------------------------------------------------------------------------
// Tuned decode kernel
// ---------------------------------------------------------------------------

constexpr int kHd = 128;          // head_dim
constexpr int kBlk = 16;          // tokens per KV block
constexpr int kWarps = 4;         // warps per CTA, each with a private ring
constexpr int kChunkBytes = 2 * kBlk * kHd * 2;  // K rows + V rows of one (block, head): 8 KiB
constexpr int kMaxGroup = 8;      // query heads per kv head (N of the MMA)
// Ring depth per warp is a template parameter: 2 stages = 65 KiB per CTA (3 CTAs per SM),
// 3 = 97 KiB (2 per SM), 4 = 129 KiB (1 per SM). The merge buffers (16.3 KiB) reuse the ring.
// After the ring: 512 bytes of barriers, then the bf16 q / k / v of the row when the kernel makes
// them itself (kMaxGroup + 2 vectors of 256 bytes).
constexpr int kStashOffset = 512;
constexpr uint32_t decode_smem_bytes(int stages) { return kWarps * stages * kChunkBytes + 4096; }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) {
  return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}
template <typename T>
__device__ __forceinline__ void st4(T *dst, float4 v);
template <>
__device__ __forceinline__ void st4<bf16>(bf16 *dst, float4 v) {
  uint2 packed;
  packed.x = pack_bf16x2(v.x, v.y);
  packed.y = pack_bf16x2(v.z, v.w);
  *reinterpret_cast<uint2 *>(dst) = packed;
}

// Device error word: bit 0 = a ring wait ran out of polls.
__device__ uint32_t g_decode_error = 0;

template <int kStages>
__global__ void __launch_bounds__(kWarps * 32)
paged_decode_kernel(const bf16 *__restrict__ q, const bf16 *__restrict__ arena, KvLayout kv,
                    uint32_t layer, AttnBatch batch, uint32_t q_heads, uint32_t splits,
                    DecodeScratch scratch, bf16 *__restrict__ out, FusedQkv fq) {
  extern __shared__ __align__(1024) uint8_t dsmem[];
  uint8_t *ring = dsmem;  // [kWarps][kStages][kChunkBytes]
  uint64_t *bars = reinterpret_cast<uint64_t *>(dsmem + kWarps * kStages * kChunkBytes);
  bf16 *stash = reinterpret_cast<bf16 *>(dsmem + kWarps * kStages * kChunkBytes + kStashOffset);  // [group + 2][kHd]

  const uint32_t kvh = blockIdx.x, row = blockIdx.y, split = blockIdx.z;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t group = q_heads / kv.num_kv_heads;
  const uint32_t ctx = batch.query_positions[row] + 1;  // attention.rs:253
  const uint32_t *table = batch.tables_flat + batch.table_offsets[batch.seq_of_row[row]];
  const uint32_t nblocks = (ctx + kBlk - 1) / kBlk;
  // Context split: a contiguous range of blocks; warps interleave inside it.
  // Splits of this row: with a length-proportional plan a row is cut into pieces of about
  // blocks_per_split blocks (a short context is not cut at all, a long one up to gridDim.z times), so
  // the CTAs of a ragged batch carry similar amounts; CTAs beyond the row's count have nothing to do.
  const uint32_t bps = scratch.blocks_per_split;
  const uint32_t my_splits = bps ? min(max((nblocks + bps / 2) / bps, 1u), splits) : splits;
  if (split >= my_splits) return;
  const uint32_t per_split = (nblocks + my_splits - 1) / my_splits;
  const uint32_t b_begin = min(split * per_split, nblocks);
  const uint32_t b_end = min(b_begin + per_split, nblocks);

  pdl_trigger();
  if (threadIdx.x < kWarps * kStages) mbar_init(&bars[threadIdx.x], 1);
  mbar_fence_init();
  __syncthreads();

  uint8_t *my_ring = ring + warp * kStages * kChunkBytes;
  uint64_t *my_bars = bars + warp * kStages;
  const size_t layer_base = (size_t)layer * kv.layer_elems();
  // Block i of this warp (i = 0, 1, ...) is logical block b_begin + warp + i*kWarps.
  const uint32_t my_count = (b_end > b_begin + warp) ? (b_end - b_begin - warp + kWarps - 1) / kWarps : 0;

  // Block-table entries are prefetched 32 at a time into one register per lane
  // (two groups in flight) so that issuing a copy never waits on a global load.
  auto load_group = [&](uint32_t g) -> uint32_t {
    const uint32_t idx = g * 32 + lane;
    return idx < my_count ? table[b_begin + warp + idx * kWarps] : 0u;
  };
  uint32_t tgroup = 0, tbl_a = load_group(0), tbl_b = load_group(1);
  auto entry = [&](uint32_t i) -> uint32_t {  // warp-uniform i, called by all lanes
    return __shfl_sync(0xffffffffu, (i >> 5) == tgroup ? tbl_a : tbl_b, i & 31);
  };
  auto issue = [&](uint32_t i, uint32_t pb) {  // lane 0 only
    const bf16 *src = arena + layer_base + ((size_t)pb * kv.num_kv_heads + kvh) * kv.chunk_elems();
    uint64_t *bar = &my_bars[i % kStages];
    mbar_arrive_expect_tx(bar, kChunkBytes);
    bulk_copy_g2s(my_ring + (i % kStages) * kChunkBytes, src, kChunkBytes, bar);
  };
  // First ring fill. Blocks written in earlier steps are fetched before the
  // dependency wait; the sequence's newest block (the one the preceding
  // RoPE/KV-write kernel is filling) and the query only after it.
  const uint32_t pre = min(my_count, (uint32_t)kStages);
  uint32_t deferred = UINT32_MAX;
  for (uint32_t i = 0; i < pre; ++i) {
    const uint32_t pb = entry(i);
    if (b_begin + warp + i * kWarps == nblocks - 1) {
      deferred = i;
      continue;
    }
    if (lane == 0) issue(i, pb);
  }
  pdl_wait();
  if (deferred != UINT32_MAX) {
    const uint32_t pb = entry(deferred);
    if (lane == 0) issue(deferred, pb);
  }

  if (fq.partial != nullptr) {
    // q heads of the group, then k, then v of this kv head, from the projection's partial sums:
    // 16 threads per head, four dims of each RoPE half per thread (tensor.rs:283-298, products
    // rounded separately like the reference).
    const uint32_t total_heads = q_heads + 2 * kv.num_kv_heads, half = kHd / 2;
    const uint32_t pos = ctx - 1, i = (threadIdx.x & 15) * 4;
    for (uint32_t hh = threadIdx.x >> 4; hh < group + 2; hh += (kWarps * 32) / 16) {
      const uint32_t head = hh < group ? kvh * group + hh
                                       : (hh == group ? q_heads + kvh : q_heads + kv.num_kv_heads + kvh);
      const float *p = fq.partial + ((size_t)row * total_heads + head) * kHd;
      float4 x0 = sum_slabs4(p + i, fq.slabs, fq.slab_stride), x1 = sum_slabs4(p + i + half, fq.slabs, fq.slab_stride);
      if (fq.bias) {
        x0 = add4(x0, ld4(fq.bias + (size_t)head * kHd + i));
        x1 = add4(x1, ld4(fq.bias + (size_t)head * kHd + i + half));
      }
      if (hh <= group) {
        const float4 c = ld4(fq.rope_cos + (size_t)pos * half + i), s = ld4(fq.rope_sin + (size_t)pos * half + i);
        const float4 r0 = make_float4(__fsub_rn(__fmul_rn(x0.x, c.x), __fmul_rn(x1.x, s.x)),
                                      __fsub_rn(__fmul_rn(x0.y, c.y), __fmul_rn(x1.y, s.y)),
                                      __fsub_rn(__fmul_rn(x0.z, c.z), __fmul_rn(x1.z, s.z)),
                                      __fsub_rn(__fmul_rn(x0.w, c.w), __fmul_rn(x1.w, s.w)));
        const float4 r1 = make_float4(__fadd_rn(__fmul_rn(x0.x, s.x), __fmul_rn(x1.x, c.x)),
                                      __fadd_rn(__fmul_rn(x0.y, s.y), __fmul_rn(x1.y, c.y)),
                                      __fadd_rn(__fmul_rn(x0.z, s.z), __fmul_rn(x1.z, c.z)),
                                      __fadd_rn(__fmul_rn(x0.w, s.w), __fmul_rn(x1.w, c.w)));
        x0 = r0;
        x1 = r1;
      }
      st4<bf16>(stash + hh * kHd + i, x0);
      st4<bf16>(stash + hh * kHd + i + half, x1);
    }
    __syncthreads();
  }

  // Q^T as the B operand (k = dim, n = head): per 16-dim chunk two packed regs.
  uint32_t qb[kHd / 16][2];
  {
    const uint32_t g = lane >> 2;
    const bf16 *qrow = fq.partial != nullptr ? stash + (g < group ? g : 0) * kHd
                                             : q + ((size_t)row * q_heads + (size_t)kvh * group + g) * kHd;
#pragma unroll
    for (int c = 0; c < kHd / 16; ++c) {
      if (g < group) {
        qb[c][0] = *reinterpret_cast<const uint32_t *>(qrow + c * 16 + (lane & 3) * 2);
        qb[c][1] = *reinterpret_cast<const uint32_t *>(qrow + c * 16 + 8 + (lane & 3) * 2);
      } else {
        qb[c][0] = 0u;
        qb[c][1] = 0u;
      }
    }
  }

  // Online softmax state for the two heads this lane sees in the C fragment
  // (columns 2*(lane%4) and +1), in the log2 domain.
  const float sl2 = 1.4426950408889634f / sqrtf((float)kHd);
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[kHd / 16][4];
#pragma unroll
  for (int t = 0; t < kHd / 16; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

  const uint32_t t_lo = lane >> 2, t_hi = t_lo + 8;  // token rows of this lane in the C fragment
  bool ok = true;
  for (uint32_t i = 0; i < my_count; ++i) {
    const uint32_t stage = i % kStages;
    if ((i >> 5) > tgroup) {  // entering the next group of 32 blocks
      tbl_a = tbl_b;
      ++tgroup;
      tbl_b = load_group(tgroup + 1);
    }
    // the outcome of the bounded wait is taken by the whole warp, so that the lanes stay
    // converged for the shuffles below even if they disagree at the deadline
    if (!__all_sync(0xffffffffu, mbar_wait(&my_bars[stage], (i / kStages) & 1))) {
      ok = false;
      break;
    }
    const uint32_t kbase = smem_u32(my_ring + stage * kChunkBytes);
    const uint32_t vbase = kbase + kBlk * kHd * 2;
    const uint32_t lb = b_begin + warp + i * kWarps;
    const uint32_t valid = min((uint32_t)kBlk, ctx - lb * kBlk);  // tokens of this block in context
    if (fq.partial != nullptr && lb == nblocks - 1) {
      // The block that holds this step's token: its k and v rows come from the stash. Lanes 0-15
      // copy the sixteen 16-byte groups of k, lanes 16-31 those of v, into the landed chunk (for
      // this step) and into the arena (for the steps to come), both in the arena's swizzled order.
      const uint32_t slot = (ctx - 1) % kBlk, j = lane & 15, is_v = lane >> 4;
      const uint4 val = *reinterpret_cast<const uint4 *>(stash + (group + is_v) * kHd + j * 8);
      const uint32_t at = (j ^ (slot & 7u)) * 8;  // element offset of the group inside the row
      *reinterpret_cast<uint4 *>(my_ring + stage * kChunkBytes + ((is_v * kBlk + slot) * kHd + at) * 2) = val;
      bf16 *dst = fq.arena + kv.row(layer, fq.slot_block[row], kvh, is_v, slot);
      *reinterpret_cast<uint4 *>(dst + at) = val;
      __syncwarp();
    }

    // S^T[t][g] = sum_d K[t][d] * Q[g][d]
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const uint32_t mi = lane >> 3, r = lane & 7;
      const uint32_t t = r + (mi & 1) * 8;
#pragma unroll
      for (int c = 0; c < kHd / 16; ++c) {
        uint32_t a[4];
        const uint32_t chunk = (uint32_t)c * 2 + (mi >> 1);
        ldmatrix_x4(a, kbase + t * (kHd * 2) + ((chunk ^ (t & 7)) << 4));
        mma_bf16_16816(s, a, qb[c][0], qb[c][1]);
      }
    }
    // scale into the log2 domain and mask slots beyond the context
    s[0] = (t_lo < valid) ? s[0] * sl2 : -INFINITY;
    s[1] = (t_lo < valid) ? s[1] * sl2 : -INFINITY;
    s[2] = (t_hi < valid) ? s[2] * sl2 : -INFINITY;
    s[3] = (t_hi < valid) ? s[3] * sl2 : -INFINITY;
    float bm0 = fmaxf(s[0], s[2]), bm1 = fmaxf(s[1], s[3]);
#pragma unroll
    for (int off = 4; off <= 16; off <<= 1) {
      bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, off));
      bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, off));
    }
    const float mn0 = fmaxf(m0, bm0), mn1 = fmaxf(m1, bm1);  // finite: token 0 is always valid
    const float c0 = fast_exp2(m0 - mn0), c1 = fast_exp2(m1 - mn1);
    const float p0 = fast_exp2(s[0] - mn0), p1 = fast_exp2(s[1] - mn1);
    const float p2 = fast_exp2(s[2] - mn0), p3 = fast_exp2(s[3] - mn1);
    l0 = l0 * c0 + p0 + p2;  // per-lane partial sums, reduced across lanes at the end
    l1 = l1 * c1 + p1 + p3;
    m0 = mn0;
    m1 = mn1;
    // P^T as the B operand (k = token, n = head)
    const uint32_t pb0 = movmatrix_trans(pack_bf16x2(p0, p1));
    const uint32_t pb1 = movmatrix_trans(pack_bf16x2(p2, p3));
    // O^T[d][g] = O^T*corr + sum_t V[t][d] * P[t][g]
    {
      const uint32_t mi = lane >> 3, r = lane & 7;
      const uint32_t t = r + (mi >> 1) * 8;
#pragma unroll
      for (int mt = 0; mt < kHd / 16; ++mt) {
        uint32_t a[4];
        const uint32_t chunk = (uint32_t)mt * 2 + (mi & 1);
        ldmatrix_x4_trans(a, vbase + t * (kHd * 2) + ((chunk ^ (t & 7)) << 4));
        o[mt][0] *= c0;
        o[mt][1] *= c1;
        o[mt][2] *= c0;
        o[mt][3] *= c1;
        mma_bf16_16816(o[mt], a, pb0, pb1);
      }
    }
    __syncwarp();
    if (i + kStages < my_count) {
      const uint32_t pb = entry(i + kStages);
      if (lane == 0) issue(i + kStages, pb);
    }
  }
  if (!ok && lane == 0) atomicOr(&g_decode_error, 1u);

  // Reduce the per-lane partial sums over the 8 lanes that share a head pair.
#pragma unroll
  for (int off = 4; off <= 16; off <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, off);
    l1 += __shfl_xor_sync(0xffffffffu, l1, off);
  }
  __syncthreads();  // every warp is done with its ring: reuse it for the merge

  float *mo = reinterpret_cast<float *>(dsmem);            // [kWarps][kMaxGroup][kHd]
  float *mml = mo + kWarps * kMaxGroup * kHd;              // [kWarps][kMaxGroup][2]
  {
    const uint32_t g0 = (lane & 3) * 2;
#pragma unroll
    for (int mt = 0; mt < kHd / 16; ++mt) {
      const uint32_t d = mt * 16 + (lane >> 2);
      float *base = mo + ((size_t)warp * kMaxGroup) * kHd;
      base[(g0 + 0) * kHd + d] = o[mt][0];
      base[(g0 + 1) * kHd + d] = o[mt][1];
      base[(g0 + 0) * kHd + d + 8] = o[mt][2];
      base[(g0 + 1) * kHd + d + 8] = o[mt][3];
    }
    if (lane < 4) {
      float *ml = mml + ((size_t)warp * kMaxGroup + g0) * 2;
      ml[0] = m0; ml[1] = l0; ml[2] = m1; ml[3] = l1;
    }
  }
  __syncthreads();
  {
    const uint32_t d = threadIdx.x;  // kWarps*32 == kHd threads: one output dim each
    for (uint32_t g = 0; g < group; ++g) {
      float mall = -INFINITY;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) mall = fmaxf(mall, mml[(w * kMaxGroup + g) * 2]);
      float acc = 0.f, L = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float mw = mml[(w * kMaxGroup + g) * 2];
        const float wgt = (mw == -INFINITY) ? 0.f : fast_exp2(mw - mall);
        acc += wgt * mo[((size_t)w * kMaxGroup + g) * kHd + d];
        L += wgt * mml[(w * kMaxGroup + g) * 2 + 1];
      }
      const uint32_t head = kvh * group + g;
      if (my_splits == 1) {
        out[((size_t)row * q_heads + head) * kHd + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
      } else {
        const size_t pi = ((size_t)row * q_heads + head) * scratch.max_splits + split;
        scratch.partial_out[pi * kHd + d] = acc;
        if (d == 0) {
          scratch.partial_ml[pi * 2] = mall;
          scratch.partial_ml[pi * 2 + 1] = L;
        }
      }
    }
  }
  if (my_splits > 1 && scratch.counters != nullptr) {
    // The CTA that arrives last at its (row, kv head) merges the splits of the group's heads: its
    // partials and everybody else's are visible (fence before the arrival, fence after it), and it
    // puts the counter back to zero for the next launch.
    __shared__ uint32_t arrived_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t *counter = scratch.counters + (size_t)row * kv.num_kv_heads + kvh;
      const uint32_t before = atomicAdd(counter, 1u);
      arrived_last = before == my_splits - 1 ? 1u : 0u;
      if (arrived_last) *counter = 0u;
    }
    __syncthreads();
    if (arrived_last) {
      __threadfence();
      // One warp per query head of the group: lane s holds the running max and sum of split s
      // (at most 32 splits), lane l the four output dims 4l .. 4l + 3 of every split.
      for (uint32_t g = warp; g < group; g += kWarps) {
        const uint32_t head = kvh * group + g;
        const size_t base = ((size_t)row * q_heads + head) * scratch.max_splits;
        float ms = -INFINITY, ls = 0.f;
        if (lane < my_splits) {
          const float2 ml = __ldcg(reinterpret_cast<const float2 *>(scratch.partial_ml + (base + lane) * 2));
          ms = ml.x;
          ls = ml.y;
        }
        const float mall = warp_max(ms);
        const float wgt = (ms == -INFINITY) ? 0.f : fast_exp2(ms - mall);
        const float L = warp_sum(wgt * ls);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t s0 = 0; s0 < my_splits; s0 += 8) {
          float4 x[8];
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j)  // eight independent loads in flight
            x[j] = s0 + j < my_splits ? __ldcg(reinterpret_cast<const float4 *>(scratch.partial_out + (base + s0 + j) * kHd) + lane)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j) {
            const float w = __shfl_sync(0xffffffffu, wgt, (s0 + j) & 31u);
            if (s0 + j < my_splits) {
              acc.x += w * x[j].x; acc.y += w * x[j].y; acc.z += w * x[j].z; acc.w += w * x[j].w;
            }
          }
        }
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        st4<bf16>(out + ((size_t)row * q_heads + head) * kHd + 4 * lane, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
      }
    }
  }
}

__global__ void __launch_bounds__(kHd)
decode_combine_kernel(DecodeScratch scratch, uint32_t splits, uint32_t q_heads, const uint32_t *__restrict__ query_positions,
                      bf16 *__restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const uint32_t row = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  if (scratch.blocks_per_split) {  // the row's own split count, as the decode kernel computed it
    const uint32_t nblocks = query_positions[row] / kBlk + 1, bps = scratch.blocks_per_split;
    splits = min(max((nblocks + bps / 2) / bps, 1u), splits);
    if (splits == 1) return;  // written by the decode kernel itself
  }
  const size_t base = ((size_t)row * q_heads + head) * scratch.max_splits;
  float mall = -INFINITY;
  for (uint32_t s = 0; s < splits; ++s) mall = fmaxf(mall, scratch.partial_ml[(base + s) * 2]);
  float acc = 0.f, L = 0.f;
  for (uint32_t s = 0; s < splits; ++s) {
    const float ms = scratch.partial_ml[(base + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : fast_exp2(ms - mall);
    acc += w * scratch.partial_out[(base + s) * kHd + d];
    L += w * scratch.partial_ml[(base + s) * 2 + 1];
  }
  out[((size_t)row * q_heads + head) * kHd + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
}

inline int after_launch(const char *stage) {
  count_launch();
  ORION_CUDA_CHECK(stage, cudaGetLastError());
  return ORION_OK;
}

}  // namespace

template <typename T>
int launch_paged_attention_generic(const T *q, const T *arena, KvLayout kv, uint32_t layer,
                                   AttnBatch batch, uint32_t q_heads, T *out,
                                   cudaStream_t stream) {
  if (batch.rows == 0) return ORION_OK;
  if (kv.head_dim > kGenThreads * kGenMaxDimsPerThread)
    return set_error(ORION_ERR_INTERNAL, "head_dim %u exceeds the attention kernel limit of %d",
                     kv.head_dim, kGenThreads * kGenMaxDimsPerThread);
  const size_t smem = (kv.head_dim + kGenChunk) * sizeof(float);
  ORION_CUDA_CHECK("paged_attention",
                   launch_pdl(paged_attention_generic_kernel<T>, dim3(batch.rows, q_heads), dim3(kGenThreads), smem,
                              stream, q, arena, kv, layer, batch, q_heads, out));
  return after_launch("paged_attention");
}
template int launch_paged_attention_generic<float>(const float *, const float *, KvLayout, uint32_t,
                                                   AttnBatch, uint32_t, float *, cudaStream_t);
template int launch_paged_attention_generic<bf16>(const bf16 *, const bf16 *, KvLayout, uint32_t,
                                                  AttnBatch, uint32_t, bf16 *, cudaStream_t);

namespace {
int g_decode_stages = 3;                 // ring depth per warp (2, 3 or 4)
uint32_t g_decode_cta_target = 2 * 148;  // CTAs the context split aims for (two per SM are resident)
// Merge of the context splits by a separate kernel (default) or by the last CTA of a (row, kv head) to
// arrive (ORION_DECODE_FUSED_COMBINE=1). Alone the two measure the same (8.3 vs 8.4 us on 64 rows x 1 kv
// head); inside a decode step the separate kernel, which overlaps the decode kernel's tail, measured
// faster (batch 8: 0.41 vs 0.50 ms of attention per step), so it stays the default.
bool g_decode_fused_combine = std::getenv("ORION_DECODE_FUSED_COMBINE") ? std::atoi(std::getenv("ORION_DECODE_FUSED_COMBINE")) != 0 : false;
// Fewest 16-token blocks a context split may hold (tuning A/B: ORION_DECODE_MIN_BLOCKS, 16 = the earlier rule).
uint32_t g_decode_min_blocks = std::getenv("ORION_DECODE_MIN_BLOCKS") ? (uint32_t)std::max(1, std::atoi(std::getenv("ORION_DECODE_MIN_BLOCKS"))) : 4;
}  // namespace

bool decode_attention_supported(KvLayout kv, uint32_t q_heads) {
  return kv.head_dim == kHd && kv.block_size == kBlk && kv.swizzle == 1 && kv.num_kv_heads > 0 &&
         q_heads % kv.num_kv_heads == 0 && q_heads / kv.num_kv_heads <= kMaxGroup;
}

size_t decode_scratch_floats(uint32_t rows, uint32_t q_heads, uint32_t head_dim,
                             uint32_t max_splits) {
  return kDecodeCounterWords + (size_t)rows * q_heads * max_splits * (head_dim + 2);
}

DecodeScratch decode_scratch_at(float *base, uint32_t rows, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                                uint32_t splits, uint32_t blocks_per_split) {
  DecodeScratch sc;
  sc.blocks_per_split = splits > 1 ? blocks_per_split : 0;
  float *partials = base + kDecodeCounterWords;
  sc.partial_out = partials;
  sc.partial_ml = partials + (size_t)rows * q_heads * splits * head_dim;
  sc.max_splits = splits;
  // the in-kernel merge keeps one split per lane
  sc.counters = (g_decode_fused_combine && splits <= 32 && (size_t)rows * kv_heads <= kDecodeCounterWords)
                    ? reinterpret_cast<uint32_t *>(base)
                    : nullptr;
  return sc;
}

uint32_t decode_choose_splits(uint32_t rows, uint32_t kv_heads, uint32_t max_position,
                              uint32_t block_size, uint32_t max_splits) {
  // Aim for two CTAs per SM. A split keeps at least one block per warp (4): at small batches the
  // kernel is bound by latency, not bandwidth, and the 28 MB that 296 CTAs keep in flight cover a
  // whole 8k context, so many short splits beat few long ones (batch 1 went from 72 to 256 CTAs).
  const uint32_t ctas = rows * kv_heads;
  if (ctas == 0) return 1;
  // as many pieces as still fit one resident wave (rounded down): 64 rows x 1 kv head cut five ways is
  // 320 CTAs for 296 places and measured 12.3 us against 8.3 us for four pieces; 256 CTAs (64 rows x
  // 4 kv heads) already reach every SM and are not cut at all
  uint32_t want = g_decode_cta_target / ctas;
  const uint32_t nblocks = max_position / block_size + 1;
  const uint32_t cap = nblocks / g_decode_min_blocks > 0 ? nblocks / g_decode_min_blocks : 1;
  if (want > cap) want = cap;
  if (want > max_splits) want = max_splits;
  return want < 1 ? 1 : want;
}

DecodePlan decode_plan(uint32_t rows, uint32_t kv_heads, uint64_t total_blocks, uint32_t max_position,
                       uint32_t block_size, uint32_t max_splits) {
  DecodePlan p{1, 0};
  const uint64_t ctas = (uint64_t)rows * kv_heads;
  if (ctas == 0 || total_blocks == 0) return p;
  // Fewer rows than SMs: every row is cut alike (measured better than pieces of equal length on
  // 8 ragged rows, 0.73 vs 0.65 of the copy peak: the short rows' pieces end early and their
  // merges overlap the long rows' streams).
  if (ctas < 148) {
    p.splits = decode_choose_splits(rows, kv_heads, max_position, block_size, max_splits);
    return p;
  }
  // Blocks one piece should hold: what makes about g_decode_cta_target CTAs out of the batch's blocks
  // (fills the machine when the batch is small), but never more than the mean row, so that in a
  // ragged batch the long rows are cut down to the size of the others. Rows of equal length are cut
  // only when there are too few of them to reach every SM.
  uint64_t per = (total_blocks * kv_heads + g_decode_cta_target - 1) / g_decode_cta_target;
  const uint64_t mean_row = (total_blocks + rows - 1) / rows;
  if (per > mean_row) per = mean_row;
  if (per < g_decode_min_blocks) per = g_decode_min_blocks;
  const uint32_t nblocks = max_position / block_size + 1;  // the longest row
  uint32_t most = (uint32_t)((nblocks + per / 2) / per);
  if (most > max_splits) most = max_splits;
  if (most <= 1) return p;
  p.splits = most;
  p.blocks_per_split = (uint32_t)per;
  return p;
}

namespace {
template <int STAGES>
int launch_decode_stages(const bf16 *q, const bf16 *arena, KvLayout kv, uint32_t layer, AttnBatch batch,
                         uint32_t q_heads, uint32_t splits, DecodeScratch scratch, bf16 *out,
                         FusedQkv fq, cudaStream_t stream) {
  static bool attr_set[kMaxDeviceOrdinals] = {};
  ORION_CUDA_CHECK("paged_decode attr",
                   ensure_dynamic_smem(paged_decode_kernel<STAGES>, (int)decode_smem_bytes(STAGES), attr_set));
  ORION_CUDA_CHECK("paged_decode",
                   launch_pdl(paged_decode_kernel<STAGES>, dim3(kv.num_kv_heads, batch.rows, splits),
                              dim3(kWarps * 32), (size_t)decode_smem_bytes(STAGES), stream, q, arena, kv, layer,
                              batch, q_heads, splits, scratch, out, fq));
  return ORION_OK;
}
}  // namespace

void decode_set_tuning(int stages, uint32_t cta_target) {
  if (stages >= 2 && stages <= 4) g_decode_stages = stages;
  if (cta_target) g_decode_cta_target = cta_target;
}

int launch_paged_attention_decode(const bf16 *q, const bf16 *arena, KvLayout kv, uint32_t layer,
                                  AttnBatch batch, uint32_t q_heads, uint32_t splits,
                                  DecodeScratch scratch, bf16 *out, cudaStream_t stream,
                                  FusedQkv fq) {
  if (batch.rows == 0) return ORION_OK;
  if (!decode_attention_supported(kv, q_heads))
    return set_error(ORION_ERR_INTERNAL, "decode attention kernel does not cover this shape");
  if (splits < 1) splits = 1;
  if (splits > 1 && (scratch.partial_out == nullptr || splits > scratch.max_splits))
    return set_error(ORION_ERR_INTERNAL, "decode attention scratch too small for %u splits",
                     splits);
  switch (g_decode_stages) {
    case 2: ORION_TRY(launch_decode_stages<2>(q, arena, kv, layer, batch, q_heads, splits, scratch, out, fq, stream)); break;
    case 4: ORION_TRY(launch_decode_stages<4>(q, arena, kv, layer, batch, q_heads, splits, scratch, out, fq, stream)); break;
    default: ORION_TRY(launch_decode_stages<3>(q, arena, kv, layer, batch, q_heads, splits, scratch, out, fq, stream)); break;
  }
  ORION_TRY(after_launch("paged_decode"));
  if (splits > 1 && scratch.counters == nullptr) {
    ORION_CUDA_CHECK("decode_combine", launch_pdl(decode_combine_kernel, dim3(batch.rows, q_heads), dim3(kHd), 0,
                                                  stream, scratch, splits, q_heads, batch.query_positions, out));
    ORION_TRY(after_launch("decode_combine"));
  }
  return ORION_OK;
}

int decode_poll_error(uint32_t *code) {
  uint32_t v = 0;
  ORION_CUDA_CHECK("decode error word", cudaMemcpyFromSymbol(&v, g_decode_error, sizeof v));
  if (v) {
    uint32_t zero = 0;
    ORION_CUDA_CHECK("decode error word", cudaMemcpyToSymbol(g_decode_error, &zero, sizeof zero));
  }
  *code = v;
  return ORION_OK;
}

// ---------------------------------------------------------------------------
// Allocation-free decode attention
// ---------------------------------------------------------------------------
//
// Some callers may not allocate device memory at the moment they need attention:
// code running while a CUDA stream is being captured into a graph, code inside a
// serving loop that has handed all of its memory to a pool it does not own, or a
// plugin that was only given buffers and a stream. For them the split-context
// decode kernel gets its per-split partial results from a fixed array that lives
// in the library image instead of from a buffer sized and allocated per call.
//
// The array costs kNoAllocScratchFloats * 4 bytes (16 MiB) on every GPU that loads
// this library, for the life of the process.
constexpr size_t kNoAllocScratchFloats = size_t(4) << 20;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

namespace {
constexpr int kMaxDevices = kMaxDeviceOrdinals;
// Device address of g_noalloc_scratch per device ordinal. The symbol's name is
// only a host-side handle; a kernel must be given the address looked up with
// cudaGetSymbolAddress while that device is current.
std::atomic<float *> g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mu;

// Makes `device` current for the scope and puts the caller's device back afterwards.
struct ScopedDevice {
  int prev = -1;
  cudaError_t status;
  explicit ScopedDevice(int device) {
    status = cudaGetDevice(&prev);
    if (status == cudaSuccess && prev != device) status = cudaSetDevice(device);
  }
  ~ScopedDevice() {
    int now = -1;
    if (prev >= 0 && cudaGetDevice(&now) == cudaSuccess && now != prev) cudaSetDevice(prev);
  }
};
}  // namespace

int noalloc_decode_attention(int device, const bf16 *q, const bf16 *arena, uint32_t num_blocks,
                             uint32_t num_kv_heads, uint32_t num_query_heads,
                             const uint32_t *query_positions, const uint32_t *seq_of_row,
                             const uint32_t *tables_flat, const uint32_t *table_offsets,
                             uint32_t rows, uint32_t max_position, uint32_t splits, bf16 *out,
                             cudaStream_t stream) {
  if (device < 0 || device >= kMaxDevices)
    return set_error(ORION_ERR_INVALID_REQUEST, "device ordinal %d outside 0..%d", device, kMaxDevices - 1);
  KvLayout kv{1, num_blocks, num_kv_heads, (uint32_t)kBlk, (uint32_t)kHd, 1u};
  if (!decode_attention_supported(kv, num_query_heads))
    return set_error(ORION_ERR_INVALID_REQUEST,
                     "allocation-free decode attention covers head_dim 128, block 16, at most 8 query "
                     "heads per kv head");
  if (rows == 0) return ORION_OK;
  if (splits == 0) splits = decode_choose_splits(rows, num_kv_heads, max_position, kBlk, 32);
  const size_t need = decode_scratch_floats(rows, num_query_heads, kHd, splits);  // counter words included
  if (splits > 1 && need > kNoAllocScratchFloats)
    return set_error(ORION_ERR_INVALID_REQUEST,
                     "allocation-free decode attention: %u rows x %u heads x %u splits needs %zu scratch "
                     "floats, the built-in array holds %zu; use fewer splits or the allocating entry point",
                     rows, num_query_heads, splits, need, kNoAllocScratchFloats);
  ScopedDevice current(device);  // the caller's current device is restored on return
  ORION_CUDA_CHECK("set device", current.status);
  float *base = g_noalloc_ptr[device].load(std::memory_order_acquire);
  if (!base) {
    // One-time set-up for this device (no allocation: the array is part of the module).
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    void *p = nullptr;
    ORION_CUDA_CHECK("scratch symbol address", cudaGetSymbolAddress(&p, g_noalloc_scratch));
    base = static_cast<float *>(p);
    g_noalloc_ptr[device].store(base, std::memory_order_release);
  }
  // Every (row, head, split) slot is written before the merge reads it, and the arrival
  // counters at the head of the array are put back to zero by the launch that used them (the
  // array starts zeroed when the module is loaded), so nothing has to be cleared between calls.
  DecodeScratch sc = decode_scratch_at(base, rows, num_query_heads, num_kv_heads, kHd, splits);
  AttnBatch ab{query_positions, seq_of_row, tables_flat, table_offsets, rows, max_position};
  return launch_paged_attention_decode(q, arena, kv, 0, ab, num_query_heads, splits, sc, out, stream);
}

}  // namespace orion

extern "C" int orion_cuda_paged_decode_attention_noalloc(
    int device, const void *q, const void *kv_arena, uint32_t num_blocks, uint32_t num_kv_heads,
    uint32_t num_query_heads, const uint32_t *query_positions, const uint32_t *seq_of_row,
    const uint32_t *block_tables_flat, const uint32_t *block_table_offsets, uint32_t rows,
    uint32_t max_position, uint32_t splits, void *out, void *stream) {
  orion::clear_error();
  if (!q || !kv_arena || !query_positions || !seq_of_row || !block_tables_flat || !block_table_offsets || !out)
    return orion::set_error(ORION_ERR_INVALID_REQUEST, "null pointer argument");
  return orion::noalloc_decode_attention(
      device, static_cast<const orion::bf16 *>(q), static_cast<const orion::bf16 *>(kv_arena), num_blocks,
      num_kv_heads, num_query_heads, query_positions, seq_of_row, block_tables_flat, block_table_offsets, rows,
      max_position, splits, static_cast<orion::bf16 *>(out), static_cast<cudaStream_t>(stream));
}
