// Bandwidth-bound elementwise kernels of the forward pass: embedding gather +
// RMSNorm, residual add + RMSNorm (which also sums the split-K slabs of the
// preceding projection), RoPE + KV-slot write, SwiGLU, greedy argmax, and the
// conversion / layout helpers used at load time and by the parity tests.
#include "kernels.h"

#include <cstdlib>

#include <cfloat>

namespace orion {

thread_local uint64_t g_launch_count = 0;
bool g_pdl_enabled = true;
uint32_t g_tuning_generation = 0;

namespace {

constexpr int kNormThreads = 256;

// Sum of squares accumulates in f64 for the f32 build (the reference does,
// tensor.rs:155) and in f32 for bf16 storage.
template <typename T>
struct NormAcc { using type = float; };
template <>
struct NormAcc<float> { using type = double; };

template <typename Acc>
__device__ __forceinline__ Acc block_sum(Acc v, Acc *shared) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) shared[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  Acc total = Acc(0);
  for (int i = 0; i < nwarps; ++i) total += shared[i];  // fixed order: deterministic
  __syncthreads();
  return total;
}

template <typename Acc>
__device__ __forceinline__ float norm_scale(Acc sum_sq, uint32_t cols, float eps);
template <>
__device__ __forceinline__ float norm_scale<double>(double sum_sq, uint32_t cols, float eps) {
  // tensor.rs:156-157: rms in f64, scale = (1/rms) as f32
  return (float)(1.0 / sqrt(sum_sq / (double)cols + (double)eps));
}
template <>
__device__ __forceinline__ float norm_scale<float>(float sum_sq, uint32_t cols, float eps) {
  return rsqrtf(sum_sq / (float)cols + eps);
}

template <typename T>
__global__ void __launch_bounds__(kNormThreads)
embed_rmsnorm_kernel(const T *__restrict__ embed, const uint32_t *__restrict__ tokens,
                     const float *__restrict__ w, float eps, float *__restrict__ hidden,
                     T *__restrict__ normed, uint32_t H) {
  using Acc = typename NormAcc<T>::type;
  __shared__ Acc red[32];
  pdl_trigger();
  pdl_wait();  // the residual stream and `normed` may still be read by the previous step
  const uint32_t row = blockIdx.x;
  const T *src = embed + (size_t)tokens[row] * H;
  float *h = hidden + (size_t)row * H;
  Acc ss = Acc(0);
  for (uint32_t c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = to_f32<T>(src[c]);
    h[c] = v;
    ss += (Acc)v * (Acc)v;
  }
  const float scale = norm_scale<Acc>(block_sum<Acc>(ss, red), H, eps);
  T *o = normed + (size_t)row * H;
  for (uint32_t c = threadIdx.x; c < H; c += blockDim.x)
    o[c] = from_f32<T>(__fmul_rn(__fmul_rn(h[c], scale), w[c]));  // (v*scale)*w, tensor.rs:159
}

template <typename T>
__global__ void __launch_bounds__(kNormThreads)
residual_rmsnorm_kernel(const float *__restrict__ partial, uint32_t splits, size_t split_stride,
                        float *__restrict__ hidden, const float *__restrict__ w, float eps,
                        T *__restrict__ out, const uint32_t *__restrict__ row_map, uint32_t H) {
  using Acc = typename NormAcc<T>::type;
  __shared__ Acc red[32];
  extern __shared__ float row_cache[];  // H floats: the updated residual row
  pdl_trigger();
  pdl_wait();
  const uint32_t src_row = row_map ? row_map[blockIdx.x] : blockIdx.x;
  float *h = hidden + (size_t)src_row * H;
  Acc ss = Acc(0);
  for (uint32_t c = threadIdx.x; c < H; c += blockDim.x) {
    float v = h[c];
    if (partial) {
      const float *p = partial + (size_t)src_row * H + c;
      float add = p[0];
      for (uint32_t s = 1; s < splits; ++s) add += p[s * split_stride];
      v = __fadd_rn(v, add);  // hidden += proj, transformer.rs:330-332
      if (!row_map) h[c] = v;
    }
    row_cache[c] = v;
    ss += (Acc)v * (Acc)v;
  }
  const float scale = norm_scale<Acc>(block_sum<Acc>(ss, red), H, eps);
  T *o = out + (size_t)blockIdx.x * H;
  for (uint32_t c = threadIdx.x; c < H; c += blockDim.x)
    o[c] = from_f32<T>(__fmul_rn(__fmul_rn(row_cache[c], scale), w[c]));
}

// ---- 128-bit vectorised variants (row widths that are multiples of 4) ------------

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) {
  return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}
template <typename T>
__device__ __forceinline__ void st4(T *dst, float4 v);
template <>
__device__ __forceinline__ void st4<float>(float *dst, float4 v) { *reinterpret_cast<float4 *>(dst) = v; }
template <>
__device__ __forceinline__ void st4<bf16>(bf16 *dst, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 packed;
  packed.x = *reinterpret_cast<uint32_t *>(&lo);
  packed.y = *reinterpret_cast<uint32_t *>(&hi);
  *reinterpret_cast<uint2 *>(dst) = packed;
}

// One CTA per output row, up to 1024 threads, CHUNKS float4 groups per thread kept
// in registers: all loads of a row (residual + every split-K slab) are in flight
// at once, so a 64-row decode batch costs one memory round trip, not sixteen.
template <typename T, int CHUNKS>
__global__ void __launch_bounds__(1024)
residual_rmsnorm_vec_kernel(const float *__restrict__ partial, uint32_t splits, size_t split_stride,
                            float *__restrict__ hidden, const float *__restrict__ w, float eps,
                            T *__restrict__ out, const uint32_t *__restrict__ row_map, uint32_t H,
                            uint32_t *__restrict__ ready) {
  using Acc = typename NormAcc<T>::type;
  __shared__ Acc red[32];
  pdl_trigger();
  const uint32_t nvec = H / 4;
  float4 wv[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {  // gains are immutable: fetched before the dependency wait
    const uint32_t idx = threadIdx.x + c * blockDim.x;
    wv[c] = idx < nvec ? ld4(w + 4 * (size_t)idx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  const uint32_t src_row = row_map ? row_map[blockIdx.x] : blockIdx.x;
  float *h = hidden + (size_t)src_row * H;
  float4 v[CHUNKS];
  Acc ss = Acc(0);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const uint32_t idx = threadIdx.x + c * blockDim.x;
    v[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (idx < nvec) {
      v[c] = ld4(h + 4 * (size_t)idx);
      if (partial) {
        const float4 add = sum_slabs4(partial + (size_t)src_row * H + 4 * (size_t)idx, splits, split_stride);
        v[c] = add4(v[c], add);  // hidden += proj, transformer.rs:330-332
        if (!row_map) *reinterpret_cast<float4 *>(h + 4 * (size_t)idx) = v[c];
      }
      ss += (Acc)v[c].x * (Acc)v[c].x + (Acc)v[c].y * (Acc)v[c].y + (Acc)v[c].z * (Acc)v[c].z +
            (Acc)v[c].w * (Acc)v[c].w;
    }
  }
  const float scale = norm_scale<Acc>(block_sum<Acc>(ss, red), H, eps);
  T *o = out + (size_t)blockIdx.x * H;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const uint32_t idx = threadIdx.x + c * blockDim.x;
    if (idx < nvec)
      st4<T>(o + 4 * (size_t)idx,
             make_float4(__fmul_rn(__fmul_rn(v[c].x, scale), wv[c].x), __fmul_rn(__fmul_rn(v[c].y, scale), wv[c].y),
                         __fmul_rn(__fmul_rn(v[c].z, scale), wv[c].z), __fmul_rn(__fmul_rn(v[c].w, scale), wv[c].w)));
  }
  if (ready) {  // the consumer polls this count instead of waiting for the kernel to complete
    __syncthreads();
    if (threadIdx.x == 0) signal_ready(ready);
  }
}

// RoPE + KV-slot write, four rotation pairs per thread: head_dim % 8 == 0.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kvwrite_vec_kernel(const float *__restrict__ partial, uint32_t splits, size_t split_stride,
                        const float *__restrict__ bias, const uint32_t *__restrict__ positions,
                        const uint32_t *__restrict__ slot_block, const uint32_t *__restrict__ slot_slot,
                        const float *__restrict__ rope_cos, const float *__restrict__ rope_sin,
                        T *__restrict__ q_out, T *__restrict__ arena, KvLayout kv, uint32_t layer,
                        uint32_t q_heads) {
  pdl_trigger();
  pdl_wait();
  const uint32_t hd = kv.head_dim, half = hd / 2, tph = half / 4;  // threads per head
  const uint32_t total_heads = q_heads + 2 * kv.num_kv_heads;
  const uint32_t row = blockIdx.x;
  const uint32_t head = blockIdx.y * (blockDim.x / tph) + threadIdx.x / tph;
  if (head >= total_heads) return;
  const uint32_t i = (threadIdx.x % tph) * 4;
  const float *p = partial + ((size_t)row * total_heads + head) * hd;
  float4 x0 = sum_slabs4(p + i, splits, split_stride), x1 = sum_slabs4(p + i + half, splits, split_stride);
  if (bias) {  // acc + bias, tensor.rs:126
    x0 = add4(x0, ld4(bias + (size_t)head * hd + i));
    x1 = add4(x1, ld4(bias + (size_t)head * hd + i + half));
  }
  const bool is_q = head < q_heads;
  const bool is_k = !is_q && head < q_heads + kv.num_kv_heads;
  if (is_q || is_k) {  // tensor.rs:291-296, products rounded separately like the reference
    const uint32_t pos = positions[row];
    const float4 c = ld4(rope_cos + (size_t)pos * half + i), s = ld4(rope_sin + (size_t)pos * half + i);
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
  if (is_q) {
    T *dst = q_out + ((size_t)row * q_heads + head) * hd;
    st4<T>(dst + i, x0);
    st4<T>(dst + i + half, x1);
  } else {
    const uint32_t kvh = is_k ? head - q_heads : head - q_heads - kv.num_kv_heads;
    const uint32_t slot = slot_slot[row];
    T *dst = arena + kv.row(layer, slot_block[row], kvh, is_k ? 0u : 1u, slot);
    st4<T>(dst + kv.col(slot, i), x0);  // i % 4 == 0: the four values stay inside one 16-byte group
    st4<T>(dst + kv.col(slot, i + half), x1);
  }
}

template <typename T>
__device__ __forceinline__ float silu_f(float g);

// SwiGLU over [rows][2*ffn] partials, four outputs per thread: ffn % 4 == 0.
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_vec_kernel(const float *__restrict__ partial, uint32_t splits, size_t split_stride,
                  T *__restrict__ act, uint32_t rows, uint32_t ffn, bool interleaved) {
  pdl_trigger();
  pdl_wait();
  const uint32_t fv = ffn / 4;
  const size_t total = (size_t)rows * fv;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / fv, f = (idx % fv) * 4;
    float4 g, u;
    if (interleaved) {  // columns 2f = gate f, 2f + 1 = up f
      const float *pg = partial + r * 2 * ffn + 2 * f;
      float4 a = ld4(pg), b = ld4(pg + 4);
      for (uint32_t s = 1; s < splits; ++s) {
        a = add4(a, ld4(pg + s * split_stride));
        b = add4(b, ld4(pg + s * split_stride + 4));
      }
      g = make_float4(a.x, a.z, b.x, b.z);
      u = make_float4(a.y, a.w, b.y, b.w);
    } else {
      const float *pg = partial + r * 2 * ffn + f;
      g = ld4(pg);
      u = ld4(pg + ffn);
      for (uint32_t s = 1; s < splits; ++s) {
        g = add4(g, ld4(pg + s * split_stride));
        u = add4(u, ld4(pg + s * split_stride + ffn));
      }
    }
    st4<T>(act + r * ffn + f,
           make_float4(__fmul_rn(silu_f<T>(g.x), u.x), __fmul_rn(silu_f<T>(g.y), u.y),
                       __fmul_rn(silu_f<T>(g.z), u.z), __fmul_rn(silu_f<T>(g.w), u.w)));  // tensor.rs:186
  }
}

template <typename T>
__global__ void rope_kvwrite_kernel(const float *__restrict__ partial, uint32_t splits,
                                    size_t split_stride, const float *__restrict__ bias,
                                    const uint32_t *__restrict__ positions,
                                    const uint32_t *__restrict__ slot_block,
                                    const uint32_t *__restrict__ slot_slot,
                                    const float *__restrict__ rope_cos,
                                    const float *__restrict__ rope_sin, T *__restrict__ q_out,
                                    T *__restrict__ arena, KvLayout kv, uint32_t layer,
                                    uint32_t q_heads) {
  pdl_trigger();
  pdl_wait();
  const uint32_t row = blockIdx.x, head = blockIdx.y;
  const uint32_t hd = kv.head_dim, half = hd / 2;
  const uint32_t n_total = (q_heads + 2 * kv.num_kv_heads) * hd;
  const float *p = partial + (size_t)row * n_total + (size_t)head * hd;
  const float *b = bias ? bias + (size_t)head * hd : nullptr;
  const uint32_t pos = positions[row];
  const float *cs = rope_cos + (size_t)pos * half, *sn = rope_sin + (size_t)pos * half;
  const bool is_q = head < q_heads;
  const bool is_k = !is_q && head < q_heads + kv.num_kv_heads;
  T *dst;
  uint32_t slot = 0;
  KvLayout lay = kv;
  if (is_q) {
    dst = q_out + ((size_t)row * q_heads + head) * hd;
    lay.swizzle = 0;  // q rows are plain
  } else {
    const uint32_t kvh = is_k ? head - q_heads : head - q_heads - kv.num_kv_heads;
    slot = slot_slot[row];
    dst = arena + kv.row(layer, slot_block[row], kvh, is_k ? 0u : 1u, slot);
  }
  for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
    float x0 = p[i], x1 = p[i + half];
    for (uint32_t s = 1; s < splits; ++s) {
      x0 += p[s * split_stride + i];
      x1 += p[s * split_stride + i + half];
    }
    if (b) {  // acc + bias, tensor.rs:126
      x0 = __fadd_rn(x0, b[i]);
      x1 = __fadd_rn(x1, b[i + half]);
    }
    if (is_q || is_k) {  // tensor.rs:291-296, unfused like the reference
      const float c = cs[i], s = sn[i];
      const float r0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
      const float r1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
      x0 = r0;
      x1 = r1;
    }
    dst[lay.col(slot, i)] = from_f32<T>(x0);
    dst[lay.col(slot, i + half)] = from_f32<T>(x1);
  }
}

template <typename T>
__global__ void rope_rows_kernel(T *__restrict__ x, const uint32_t *__restrict__ positions,
                                 const float *__restrict__ rope_cos,
                                 const float *__restrict__ rope_sin, uint32_t heads, uint32_t hd) {
  const uint32_t row = blockIdx.x, head = blockIdx.y, half = hd / 2;
  T *v = x + ((size_t)row * heads + head) * hd;
  const float *cs = rope_cos + (size_t)positions[row] * half;
  const float *sn = rope_sin + (size_t)positions[row] * half;
  for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
    const float x0 = to_f32<T>(v[i]), x1 = to_f32<T>(v[i + half]);
    v[i] = from_f32<T>(__fsub_rn(__fmul_rn(x0, cs[i]), __fmul_rn(x1, sn[i])));
    v[i + half] = from_f32<T>(__fadd_rn(__fmul_rn(x0, sn[i]), __fmul_rn(x1, cs[i])));
  }
}

template <typename T>
__device__ __forceinline__ float silu_f(float g);
template <>
__device__ __forceinline__ float silu_f<float>(float g) { return g / (1.0f + expf(-g)); }
template <>
__device__ __forceinline__ float silu_f<bf16>(float g) { return g / (1.0f + __expf(-g)); }

template <typename T>
__global__ void swiglu_kernel(const float *__restrict__ partial, uint32_t splits,
                              size_t split_stride, T *__restrict__ act, uint32_t rows,
                              uint32_t ffn, bool interleaved) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)rows * ffn;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / ffn, f = idx % ffn;
    const float *pg = partial + r * 2 * ffn + (interleaved ? 2 * f : f);
    const size_t up = interleaved ? 1 : ffn;
    float g = pg[0], u = pg[up];
    for (uint32_t s = 1; s < splits; ++s) {
      g += pg[s * split_stride];
      u += pg[s * split_stride + up];
    }
    act[idx] = from_f32<T>(__fmul_rn(silu_f<T>(g), u));  // tensor.rs:186
  }
}

__global__ void finish_linear_kernel(const float *__restrict__ partial, uint32_t splits,
                                     size_t split_stride, const float *__restrict__ bias,
                                     float *__restrict__ out, uint32_t rows, uint32_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)rows * n;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    float v = partial[idx];
    for (uint32_t s = 1; s < splits; ++s) v += partial[s * split_stride + idx];
    out[idx] = __fadd_rn(v, bias ? bias[idx % n] : 0.0f);
  }
}

__global__ void __launch_bounds__(1024)
argmax_kernel(const float *__restrict__ logits, uint32_t cols, uint32_t *__restrict__ out) {
  __shared__ float s_val[32];
  __shared__ uint32_t s_idx[32];
  pdl_trigger();
  pdl_wait();
  const float *row = logits + (size_t)blockIdx.x * cols;
  float best = -INFINITY;
  uint32_t best_i = UINT32_MAX;
  // strict comparisons in ascending index order: the lowest index of equal maxima survives and
  // NaN never wins (sampling.rs:196-206)
  if ((cols & 3u) == 0 && (reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
    const float4 *row4 = reinterpret_cast<const float4 *>(row);
    for (uint32_t c = threadIdx.x; c < cols / 4; c += blockDim.x) {
      const float4 v = row4[c];
      if (v.x > best) { best = v.x; best_i = 4 * c; }
      if (v.y > best) { best = v.y; best_i = 4 * c + 1; }
      if (v.z > best) { best = v.z; best_i = 4 * c + 2; }
      if (v.w > best) { best = v.w; best_i = 4 * c + 3; }
    }
  } else {
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float v = row[c];
      if (v > best) {
        best = v;
        best_i = c;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    s_val[threadIdx.x >> 5] = best;
    s_idx[threadIdx.x >> 5] = best_i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (uint32_t w = 1; w < blockDim.x / 32; ++w) {
      if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) {
        best = s_val[w];
        best_i = s_idx[w];
      }
    }
    out[blockIdx.x] = best_i;
  }
}

template <typename T>
__global__ void convert_from_f32_kernel(const float *__restrict__ src, T *__restrict__ dst,
                                        size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    dst[i] = from_f32<T>(src[i]);
}
template <typename T>
__global__ void convert_to_f32_kernel(const T *__restrict__ src, float *__restrict__ dst,
                                      size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    dst[i] = to_f32<T>(src[i]);
}
template <typename T>
__global__ void scale_convert_kernel(const float *__restrict__ src, T *__restrict__ dst, size_t n,
                                     float scale) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    dst[i] = from_f32<T>(src[i] * scale);
}
__global__ void f16_to_f32_kernel(const uint16_t *__restrict__ src, float *__restrict__ dst,
                                  size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __half2float(__ushort_as_half(src[i]));
}

// One thread per arena element, indexed in reference order.
template <typename T, bool kToReference>
__global__ void arena_reorder_kernel(T *__restrict__ arena, KvLayout kv, float *__restrict__ ref,
                                     size_t total) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    size_t r = idx;
    const uint32_t d = r % kv.head_dim; r /= kv.head_dim;
    const uint32_t head = r % kv.num_kv_heads; r /= kv.num_kv_heads;
    const uint32_t slot = r % kv.block_size; r /= kv.block_size;
    const uint32_t is_v = r % 2; r /= 2;
    const uint32_t block = r % kv.num_blocks; r /= kv.num_blocks;
    const uint32_t layer = (uint32_t)r;
    const size_t a = kv.row(layer, block, head, is_v, slot) + kv.col(slot, d);
    if (kToReference) ref[idx] = to_f32<T>(arena[a]);
    else arena[a] = from_f32<T>(ref[idx]);
  }
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

template <typename T>
__global__ void fill_normal_kernel(T *__restrict__ dst, size_t n, uint64_t seed) {
  // Box-Muller on a counter-based stream: element pair (2i, 2i+1) from counter i.
  const size_t pairs = (n + 1) / 2;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs;
       i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t bits = splitmix64(seed ^ (i * 0xD1B54A32D192ED03ull));
    const float u1 = ((uint32_t)(bits >> 40) + 1.0f) * (1.0f / 16777217.0f);
    const float u2 = (uint32_t)(bits & 0xffffffu) * (1.0f / 16777216.0f);
    const float r = sqrtf(-2.0f * __logf(u1));
    float s, c;
    __sincosf(6.28318530718f * u2, &s, &c);
    dst[2 * i] = from_f32<T>(r * c);
    if (2 * i + 1 < n) dst[2 * i + 1] = from_f32<T>(r * s);
  }
}

inline uint32_t grid_for(size_t n, int threads) {
  size_t g = (n + threads - 1) / threads;
  const size_t cap = 148 * 16;  // a few waves over the 148 SMs; grid-stride covers the rest
  return (uint32_t)(g < 1 ? 1 : (g > cap ? cap : g));
}

inline int after_launch(const char *stage) {
  count_launch();
  ORION_CUDA_CHECK(stage, cudaGetLastError());
  return ORION_OK;
}

}  // namespace

template <typename T>
int launch_embed_rmsnorm(const T *embed, const uint32_t *tokens, const float *norm_w, float eps,
                         float *hidden, T *normed, uint32_t rows, uint32_t hidden_size,
                         cudaStream_t stream) {
  if (rows == 0) return ORION_OK;
  ORION_CUDA_CHECK("embed_rmsnorm", launch_pdl(embed_rmsnorm_kernel<T>, dim3(rows), dim3(kNormThreads), 0,
                                               stream, embed, tokens, norm_w, eps, hidden, normed,
                                               hidden_size));
  return after_launch("embed_rmsnorm");
}

namespace {
template <typename T, int CHUNKS>
int launch_residual_vec(const float *partial, uint32_t splits, size_t split_stride, float *hidden,
                        const float *norm_w, float eps, T *out, const uint32_t *row_map,
                        uint32_t out_rows, uint32_t H, uint32_t threads, cudaStream_t stream, uint32_t *ready) {
  ORION_CUDA_CHECK("residual_rmsnorm",
                   launch_pdl(residual_rmsnorm_vec_kernel<T, CHUNKS>, dim3(out_rows), dim3(threads), 0, stream,
                              partial, splits, split_stride, hidden, norm_w, eps, out, row_map, H, ready));
  return after_launch("residual_rmsnorm");
}
}  // namespace

template <typename T>
int launch_residual_rmsnorm(const float *partial, uint32_t splits, size_t split_stride,
                            float *hidden, const float *norm_w, float eps, T *out,
                            const uint32_t *row_map, uint32_t out_rows, uint32_t hidden_size,
                            cudaStream_t stream, uint32_t *ready) {
  if (out_rows == 0) return ORION_OK;
  if (hidden_size % 4 == 0 && hidden_size / 4 <= 4096 && split_stride % 4 == 0) {
    const uint32_t nvec = hidden_size / 4;
    const uint32_t threads = nvec >= 1024 ? 1024 : ((nvec + 31) / 32) * 32;
    const uint32_t chunks = (nvec + threads - 1) / threads;
    if (chunks == 1)
      return launch_residual_vec<T, 1>(partial, splits, split_stride, hidden, norm_w, eps, out, row_map,
                                       out_rows, hidden_size, threads, stream, ready);
    if (chunks == 2)
      return launch_residual_vec<T, 2>(partial, splits, split_stride, hidden, norm_w, eps, out, row_map,
                                       out_rows, hidden_size, threads, stream, ready);
    return launch_residual_vec<T, 4>(partial, splits, split_stride, hidden, norm_w, eps, out, row_map,
                                     out_rows, hidden_size, threads, stream, ready);
  }
  if (ready) return set_error(ORION_ERR_INTERNAL, "the scalar norm kernel counts no finished rows");
  const size_t smem = (size_t)hidden_size * sizeof(float);
  if (smem > 200 * 1024)
    return set_error(ORION_ERR_INTERNAL, "hidden size %u too large for the fused norm kernel",
                     hidden_size);
  if (smem > 48 * 1024)
    ORION_CUDA_CHECK("residual_rmsnorm attr",
                     cudaFuncSetAttribute(residual_rmsnorm_kernel<T>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  ORION_CUDA_CHECK("residual_rmsnorm",
                   launch_pdl(residual_rmsnorm_kernel<T>, dim3(out_rows), dim3(kNormThreads), smem, stream,
                              partial, splits, split_stride, hidden, norm_w, eps, out, row_map, hidden_size));
  return after_launch("residual_rmsnorm");
}

template <typename T>
int launch_rmsnorm_rows(const float *x, const float *norm_w, float eps, T *out, uint32_t rows,
                        uint32_t cols, cudaStream_t stream) {
  return launch_residual_rmsnorm<T>(nullptr, 0, 0, const_cast<float *>(x), norm_w, eps, out,
                                    nullptr, rows, cols, stream, nullptr);
}

template <typename T>
int launch_rope_kvwrite(const float *partial, uint32_t splits, size_t split_stride,
                        const float *bias, const uint32_t *positions, const uint32_t *slot_block,
                        const uint32_t *slot_slot, const float *rope_cos, const float *rope_sin,
                        T *q_out, T *arena, KvLayout kv, uint32_t layer, uint32_t rows,
                        uint32_t q_heads, cudaStream_t stream) {
  if (rows == 0) return ORION_OK;
  const uint32_t half = kv.head_dim / 2;
  const uint32_t total_heads = q_heads + 2 * kv.num_kv_heads;
  if (kv.head_dim % 8 == 0 && half / 4 <= 256 && 256 % (half / 4) == 0 && split_stride % 4 == 0) {
    const uint32_t heads_per_block = 256 / (half / 4);
    dim3 grid(rows, (total_heads + heads_per_block - 1) / heads_per_block);
    ORION_CUDA_CHECK("rope_kvwrite",
                     launch_pdl(rope_kvwrite_vec_kernel<T>, grid, dim3(256), 0, stream, partial, splits,
                                split_stride, bias, positions, slot_block, slot_slot, rope_cos, rope_sin,
                                q_out, arena, kv, layer, q_heads));
    return after_launch("rope_kvwrite");
  }
  const uint32_t threads = half >= 128 ? 128 : (half < 32 ? 32 : ((half + 31) / 32) * 32);
  dim3 grid(rows, total_heads);
  ORION_CUDA_CHECK("rope_kvwrite",
                   launch_pdl(rope_kvwrite_kernel<T>, grid, dim3(threads), 0, stream, partial, splits,
                              split_stride, bias, positions, slot_block, slot_slot, rope_cos, rope_sin, q_out,
                              arena, kv, layer, q_heads));
  return after_launch("rope_kvwrite");
}

template <typename T>
int launch_rope_rows(T *x, const uint32_t *positions, const float *rope_cos, const float *rope_sin,
                     uint32_t rows, uint32_t heads, uint32_t head_dim, cudaStream_t stream) {
  if (rows == 0 || heads == 0) return ORION_OK;
  rope_rows_kernel<T><<<dim3(rows, heads), 64, 0, stream>>>(x, positions, rope_cos, rope_sin, heads,
                                                            head_dim);
  return after_launch("rope");
}

template <typename T>
int launch_swiglu(const float *partial, uint32_t splits, size_t split_stride, T *act, uint32_t rows,
                  uint32_t ffn, cudaStream_t stream, bool interleaved) {
  if (rows == 0 || ffn == 0) return ORION_OK;
  if (ffn % 4 == 0 && split_stride % 4 == 0) {
    ORION_CUDA_CHECK("swiglu", launch_pdl(swiglu_vec_kernel<T>, dim3(grid_for((size_t)rows * ffn / 4, 256)),
                                          dim3(256), 0, stream, partial, splits, split_stride, act, rows, ffn, interleaved));
    return after_launch("swiglu");
  }
  ORION_CUDA_CHECK("swiglu", launch_pdl(swiglu_kernel<T>, dim3(grid_for((size_t)rows * ffn, 256)), dim3(256), 0,
                                        stream, partial, splits, split_stride, act, rows, ffn, interleaved));
  return after_launch("swiglu");
}

// dst[r * dst_stride + c] = src[r * cols + c]: spreads the rows of a contiguous matrix over a
// strided destination (the gate and up projections are stored row-interleaved).
template <typename T>
__global__ void copy_rows_strided_kernel(const T *__restrict__ src, T *__restrict__ dst, size_t rows, size_t cols,
                                         size_t dst_stride) {
  const size_t total = rows * cols;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
    dst[(idx / cols) * dst_stride + idx % cols] = src[idx];
}

template <typename T>
int launch_copy_rows_strided(const T *src, T *dst, size_t rows, size_t cols, size_t dst_stride, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return ORION_OK;
  copy_rows_strided_kernel<T><<<grid_for(rows * cols, 256), 256, 0, stream>>>(src, dst, rows, cols, dst_stride);
  return after_launch("copy_rows_strided");
}

int launch_finish_linear(const float *partial, uint32_t splits, size_t split_stride,
                         const float *bias, float *out, uint32_t rows, uint32_t n,
                         cudaStream_t stream) {
  if (rows == 0 || n == 0) return ORION_OK;
  ORION_CUDA_CHECK("finish_linear",
                   launch_pdl(finish_linear_kernel, dim3(grid_for((size_t)rows * n, 256)), dim3(256), 0, stream,
                              partial, splits, split_stride, bias, out, rows, n));
  return after_launch("finish_linear");
}

int launch_argmax(const float *logits, uint32_t rows, uint32_t cols, uint32_t *out,
                  cudaStream_t stream) {
  if (rows == 0) return ORION_OK;
  const uint32_t threads = cols >= 16384 ? 1024 : 256;
  ORION_CUDA_CHECK("argmax", launch_pdl(argmax_kernel, dim3(rows), dim3(threads), 0, stream, logits, cols, out));
  return after_launch("argmax");
}

template <typename T>
int launch_convert_from_f32(const float *src, T *dst, size_t n, cudaStream_t stream) {
  if (n == 0) return ORION_OK;
  convert_from_f32_kernel<T><<<grid_for(n, 256), 256, 0, stream>>>(src, dst, n);
  return after_launch("convert_from_f32");
}
template <typename T>
int launch_convert_to_f32(const T *src, float *dst, size_t n, cudaStream_t stream) {
  if (n == 0) return ORION_OK;
  convert_to_f32_kernel<T><<<grid_for(n, 256), 256, 0, stream>>>(src, dst, n);
  return after_launch("convert_to_f32");
}
int launch_f16_to_f32(const uint16_t *src, float *dst, size_t n, cudaStream_t stream) {
  if (n == 0) return ORION_OK;
  f16_to_f32_kernel<<<grid_for(n, 256), 256, 0, stream>>>(src, dst, n);
  return after_launch("f16_to_f32");
}

namespace {
template <typename T>
__global__ void gather_rows_kernel(const T *__restrict__ src, const uint32_t *__restrict__ row_map,
                                   T *__restrict__ dst, uint32_t cols) {
  pdl_trigger();
  pdl_wait();
  const T *s = src + (size_t)row_map[blockIdx.x] * cols;
  T *d = dst + (size_t)blockIdx.x * cols;
  for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) d[c] = s[c];
}
}  // namespace

template <typename T>
int launch_gather_rows(const T *src, const uint32_t *row_map, T *dst, uint32_t rows, uint32_t cols,
                       cudaStream_t stream) {
  if (rows == 0) return ORION_OK;
  ORION_CUDA_CHECK("gather_rows", launch_pdl(gather_rows_kernel<T>, dim3(rows), dim3(256), 0, stream, src, row_map,
                                             dst, cols));
  return after_launch("gather_rows");
}

template <typename T>
int launch_scale_convert(const float *src, T *dst, size_t n, float scale, cudaStream_t stream) {
  if (n == 0) return ORION_OK;
  scale_convert_kernel<T><<<grid_for(n, 256), 256, 0, stream>>>(src, dst, n, scale);
  return after_launch("scale_convert");
}

template <typename T>
int launch_arena_to_reference_order(const T *arena, KvLayout kv, float *out, cudaStream_t stream) {
  const size_t total = kv.layer_elems() * kv.num_layers;
  if (total == 0) return ORION_OK;
  arena_reorder_kernel<T, true><<<grid_for(total, 256), 256, 0, stream>>>(const_cast<T *>(arena),
                                                                          kv, out, total);
  return after_launch("arena_to_reference_order");
}
template <typename T>
int launch_arena_from_reference_order(const float *ref, KvLayout kv, T *arena,
                                      cudaStream_t stream) {
  const size_t total = kv.layer_elems() * kv.num_layers;
  if (total == 0) return ORION_OK;
  arena_reorder_kernel<T, false><<<grid_for(total, 256), 256, 0, stream>>>(
      arena, kv, const_cast<float *>(ref), total);
  return after_launch("arena_from_reference_order");
}

template <typename T>
int launch_fill_normal(T *dst, size_t n, uint64_t seed, cudaStream_t stream) {
  if (n == 0) return ORION_OK;
  fill_normal_kernel<T><<<grid_for((n + 1) / 2, 256), 256, 0, stream>>>(dst, n, seed);
  return after_launch("fill_normal");
}

#define ORION_INSTANTIATE(T)                                                                      \
  template int launch_embed_rmsnorm<T>(const T *, const uint32_t *, const float *, float, float *, \
                                       T *, uint32_t, uint32_t, cudaStream_t);                    \
  template int launch_residual_rmsnorm<T>(const float *, uint32_t, size_t, float *, const float *, \
                                          float, T *, const uint32_t *, uint32_t, uint32_t,       \
                                          cudaStream_t, uint32_t *);                              \
  template int launch_rmsnorm_rows<T>(const float *, const float *, float, T *, uint32_t,         \
                                      uint32_t, cudaStream_t);                                    \
  template int launch_rope_kvwrite<T>(const float *, uint32_t, size_t, const float *,             \
                                      const uint32_t *, const uint32_t *, const uint32_t *,       \
                                      const float *, const float *, T *, T *, KvLayout, uint32_t, \
                                      uint32_t, uint32_t, cudaStream_t);                          \
  template int launch_rope_rows<T>(T *, const uint32_t *, const float *, const float *, uint32_t, \
                                   uint32_t, uint32_t, cudaStream_t);                             \
  template int launch_copy_rows_strided<T>(const T *, T *, size_t, size_t, size_t, cudaStream_t);   \
  template int launch_swiglu<T>(const float *, uint32_t, size_t, T *, uint32_t, uint32_t,         \
                                cudaStream_t, bool);                                              \
  template int launch_convert_from_f32<T>(const float *, T *, size_t, cudaStream_t);              \
  template int launch_convert_to_f32<T>(const T *, float *, size_t, cudaStream_t);                \
  template int launch_arena_to_reference_order<T>(const T *, KvLayout, float *, cudaStream_t);    \
  template int launch_arena_from_reference_order<T>(const float *, KvLayout, T *, cudaStream_t);  \
  template int launch_scale_convert<T>(const float *, T *, size_t, float, cudaStream_t);           \
  template int launch_gather_rows<T>(const T *, const uint32_t *, T *, uint32_t, uint32_t, cudaStream_t); \
  template int launch_fill_normal<T>(T *, size_t, uint64_t, cudaStream_t);

ORION_INSTANTIATE(float)
ORION_INSTANTIATE(bf16)

}  // namespace orion
