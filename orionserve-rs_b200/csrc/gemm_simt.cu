// SIMT GEMM  out[r][n] = sum_k x[r][k] * w[n][k]  (tensor.rs:114-128 without bias).
//
// This is the arithmetic of the f32 correctness build and the fallback for bf16
// shapes the tensor-core kernel does not take (K not a multiple of 8, unaligned
// rows). Every output element is accumulated by ONE thread with k ascending;
// for f32 storage the multiply and the add are rounded separately (no FMA), so
// the result equals the reference's `acc += a * b` loop bit for bit.
#include "kernels.h"

namespace orion {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T>
__device__ __forceinline__ float mac(float acc, float a, float b);
template <>
__device__ __forceinline__ float mac<float>(float acc, float a, float b) {
  return __fadd_rn(acc, __fmul_rn(a, b));
}
template <>
__device__ __forceinline__ float mac<bf16>(float acc, float a, float b) {
  return fmaf(a, b, acc);
}

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T *__restrict__ x, uint32_t ldx, const T *__restrict__ w, uint32_t ldw,
                 float *__restrict__ out, uint32_t M, uint32_t N, uint32_t K) {
  __shared__ float xs[BK][BM + 1];
  __shared__ float ws[BK][BN + 1];
  pdl_trigger();
  pdl_wait();
  const uint32_t m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const uint32_t tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // tx -> n, ty -> m
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  for (uint32_t k0 = 0; k0 < K; k0 += BK) {
    for (uint32_t idx = threadIdx.x; idx < BM * BK; idx += 256) {
      const uint32_t r = idx / BK, kk = idx % BK;
      const uint32_t gm = m0 + r, gk = k0 + kk;
      xs[kk][r] = (gm < M && gk < K) ? to_f32<T>(x[(size_t)gm * ldx + gk]) : 0.0f;
    }
    for (uint32_t idx = threadIdx.x; idx < BN * BK; idx += 256) {
      const uint32_t r = idx / BK, kk = idx % BK;
      const uint32_t gn = n0 + r, gk = k0 + kk;
      ws[kk][r] = (gn < N && gk < K) ? to_f32<T>(w[(size_t)gn * ldw + gk]) : 0.0f;
    }
    __syncthreads();
    const uint32_t kmax = min((uint32_t)BK, K - k0);  // never accumulate padded k (keeps -0.0 exact)
    for (uint32_t kk = 0; kk < kmax; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = mac<T>(acc[i][j], a[i], b[j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const uint32_t gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const uint32_t gn = n0 + tx * TN + j;
      if (gn < N) out[(size_t)gm * N + gn] = acc[i][j];
    }
  }
}

}  // namespace

template <typename T>
int launch_gemm_simt(const T *x, uint32_t ldx, const T *w, uint32_t ldw, float *out, uint32_t rows,
                     uint32_t n, uint32_t k, cudaStream_t stream) {
  if (rows == 0 || n == 0) return ORION_OK;
  dim3 grid((n + BN - 1) / BN, (rows + BM - 1) / BM);
  ORION_CUDA_CHECK("gemm_simt", launch_pdl(gemm_simt_kernel<T>, grid, dim3(256), 0, stream, x, ldx, w, ldw, out,
                                           rows, n, k));
  count_launch();
  ORION_CUDA_CHECK("gemm_simt", cudaGetLastError());
  return ORION_OK;
}
template int launch_gemm_simt<float>(const float *, uint32_t, const float *, uint32_t, float *,
                                     uint32_t, uint32_t, uint32_t, cudaStream_t);
template int launch_gemm_simt<bf16>(const bf16 *, uint32_t, const bf16 *, uint32_t, float *,
                                    uint32_t, uint32_t, uint32_t, cudaStream_t);

}  // namespace orion
