// True 32-bit matrix product for the float32 path: out[m, n] = sum_k x[m, k] * w[n, k] (+ bias[n]).
//
// FFMA on the CUDA cores, no tensor-core mode of reduced precision. Every output
// element is summed over k in the same order whatever M is, so a token's result does
// not depend on what else is in the batch. The reference's products are library calls
// (llm-core/src/backends/candle.rs:1276-1340: weight [out, in], used transposed,
// optional bias added after).
#include "common.cuh"

constexpr int GF_BM = 64, GF_BN = 64, GF_BK = 16, GF_THREADS = 256;

__global__ void __launch_bounds__(GF_THREADS)
gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                float* __restrict__ out, int M, int N, int K, long long x_stride, long long out_stride) {
  __shared__ float As[GF_BK][GF_BM + 4];
  __shared__ float Bs[GF_BK][GF_BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
  const int tr = tid / 16, tc = tid % 16;  // this thread's 4x4 block: rows tr*4.., cols tc*4..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // Each thread loads 4 consecutive k of one row of each tile.
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += GF_BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int m = m0 + lrow, n = n0 + lrow;
      As[lk + e][lrow] = (m < M && k < K) ? x[(size_t)m * x_stride + k] : 0.f;
      Bs[lk + e][lrow] = (n < N && k < K) ? w[(size_t)n * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GF_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][tr * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tc * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + tr * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tc * 4 + j;
      if (n < N) out[(size_t)m * out_stride + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

LLMRS_API int llmrs_gemm_f32(const float* x, long long x_stride, const float* w, const float* bias, float* out,
                             long long out_stride, int M, int N, int K, cudaStream_t stream) {
  LLMRS_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
  if (M == 0) return 0;
  dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
  LLMRS_REQUIRE(grid.y <= 65535, "gemm_f32: M=%d is too large", M);
  gemm_f32_kernel<<<grid, GF_THREADS, 0, stream>>>(x, w, bias, out, M, N, K, x_stride, out_stride);
  return llmrs_launch_status("gemm_f32");
}
