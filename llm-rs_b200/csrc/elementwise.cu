// Embedding gather, residual add fused with RMSNorm, and SiLU(gate)*up.
//
// The residual stream is float32 in both precisions: every sum into it and every norm
// statistic is computed in 32-bit; only the normed activations that feed a matrix
// product are rounded to the activation type.
#include "common.cuh"

// ---------------------------------------------------------------------------------
// Embedding: h[t, :] = table[id[t], :] widened to float32.
// (llm-core/src/backends/candle.rs:1238-1261: index_select on the table, no scale.)
// ---------------------------------------------------------------------------------
template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab) {
  const int t = blockIdx.x;
  int id = ids[t];
  // Ids are checked on the host; clamp all the same so that a bad id reads inside the table.
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const TW* row = table + (size_t)id * hidden;
  float* o = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]);
}

LLMRS_API int llmrs_embedding(const void* table, int table_dtype, const int* ids, float* out,
                              int n_tokens, int hidden, int vocab, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes");
  if (n_tokens == 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == LLMRS_F32)
    embedding_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)table, ids, out, hidden, vocab);
  else if (table_dtype == LLMRS_BF16)
    embedding_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>((const __nv_bfloat16*)table, ids, out,
                                                                       hidden, vocab);
  else
    return llmrs_fail("embedding: unknown table dtype %d", table_dtype);
  return llmrs_launch_status("embedding");
}

// ---------------------------------------------------------------------------------
// h += delta (optional); y = h / sqrt(mean(h^2) + eps) * w, rounded once to TA.
// Formula: llm-core/src/backends/attention.rs:55-68,98-104 (float32 statistics, plain
// weight, no 1+w). One block per row; the row is held in registers between the passes
// when it fits, else read again from h.
//
// With `rows` != nullptr the kernel reads row rows[i] of h and delta, writes y[i] and
// leaves h untouched (the final norm, which only the wanted positions need).
// ---------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;
constexpr int NORM_KEEP = 8;  // values per thread kept in registers

template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TA* __restrict__ delta,
                                   const float* __restrict__ weight, TA* __restrict__ y,
                                   const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float red[33];
  const int i = blockIdx.x;
  const int src = rows ? rows[i] : i;
  float* hr = h + (size_t)src * hidden;
  const TA* dr = delta ? delta + (size_t)src * hidden : nullptr;
  float keep[NORM_KEEP];
  float ss = 0.f;
  int n = 0;
  for (int c = threadIdx.x; c < hidden; c += NORM_THREADS, ++n) {
    float v = hr[c];
    if (dr) v += to_float(dr[c]);
    if (!rows && dr) hr[c] = v;
    if (n < NORM_KEEP) keep[n] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  TA* yr = y + (size_t)i * hidden;
  n = 0;
  for (int c = threadIdx.x; c < hidden; c += NORM_THREADS, ++n) {
    float v;
    if (n < NORM_KEEP) {
      v = keep[n];
    } else {
      v = hr[c];
      if (rows && dr) v += to_float(dr[c]);
    }
    yr[c] = from_float<TA>(v * inv * weight[c]);
  }
}

LLMRS_API int llmrs_add_rmsnorm(float* h, const void* delta, const float* weight, void* y, const int* rows,
                                int n_rows, int hidden, float eps, int act_dtype, cudaStream_t stream) {
  LLMRS_REQUIRE(n_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes");
  if (n_rows == 0) return 0;
  if (act_dtype == LLMRS_F32)
    add_rmsnorm_kernel<float><<<n_rows, NORM_THREADS, 0, stream>>>(h, (const float*)delta, weight, (float*)y, rows,
                                                                    hidden, eps);
  else if (act_dtype == LLMRS_BF16)
    add_rmsnorm_kernel<__nv_bfloat16><<<n_rows, NORM_THREADS, 0, stream>>>(
        h, (const __nv_bfloat16*)delta, weight, (__nv_bfloat16*)y, rows, hidden, eps);
  else
    return llmrs_fail("add_rmsnorm: unknown activation dtype %d", act_dtype);
  return llmrs_launch_status("add_rmsnorm");
}

// ---------------------------------------------------------------------------------
// h += delta without a norm (the last residual sum when no norm follows, and toy blocks).
// ---------------------------------------------------------------------------------
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ h, const TA* __restrict__ delta, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) h[i] += to_float(delta[i]);
}

LLMRS_API int llmrs_residual_add(float* h, const void* delta, long long n, int act_dtype, cudaStream_t stream) {
  LLMRS_REQUIRE(n >= 0, "residual_add: bad size");
  if (n == 0) return 0;
  const int threads = 256;
  const int blocks = (int)((n + threads - 1) / threads < 148 * 8 ? (n + threads - 1) / threads : 148 * 8);
  if (act_dtype == LLMRS_F32)
    residual_add_kernel<float><<<blocks, threads, 0, stream>>>(h, (const float*)delta, (size_t)n);
  else if (act_dtype == LLMRS_BF16)
    residual_add_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(h, (const __nv_bfloat16*)delta, (size_t)n);
  else
    return llmrs_fail("residual_add: unknown activation dtype %d", act_dtype);
  return llmrs_launch_status("residual_add");
}

// ---------------------------------------------------------------------------------
// out[t, c] = silu(gu[t, c]) * gu[t, inter + c]; silu(x) = x * 1/(1+exp(-x)) in float32.
// (llm-core/src/backends/candle.rs:1645-1663: SiLU as x*sigmoid(x), then Mul.)
// ---------------------------------------------------------------------------------
template <typename TA>
__global__ void silu_mul_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int inter, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / inter;
    const int c = (int)(i - t * inter);
    const float g = to_float(gu[t * 2 * inter + c]);
    const float u = to_float(gu[t * 2 * inter + inter + c]);
    const float s = g / (1.0f + expf(-g));
    out[i] = from_float<TA>(s * u);
  }
}

LLMRS_API int llmrs_silu_mul(const void* gu, void* out, int n_tokens, int inter, int act_dtype,
                             cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && inter > 0, "silu_mul: bad sizes");
  const size_t total = (size_t)n_tokens * inter;
  if (total == 0) return 0;
  const int threads = 256;
  const size_t want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (act_dtype == LLMRS_F32)
    silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, inter, total);
  else if (act_dtype == LLMRS_BF16)
    silu_mul_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                                                                    inter, total);
  else
    return llmrs_fail("silu_mul: unknown activation dtype %d", act_dtype);
  return llmrs_launch_status("silu_mul");
}
