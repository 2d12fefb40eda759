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
#ifdef LLMRS_DEBUG_CHECKS
  id = llmrs_checked(id, 0, vocab, 1, t, 0);
#endif
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

// The same, for rows whose length is a multiple of 4 and at most 4 * NORM_THREADS * CHUNKS:
// every thread loads all of its values (16 bytes at a time) before anything is stored,
// so the loads of a row are in flight together instead of one behind the other.
template <typename TA> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

template <typename TA, int CHUNKS>
__global__ void __launch_bounds__(NORM_THREADS)
add_rmsnorm_vec_kernel(float* __restrict__ h, const TA* __restrict__ delta, const float* __restrict__ weight,
                       TA* __restrict__ y, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x;
  const int src = rows ? rows[i] : i;
  float* hr = h + (size_t)src * hidden;
  const TA* dr = delta ? delta + (size_t)src * hidden : nullptr;
  float4 v[CHUNKS];
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k) {
    const int c = (k * NORM_THREADS + threadIdx.x) * 4;
    v[k] = c < hidden ? Vec4<float>::load(hr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (dr) {
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = (k * NORM_THREADS + threadIdx.x) * 4;
      if (c < hidden) {
        const float4 d = Vec4<TA>::load(dr + c);
        v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k) {
    const int c = (k * NORM_THREADS + threadIdx.x) * 4;
    ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    if (!rows && dr && c < hidden) Vec4<float>::store(hr + c, v[k]);
  }
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  TA* yr = y + (size_t)i * hidden;
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k) {
    const int c = (k * NORM_THREADS + threadIdx.x) * 4;
    if (c < hidden) {
      const float4 w = Vec4<float>::load(weight + c);
      Vec4<TA>::store(yr + c, make_float4(v[k].x * inv * w.x, v[k].y * inv * w.y, v[k].z * inv * w.z,
                                          v[k].w * inv * w.w));
    }
  }
}

template <typename TA>
static void launch_add_rmsnorm(float* h, const TA* delta, const float* weight, TA* y, const int* rows, int n_rows,
                               int hidden, float eps, cudaStream_t stream) {
  const int per_chunk = 4 * NORM_THREADS;
  if (hidden % 4 == 0 && hidden <= 8 * per_chunk) {
    if (hidden <= per_chunk)
      llmrs_launch(add_rmsnorm_vec_kernel<TA, 1>, dim3(n_rows), dim3(NORM_THREADS), 0, stream, true, h, delta, weight, y, rows,
                   hidden, eps);
    else if (hidden <= 2 * per_chunk)
      llmrs_launch(add_rmsnorm_vec_kernel<TA, 2>, dim3(n_rows), dim3(NORM_THREADS), 0, stream, true, h, delta, weight, y, rows,
                   hidden, eps);
    else if (hidden <= 4 * per_chunk)
      llmrs_launch(add_rmsnorm_vec_kernel<TA, 4>, dim3(n_rows), dim3(NORM_THREADS), 0, stream, true, h, delta, weight, y, rows,
                   hidden, eps);
    else
      llmrs_launch(add_rmsnorm_vec_kernel<TA, 8>, dim3(n_rows), dim3(NORM_THREADS), 0, stream, true, h, delta, weight, y, rows,
                   hidden, eps);
  } else {
    add_rmsnorm_kernel<TA><<<n_rows, NORM_THREADS, 0, stream>>>(h, delta, weight, y, rows, hidden, eps);
  }
}

LLMRS_API int llmrs_add_rmsnorm(float* h, const void* delta, const float* weight, void* y, const int* rows,
                                int n_rows, int hidden, float eps, int act_dtype, cudaStream_t stream) {
  LLMRS_REQUIRE(n_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes");
  if (n_rows == 0) return 0;
  if (act_dtype == LLMRS_F32)
    launch_add_rmsnorm<float>(h, (const float*)delta, weight, (float*)y, rows, n_rows, hidden, eps, stream);
  else if (act_dtype == LLMRS_BF16)
    launch_add_rmsnorm<__nv_bfloat16>(h, (const __nv_bfloat16*)delta, weight, (__nv_bfloat16*)y, rows, n_rows,
                                      hidden, eps, stream);
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
// out[t, c] = silu(gate(t, c)) * up(t, c); silu(x) = x * 1/(1+exp(-x)) in float32.
// (llm-core/src/backends/candle.rs:1645-1663: SiLU as x*sigmoid(x), then Mul.)
// gu holds gate and up in alternating runs of `block` columns: column c of the output has
// its gate at (c / block) * 2 * block + c % block and its up `block` columns further.
// block = inter is the plain layout [gate | up].
// ---------------------------------------------------------------------------------
template <typename TA>
__global__ void silu_mul_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int inter, int block, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / inter;
    const int c = (int)(i - t * inter);
    const size_t gcol = (size_t)(c / block) * 2 * block + c % block;
    const float g = to_float(gu[t * 2 * inter + gcol]);
    const float u = to_float(gu[t * 2 * inter + gcol + block]);
    const float s = g / (1.0f + expf(-g));
    out[i] = from_float<TA>(s * u);
  }
}

// Eight (bfloat16) or four (float32) columns per thread, 16 bytes per load, when the
// width allows; no division per element.
template <typename TA>
__global__ void silu_mul_vec_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int inter, int block,
                                    int n_tokens) {
  constexpr int PER = 16 / sizeof(TA);
  // One token per blockIdx.y, one 16-byte run of outputs per thread: no division by the row length.
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * PER;
  if (c >= inter) return;
  const int blk = c / block, r = c - blk * block;
  for (int t = blockIdx.y; t < n_tokens; t += gridDim.y) {
    const TA* gp = gu + (size_t)t * 2 * inter + (size_t)blk * 2 * block + r;
    float g[PER], u[PER];
#pragma unroll
    for (int k = 0; k < PER; k += 4) {
      const float4 a = Vec4<TA>::load(gp + k), b = Vec4<TA>::load(gp + block + k);
      g[k] = a.x; g[k + 1] = a.y; g[k + 2] = a.z; g[k + 3] = a.w;
      u[k] = b.x; u[k + 1] = b.y; u[k + 2] = b.z; u[k + 3] = b.w;
    }
#pragma unroll
    for (int k = 0; k < PER; ++k) g[k] = g[k] / (1.0f + expf(-g[k])) * u[k];
#pragma unroll
    for (int k = 0; k < PER; k += 4)
      Vec4<TA>::store(out + (size_t)t * inter + c + k, make_float4(g[k], g[k + 1], g[k + 2], g[k + 3]));
  }
}

template <typename TA>
static void launch_silu_mul(const TA* gu, TA* out, int n_tokens, int inter, int block, cudaStream_t stream) {
  constexpr int PER = 16 / sizeof(TA);
  const int threads = 256;
  if (inter % PER == 0 && block % PER == 0) {
    dim3 grid((inter / PER + threads - 1) / threads, n_tokens < 65535 ? n_tokens : 65535);
    silu_mul_vec_kernel<TA><<<grid, threads, 0, stream>>>(gu, out, inter, block, n_tokens);
  } else {
    const size_t total = (size_t)n_tokens * inter;
    const size_t want = (total + threads - 1) / threads;
    silu_mul_kernel<TA><<<(int)(want < 148 * 16 ? want : 148 * 16), threads, 0, stream>>>(gu, out, inter, block, total);
  }
}

LLMRS_API int llmrs_silu_mul(const void* gu, void* out, int n_tokens, int inter, int block, int act_dtype,
                             cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && inter > 0 && block > 0 && inter % block == 0,
                "silu_mul: bad sizes (width %d, runs of %d)", inter, block);
  if ((size_t)n_tokens * inter == 0) return 0;
  if (act_dtype == LLMRS_F32)
    launch_silu_mul<float>((const float*)gu, (float*)out, n_tokens, inter, block, stream);
  else if (act_dtype == LLMRS_BF16)
    launch_silu_mul<__nv_bfloat16>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n_tokens, inter, block, stream);
  else
    return llmrs_fail("silu_mul: unknown activation dtype %d", act_dtype);
  return llmrs_launch_status("silu_mul");
}

// ---------------------------------------------------------------------------------
// dst[dst_idx[i]] = src[src_idx[i]] for the pairs with dst_idx[i] >= 0: token ids that an
// earlier step sampled go into this step's input without a trip through the host.
// ---------------------------------------------------------------------------------
__global__ void scatter_tokens_kernel(int* __restrict__ dst, const int* __restrict__ dst_idx,
                                      const int* __restrict__ src, const int* __restrict__ src_idx, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && dst_idx[i] >= 0) dst[dst_idx[i]] = src[src_idx[i]];
}

LLMRS_API int llmrs_scatter_tokens(int* dst, const int* dst_idx, const int* src, const int* src_idx, int n,
                                   cudaStream_t stream) {
  LLMRS_REQUIRE(n >= 0, "scatter_tokens: bad size");
  if (n == 0) return 0;
  scatter_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(dst, dst_idx, src, src_idx, n);
  return llmrs_launch_status("scatter_tokens");
}
