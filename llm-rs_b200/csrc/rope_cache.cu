// Per-head RMSNorm of queries and keys, rotation by position, and the write of the new
// keys and values into the pages of the cache: one pass over the projection's output.
//
// Order and formulas: per-head norm over head_dim with a shared [head_dim] weight, before
// the rotation (llm-core/src/graph/builder.rs:123-153, llm-core/src/backends/attention.rs:70-97);
// rotation angles pos * theta^(-2i/d) (attention.rs:178-214), applied in the rotate-half
// pairing (x[i], x[i + r/2]) that the published Qwen3 weights assume, where the reference
// pairs (x[2i], x[2i+1]) (attention.rs:216-233); the new key and value go to page
// table[(cached+t)/P], slot (cached+t)%P (llm-core/src/backends/candle.rs:1440-1534).
// Norm and rotation run in float32 and the result is rounded once.
#include "common.cuh"

constexpr int ROPE_THREADS = 128;  // one warp per (token, head); grid.y covers the heads
constexpr int ROPE_WARPS = ROPE_THREADS / 32;

template <typename T>
__global__ void qk_norm_rope_kvwrite_kernel(
    T* __restrict__ q, long long q_stride,          // [n_tokens, n_q_heads*d], rotated in place
    const T* __restrict__ k, long long k_stride,    // [n_tokens, n_kv_heads*d] or null (reads another cache)
    const T* __restrict__ v, long long v_stride,
    const float* __restrict__ q_norm_w,             // [d] or null
    const float* __restrict__ k_norm_w,             // [d] or null
    const float* __restrict__ cos_sin,              // [max_pos, rotary_dim/2, 2] or null (no rotation)
    const int* __restrict__ positions,              // [n_tokens]
    const int* __restrict__ token_req,              // [n_tokens] row of the block table
    const int* __restrict__ block_table, int table_stride,
    T* __restrict__ cache,                          // [n_pages, n_kv_heads, 2, page_size, d]
    int n_q_heads, int n_kv_heads, int d, int rotary_dim, int page_size, float eps) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* x = smem + warp * d;
  const int pos = positions[t];
  const int half = rotary_dim / 2;
  const float* cs = cos_sin ? cos_sin + (size_t)pos * rotary_dim : nullptr;
  const int n_heads_total = n_q_heads + (k ? 2 * n_kv_heads : 0);

  for (int hh = blockIdx.y * ROPE_WARPS + warp; hh < n_heads_total; hh += gridDim.y * ROPE_WARPS) {
    // Which tensor this head belongs to.
    int kind, head;
    if (hh < n_q_heads) { kind = 0; head = hh; }
    else if (hh < n_q_heads + n_kv_heads) { kind = 1; head = hh - n_q_heads; }
    else { kind = 2; head = hh - n_q_heads - n_kv_heads; }
    const T* src = kind == 0 ? q + (size_t)t * q_stride + (size_t)head * d
                 : kind == 1 ? k + (size_t)t * k_stride + (size_t)head * d
                             : v + (size_t)t * v_stride + (size_t)head * d;
    T* dst;
    if (kind == 0) {
      dst = q + (size_t)t * q_stride + (size_t)head * d;
    } else {
      const int page = block_table[(size_t)token_req[t] * table_stride + pos / page_size];
      dst = cache + kv_tile_offset(page, head, kind - 1, n_kv_heads, page_size, d) + (size_t)(pos % page_size) * d;
    }
    if (kind == 2) {
      for (int i = lane; i < d; i += 32) dst[i] = src[i];
      continue;
    }
    const float* w = kind == 0 ? q_norm_w : k_norm_w;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float f = to_float(src[i]);
      x[i] = f;
      ss += f * f;
    }
    ss = warp_sum(ss);
    __syncwarp();
    const float inv = w ? 1.0f / sqrtf(ss / (float)d + eps) : 1.0f;
    for (int i = lane; i < d; i += 32) {
      float a = x[i] * inv * (w ? w[i] : 1.0f);
      if (cs && i < rotary_dim) {
        const int j = i < half ? i : i - half;
        const int pi = i < half ? i + half : i - half;
        const float b = x[pi] * inv * (w ? w[pi] : 1.0f);
        const float c = cs[2 * j], s = cs[2 * j + 1];
        a = i < half ? a * c - b * s : a * c + b * s;
      }
      dst[i] = from_float<T>(a);
    }
    __syncwarp();
  }
}

// The same for bfloat16 heads of 128 elements that are rotated whole (or not at all): a lane
// holds four consecutive elements (one 8-byte load), its partner in the rotation is lane ^ 16,
// nothing goes through shared memory.
__global__ void __launch_bounds__(ROPE_THREADS)
qk_norm_rope_kvwrite_d128_kernel(__nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ k,
                                 long long k_stride, const __nv_bfloat16* __restrict__ v, long long v_stride,
                                 const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                                 const float* __restrict__ cos_sin, const int* __restrict__ positions,
                                 const int* __restrict__ token_req, const int* __restrict__ block_table,
                                 int table_stride, __nv_bfloat16* __restrict__ cache, int n_q_heads, int n_kv_heads,
                                 int page_size, float eps) {
  constexpr int D = 128;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hh = blockIdx.y * ROPE_WARPS + warp;
  const int n_heads_total = n_q_heads + (k ? 2 * n_kv_heads : 0);
  if (hh >= n_heads_total) return;
  const int pos = positions[t];
  int kind, head;
  if (hh < n_q_heads) { kind = 0; head = hh; }
  else if (hh < n_q_heads + n_kv_heads) { kind = 1; head = hh - n_q_heads; }
  else { kind = 2; head = hh - n_q_heads - n_kv_heads; }
  const __nv_bfloat16* src = kind == 0 ? q + (size_t)t * q_stride + (size_t)head * D
                           : kind == 1 ? k + (size_t)t * k_stride + (size_t)head * D
                                       : v + (size_t)t * v_stride + (size_t)head * D;
  __nv_bfloat16* dst;
  if (kind == 0) {
    dst = q + (size_t)t * q_stride + (size_t)head * D;
  } else {
    const int page = block_table[(size_t)token_req[t] * table_stride + pos / page_size];
    dst = cache + kv_tile_offset(page, head, kind - 1, n_kv_heads, page_size, D) + (size_t)(pos % page_size) * D;
  }
  const uint2 raw = *reinterpret_cast<const uint2*>(src + lane * 4);
  if (kind == 2) {
    *reinterpret_cast<uint2*>(dst + lane * 4) = raw;
    return;
  }
  const float2 a01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 a23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  float x[4] = {a01.x, a01.y, a23.x, a23.y};
  const float* w = kind == 0 ? q_norm_w : k_norm_w;
  if (w) {
    const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
    const float inv = 1.0f / sqrtf(ss / (float)D + eps);
    const float4 wv = *reinterpret_cast<const float4*>(w + lane * 4);
    x[0] *= inv * wv.x; x[1] *= inv * wv.y; x[2] *= inv * wv.z; x[3] *= inv * wv.w;
  }
  if (cos_sin) {
    // Element i < 64 pairs with i + 64: lanes 0-15 hold the first half, lane ^ 16 the partner.
    const float* cs = cos_sin + (size_t)pos * D + (size_t)(lane & 15) * 8;   // (cos, sin) of 4 frequencies
    const float4 cs01 = *reinterpret_cast<const float4*>(cs), cs23 = *reinterpret_cast<const float4*>(cs + 4);
    const float c[4] = {cs01.x, cs01.z, cs23.x, cs23.z}, sn[4] = {cs01.y, cs01.w, cs23.y, cs23.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
      x[e] = lane < 16 ? x[e] * c[e] - other * sn[e] : x[e] * c[e] + other * sn[e];
    }
  }
  uint2 o;
  *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(x[0], x[1]);
  *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(x[2], x[3]);
  *reinterpret_cast<uint2*>(dst + lane * 4) = o;
}

LLMRS_API int llmrs_qk_norm_rope_kvwrite(void* q, long long q_stride, const void* k, long long k_stride,
                                         const void* v, long long v_stride, const float* q_norm_w,
                                         const float* k_norm_w, const float* cos_sin, const int* positions,
                                         const int* token_req, const int* block_table, int table_stride,
                                         void* cache, int n_tokens, int n_q_heads, int n_kv_heads, int d,
                                         int rotary_dim, int page_size, float eps, int dtype,
                                         cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && n_q_heads > 0 && n_kv_heads > 0 && d > 0 && page_size > 0,
                "qk_norm_rope_kvwrite: bad sizes");
  LLMRS_REQUIRE(rotary_dim >= 0 && rotary_dim <= d && rotary_dim % 2 == 0,
                "qk_norm_rope_kvwrite: rotary_dim %d must be even and at most head_dim %d", rotary_dim, d);
  LLMRS_REQUIRE(d <= 1024, "qk_norm_rope_kvwrite: head_dim %d above 1024 is not supported", d);
  if (n_tokens == 0) return 0;
  const size_t smem = (size_t)ROPE_WARPS * d * sizeof(float);
  const int heads_total = n_q_heads + (k ? 2 * n_kv_heads : 0);
  dim3 grid(n_tokens, (heads_total + ROPE_WARPS - 1) / ROPE_WARPS);
  const bool aligned8 = ((uintptr_t)q % 8 == 0) && q_stride % 4 == 0 && (!k || ((uintptr_t)k % 8 == 0 && k_stride % 4 == 0)) &&
                        (!v || ((uintptr_t)v % 8 == 0 && v_stride % 4 == 0));
  if (dtype == LLMRS_BF16 && d == 128 && (rotary_dim == 128 || rotary_dim == 0 || !cos_sin) && aligned8) {
    llmrs_launch(qk_norm_rope_kvwrite_d128_kernel, grid, dim3(ROPE_THREADS), 0, stream, true, (__nv_bfloat16*)q,
                 q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, q_norm_w, k_norm_w,
                 (rotary_dim == 128 ? cos_sin : (const float*)nullptr), positions, token_req, block_table, table_stride,
                 (__nv_bfloat16*)cache, n_q_heads, n_kv_heads, page_size, eps);
    return llmrs_launch_status("qk_norm_rope_kvwrite");
  }
  if (dtype == LLMRS_F32)
    llmrs_launch(qk_norm_rope_kvwrite_kernel<float>, grid, dim3(ROPE_THREADS), smem, stream, true,
        (float*)q, q_stride, (const float*)k, k_stride, (const float*)v, v_stride, q_norm_w, k_norm_w, cos_sin,
        positions, token_req, block_table, table_stride, (float*)cache, n_q_heads, n_kv_heads, d, rotary_dim,
        page_size, eps);
  else if (dtype == LLMRS_BF16)
    llmrs_launch(qk_norm_rope_kvwrite_kernel<__nv_bfloat16>, grid, dim3(ROPE_THREADS), smem, stream, true,
        (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, q_norm_w,
        k_norm_w, cos_sin, positions, token_req, block_table, table_stride, (__nv_bfloat16*)cache, n_q_heads,
        n_kv_heads, d, rotary_dim, page_size, eps);
  else
    return llmrs_fail("qk_norm_rope_kvwrite: unknown dtype %d", dtype);
  return llmrs_launch_status("qk_norm_rope_kvwrite");
}
