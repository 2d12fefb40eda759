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
      const int page = LLMRS_CHECKED_PAGE(block_table[(size_t)token_req[t] * table_stride + pos / page_size], 2, t);
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

// The same for bfloat16 heads of 128 elements that are rotated whole (or not at all). Sixteen lanes
// hold a head (eight consecutive elements = one 16-byte load each; the partner in the rotation is
// lane ^ 8), so a warp works on two heads at a time, and it takes PASSES such pairs of one token one
// after the other with all their loads in flight together: the position, the page and the row of
// (cos, sin) are fetched once for all of them. A block walks tokens blockIdx.x, blockIdx.x + gridDim.x,
// ... Steps of few tokens take one pair per warp (more warps at once, a shorter chain each). Nothing
// goes through shared memory.
constexpr int D128_WARPS = 4;

template <int D128_PASSES>
__global__ void __launch_bounds__(D128_WARPS * 32)
qk_norm_rope_kvwrite_d128_kernel(__nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ k,
                                 long long k_stride, const __nv_bfloat16* __restrict__ v, long long v_stride,
                                 const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                                 const float* __restrict__ cos_sin, const int* __restrict__ positions,
                                 const int* __restrict__ token_req, const int* __restrict__ block_table,
                                 int table_stride, __nv_bfloat16* __restrict__ cache, int n_q_heads, int n_kv_heads,
                                 int page_size, float eps, int n_tokens) {
  constexpr int D = 128;
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 4, l16 = lane & 15;          // which head of the pair, and the lane's place in it
  const int n_heads_total = n_q_heads + (k ? 2 * n_kv_heads : 0);
  const int first = ((blockIdx.y * D128_WARPS + warp) * D128_PASSES) * 2 + sub;   // this half-warp's heads: first, first + 2, ...
  if (first - sub >= n_heads_total) return;
  for (int t = blockIdx.x; t < n_tokens; t += gridDim.x) {
  const int pos = positions[t];
  const size_t page_base = k ? (size_t)LLMRS_CHECKED_PAGE(block_table[(size_t)token_req[t] * table_stride + pos / page_size], 2, t) : 0;

  const __nv_bfloat16* src[D128_PASSES];
  __nv_bfloat16* dst[D128_PASSES];
  int kind[D128_PASSES];
  uint4 raw[D128_PASSES];
#pragma unroll
  for (int p = 0; p < D128_PASSES; ++p) {
    const int hh = first + 2 * p;
    kind[p] = -1;
    src[p] = q;
    dst[p] = q;
    if (hh < n_heads_total) {
      int head;
      if (hh < n_q_heads) { kind[p] = 0; head = hh; }
      else if (hh < n_q_heads + n_kv_heads) { kind[p] = 1; head = hh - n_q_heads; }
      else { kind[p] = 2; head = hh - n_q_heads - n_kv_heads; }
      src[p] = kind[p] == 0 ? q + (size_t)t * q_stride + (size_t)head * D
             : kind[p] == 1 ? k + (size_t)t * k_stride + (size_t)head * D
                            : v + (size_t)t * v_stride + (size_t)head * D;
      dst[p] = kind[p] == 0 ? q + (size_t)t * q_stride + (size_t)head * D
                            : cache + kv_tile_offset((int)page_base, head, kind[p] - 1, n_kv_heads, page_size, D) +
                                  (size_t)(pos % page_size) * D;
      raw[p] = *reinterpret_cast<const uint4*>(src[p] + l16 * 8);
    }
  }
  // (cos, sin) of this lane's eight frequencies: element i < 64 pairs with i + 64, lanes 0-7 of a head
  // hold the first half, lane ^ 8 the partner.
  float c[8], sn[8];
  if (cos_sin) {
    const float4* cs = reinterpret_cast<const float4*>(cos_sin + (size_t)pos * D + (size_t)(l16 & 7) * 16);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float4 x = cs[e];
      c[2 * e] = x.x; sn[2 * e] = x.y; c[2 * e + 1] = x.z; sn[2 * e + 1] = x.w;
    }
  }
#pragma unroll
  for (int p = 0; p < D128_PASSES; ++p) {
    // Both halves of the warp take every step together (the shuffles are warp-wide); a half without a
    // head, or with a head of V, computes on what it has and stores nothing of it.
    const bool live = kind[p] >= 0;
    if (kind[p] == 2) *reinterpret_cast<uint4*>(dst[p] + l16 * 8) = raw[p];
    float x[8];
    {
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[p]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = live ? __bfloat1622float2(h2[e]) : make_float2(0.f, 0.f);
        x[2 * e] = f.x; x[2 * e + 1] = f.y;
      }
    }
    const float* w = kind[p] == 0 ? q_norm_w : kind[p] == 1 ? k_norm_w : nullptr;
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // within the 16 lanes of a head
    if (w) {
      const float inv = 1.0f / sqrtf(ss / (float)D + eps);
      const float4 w0 = *reinterpret_cast<const float4*>(w + l16 * 8), w1 = *reinterpret_cast<const float4*>(w + l16 * 8 + 4);
      x[0] *= inv * w0.x; x[1] *= inv * w0.y; x[2] *= inv * w0.z; x[3] *= inv * w0.w;
      x[4] *= inv * w1.x; x[5] *= inv * w1.y; x[6] *= inv * w1.z; x[7] *= inv * w1.w;
    }
    if (cos_sin) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, x[e], 8);
        x[e] = l16 < 8 ? x[e] * c[e] - other * sn[e] : x[e] * c[e] + other * sn[e];
      }
    }
    if (kind[p] == 0 || kind[p] == 1) {
      uint4 o;
      __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
      *reinterpret_cast<uint4*>(dst[p] + l16 * 8) = o;
    }
  }
  }
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
  const bool aligned16 = ((uintptr_t)q % 16 == 0) && q_stride % 8 == 0 && (!k || ((uintptr_t)k % 16 == 0 && k_stride % 8 == 0)) &&
                         (!v || ((uintptr_t)v % 16 == 0 && v_stride % 8 == 0)) && (!cache || (uintptr_t)cache % 16 == 0);
  if (dtype == LLMRS_BF16 && d == 128 && (rotary_dim == 128 || rotary_dim == 0 || !cos_sin) && aligned16) {
    const float* cs = rotary_dim == 128 ? cos_sin : (const float*)nullptr;
    if (n_tokens <= 64) {
      const int per_block = D128_WARPS * 2;   // heads per block
      const dim3 grid128(n_tokens, (heads_total + per_block - 1) / per_block);
      llmrs_launch(qk_norm_rope_kvwrite_d128_kernel<1>, grid128, dim3(D128_WARPS * 32), 0, stream, true, (__nv_bfloat16*)q,
                   q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, q_norm_w, k_norm_w,
                   cs, positions, token_req, block_table, table_stride, (__nv_bfloat16*)cache, n_q_heads, n_kv_heads,
                   page_size, eps, n_tokens);
    } else {
      const int per_block = D128_WARPS * 3 * 2;
      const int gy = (heads_total + per_block - 1) / per_block;
      const int gx = n_tokens < 148 * 16 / gy ? n_tokens : 148 * 16 / gy;
      llmrs_launch(qk_norm_rope_kvwrite_d128_kernel<3>, dim3(gx > 0 ? gx : 1, gy), dim3(D128_WARPS * 32), 0, stream, true,
                   (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride,
                   q_norm_w, k_norm_w, cs, positions, token_req, block_table, table_stride, (__nv_bfloat16*)cache,
                   n_q_heads, n_kv_heads, page_size, eps, n_tokens);
    }
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
