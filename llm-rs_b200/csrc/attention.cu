// Attention over the paged cache, for every element type and head size (head_dim in
// steps of 16, any number of heads and groups).
//
//   prefill: 16 query tokens of one request against all keys they may see (earlier
//            portions from the cache plus their own causal part), online softmax. The
//            tile list names tiles of 64 queries; grid.z picks the quarter.
//   decode:  one query token per request; the keys are cut into splits of a fixed
//            number that run as separate blocks and are merged by a combine kernel.
//
// Scores, softmax and the weighted sum of values are float32. The mask is causal, with
// an optional window: query at position p sees keys p-window+1 .. p.
// Math: llm-core/src/backends/candle.rs:1587-1640 (head j of the keys serves query heads
// j*G .. j*G+G-1, scores scaled by 1/sqrt(d) after the product, -inf above the diagonal,
// softmax over keys, product with values).
#include "common.cuh"

// Tensor-core kernels for bfloat16 with head_dim <= 128 (attention_mma.cu).
int llmrs_attn_prefill_mma(const void* q, long long q_stride, void* out, long long out_stride, const void* cache,
                           const int* tiles, int n_tiles, const int* q_start, const int* n_new,
                           const int* cached_len, const int* block_table, int table_stride, int n_q_heads,
                           int n_kv_heads, int d, int page_size, int window, float scale, cudaStream_t stream);
int llmrs_attn_decode_split_mma(const void* q, long long q_stride, const void* cache, const int* dec_reqs, int n_dec,
                                const int* q_start, const int* cached_len, const int* block_table, int table_stride,
                                float* scratch, int max_splits, int split_keys, int n_q_heads, int n_kv_heads, int d,
                                int page_size, int window, float scale, void* out, long long out_stride,
                                int* counters, int cluster_merge, const L2Prefetch& next, cudaStream_t stream);

bool llmrs_attn_prefill_tc_supported(const void* q, long long q_stride, const void* cache, int d, int page_size,
                                     float scale);
int llmrs_attn_prefill_tc(const void* q, long long q_stride, int n_tokens, void* out, long long out_stride,
                          const void* cache, long long cache_rows, const int* tiles, int n_tiles, const int* q_start,
                          const int* n_new, const int* cached_len, const int* block_table, int table_stride,
                          int n_q_heads, int n_kv_heads, int page_size, int window, float scale, int* error_flag,
                          cudaStream_t stream);

// 1: bfloat16 also takes the generic kernels (tests compare the two implementations).
static int g_generic_only = 0;
LLMRS_API void llmrs_attention_generic_only(int on) { g_generic_only = on; }

// ---------------------------------------------------------------------------------
// Prefill
// ---------------------------------------------------------------------------------
constexpr int PF_BQ = 16;        // query rows per block
constexpr int PF_TILE = 64;      // query rows per entry of the tile list
constexpr int PF_BK = 32;        // keys per iteration
constexpr int PF_THREADS = 256;  // 16 threads per query row
constexpr int PF_MAX_DCHUNK = 16;  // head_dim / 16 <= 16  => head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(PF_THREADS)
attn_prefill_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                    const T* __restrict__ cache, const int* __restrict__ tiles,
                    const int* __restrict__ q_start, const int* __restrict__ n_new,
                    const int* __restrict__ cached_len, const int* __restrict__ block_table, int table_stride,
                    int n_q_heads, int n_kv_heads, int d, int page_size, int window, float scale) {
  extern __shared__ float smem[];
  float* Qs = smem;                       // [PF_BQ][d]
  float* Ks = Qs + PF_BQ * d;             // [PF_BK][d + 1]
  float* Vs = Ks + PF_BK * (d + 1);       // [PF_BK][d]
  float* Ps = Vs + PF_BK * d;             // [PF_BQ][PF_BK]

  const int tile = blockIdx.x, head = blockIdx.y;
  const int kvh = head / (n_q_heads / n_kv_heads);
  const int req = tiles[2 * tile], q_off = tiles[2 * tile + 1] + blockIdx.z * PF_BQ;
  if (q_off >= n_new[req]) return;
  const int rows = min(PF_BQ, n_new[req] - q_off);
  const int cached = cached_len[req];
  const int tok0 = q_start[req] + q_off;
  const int pos0 = cached + q_off;              // position of row 0
  const int kv_hi = pos0 + rows;                // keys [kv_lo, kv_hi)
  int kv_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  kv_lo = (kv_lo / page_size) * page_size;      // start on a page's edge; the mask cuts the rest
  const int* table = block_table + (size_t)req * table_stride;

  const int tid = threadIdx.x;
  const int r = tid >> 4, c = tid & 15;
  const int nd = d >> 4;  // columns of the output this thread owns: c + 16*j

  for (int i = tid; i < PF_BQ * d; i += PF_THREADS) {
    const int rr = i / d, cc = i - rr * d;
    Qs[i] = rr < rows ? to_float(q[(size_t)(tok0 + rr) * q_stride + (size_t)head * d + cc]) * scale : 0.f;
  }
  float acc[PF_MAX_DCHUNK];
#pragma unroll
  for (int j = 0; j < PF_MAX_DCHUNK; ++j) acc[j] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int my_pos = pos0 + r;

  for (int kb = kv_lo; kb < kv_hi; kb += PF_BK) {
    __syncthreads();
    for (int i = tid; i < PF_BK * d; i += PF_THREADS) {
      const int kk = i / d, cc = i - kk * d;
      const int key = kb + kk;
      float kf = 0.f, vf = 0.f;
      if (key < kv_hi) {
        const int page = LLMRS_CHECKED_PAGE(table[key / page_size], 3, key);
        const size_t base = kv_tile_offset(page, kvh, 0, n_kv_heads, page_size, d) + (size_t)(key % page_size) * d + cc;
        kf = to_float(cache[base]);
        vf = to_float(cache[base + (size_t)page_size * d]);
      }
      Ks[kk * (d + 1) + cc] = kf;
      Vs[kk * d + cc] = vf;
    }
    __syncthreads();
    // Scores of row r against keys c and c+16.
    float s[PF_BK / 16];
#pragma unroll
    for (int jj = 0; jj < PF_BK / 16; ++jj) {
      const int kk = c + 16 * jj;
      const int key = kb + kk;
      const float* qr = Qs + r * d;
      const float* kr = Ks + kk * (d + 1);
      float dot = 0.f;
      for (int e = 0; e < d; ++e) dot = fmaf(qr[e], kr[e], dot);
      const bool seen = r < rows && key < kv_hi && key <= my_pos && (window <= 0 || key > my_pos - window);
      s[jj] = seen ? dot : -INFINITY;
    }
    float bm = s[0];
#pragma unroll
    for (int jj = 1; jj < PF_BK / 16; ++jj) bm = fmaxf(bm, s[jj]);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o, 16));
    const float m_new = fmaxf(m, bm);
    float corr = 1.f, bs = 0.f;
    if (m_new > -INFINITY) {
      corr = expf(m - m_new);  // m = -inf gives 0
#pragma unroll
      for (int jj = 0; jj < PF_BK / 16; ++jj) {
        const float p = expf(s[jj] - m_new);
        Ps[r * PF_BK + c + 16 * jj] = p;
        bs += p;
      }
    } else {
#pragma unroll
      for (int jj = 0; jj < PF_BK / 16; ++jj) Ps[r * PF_BK + c + 16 * jj] = 0.f;
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) bs += __shfl_xor_sync(0xffffffffu, bs, o, 16);
    l = l * corr + bs;
    m = m_new;
    __syncwarp();  // the 16 threads of a row sit in one warp
    const float* pr = Ps + r * PF_BK;
#pragma unroll
    for (int j = 0; j < PF_MAX_DCHUNK; ++j) {
      if (j < nd) {
        float a = acc[j] * corr;
        const int col = c + 16 * j;
        for (int kk = 0; kk < PF_BK; ++kk) a = fmaf(pr[kk], Vs[kk * d + col], a);
        acc[j] = a;
      }
    }
  }
  if (r < rows) {
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* o = out + (size_t)(tok0 + r) * out_stride + (size_t)head * d;
#pragma unroll
    for (int j = 0; j < PF_MAX_DCHUNK; ++j)
      if (j < nd) o[c + 16 * j] = from_float<T>(acc[j] * inv);
  }
}

// `n_tokens` rows of q and out; `n_pages` pages in `cache`. `prefer_tc` = 1 asks for the tcgen05
// kernel (128-query blocks; worth it when the portions are long) where it applies: bfloat16,
// head_dim 128, pages of a multiple of 16 keys. That kernel's waits are bounded; a block that gives up
// writes 2 into *error_flag (an int of the caller's on the device; null: a word inside the library that
// llmrs_attention_tc_error reads).
LLMRS_API int llmrs_attn_prefill(const void* q, long long q_stride, void* out, long long out_stride,
                                 const void* cache, const int* tiles, int n_tiles, const int* q_start,
                                 const int* n_new, const int* cached_len, const int* block_table,
                                 int table_stride, int n_q_heads, int n_kv_heads, int d, int page_size,
                                 int window, float scale, int dtype, int n_tokens, int n_pages, int prefer_tc,
                                 int* error_flag, cudaStream_t stream) {
  LLMRS_REQUIRE(n_tiles >= 0 && n_q_heads > 0 && n_kv_heads > 0 && page_size > 0, "attn_prefill: bad sizes");
  LLMRS_REQUIRE(n_q_heads % n_kv_heads == 0, "attn_prefill: %d query heads are no multiple of %d key heads",
                n_q_heads, n_kv_heads);
  LLMRS_REQUIRE(d >= 16 && d % 16 == 0 && d <= 16 * PF_MAX_DCHUNK,
                "attn_prefill: head_dim %d must be a multiple of 16 between 16 and %d", d, 16 * PF_MAX_DCHUNK);
  if (n_tiles == 0) return 0;
  const size_t smem = (size_t)(PF_BQ * d + PF_BK * (d + 1) + PF_BK * d + PF_BQ * PF_BK) * sizeof(float);
  dim3 grid(n_tiles, n_q_heads, PF_TILE / PF_BQ);
  cudaError_t e;
  // (The tcgen05 kernel notes the list's 128-row tiles in shared memory: at most 8,192 entries.)
  if (dtype == LLMRS_BF16 && prefer_tc && !g_generic_only && n_tiles <= 8192 &&
      llmrs_attn_prefill_tc_supported(q, q_stride, cache, d, page_size, scale))
    return llmrs_attn_prefill_tc(q, q_stride, n_tokens, out, out_stride, cache,
                                 (long long)n_pages * n_kv_heads * 2 * page_size, tiles, n_tiles, q_start, n_new,
                                 cached_len, block_table, table_stride, n_q_heads, n_kv_heads, page_size, window, scale,
                                 error_flag, stream);
  if (dtype == LLMRS_BF16 && d <= 128 && !g_generic_only && scale > 0.f)
    return llmrs_attn_prefill_mma(q, q_stride, out, out_stride, cache, tiles, n_tiles, q_start, n_new, cached_len,
                                  block_table, table_stride, n_q_heads, n_kv_heads, d, page_size, window, scale,
                                  stream);
  if (dtype == LLMRS_F32) {
    e = cudaFuncSetAttribute(attn_prefill_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llmrs_fail("attn_prefill: shared memory %zu: %s", smem, cudaGetErrorString(e));
    attn_prefill_kernel<float><<<grid, PF_THREADS, smem, stream>>>(
        (const float*)q, q_stride, (float*)out, out_stride, (const float*)cache, tiles, q_start, n_new, cached_len,
        block_table, table_stride, n_q_heads, n_kv_heads, d, page_size, window, scale);
  } else if (dtype == LLMRS_BF16) {
    e = cudaFuncSetAttribute(attn_prefill_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return llmrs_fail("attn_prefill: shared memory %zu: %s", smem, cudaGetErrorString(e));
    attn_prefill_kernel<__nv_bfloat16><<<grid, PF_THREADS, smem, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)cache, tiles,
        q_start, n_new, cached_len, block_table, table_stride, n_q_heads, n_kv_heads, d, page_size, window, scale);
  } else {
    return llmrs_fail("attn_prefill: unknown dtype %d", dtype);
  }
  return llmrs_launch_status("attn_prefill");
}

// ---------------------------------------------------------------------------------
// Decode: split over keys, then combine.
// ---------------------------------------------------------------------------------
constexpr int DC_THREADS = 256;
constexpr int DC_HG = 8;  // query heads of one key head handled by one block

// Scratch of one (decode request, query head, split): m, l, then d floats of the
// unnormalised weighted sum of values.
__host__ __device__ inline size_t dc_part_stride(int d) { return (size_t)d + 2; }

template <typename T, int VEC>
__global__ void __launch_bounds__(DC_THREADS)
attn_decode_split_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ cache,
                         const int* __restrict__ dec_reqs, const int* __restrict__ q_start,
                         const int* __restrict__ cached_len, const int* __restrict__ block_table,
                         int table_stride, float* __restrict__ part, int max_splits, int split_keys,
                         int n_q_heads, int n_kv_heads, int d, int page_size, int window, float scale) {
  extern __shared__ float smem[];
  const int G = n_q_heads / n_kv_heads;
  const int groups_per_kv = (G + DC_HG - 1) / DC_HG;
  const int di = blockIdx.x;
  const int kvh = blockIdx.y / groups_per_kv;
  const int g0 = (blockIdx.y % groups_per_kv) * DC_HG;
  const int ng = min(DC_HG, G - g0);
  const int split = blockIdx.z;
  const int req = dec_reqs[di];
  const int kv_len = cached_len[req] + 1;  // the new token's key is already in the cache
  const int kv_lo = window > 0 ? max(0, kv_len - window) : 0;
  const int k_begin = max(split * split_keys, kv_lo);
  const int k_end = min((split + 1) * split_keys, kv_len);
  if (k_begin >= k_end) return;
  const int nk = k_end - k_begin;
  const int* table = block_table + (size_t)req * table_stride;
  const int tid = threadIdx.x;

  float* Qs = smem;                        // [DC_HG][d], scaled
  float* Ss = Qs + DC_HG * d;              // [DC_HG][split_keys]
  float* Rs = Ss + DC_HG * split_keys;     // reduction: [subsets][DC_HG][d]
  __shared__ float row_m[DC_HG], row_l[DC_HG];

  const int tok = q_start[req];
  for (int i = tid; i < ng * d; i += DC_THREADS) {
    const int g = i / d, e = i - g * d;
    Qs[g * d + e] = to_float(q[(size_t)tok * q_stride + (size_t)(kvh * G + g0 + g) * d + e]) * scale;
  }
  __syncthreads();

  // Phase 1: scores. TPK threads share one key; each reads VEC elements at a time.
  const int nvec = d / VEC;
  int tpk = 1;
  while (tpk < 8 && nvec % (tpk * 2) == 0) tpk *= 2;
  const int sub = tid % tpk, kslot = tid / tpk, kstep = DC_THREADS / tpk;
  // Every thread runs the same number of rounds: the shuffles below need the whole warp.
  for (int kbase = 0; kbase < nk; kbase += kstep) {
    const int kk = kbase + kslot;
    const bool live = kk < nk;
    const int key = k_begin + (live ? kk : 0);
    const int page = LLMRS_CHECKED_PAGE(table[key / page_size], 3, key);
    const T* kr = cache + kv_tile_offset(page, kvh, 0, n_kv_heads, page_size, d) + (size_t)(key % page_size) * d;
    float dot[DC_HG];
#pragma unroll
    for (int g = 0; g < DC_HG; ++g) dot[g] = 0.f;
    for (int vi = sub; live && vi < nvec; vi += tpk) {
      float kf[VEC];
      if constexpr (sizeof(T) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4*>(kr + vi * VEC);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < VEC / 2; ++e) {
          const float2 f = __bfloat1622float2(p2[e]);
          kf[2 * e] = f.x;
          kf[2 * e + 1] = f.y;
        }
      } else {
        const float4 raw = *reinterpret_cast<const float4*>(kr + vi * VEC);
        kf[0] = raw.x; kf[1] = raw.y; kf[2] = raw.z; kf[3] = raw.w;
      }
#pragma unroll
      for (int g = 0; g < DC_HG; ++g) {
        if (g < ng) {
          const float* qg = Qs + g * d + vi * VEC;
#pragma unroll
          for (int e = 0; e < VEC; ++e) dot[g] = fmaf(qg[e], kf[e], dot[g]);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < DC_HG; ++g) {
      float v = dot[g];
      for (int o = tpk >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (live && sub == 0 && g < ng) Ss[g * split_keys + kk] = v;
    }
  }
  __syncthreads();

  // Phase 2: softmax over this split, one warp per head.
  const int warp = tid >> 5, lane = tid & 31;
  for (int g = warp; g < ng; g += DC_THREADS / 32) {
    float* sr = Ss + g * split_keys;
    float mx = -INFINITY;
    for (int kk = lane; kk < nk; kk += 32) mx = fmaxf(mx, sr[kk]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int kk = lane; kk < nk; kk += 32) {
      const float p = expf(sr[kk] - mx);
      sr[kk] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    if (lane == 0) { row_m[g] = mx; row_l[g] = sum; }
  }
  __syncthreads();

  // Phase 3: weighted sum of values. tpr threads cover one value row (4 elements each);
  // the key range is dealt out to the row groups ("subsets") and reduced afterwards.
  const int tpr = d / 4;
  const int n_sub = DC_THREADS / tpr;
  const int my_sub = tid / tpr, col = (tid % tpr) * 4;
  float acc[DC_HG][4];
#pragma unroll
  for (int g = 0; g < DC_HG; ++g) acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
  if (my_sub < n_sub) {
    for (int kk = my_sub; kk < nk; kk += n_sub) {
      const int key = k_begin + kk;
      const int page = LLMRS_CHECKED_PAGE(table[key / page_size], 3, key);
      const T* vr = cache + kv_tile_offset(page, kvh, 1, n_kv_heads, page_size, d) + (size_t)(key % page_size) * d + col;
      float vf[4];
      if constexpr (sizeof(T) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(vr);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(p2[0]), b = __bfloat1622float2(p2[1]);
        vf[0] = a.x; vf[1] = a.y; vf[2] = b.x; vf[3] = b.y;
      } else {
        const float4 raw = *reinterpret_cast<const float4*>(vr);
        vf[0] = raw.x; vf[1] = raw.y; vf[2] = raw.z; vf[3] = raw.w;
      }
#pragma unroll
      for (int g = 0; g < DC_HG; ++g) {
        if (g < ng) {
          const float p = Ss[g * split_keys + kk];
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[g][e] = fmaf(p, vf[e], acc[g][e]);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < DC_HG; ++g) {
      if (g < ng) {
        float* rr = Rs + ((size_t)my_sub * DC_HG + g) * d + col;
        rr[0] = acc[g][0]; rr[1] = acc[g][1]; rr[2] = acc[g][2]; rr[3] = acc[g][3];
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < ng * d; i += DC_THREADS) {
    const int g = i / d, e = i - g * d;
    float s = 0.f;
    for (int sb = 0; sb < n_sub; ++sb) s += Rs[((size_t)sb * DC_HG + g) * d + e];
    const int head = kvh * G + g0 + g;
    float* pp = part + ((size_t)((size_t)di * n_q_heads + head) * max_splits + split) * dc_part_stride(d);
    pp[2 + e] = s;
    if (e == 0) { pp[0] = row_m[g]; pp[1] = row_l[g]; }
  }
}

template <typename T>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part, T* __restrict__ out, long long out_stride,
                                           const int* __restrict__ dec_reqs, const int* __restrict__ q_start,
                                           const int* __restrict__ cached_len, int max_splits, int split_keys,
                                           int n_q_heads, int d, int window) {
  pdl_launch_dependents();
  pdl_wait();
  const int di = blockIdx.x, head = blockIdx.y;
  const int req = dec_reqs[di];
  const int kv_len = cached_len[req] + 1;
  const int kv_lo = window > 0 ? max(0, kv_len - window) : 0;
  const int s_first = kv_lo / split_keys, s_last = (kv_len - 1) / split_keys;
  const float* base = part + ((size_t)((size_t)di * n_q_heads + head) * max_splits) * dc_part_stride(d);
  float m = -INFINITY;
  for (int s = s_first; s <= s_last; ++s) m = fmaxf(m, base[(size_t)s * dc_part_stride(d)]);
  float l = 0.f;
  for (int s = s_first; s <= s_last; ++s) {
    const float* pp = base + (size_t)s * dc_part_stride(d);
    l += pp[1] * expf(pp[0] - m);
  }
  const float inv = 1.0f / l;
  T* o = out + (size_t)q_start[req] * out_stride + (size_t)head * d;
  for (int e = threadIdx.x; e < d; e += blockDim.x) {
    float a = 0.f;
    for (int s = s_first; s <= s_last; ++s) {
      const float* pp = base + (size_t)s * dc_part_stride(d);
      a += pp[2 + e] * expf(pp[0] - m);
    }
    o[e] = from_float<T>(a * inv);
  }
}

// Number of floats of scratch that llmrs_attn_decode needs (the splits' records).
LLMRS_API long long llmrs_attn_decode_scratch_floats(int n_dec, int n_q_heads, int d, int max_splits) {
  return (long long)n_dec * n_q_heads * max_splits * (long long)dc_part_stride(d);
}

template <typename T, int VEC>
static int launch_decode(const void* q, long long q_stride, void* out, long long out_stride, const void* cache,
                         const int* dec_reqs, int n_dec, const int* q_start, const int* cached_len,
                         const int* block_table, int table_stride, float* scratch, int max_splits, int split_keys,
                         int n_q_heads, int n_kv_heads, int d, int page_size, int window, float scale,
                         cudaStream_t stream) {
  const int G = n_q_heads / n_kv_heads;
  const int groups_per_kv = (G + DC_HG - 1) / DC_HG;
  const int tpr = d / 4;
  const int n_sub = DC_THREADS / tpr;
  const size_t smem = ((size_t)DC_HG * d + (size_t)DC_HG * split_keys + (size_t)n_sub * DC_HG * d) * sizeof(float);
  LLMRS_REQUIRE(smem <= 200 * 1024, "attn_decode: %zu bytes of shared memory needed (split of %d keys)", smem,
                split_keys);
  static size_t configured = 0;  // per instantiation; raised only when a launch needs more
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_split_kernel<T, VEC>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return llmrs_fail("attn_decode: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  dim3 grid(n_dec, n_kv_heads * groups_per_kv, max_splits);
  attn_decode_split_kernel<T, VEC><<<grid, DC_THREADS, smem, stream>>>(
      (const T*)q, q_stride, (const T*)cache, dec_reqs, q_start, cached_len, block_table, table_stride, scratch,
      max_splits, split_keys, n_q_heads, n_kv_heads, d, page_size, window, scale);
  int rc = llmrs_launch_status("attn_decode_split");
  if (rc) return rc;
  dim3 cgrid(n_dec, n_q_heads);
  llmrs_launch(attn_decode_combine_kernel<T>, cgrid, dim3(128), 0, stream, true, (const float*)scratch, (T*)out,
               out_stride, dec_reqs, q_start, cached_len, max_splits, split_keys, n_q_heads, d, window);
  return llmrs_launch_status("attn_decode_combine");
}

// Decode attention for the requests listed in dec_reqs (one new token each, whose key
// and value are already written). `max_splits` * `split_keys` must cover the longest
// request; `scratch` holds llmrs_attn_decode_scratch_floats() floats. `counters` is either
// null (the splits are merged by a second kernel) or n_dec * n_q_heads ints that are zero
// when the call starts: the tensor-core kernel then merges the splits itself, in the
// block that finishes last, and leaves the counters at zero.
LLMRS_API int llmrs_attn_decode(const void* q, long long q_stride, void* out, long long out_stride,
                                const void* cache, const int* dec_reqs, int n_dec, const int* q_start,
                                const int* cached_len, const int* block_table, int table_stride, float* scratch,
                                int* counters, int max_splits, int split_keys, int n_q_heads, int n_kv_heads,
                                int d, int page_size, int window, float scale, int dtype, cudaStream_t stream) {
  LLMRS_REQUIRE(n_dec >= 0 && n_q_heads > 0 && n_kv_heads > 0 && page_size > 0 && max_splits > 0 && split_keys > 0,
                "attn_decode: bad sizes");
  LLMRS_REQUIRE(n_q_heads % n_kv_heads == 0, "attn_decode: %d query heads are no multiple of %d key heads",
                n_q_heads, n_kv_heads);
  LLMRS_REQUIRE(d >= 16 && d % 16 == 0 && d <= 1024, "attn_decode: head_dim %d must be a multiple of 16 up to 1024", d);
  const L2Prefetch next = llmrs_take_next_prefetch();   // for the tensor-core kernel; the others drop it
  if (n_dec == 0) return 0;
  if (dtype == LLMRS_F32)
    return launch_decode<float, 4>(q, q_stride, out, out_stride, cache, dec_reqs, n_dec, q_start, cached_len,
                                   block_table, table_stride, scratch, max_splits, split_keys, n_q_heads, n_kv_heads,
                                   d, page_size, window, scale, stream);
  if (dtype == LLMRS_BF16 && d <= 128 && !g_generic_only && scale > 0.f) {
    if (counters == nullptr && max_splits <= 16)  // the splits merge inside the kernel, as a cluster
      return llmrs_attn_decode_split_mma(q, q_stride, cache, dec_reqs, n_dec, q_start, cached_len, block_table,
                                         table_stride, scratch, max_splits, split_keys, n_q_heads, n_kv_heads, d,
                                         page_size, window, scale, out, out_stride, nullptr, 1, next, stream);
    if (counters == nullptr) {
      int rc = llmrs_attn_decode_split_mma(q, q_stride, cache, dec_reqs, n_dec, q_start, cached_len, block_table,
                                           table_stride, scratch, max_splits, split_keys, n_q_heads, n_kv_heads, d,
                                           page_size, window, scale, out, out_stride, nullptr, 0, next, stream);
      if (rc) return rc;
      dim3 cgrid(n_dec, n_q_heads);
      llmrs_launch(attn_decode_combine_kernel<__nv_bfloat16>, cgrid, dim3(128), 0, stream, true,
                   (const float*)scratch, (__nv_bfloat16*)out, out_stride, dec_reqs, q_start, cached_len, max_splits,
                   split_keys, n_q_heads, d, window);
      return llmrs_launch_status("attn_decode_combine");
    }
    return llmrs_attn_decode_split_mma(q, q_stride, cache, dec_reqs, n_dec, q_start, cached_len, block_table,
                                       table_stride, scratch, max_splits, split_keys, n_q_heads, n_kv_heads, d,
                                       page_size, window, scale, out, out_stride, counters, 0, next, stream);
  }
  if (dtype == LLMRS_BF16)
    return launch_decode<__nv_bfloat16, 8>(q, q_stride, out, out_stride, cache, dec_reqs, n_dec, q_start, cached_len,
                                           block_table, table_stride, scratch, max_splits, split_keys, n_q_heads,
                                           n_kv_heads, d, page_size, window, scale, stream);
  return llmrs_fail("attn_decode: unknown dtype %d", dtype);
}
