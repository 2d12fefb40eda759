// Next-token choice on the device: one block per row of float32 logits.
//
// Order of operations as in llm-core/src/sampler.rs:25-125: repetition penalty (divide a
// positive logit, multiply a negative one, once per distinct token of the history) ->
// greedy when temperature <= 1e-5 (first maximum wins, strict '>') -> divide by the
// temperature -> softmax -> keep the top_k most probable -> keep the smallest set of
// most probable tokens whose mass reaches top_p -> draw.
//
// Where the reference sorts and draws from an unseeded generator, this kernel finds
// the two cut-off values by bisection on the float bit pattern, keeps ties at a cut-off,
// and draws in vocabulary order with a Philox4x32-10 number keyed by (seed; request id,
// index of the generated token), so a request's tokens do not depend on what else is
// in the batch. The distribution drawn from is the reference's.
#include "common.cuh"

constexpr int SM_THREADS = 1024;

__device__ __host__ inline void philox4x32_10(uint32_t key0, uint32_t key1, uint32_t c0, uint32_t c1, uint32_t c2,
                                              uint32_t c3, uint32_t out[4]) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  for (int round = 0; round < 10; ++round) {
    const uint64_t p0 = (uint64_t)M0 * c0, p1 = (uint64_t)M1 * c2;
    const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
    const uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
    const uint32_t n0 = hi1 ^ c1 ^ key0, n1 = lo1, n2 = hi0 ^ c3 ^ key1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    key0 += W0; key1 += W1;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Uniform number in [0, 1) with 24 bits, for tests and the host-side plain sampler.
LLMRS_API float llmrs_philox_uniform(unsigned long long seed, unsigned long long request_id, unsigned int index) {
  uint32_t r[4];
  philox4x32_10((uint32_t)seed, (uint32_t)(seed >> 32), (uint32_t)request_id, (uint32_t)(request_id >> 32), index, 0u,
                r);
  return (float)(r[0] >> 8) * (1.0f / 16777216.0f);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  // Larger value wins; equal values: the lower index (the reference scans with strict '>').
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax a, ArgMax* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  __syncthreads();
  if (lane == 0) red[warp] = a;
  __syncthreads();
  if (warp == 0) {
    ArgMax t = lane < (blockDim.x >> 5) ? red[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax b;
      b.v = __shfl_xor_sync(0xffffffffu, t.v, o);
      b.i = __shfl_xor_sync(0xffffffffu, t.i, o);
      t = better(t, b);
    }
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// logits [n_rows, vocab] are changed in place (penalty, then exp(x - max)).
__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ penalty,
              const int* __restrict__ hist_tokens, const int* __restrict__ hist_offsets,
              const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ request_ids,
              const int* __restrict__ gen_index, int* __restrict__ out_tokens) {
  __shared__ float red[33];
  __shared__ ArgMax ared[33];
  __shared__ float scan[SM_THREADS];
  __shared__ int chosen;
  const int row = blockIdx.x, tid = threadIdx.x;
  float* x = logits + (size_t)row * vocab;

  const float pen = penalty ? penalty[row] : 1.0f;
  if (pen != 1.0f && hist_offsets) {
    for (int j = hist_offsets[row] + tid; j < hist_offsets[row + 1]; j += SM_THREADS) {
      const int idx = hist_tokens[j];  // distinct tokens: each index is touched once
      if (idx >= 0 && idx < vocab) {
        const float v = x[idx];
        x[idx] = v > 0.f ? v / pen : v * pen;
      }
    }
    __syncthreads();
  }

  const float T = temperature ? temperature[row] : 0.f;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = tid; i < vocab; i += SM_THREADS) best = better(best, ArgMax{x[i], i});
  best = block_argmax(best, ared);
  if (best.i >= vocab) best.i = 0;  // a row of NaN has no maximum
  if (T <= 1e-5f) {
    if (tid == 0) out_tokens[row] = best.i;
    return;
  }

  // e_i = exp(x_i / T - max / T); contiguous chunk per thread so that sums run in vocabulary order.
  const int chunk = (vocab + SM_THREADS - 1) / SM_THREADS;
  const int lo = min(tid * chunk, vocab), hi = min(lo + chunk, vocab);
  const float mx = best.v / T;
  float mass = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float e = expf(x[i] / T - mx);
    x[i] = e;
    mass += e;
  }
  __syncthreads();

  float cut = 0.f;  // keep e_i >= cut
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < vocab) {
    // Largest t with count(e >= t) >= k, by bisection on the bit pattern (e >= 0: bits are ordered).
    uint32_t lo_b = 0u, hi_b = 0x3f800000u;  // e lies in [0, 1]
    while (lo_b < hi_b) {
      const uint32_t mid = lo_b + (hi_b - lo_b + 1) / 2;
      const float t = __uint_as_float(mid);
      float cnt = 0.f;
      for (int i = lo; i < hi; ++i) cnt += x[i] >= t ? 1.f : 0.f;
      cnt = block_sum(cnt, red);
      if (cnt >= (float)k) lo_b = mid; else hi_b = mid - 1;
    }
    cut = __uint_as_float(lo_b);
    mass = 0.f;
    for (int i = lo; i < hi; ++i) mass += x[i] >= cut ? x[i] : 0.f;
  }
  float total = block_sum(mass, red);
  const float p = top_p ? top_p[row] : 1.0f;
  if (p < 1.0f) {
    // Largest t >= cut with mass(e >= t) >= p * total.
    const float need = p * total;
    uint32_t lo_b = __float_as_uint(cut), hi_b = 0x3f800000u;
    while (lo_b < hi_b) {
      const uint32_t mid = lo_b + (hi_b - lo_b + 1) / 2;
      const float t = __uint_as_float(mid);
      float ms = 0.f;
      for (int i = lo; i < hi; ++i) ms += x[i] >= t ? x[i] : 0.f;
      ms = block_sum(ms, red);
      if (ms >= need) lo_b = mid; else hi_b = mid - 1;
    }
    cut = __uint_as_float(lo_b);
    mass = 0.f;
    for (int i = lo; i < hi; ++i) mass += x[i] >= cut ? x[i] : 0.f;
    total = block_sum(mass, red);
  }

  // Draw: first index, in vocabulary order, whose running sum of kept e exceeds u * total.
  uint32_t r[4];
  const unsigned long long seed = seeds ? seeds[row] : 0ull, rid = request_ids ? request_ids[row] : 0ull;
  philox4x32_10((uint32_t)seed, (uint32_t)(seed >> 32), (uint32_t)rid, (uint32_t)(rid >> 32),
                gen_index ? (uint32_t)gen_index[row] : 0u, 0u, r);
  const float u = (float)(r[0] >> 8) * (1.0f / 16777216.0f);
  const float target = u * total;
  scan[tid] = mass;
  if (tid == 0) chosen = -1;
  __syncthreads();
  if (tid == 0) {
    // Serial scan over the 1024 chunk sums keeps the order of the additions fixed.
    float run = 0.f;
    int owner = -1;
    float before = 0.f;
    for (int t = 0; t < SM_THREADS; ++t) {
      const float next = run + scan[t];
      if (owner < 0 && next > target) { owner = t; before = run; }
      run = next;
    }
    if (owner < 0) {
      // Rounding left the target at or above the sum: the last chunk with kept mass owns it.
      for (int t = SM_THREADS - 1; t >= 0; --t)
        if (scan[t] > 0.f) { owner = t; break; }
      before = -1.f;
    }
    scan[0] = before;
    chosen = owner;  // chunk index for now
  }
  __syncthreads();
  const int owner = chosen;
  const float before = scan[0];
  __syncthreads();
  if (tid == owner) {
    int pick = -1, last_kept = -1;
    float run = before;
    for (int i = lo; i < hi; ++i) {
      if (x[i] >= cut && x[i] > 0.f) {
        last_kept = i;
        if (before >= 0.f) {
          run += x[i];
          if (run > target) { pick = i; break; }
        }
      }
    }
    // The loop ran to the chunk's end without a pick: rounding; take the chunk's last kept token.
    if (pick < 0) pick = last_kept >= 0 ? last_kept : best.i;
    out_tokens[row] = pick;
  }
  if (owner < 0 && tid == 0) out_tokens[row] = best.i;
}

LLMRS_API int llmrs_sample(float* logits, int n_rows, int vocab, const float* temperature, const int* top_k,
                           const float* top_p, const float* penalty, const int* hist_tokens,
                           const int* hist_offsets, const unsigned long long* seeds,
                           const unsigned long long* request_ids, const int* gen_index, int* out_tokens,
                           cudaStream_t stream) {
  LLMRS_REQUIRE(n_rows >= 0 && vocab > 0, "sample: bad sizes");
  if (n_rows == 0) return 0;
  sample_kernel<<<n_rows, SM_THREADS, 0, stream>>>(logits, vocab, temperature, top_k, top_p, penalty, hist_tokens,
                                                   hist_offsets, seeds, request_ids, gen_index, out_tokens);
  return llmrs_launch_status("sample");
}

// Greedy choice only: out[row] = index of the first maximum. Leaves the logits untouched.
__global__ void __launch_bounds__(SM_THREADS)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out_tokens) {
  __shared__ ArgMax ared[33];
  const float* x = logits + (size_t)blockIdx.x * vocab;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += SM_THREADS) best = better(best, ArgMax{x[i], i});
  best = block_argmax(best, ared);
  if (threadIdx.x == 0) out_tokens[blockIdx.x] = best.i < vocab ? best.i : 0;  // a row of NaN has no maximum
}

LLMRS_API int llmrs_argmax(const float* logits, int n_rows, int vocab, int* out_tokens, cudaStream_t stream) {
  LLMRS_REQUIRE(n_rows >= 0 && vocab > 0, "argmax: bad sizes");
  if (n_rows == 0) return 0;
  argmax_kernel<<<n_rows, SM_THREADS, 0, stream>>>(logits, vocab, out_tokens);
  return llmrs_launch_status("argmax");
}
