// Next-token choice on the device: one block per row of float32 logits.
//
// Order of operations as in llm-core/src/sampler.rs:25-125: repetition penalty (divide a
// positive logit, multiply a negative one, once per distinct token of the history) ->
// greedy when temperature <= 1e-5 (first maximum wins, strict '>') -> divide by the
// temperature -> softmax -> keep the top_k most probable -> keep the smallest set of
// most probable tokens whose mass reaches top_p -> draw.
//
// Where the reference sorts and draws from an unseeded generator, this kernel finds
// the two cut-off values digit by digit on the float bit pattern, keeps ties at a cut-off,
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

// Calls f(index, value) for every element of a row, the block's threads striding over it; four
// elements per load when the row allows it (every row then starts on a 16-byte boundary).
template <typename F>
__device__ __forceinline__ void for_each_elem(const float* __restrict__ x, int vocab, F&& f) {
  if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    // Four loads in flight per thread: one block reads the whole row, and with a single load per
    // thread it waits for the memory's latency on every step.
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const int n4 = vocab / 4, bd = blockDim.x;
    int i = threadIdx.x;
    for (; i + 3 * bd < n4; i += 4 * bd) {
      const float4 v0 = x4[i], v1 = x4[i + bd], v2 = x4[i + 2 * bd], v3 = x4[i + 3 * bd];
      f(4 * i, v0.x); f(4 * i + 1, v0.y); f(4 * i + 2, v0.z); f(4 * i + 3, v0.w);
      f(4 * (i + bd), v1.x); f(4 * (i + bd) + 1, v1.y); f(4 * (i + bd) + 2, v1.z); f(4 * (i + bd) + 3, v1.w);
      f(4 * (i + 2 * bd), v2.x); f(4 * (i + 2 * bd) + 1, v2.y); f(4 * (i + 2 * bd) + 2, v2.z); f(4 * (i + 2 * bd) + 3, v2.w);
      f(4 * (i + 3 * bd), v3.x); f(4 * (i + 3 * bd) + 1, v3.y); f(4 * (i + 3 * bd) + 2, v3.z); f(4 * (i + 3 * bd) + 3, v3.w);
    }
    for (; i < n4; i += bd) {
      const float4 v = x4[i];
      f(4 * i, v.x); f(4 * i + 1, v.y); f(4 * i + 2, v.z); f(4 * i + 3, v.w);
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) f(i, x[i]);
  }
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

// ---- selection of a cut-off value by digits ------------------------------------------------
// The values e are floats in [0, 1], whose bit patterns are ordered like the values. A cut-off is
// found digit by digit (11, 11 and 8 bits, highest first): one pass over the row builds a histogram
// of the current digit among the values that share the digits found so far, and the digit is the
// highest bin at which the running total from the top reaches what is asked: a number of values
// (top_k) or a mass (top_p). Three passes instead of the thirty of a bisection, and every pass
// reads the row in coalesced order. Masses are added as 64-bit fixed point (2^-40 units), so the
// histogram does not depend on the order in which the threads arrive.
constexpr int SEL_BINS = 2048;
constexpr float SEL_FIX = 1099511627776.0f;   // 2^40

struct SelectScratch {
  // Counts or fixed-point masses, as two 32-bit halves: shared memory adds 32-bit words natively, while a
  // 64-bit add is a compare-and-swap loop that crawls when many threads meet in one bin.
  uint32_t lo[SEL_BINS], hi[SEL_BINS];
  unsigned long long warp_tot[32];
  unsigned long long found_above;
  int found_bin;
};

__device__ __forceinline__ unsigned long long to_fixed(float e) { return (unsigned long long)(e * SEL_FIX); }

// bins[b] += add, exactly: the low word's carry goes into the high word.
__device__ __forceinline__ void bin_add(SelectScratch* sc, uint32_t b, unsigned long long add) {
  const uint32_t lo = (uint32_t)add;
  uint32_t hi = (uint32_t)(add >> 32);
  if (lo) {
    const uint32_t old = atomicAdd(&sc->lo[b], lo);
    if (old > 0xffffffffu - lo) ++hi;
  }
  if (hi) atomicAdd(&sc->hi[b], hi);
}
__device__ __forceinline__ unsigned long long bin_value(const SelectScratch* sc, int b) {
  return ((unsigned long long)sc->hi[b] << 32) | sc->lo[b];
}

// Highest bin b with sum(bins[b..]) >= need; returns b (or -1) and leaves sum(bins[b+1..]) in sc->found_above.
// All threads of the block call it; bins are read top-down, two per thread.
__device__ int find_bin(SelectScratch* sc, unsigned long long need) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b0 = SEL_BINS - 1 - 2 * tid, b1 = b0 - 1;            // this thread's two bins, the higher first
  const unsigned long long v0 = bin_value(sc, b0), v1 = bin_value(sc, b1);
  unsigned long long incl = v0 + v1;                              // inclusive scan over threads, top-down
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (tid == 0) sc->found_bin = -1;
  if (lane == 31) sc->warp_tot[warp] = incl;
  __syncthreads();
  unsigned long long before = 0;                                  // everything above this thread's bins
  for (int w = 0; w < warp; ++w) before += sc->warp_tot[w];
  before += incl - (v0 + v1);
  // Exactly one thread sees the running total cross `need` (need >= 1).
  if (before < need && before + v0 >= need) { sc->found_bin = b0; sc->found_above = before; }
  else if (before + v0 < need && before + v0 + v1 >= need) { sc->found_bin = b1; sc->found_above = before + v0; }
  __syncthreads();
  return sc->found_bin;
}

// The largest t >= floor_bits (as a bit pattern) such that the values e >= t number at least
// `need` (by_mass = false) or weigh at least `need` in fixed point (by_mass = true). Values below
// `floor_bits` do not take part. Returns floor_bits when nothing qualifies.
__device__ uint32_t select_cut(const float* __restrict__ x, int vocab, uint32_t floor_bits, unsigned long long need,
                               bool by_mass, SelectScratch* sc) {
  const int tid = threadIdx.x;
  uint32_t prefix = 0;            // digits found so far, in place
  uint32_t prefix_mask = 0;
  const int shifts[3] = {19, 8, 0}, widths[3] = {11, 11, 8};
  if (need == 0) need = 1;
#pragma unroll 1
  for (int level = 0; level < 3; ++level) {
    for (int i = tid; i < SEL_BINS; i += SM_THREADS) sc->lo[i] = sc->hi[i] = 0u;
    __syncthreads();
    const int shift = shifts[level];
    const uint32_t digit_mask = (1u << widths[level]) - 1u;
    for_each_elem(x, vocab, [&](int, float e) {
      const uint32_t bits = __float_as_uint(e);
      if (bits >= floor_bits && (bits & prefix_mask) == prefix)
        bin_add(sc, (bits >> shift) & digit_mask, by_mass ? to_fixed(e) : 1ull);
    });
    __syncthreads();
    const int bin = find_bin(sc, need);
    if (bin < 0) return floor_bits;
    need -= sc->found_above;
    prefix |= (uint32_t)bin << shift;
    prefix_mask |= digit_mask << shift;
    __syncthreads();
  }
  return prefix > floor_bits ? prefix : floor_bits;
}

// logits [n_rows, vocab] are changed in place (penalty, then exp(x - max)).
__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ penalty,
              const int* __restrict__ hist_tokens, const int* __restrict__ hist_offsets,
              const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ request_ids,
              const int* __restrict__ gen_index, int* __restrict__ out_tokens) {
  __shared__ ArgMax ared[33];
  __shared__ SelectScratch sel;
  __shared__ float scan[SM_THREADS];
  __shared__ int chosen;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
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
  for_each_elem(x, vocab, [&](int i, float v) { best = better(best, ArgMax{v, i}); });
  best = block_argmax(best, ared);
  if (best.i >= vocab) best.i = 0;  // a row of NaN has no maximum
  if (T <= 1e-5f) {
    if (tid == 0) out_tokens[row] = best.i;
    return;
  }

  // e_i = exp(x_i / T - max / T), in [0, 1].
  const float mx = best.v / T;
  if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    float4* x4 = reinterpret_cast<float4*>(x);
    const int n4 = vocab / 4;
    for (int i0 = tid; i0 < n4; i0 += 4 * SM_THREADS) {
      float4 v[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (i0 + q * SM_THREADS < n4) v[q] = x4[i0 + q * SM_THREADS];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (i0 + q * SM_THREADS >= n4) break;
        float* e = reinterpret_cast<float*>(&v[q]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float y = expf(e[c] / T - mx);
          e[c] = y >= 0.f ? y : 0.f;   // a NaN logit keeps no mass
        }
        x4[i0 + q * SM_THREADS] = v[q];
      }
    }
  } else {
    for (int i = tid; i < vocab; i += SM_THREADS) {
      const float e = expf(x[i] / T - mx);
      x[i] = e >= 0.f ? e : 0.f;
    }
  }
  __syncthreads();

  uint32_t cut_bits = 0u;  // keep e_i >= cut
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < vocab) cut_bits = select_cut(x, vocab, 0u, (unsigned long long)k, false, &sel);   // the k-th largest value
  const float p = top_p ? top_p[row] : 1.0f;
  if (p < 1.0f) {
    // Mass of what top_k kept, then the largest t >= cut with mass(e >= t) >= p * that mass.
    unsigned long long part = 0;
    for_each_elem(x, vocab, [&](int, float e) {
      if (__float_as_uint(e) >= cut_bits) part += to_fixed(e);
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    __syncthreads();
    if (lane == 0) sel.warp_tot[warp] = part;
    __syncthreads();
    unsigned long long total_fx = 0;
    for (int w = 0; w < SM_THREADS / 32; ++w) total_fx += sel.warp_tot[w];
    __syncthreads();
    const unsigned long long need = (unsigned long long)((double)total_fx * (double)p);
    cut_bits = select_cut(x, vocab, cut_bits, need, true, &sel);
  }
  const float cut = __uint_as_float(cut_bits);

  // Draw: first index, in vocabulary order, whose running sum of kept e exceeds u * total. The
  // vocabulary is cut into 1024 runs of consecutive indices; a warp sums 32 of the runs (coalesced
  // loads, a fixed order of additions), one thread walks the 1024 sums in order, and the thread
  // that owns the run in which the target falls walks that run.
  const int chunk = (vocab + SM_THREADS - 1) / SM_THREADS;
  for (int c = warp * 32; c < warp * 32 + 32; c += 4) {   // four runs at a time: their loads are in flight together
    float part[4] = {0.f, 0.f, 0.f, 0.f};
    for (int off = lane; off < chunk; off += 32) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int lo_c = min((c + q) * chunk, vocab), hi_c = min(lo_c + chunk, vocab);
        const float e = lo_c + off < hi_c ? x[lo_c + off] : 0.f;
        part[q] += e >= cut ? e : 0.f;
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part[q] += __shfl_xor_sync(0xffffffffu, part[q], o);
      if (lane == 0) scan[c + q] = part[q];
    }
  }
  if (tid == 0) chosen = -1;
  __syncthreads();
  uint32_t r[4];
  const unsigned long long seed = seeds ? seeds[row] : 0ull, rid = request_ids ? request_ids[row] : 0ull;
  philox4x32_10((uint32_t)seed, (uint32_t)(seed >> 32), (uint32_t)rid, (uint32_t)(rid >> 32),
                gen_index ? (uint32_t)gen_index[row] : 0u, 0u, r);
  const float u = (float)(r[0] >> 8) * (1.0f / 16777216.0f);
  __shared__ float s_target, s_before, wsum[32];
  __shared__ int wfirst[32], wlast[32];
  {
    // Running sums of the 1024 runs by a block-wide scan (a fixed order of additions), then the first
    // run whose running sum exceeds the target.
    const float v = scan[tid];
    float incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    float before_warp = 0.f, total = 0.f;
    for (int w = 0; w < SM_THREADS / 32; ++w) {
      if (w == warp) before_warp = total;
      total += wsum[w];
    }
    incl += before_warp;
    const float target = u * total;
    const unsigned hit = __ballot_sync(0xffffffffu, incl > target);
    const unsigned kept = __ballot_sync(0xffffffffu, v > 0.f);
    if (lane == 0) {
      wfirst[warp] = hit ? warp * 32 + __ffs(hit) - 1 : 0x7fffffff;
      wlast[warp] = kept ? warp * 32 + 31 - __clz(kept) : -1;
    }
    __syncthreads();
    int first = 0x7fffffff, last = -1;
    for (int w = 0; w < SM_THREADS / 32; ++w) {
      first = min(first, wfirst[w]);
      last = max(last, wlast[w]);
    }
    if (first != 0x7fffffff) {
      if (tid == first) { s_before = incl - v; s_target = target; chosen = first; }
    } else if (tid == 0) {
      // Rounding left the target at or above the sum: the last run with kept mass owns it.
      s_before = -1.f;
      s_target = target;
      chosen = last;
    }
  }
  __syncthreads();
  const int owner = chosen;
  if (tid == 0) {
    if (owner < 0) {
      out_tokens[row] = best.i;
    } else {
      const float target = s_target, before = s_before;
      const int lo = min(owner * chunk, vocab), hi = min(lo + chunk, vocab);
      int pick = -1, last_kept = -1;
      float run = before;
      for (int i = lo; i < hi; ++i) {
        const float e = x[i];
        if (e >= cut && e > 0.f) {
          last_kept = i;
          if (before >= 0.f) {
            run += e;
            if (run > target) { pick = i; break; }
          }
        }
      }
      // The walk reached the run's end without a pick: rounding; take the run's last kept token.
      if (pick < 0) pick = last_kept >= 0 ? last_kept : best.i;
      out_tokens[row] = pick;
    }
  }
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
  for_each_elem(x, vocab, [&](int i, float v) { best = better(best, ArgMax{v, i}); });
  best = block_argmax(best, ared);
  if (threadIdx.x == 0) out_tokens[blockIdx.x] = best.i < vocab ? best.i : 0;  // a row of NaN has no maximum
}

LLMRS_API int llmrs_argmax(const float* logits, int n_rows, int vocab, int* out_tokens, cudaStream_t stream) {
  LLMRS_REQUIRE(n_rows >= 0 && vocab > 0, "argmax: bad sizes");
  if (n_rows == 0) return 0;
  argmax_kernel<<<n_rows, SM_THREADS, 0, stream>>>(logits, vocab, out_tokens);
  return llmrs_launch_status("argmax");
}
