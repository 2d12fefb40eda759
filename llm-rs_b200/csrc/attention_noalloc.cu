// Decode attention with built-in workspace, for callers that cannot allocate on the
// device (see llmrs_noalloc.h for who they are and what the rules are). It runs the same
// split and combine kernels as llmrs_attn_decode; the only difference is where the
// partial results of the splits live: in the fixed array below instead of a buffer
// from the caller. Not part of mashriram/llm-rs.
#include <mutex>

#include "common.cuh"
#include "llmrs_noalloc.h"

// The regular entry point and its workspace formula (attention.cu).
extern "C" int llmrs_attn_decode(const void* q, long long q_stride, void* out, long long out_stride,
                                 const void* cache, const int* dec_reqs, int n_dec, const int* q_start,
                                 const int* cached_len, const int* block_table, int table_stride, float* scratch,
                                 int* counters, int max_splits, int split_keys, int n_q_heads, int n_kv_heads,
                                 int d, int page_size, int window, float scale, int dtype, cudaStream_t stream);
extern "C" long long llmrs_attn_decode_scratch_floats(int n_dec, int n_q_heads, int d, int max_splits);

// 8 MiB per GPU, held from the moment this file's device code is loaded on it (with lazy module
// loading: the first cudaGetSymbolAddress below) to process exit. In host code this name is only
// a handle for cudaGetSymbolAddress, never an address to hand to a kernel.
static __device__ __align__(256) float g_static_scratch[LLMRS_NOALLOC_SCRATCH_BYTES / sizeof(float)];

constexpr int kMaxDevices = 64;
static float* g_scratch_addr[kMaxDevices] = {};
static std::mutex g_scratch_mutex;

// Device address of the array on the current device; looked up at the first call per device.
static int static_scratch_address(float** addr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return llmrs_fail("attn_decode_static_scratch: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return llmrs_fail("attn_decode_static_scratch: device %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return llmrs_fail("attn_decode_static_scratch: cudaGetSymbolAddress on device %d: %s", dev,
                        cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *addr = g_scratch_addr[dev];
  return 0;
}

LLMRS_API int llmrs_attn_decode_static_scratch(const void* q, long long q_stride, void* out, long long out_stride,
                                               const void* cache, const int* dec_reqs, int n_dec,
                                               const int* q_start, const int* cached_len, const int* block_table,
                                               int table_stride, int max_splits, int split_keys, int n_q_heads,
                                               int n_kv_heads, int d, int page_size, int window, float scale,
                                               int dtype, cudaStream_t stream) {
  LLMRS_REQUIRE(n_dec >= 0 && n_q_heads > 0 && d > 0 && max_splits > 0, "attn_decode_static_scratch: bad sizes");
  const long long need = llmrs_attn_decode_scratch_floats(n_dec, n_q_heads, d, max_splits);
  const long long have = (long long)(LLMRS_NOALLOC_SCRATCH_BYTES / sizeof(float));
  LLMRS_REQUIRE(need <= have,
                "attn_decode_static_scratch: %d requests x %d heads x %d splits x (%d+2) floats = %lld floats do "
                "not fit the built-in workspace of %lld floats (%u bytes); use llmrs_attn_decode with a buffer "
                "of your own",
                n_dec, n_q_heads, max_splits, d, need, have, (unsigned)LLMRS_NOALLOC_SCRATCH_BYTES);
  float* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc) return rc;
  return llmrs_attn_decode(q, q_stride, out, out_stride, cache, dec_reqs, n_dec, q_start, cached_len, block_table,
                           table_stride, scratch, /*counters=*/nullptr, max_splits, split_keys, n_q_heads, n_kv_heads, d,
                           page_size, window, scale, dtype, stream);
}
