// Shared helpers of the kernel library: element types, loads and stores that widen to
// float, warp and block reductions, and the error record of the C entry points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLMRS_API extern "C" __attribute__((visibility("default")))

// Element types as the Python side names them.
enum LlmrsDtype : int { LLMRS_F32 = 0, LLMRS_BF16 = 1 };

// Records a message for llmrs_last_error() and returns the negative code that entry
// points hand back when they refuse their arguments (no kernel was launched).
int llmrs_fail(const char* fmt, ...);
// cudaGetLastError() as the entry point's return value (0 = launched).
int llmrs_launch_status(const char* what);

// Programmatic dependent launch. A kernel launched through llmrs_launch() with pdl = true
// may start while the kernel before it in the stream is still running: it calls
// pdl_launch_dependents() at its top (the kernel after it may be scheduled early in turn)
// and pdl_wait() before its first read or write of anything an earlier kernel touches;
// what it does before that wait (barrier set-up, loads of weights) overlaps the tail of
// its predecessor. Without the launch attribute both calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 1: kernels that support it are launched with the programmatic-serialization attribute.
extern int g_llmrs_pdl;

// Warming the L2 for the kernel that runs next. A decode step is a chain of kernels that each stream some
// tens of megabytes once; between the end of one kernel's stream and the first bytes of the next the memory
// system idles (epilogues, barriers, launch). A kernel that was given a hint (llmrs_set_next_prefetch, consumed
// by the next launch that supports it) asks, when its own last loads are on their way, for the start of the
// NEXT kernel's weights to be brought into the L2 (126 MB on a B200): every block asks for its slice.
struct L2Prefetch {
  const char* ptr;              // 16-byte aligned, or null
  unsigned long long bytes;     // a multiple of 16
};
L2Prefetch llmrs_take_next_prefetch();    // the pending hint (and clears it)

// This block's slice of `pf` (blocks numbered over the whole grid), requested in pieces of 16 KB by the calling thread.
__device__ __forceinline__ void l2_prefetch_slice(const L2Prefetch& pf) {
  if (pf.ptr == nullptr || pf.bytes == 0) return;
  const unsigned long long nb = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
  const unsigned long long b = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
  const unsigned long long chunk = (((pf.bytes + nb - 1) / nb) + 127ull) & ~127ull;
  const unsigned long long lo = b * chunk;
  const unsigned long long hi = lo + chunk < pf.bytes ? lo + chunk : pf.bytes;
  for (unsigned long long a = lo; a < hi; a += 16384ull) {
    const unsigned int n = (unsigned int)(hi - a < 16384ull ? hi - a : 16384ull);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pf.ptr + a), "r"(n) : "memory");
  }
}

template <typename... KArgs, typename... Args>
inline cudaError_t llmrs_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  unsigned n = 0;
  if (pdl && g_llmrs_pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    n = 1;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- the debug build (-DLLMRS_DEBUG_CHECKS; LLMRS_DEBUG_KERNELS=1 at import) ---------------------------
// Where a memory checker cannot be run, the kernels check the indices they are about to use themselves: a page
// id taken from a block table (the realistic fault is -1, a page that a window has released), a token id. A bad
// one is recorded (the first one with its values, and how many there were) and replaced by one that stays inside
// the buffer; nothing traps. llmrs_debug_take() reads and clears the record of every file of the library.
//   codes: 1 token id (embedding), 2 page for a cache write, 3/4 page read by the generic / mma.sync attention,
//          5 page in the q|k|v epilogue, 6 page read by the tcgen05 attention
#ifdef LLMRS_DEBUG_CHECKS
static __device__ int g_llmrs_debug[4];   // code, value, where, count (one record per file of the library)
struct LlmrsDebugReader { explicit LlmrsDebugReader(int (*read)(int*)); };   // errors.cu keeps the list
static int llmrs_debug_read_file(int* out4) {
  const int zero[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(out4, g_llmrs_debug, sizeof(zero)) != cudaSuccess) return -1;
  if (out4[3]) cudaMemcpyToSymbol(g_llmrs_debug, zero, sizeof(zero));
  return 0;
}
static LlmrsDebugReader g_llmrs_debug_reader(&llmrs_debug_read_file);
__device__ __forceinline__ int llmrs_checked(int value, int lo, int hi, int code, int where, int fallback) {
  if (value >= lo && value < hi) return value;
  if (atomicAdd(&g_llmrs_debug[3], 1) == 0) {
    g_llmrs_debug[0] = code;
    g_llmrs_debug[1] = value;
    g_llmrs_debug[2] = where;
  }
  return fallback;
}
#define LLMRS_CHECKED_PAGE(page, code, where) llmrs_checked((page), 0, 0x7fffffff, (code), (where), 0)
#else
#define LLMRS_CHECKED_PAGE(page, code, where) (page)
#endif

#define LLMRS_REQUIRE(cond, ...)                     \
  do {                                               \
    if (!(cond)) return llmrs_fail(__VA_ARGS__);     \
  } while (0)

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// Element offset of (page, kv head, K|V, slot in page, 0) in one layer's cache:
// [n_pages, n_kv_heads, 2, page_size, head_dim]. The keys of one (page, head) and its
// values are two adjacent contiguous tiles, so one tile is one straight copy.
__device__ __host__ __forceinline__ size_t kv_tile_offset(int page, int kvh, int which, int n_kv_heads,
                                                           int page_size, int head_dim) {
  return ((size_t)((size_t)page * n_kv_heads + kvh) * 2 + which) * page_size * head_dim;
}
