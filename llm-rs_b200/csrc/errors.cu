// Error record of the C entry points.
#include <stdarg.h>
#include <stdio.h>
#include "common.cuh"

static thread_local char g_last_error[512] = "";

int llmrs_fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return -1;
}

int llmrs_launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

// The message of the last refusal or failed launch on this thread.
LLMRS_API const char* llmrs_last_error() { return g_last_error; }

int g_llmrs_pdl = 1;
// Switch programmatic dependent launch on (1, the default) or off (0) for the kernels that support it.
LLMRS_API void llmrs_set_pdl(int on) { g_llmrs_pdl = on; }

// The hint for the next launch that can warm the L2 (see L2Prefetch in common.cuh): the start of the weights that
// the kernel AFTER that launch will stream. One-shot: the launch takes it, and a launch that cannot use it drops it.
static thread_local L2Prefetch g_next_prefetch = {nullptr, 0};
LLMRS_API int llmrs_set_next_prefetch(const void* ptr, long long bytes) {
  LLMRS_REQUIRE(bytes >= 0 && bytes % 16 == 0 && ((uintptr_t)ptr & 15) == 0,
                "set_next_prefetch: the range must be 16-byte aligned and a multiple of 16 bytes long");
  g_next_prefetch.ptr = bytes ? (const char*)ptr : nullptr;
  g_next_prefetch.bytes = ptr ? (unsigned long long)bytes : 0ull;
  return 0;
}
L2Prefetch llmrs_take_next_prefetch() {
  L2Prefetch p = g_next_prefetch;
  g_next_prefetch = {nullptr, 0};
  return p;
}

// The debug build's records (see common.cuh): every file of the library that checks indices registers its reader.
static int (*g_debug_readers[32])(int*);
static int g_n_debug_readers = 0;
#ifdef LLMRS_DEBUG_CHECKS
LlmrsDebugReader::LlmrsDebugReader(int (*read)(int*)) {
  if (g_n_debug_readers < 32) g_debug_readers[g_n_debug_readers++] = read;
}
#endif
// out4 receives code, value, where and the number of failed checks since the last call (all files together; the
// first record found wins). Returns 1 in a debug build, 0 in a normal one (nothing is checked), -1 on a CUDA error.
LLMRS_API int llmrs_debug_take(int* out4) {
  out4[0] = out4[1] = out4[2] = out4[3] = 0;
#ifdef LLMRS_DEBUG_CHECKS
  for (int i = 0; i < g_n_debug_readers; ++i) {
    int r[4] = {0, 0, 0, 0};
    if (g_debug_readers[i](r) != 0) return -1;
    if (r[3] && !out4[3]) { out4[0] = r[0]; out4[1] = r[1]; out4[2] = r[2]; }
    out4[3] += r[3];
  }
  return 1;
#else
  return 0;
#endif
}

// Version of the entry points' signatures; the Python side checks it after loading.
LLMRS_API int llmrs_abi_version() { return 4; }
