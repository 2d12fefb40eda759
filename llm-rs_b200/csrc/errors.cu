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

// Version of the entry points' signatures; the Python side checks it after loading.
LLMRS_API int llmrs_abi_version() { return 4; }
