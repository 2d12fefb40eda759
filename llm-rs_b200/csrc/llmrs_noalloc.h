/* Decode attention for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in mashriram/llm-rs; it exists for users of this
 * library only.
 *
 * Who needs it: code that runs where a device allocation is not allowed or not safe.
 * Typical cases are a real-time or latency-bound serving loop that has promised its
 * host never to call cudaMalloc after start-up (an allocation may synchronise the whole
 * device and stall every stream), a plug-in that lives inside another process's memory
 * budget and is handed fixed buffers, and a host that works under a memory pool it does
 * not own, so that it has nothing to carve kernel workspace from. The regular entry
 * point, llmrs_attn_decode, wants such a workspace from its caller (the partial results
 * of the key splits, merged by its combine step). This variant brings its own: a fixed
 * array in the library's device image.
 *
 * What it costs: LLMRS_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory on every GPU
 * on which the library's device code is loaded, until the process exits, used or not.
 * With CUDA's lazy module loading (the default) that moment is the first call of this
 * entry point on the device, not the loading of the shared library: the driver brings
 * the array into being inside that call. A caller that must not see any allocation
 * after start-up therefore makes one call per device at start-up; a call with
 * n_dec = 0 does the look-up, launches nothing and needs no valid pointers.
 *
 * Limits and rules:
 *  - n_dec * n_q_heads * max_splits * (head_dim + 2) floats must fit in the array;
 *    a larger request is refused with a message (llmrs_last_error) and nothing runs.
 *  - The first call on each device looks up the array's device address (once per device,
 *    for the device that is current at the call; see "What it costs"). Make that first
 *    call at start-up and outside any stream capture.
 *  - All calls share the one array, and it keeps what the last call left in it. The
 *    kernels write every slot they later read, so nothing needs clearing between calls.
 *    Two calls whose kernels may overlap on the GPU (different streams, no dependency
 *    between them) race on the array: order them.
 *  - It allocates nothing: no cudaMalloc, no cudaFree, no library routine that allocates.
 *    Inputs and outputs are the caller's, exactly as for llmrs_attn_decode.
 *
 * Arguments and return value are those of llmrs_attn_decode without `scratch`.
 */
#ifndef LLMRS_NOALLOC_H
#define LLMRS_NOALLOC_H

#include <cuda_runtime.h>

#define LLMRS_NOALLOC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int llmrs_attn_decode_static_scratch(const void* q, long long q_stride, void* out, long long out_stride,
                                     const void* cache, const int* dec_reqs, int n_dec, const int* q_start,
                                     const int* cached_len, const int* block_table, int table_stride,
                                     int max_splits, int split_keys, int n_q_heads, int n_kv_heads, int d,
                                     int page_size, int window, float scale, int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
