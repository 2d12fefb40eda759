/* C entry points of the host library (cache bookkeeping and step packing). Every function
 * returns a status (0 = ok, 1 = cache error, 2 = out of pages, 3 = no free request slot,
 * 4 = bad argument); llmrs_host_last_error() gives the message of the calling thread's
 * last failure. Handles are owned by the caller and freed with the matching destroy. */
#ifndef LLMRS_HOST_H
#define LLMRS_HOST_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int llmrs_host_abi_version(void);
const char* llmrs_host_last_error(void);

/* A stand-alone page pool. */
int llmrs_pool_create(int capacity, void** pool);
void llmrs_pool_destroy(void* pool);
int llmrs_pool_allocate(void* pool, int32_t* page);
int llmrs_pool_free(void* pool, int32_t page, int* went_back);
int llmrs_pool_increment_ref(void* pool, int32_t page);
int llmrs_pool_ref_count(void* pool, int32_t page, int* count);
int llmrs_pool_counts(void* pool, int* free_pages, int* capacity);

/* The cache manager. windows[g] = 0 for a group that keeps every key. */
int llmrs_cm_create(const int* n_pages, const int* windows, int n_groups, int page_size, int n_slots, void** cm);
void llmrs_cm_destroy(void* cm);
int llmrs_cm_admit(void* cm, int64_t id, int* slot);
int llmrs_cm_release(void* cm, int64_t id);
int llmrs_cm_pages_needed(void* cm, int live, int64_t id, int n_new, int cached_len, int* out);
int llmrs_cm_reserve(void* cm, int64_t id, int n_new);
int llmrs_cm_cancel(void* cm, int64_t id);
int llmrs_cm_commit(void* cm, int64_t id, int n_new);
/* info: slot, cached_len, reserved_len; edits counts table changes other than appends. */
int llmrs_cm_info(void* cm, int64_t id, int* info3, int64_t* edits);
/* Copies at most `capacity` entries of the block table; *length is the table's length. */
int llmrs_cm_table(void* cm, int64_t id, int group, int32_t* out, int capacity, int* length);
int llmrs_cm_pool_counts(void* cm, int group, int* free_pages, int* capacity);
int llmrs_cm_check_invariants(void* cm);

/* Packs one step (layout: see StepArray in cache_manager.hpp). shape8 receives n_tokens,
 * n_requests, n_want, n_prefill_tiles, n_decode, max_decode_kv_len, long_portions, 0;
 * *total the int32 elements needed. When capacity < *total nothing is written and
 * *written is 0. */
int llmrs_pack_step(void* cm, int n_entries, const int64_t* ids, const int32_t* n_tokens, const int32_t* tokens,
                    const int32_t* n_want, const int32_t* want, const int32_t* device_token, int table_round,
                    int prefill_tile, int32_t* out, int64_t capacity, int64_t* offsets, int64_t* sizes,
                    int32_t* widths, int32_t* shape8, int64_t* total, int* written);

#ifdef __cplusplus
}
#endif
#endif
