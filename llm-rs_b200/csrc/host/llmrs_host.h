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

/* Packs the index arrays of one step that every part may read (layout: see StepArray in
 * cache_manager.hpp). shape4 receives n_tokens, n_requests, n_want, 0; *total the int32 elements
 * needed. When capacity < *total nothing is written and *written is 0. */
int llmrs_pack_step(void* cm, int n_entries, const int64_t* ids, const int32_t* n_tokens, const int32_t* tokens,
                    const int32_t* n_want, const int32_t* want, const int32_t* device_token, int table_round,
                    int32_t* out, int64_t capacity, int64_t* offsets, int64_t* sizes,
                    int32_t* widths, int32_t* shape4, int64_t* total, int* written);

/* The plan of paged attention for one step: requests with one new token go to decode_out, longer
 * portions are cut into tiles of `tile` queries, written to tiles_out as (request row, offset)
 * pairs. plan4 receives n_tiles, n_decode, max_decode_kv_len, long_portions. When a capacity
 * (in tiles, in requests) is too small nothing is written and *written is 0. */
int llmrs_plan_paged_attention(int n_requests, const int32_t* n_new, const int32_t* cached_len, int tile,
                               int32_t* tiles_out, int64_t tiles_capacity, int32_t* decode_out,
                               int64_t decode_capacity, int32_t* plan4, int* written);

/* The scheduler (decisions only; see scheduler.hpp). It reads the cache manager `cm`, which must
 * outlive it, and never changes it: after every call that returns `n_release > 0` ids through
 * llmrs_sched_take, the caller releases those requests in the manager before it calls again.
 * Finish reasons: 0 none, 1 stop (EOS), 2 length, 3 too long for the pool, 4 a step failed. */
int llmrs_sched_create(void* cm, int max_positions, const int32_t* eos, int n_eos, int max_tokens_per_step,
                       int prefill_chunk, int max_requests_per_step, void** sched);
void llmrs_sched_destroy(void* sched);
int llmrs_sched_add(void* sched, int64_t id, int prompt_len, int max_new_tokens, int ignore_eos);
int llmrs_sched_has_work(void* sched, int* out);
/* entries: per entry id, and 4 ints: start (-1: the token in flight), n_tokens, sample, pending. *batch: handle, 0 if empty. */
int llmrs_sched_schedule(void* sched, int64_t* ids, int32_t* fields4, int capacity, int* n, int64_t* batch);
int llmrs_sched_on_launched(void* sched, int64_t batch);
int llmrs_sched_cancel(void* sched, int64_t batch);
/* tokens: one per sampling entry of the batch, in order. outs: per output id, and 3 ints: token (-1 none), finished, reason. */
int llmrs_sched_on_result(void* sched, int64_t batch, const int32_t* tokens, int n_tokens, int64_t* out_ids,
                          int32_t* out_fields3, int capacity, int* n_out);
int llmrs_sched_abort_all(void* sched, int reason, int64_t* out_ids, int32_t* out_fields3, int capacity, int* n_out);
/* which = 0: requests to release now; 1: requests whose state changed; 2: waiting queue; 3: running list. */
int llmrs_sched_take(void* sched, int which, int64_t* ids, int capacity, int* n);
/* state6: status (0 waiting, 1 running, 2 finished), finish reason, n_output, n_computed, n_inflight, preemptions */
int llmrs_sched_get(void* sched, int64_t id, int32_t* state6);
int llmrs_sched_forget(void* sched, int64_t id);
int llmrs_sched_stats(void* sched, int64_t* stats3);

#ifdef __cplusplus
}
#endif
#endif
