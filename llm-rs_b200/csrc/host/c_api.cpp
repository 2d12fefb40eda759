#include "llmrs_host.h"

#include <exception>
#include <string>

#include "cache_manager.hpp"
#include "scheduler.hpp"

using namespace llmrs_host;

namespace {
thread_local std::string g_error;

template <typename F>
int guarded(F&& body) {
    try {
        body();
        return kOk;
    } catch (const Failure& f) {
        g_error = f.message;
        return f.status;
    } catch (const std::exception& e) {
        g_error = e.what();
        return kBadArgument;
    }
}

template <typename T>
T* as(void* handle, const char* what) {
    if (handle == nullptr) throw Failure{kBadArgument, std::string("null ") + what + " handle"};
    return static_cast<T*>(handle);
}
}  // namespace

extern "C" {

int llmrs_host_abi_version(void) { return 3; }
const char* llmrs_host_last_error(void) { return g_error.c_str(); }

int llmrs_pool_create(int capacity, void** pool) {
    return guarded([&] { *pool = new PagePool(capacity); });
}
void llmrs_pool_destroy(void* pool) { delete static_cast<PagePool*>(pool); }
int llmrs_pool_allocate(void* pool, int32_t* page) {
    return guarded([&] { *page = as<PagePool>(pool, "pool")->allocate(); });
}
int llmrs_pool_free(void* pool, int32_t page, int* went_back) {
    return guarded([&] { *went_back = as<PagePool>(pool, "pool")->free(page) ? 1 : 0; });
}
int llmrs_pool_increment_ref(void* pool, int32_t page) {
    return guarded([&] { as<PagePool>(pool, "pool")->increment_ref(page); });
}
int llmrs_pool_ref_count(void* pool, int32_t page, int* count) {
    return guarded([&] { *count = as<PagePool>(pool, "pool")->ref_count(page); });
}
int llmrs_pool_counts(void* pool, int* free_pages, int* capacity) {
    return guarded([&] {
        auto* p = as<PagePool>(pool, "pool");
        *free_pages = p->free_pages();
        *capacity = p->capacity();
    });
}

int llmrs_cm_create(const int* n_pages, const int* windows, int n_groups, int page_size, int n_slots, void** cm) {
    return guarded([&] { *cm = new CacheManager(n_pages, windows, n_groups, page_size, n_slots); });
}
void llmrs_cm_destroy(void* cm) { delete static_cast<CacheManager*>(cm); }
int llmrs_cm_admit(void* cm, int64_t id, int* slot) {
    return guarded([&] { *slot = as<CacheManager>(cm, "manager")->admit(id).slot; });
}
int llmrs_cm_release(void* cm, int64_t id) {
    return guarded([&] { as<CacheManager>(cm, "manager")->release(id); });
}
int llmrs_cm_pages_needed(void* cm, int live, int64_t id, int n_new, int cached_len, int* out) {
    return guarded([&] { as<CacheManager>(cm, "manager")->pages_needed(live != 0, id, n_new, cached_len, out); });
}
int llmrs_cm_reserve(void* cm, int64_t id, int n_new) {
    return guarded([&] { as<CacheManager>(cm, "manager")->reserve(id, n_new); });
}
int llmrs_cm_cancel(void* cm, int64_t id) {
    return guarded([&] { as<CacheManager>(cm, "manager")->cancel(id); });
}
int llmrs_cm_commit(void* cm, int64_t id, int n_new) {
    return guarded([&] { as<CacheManager>(cm, "manager")->commit(id, n_new); });
}
int llmrs_cm_info(void* cm, int64_t id, int* info3, int64_t* edits) {
    return guarded([&] {
        const Record& rec = as<CacheManager>(cm, "manager")->record(id);
        info3[0] = rec.slot;
        info3[1] = rec.cached_len;
        info3[2] = rec.reserved_len;
        *edits = rec.edits;
    });
}
int llmrs_cm_table(void* cm, int64_t id, int group, int32_t* out, int capacity, int* length) {
    return guarded([&] {
        auto* m = as<CacheManager>(cm, "manager");
        m->pool(group);  // checks the group
        const auto& table = m->record(id).tables[group];
        *length = static_cast<int>(table.size());
        for (int i = 0; i < *length && i < capacity; ++i) out[i] = table[i];
    });
}
int llmrs_cm_pool_counts(void* cm, int group, int* free_pages, int* capacity) {
    return guarded([&] {
        const PagePool& p = as<CacheManager>(cm, "manager")->pool(group);
        *free_pages = p.free_pages();
        *capacity = p.capacity();
    });
}
int llmrs_cm_check_invariants(void* cm) {
    return guarded([&] { as<CacheManager>(cm, "manager")->check_invariants(); });
}

int llmrs_pack_step(void* cm, int n_entries, const int64_t* ids, const int32_t* n_tokens, const int32_t* tokens,
                    const int32_t* n_want, const int32_t* want, const int32_t* device_token, int table_round,
                    int32_t* out, int64_t capacity, int64_t* offsets, int64_t* sizes,
                    int32_t* widths, int32_t* shape4, int64_t* total, int* written) {
    return guarded([&] {
        StepShape s;
        bool ok = pack_step(*as<CacheManager>(cm, "manager"), n_entries, ids, n_tokens, tokens, n_want, want,
                            device_token, table_round, out, capacity, offsets, sizes, widths, &s);
        shape4[0] = s.n_tokens;
        shape4[1] = s.n_requests;
        shape4[2] = s.n_want;
        shape4[3] = 0;
        *total = s.total;
        *written = ok ? 1 : 0;
    });
}

int llmrs_plan_paged_attention(int n_requests, const int32_t* n_new, const int32_t* cached_len, int tile,
                               int32_t* tiles_out, int64_t tiles_capacity, int32_t* decode_out,
                               int64_t decode_capacity, int32_t* plan4, int* written) {
    return guarded([&] {
        AttentionPlan a;
        bool ok = plan_paged_attention(n_requests, n_new, cached_len, tile, tiles_out, tiles_capacity, decode_out,
                                       decode_capacity, &a);
        plan4[0] = a.n_tiles;
        plan4[1] = a.n_decode;
        plan4[2] = a.max_decode_kv_len;
        plan4[3] = a.long_portions;
        *written = ok ? 1 : 0;
    });
}


int llmrs_sched_create(void* cm, int max_positions, const int32_t* eos, int n_eos, int max_tokens_per_step,
                       int prefill_chunk, int max_requests_per_step, void** sched) {
    return guarded([&] {
        *sched = new Scheduler(as<CacheManager>(cm, "manager"), max_positions, eos, n_eos, max_tokens_per_step,
                               prefill_chunk, max_requests_per_step);
    });
}
void llmrs_sched_destroy(void* sched) { delete static_cast<Scheduler*>(sched); }
int llmrs_sched_add(void* sched, int64_t id, int prompt_len, int max_new_tokens, int ignore_eos) {
    return guarded([&] { as<Scheduler>(sched, "scheduler")->add(id, prompt_len, max_new_tokens, ignore_eos != 0); });
}
int llmrs_sched_has_work(void* sched, int* out) {
    return guarded([&] { *out = as<Scheduler>(sched, "scheduler")->has_work() ? 1 : 0; });
}
int llmrs_sched_schedule(void* sched, int64_t* ids, int32_t* fields4, int capacity, int* n, int64_t* batch) {
    return guarded([&] {
        std::vector<SchedEntry> entries;
        *batch = as<Scheduler>(sched, "scheduler")->schedule(&entries);
        *n = static_cast<int>(entries.size());
        if (*n > capacity) throw Failure{kBadArgument, "the buffer for the step's entries is too small"};
        for (int i = 0; i < *n; ++i) {
            ids[i] = entries[i].id;
            fields4[4 * i] = entries[i].start;
            fields4[4 * i + 1] = entries[i].n_tokens;
            fields4[4 * i + 2] = entries[i].sample ? 1 : 0;
            fields4[4 * i + 3] = entries[i].pending ? 1 : 0;
        }
    });
}
int llmrs_sched_on_launched(void* sched, int64_t batch) {
    return guarded([&] { as<Scheduler>(sched, "scheduler")->on_launched(batch); });
}

int llmrs_sched_cancel(void* sched, int64_t batch) {
    return guarded([&] { as<Scheduler>(sched, "scheduler")->cancel(batch); });
}
namespace {
void copy_outputs(const std::vector<SchedOutput>& outs, int64_t* out_ids, int32_t* out_fields3, int capacity, int* n_out) {
    *n_out = static_cast<int>(outs.size());
    if (*n_out > capacity) throw Failure{kBadArgument, "the buffer for the outputs is too small"};
    for (int i = 0; i < *n_out; ++i) {
        out_ids[i] = outs[i].id;
        out_fields3[3 * i] = outs[i].token;
        out_fields3[3 * i + 1] = outs[i].finished ? 1 : 0;
        out_fields3[3 * i + 2] = outs[i].reason;
    }
}
}  // namespace
int llmrs_sched_on_result(void* sched, int64_t batch, const int32_t* tokens, int n_tokens, int64_t* out_ids,
                          int32_t* out_fields3, int capacity, int* n_out) {
    return guarded([&] {
        std::vector<SchedOutput> outs;
        as<Scheduler>(sched, "scheduler")->on_result(batch, tokens, n_tokens, &outs);
        copy_outputs(outs, out_ids, out_fields3, capacity, n_out);
    });
}
int llmrs_sched_abort_all(void* sched, int reason, int64_t* out_ids, int32_t* out_fields3, int capacity, int* n_out) {
    return guarded([&] {
        std::vector<SchedOutput> outs;
        as<Scheduler>(sched, "scheduler")->abort_all(reason, &outs);
        copy_outputs(outs, out_ids, out_fields3, capacity, n_out);
    });
}
int llmrs_sched_take(void* sched, int which, int64_t* ids, int capacity, int* n) {
    return guarded([&] {
        auto* s = as<Scheduler>(sched, "scheduler");
        std::vector<int64_t> v;
        if (which == 0) s->take_releases(&v);
        else if (which == 1) s->take_changed(&v);
        else if (which == 2) v.assign(s->waiting().begin(), s->waiting().end());
        else if (which == 3) v = s->running();
        else throw Failure{kBadArgument, "llmrs_sched_take: which must be 0..3"};
        *n = static_cast<int>(v.size());
        // Lists that are taken (0, 1) must not be lost to a small buffer: the caller sizes it by the
        // number of requests it has ever added.
        if (*n > capacity) throw Failure{kBadArgument, "the buffer for the request ids is too small"};
        for (int i = 0; i < *n; ++i) ids[i] = v[i];
    });
}
int llmrs_sched_get(void* sched, int64_t id, int32_t* state6) {
    return guarded([&] {
        const SchedRequest& r = as<Scheduler>(sched, "scheduler")->request(id);
        state6[0] = r.status;
        state6[1] = r.finish_reason;
        state6[2] = r.n_output;
        state6[3] = r.n_computed;
        state6[4] = r.n_inflight;
        state6[5] = r.preemptions;
    });
}
int llmrs_sched_forget(void* sched, int64_t id) {
    return guarded([&] { as<Scheduler>(sched, "scheduler")->forget(id); });
}
int llmrs_sched_stats(void* sched, int64_t* stats3) {
    return guarded([&] { as<Scheduler>(sched, "scheduler")->stats(stats3, stats3 + 1, stats3 + 2); });
}

}  // extern "C"
