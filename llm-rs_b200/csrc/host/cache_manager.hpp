// Host-side bookkeeping of the paged cache: a page pool per group of layers, a block
// table per request and group, and one slot per live request for fixed-size state.
// No device memory is touched here; the device tensors are indexed by what this hands out.
//
// The pool keeps the contract of llm-scheduler/src/block_allocator.rs:8-80 (ids
// 0..capacity-1, FIFO free list, reference counts, double free and bad ids are errors).
// Unlike the reference (llm-scheduler/src/scheduler.rs:161-167 grows a table by one page
// after a step) pages are reserved before a step for exactly its tokens and the cached
// length moves at commit, so a step that fails leaves nothing behind.
#pragma once

#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

namespace llmrs_host {

enum Status : int { kOk = 0, kCacheError = 1, kOutOfPages = 2, kNoFreeSlot = 3, kBadArgument = 4 };

// Thrown inside the library, turned into a status and a message at the C boundary.
struct Failure {
    Status status;
    std::string message;
};

constexpr int32_t kReleased = -1;  // table entry of a page that a window has passed

class PagePool {
public:
    explicit PagePool(int capacity);
    int capacity() const { return capacity_; }
    int free_pages() const { return static_cast<int>(free_.size()); }
    int used_pages() const { return capacity_ - free_pages(); }
    int32_t allocate();
    void increment_ref(int32_t page);
    int ref_count(int32_t page) const;
    bool free(int32_t page);  // true if the page went back to the free list
    const std::deque<int32_t>& free_list() const { return free_; }

private:
    void check(int32_t page) const;
    int capacity_;
    std::deque<int32_t> free_;
    std::vector<int32_t> refs_;
};

struct Record {
    int64_t id = 0;
    int slot = 0;
    int cached_len = 0;
    int reserved_len = 0;  // tokens the tables cover (>= cached_len between reserve and commit)
    std::vector<std::vector<int32_t>> tables;  // per group: logical page -> physical page
    int64_t edits = 0;     // changes to the tables other than appending a page
};

class CacheManager {
public:
    // windows[g] == 0: the group keeps every key; > 0: only the last `window` keys are read.
    CacheManager(const int* n_pages, const int* windows, int n_groups, int page_size, int n_slots);

    int n_groups() const { return static_cast<int>(pools_.size()); }
    int page_size() const { return page_size_; }
    int n_slots() const { return n_slots_; }
    int n_live() const { return static_cast<int>(requests_.size()); }
    bool is_live(int64_t id) const { return requests_.count(id) != 0; }
    bool has_free_slot() const { return !free_slots_.empty(); }
    const PagePool& pool(int g) const;

    const Record& admit(int64_t id);
    const Record& record(int64_t id) const;
    void release(int64_t id);

    // Pages per group that reserve(id, n_new) would take. For a request that is not live
    // pass live = false and the cached length it would start from.
    void pages_needed(bool live, int64_t id, int n_new, int cached_len, int* out) const;
    bool can_reserve(bool live, int64_t id, int n_new, int cached_len) const;
    void reserve(int64_t id, int n_new);
    void cancel(int64_t id);
    void commit(int64_t id, int n_new);
    void check_invariants() const;

private:
    Record& record_mut(int64_t id);
    int first_needed_page(int g, int first_query_pos) const;

    int page_size_;
    int n_slots_;
    std::vector<PagePool> pools_;
    std::vector<int> windows_;
    std::vector<int> free_slots_;
    std::unordered_map<int64_t, Record> requests_;
};

// Where each array of a packed step lies in the step's int32 buffer.
enum StepArray : int {
    kTokenIds = 0, kPositions, kTokenReq, kQStart, kNNew, kCachedLen, kSlotIds, kWantRows,
    kPendDst, kPendSrc, kFirstTable  // kFirstTable + g: block table of group g
};

struct StepShape {
    int n_tokens = 0, n_requests = 0, n_want = 0;
    int64_t total = 0;  // int32 elements the packed step takes
};

// Packs the index arrays of one step that every part may read (tokens, positions, request rows,
// per-request lengths, wanted rows, pending device tokens, block tables padded to `table_round`
// pages) into `out`. What a mixer plans for itself (tiles, lists, cuts) is not in here: it comes
// from the mixer's own plan and is appended by the caller. Every array starts at a multiple of 4
// elements. offsets/sizes have kFirstTable + n_groups entries; widths has n_groups.
// Returns false, with shape->total set, when `capacity` is too small (nothing is written).
bool pack_step(const CacheManager& cm, int n_entries, const int64_t* ids, const int32_t* n_tokens,
               const int32_t* tokens, const int32_t* n_want, const int32_t* want,
               const int32_t* device_token, int table_round,
               int32_t* out, int64_t capacity, int64_t* offsets, int64_t* sizes, int32_t* widths,
               StepShape* shape);

// The plan of paged attention for one step, from the step's per-request numbers alone: requests
// that bring one token go to the decode list, longer portions are cut into tiles of `tile`
// queries (request row, offset of the tile's first query).
struct AttentionPlan {
    int n_tiles = 0, n_decode = 0;
    int max_decode_kv_len = 0;   // most keys a decoding request sees (its cached length + 1)
    int long_portions = 0;       // blocks of 128 queries would be at least half full on average
};

// tiles_out holds 2 * tiles_capacity ints, decode_out decode_capacity ints. Returns false (and only
// the counts in *plan) when either is too small.
bool plan_paged_attention(int n_requests, const int32_t* n_new, const int32_t* cached_len, int tile,
                          int32_t* tiles_out, int64_t tiles_capacity, int32_t* decode_out,
                          int64_t decode_capacity, AttentionPlan* plan);

}  // namespace llmrs_host
