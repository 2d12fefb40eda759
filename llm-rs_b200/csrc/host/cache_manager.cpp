#include "cache_manager.hpp"

#include <algorithm>
#include <unordered_set>

namespace llmrs_host {

namespace {
[[noreturn]] void fail(Status s, std::string msg) { throw Failure{s, std::move(msg)}; }
int pages_for(int n_tokens, int page_size) { return (n_tokens + page_size - 1) / page_size; }
std::string req(int64_t id) { return "request #" + std::to_string(id); }
}  // namespace

// ---------------------------------------------------------------- page pool
PagePool::PagePool(int capacity) : capacity_(capacity), refs_(capacity > 0 ? capacity : 0, 0) {
    if (capacity < 0) fail(kBadArgument, "capacity must not be negative");
    for (int i = 0; i < capacity; ++i) free_.push_back(i);
}

void PagePool::check(int32_t page) const {
    if (page < 0 || page >= capacity_) fail(kCacheError, "invalid page id " + std::to_string(page));
}

int32_t PagePool::allocate() {
    if (free_.empty()) fail(kOutOfPages, "out of pages in the cache pool");
    int32_t page = free_.front();
    free_.pop_front();
    refs_[page] = 1;
    return page;
}

void PagePool::increment_ref(int32_t page) {
    check(page);
    if (refs_[page] == 0) fail(kCacheError, "cannot share page " + std::to_string(page) + ": it is not allocated");
    ++refs_[page];
}

int PagePool::ref_count(int32_t page) const {
    check(page);
    return refs_[page];
}

bool PagePool::free(int32_t page) {
    check(page);
    if (refs_[page] == 0) fail(kCacheError, "double free of page " + std::to_string(page));
    if (--refs_[page] == 0) {
        free_.push_back(page);
        return true;
    }
    return false;
}

// ---------------------------------------------------------------- cache manager
CacheManager::CacheManager(const int* n_pages, const int* windows, int n_groups, int page_size, int n_slots)
    : page_size_(page_size), n_slots_(n_slots) {
    if (page_size < 1) fail(kBadArgument, "page_size must be positive");
    if (n_groups < 0 || n_slots < 0) fail(kBadArgument, "group and slot counts must not be negative");
    for (int g = 0; g < n_groups; ++g) {
        pools_.emplace_back(n_pages[g]);
        windows_.push_back(windows[g] > 0 ? windows[g] : 0);
    }
    for (int s = n_slots - 1; s >= 0; --s) free_slots_.push_back(s);
}

const PagePool& CacheManager::pool(int g) const {
    if (g < 0 || g >= n_groups()) fail(kBadArgument, "no cache group " + std::to_string(g));
    return pools_[g];
}

const Record& CacheManager::admit(int64_t id) {
    if (is_live(id)) fail(kCacheError, req(id) + " is already live");
    if (free_slots_.empty()) fail(kNoFreeSlot, "all " + std::to_string(n_slots_) + " request slots are taken");
    Record rec;
    rec.id = id;
    rec.slot = free_slots_.back();
    free_slots_.pop_back();
    rec.tables.resize(pools_.size());
    return requests_.emplace(id, std::move(rec)).first->second;
}

const Record& CacheManager::record(int64_t id) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) fail(kCacheError, req(id) + " is not live");
    return it->second;
}

Record& CacheManager::record_mut(int64_t id) { return const_cast<Record&>(record(id)); }

void CacheManager::release(int64_t id) {
    Record& rec = record_mut(id);
    for (size_t g = 0; g < rec.tables.size(); ++g)
        for (int32_t page : rec.tables[g])
            if (page != kReleased) pools_[g].free(page);
    free_slots_.push_back(rec.slot);
    requests_.erase(id);
}

// Logical page of the oldest key that a query at first_query_pos reads.
int CacheManager::first_needed_page(int g, int first_query_pos) const {
    int window = windows_[g];
    if (window <= 0) return 0;
    return std::max(0, first_query_pos - window + 1) / page_size_;
}

void CacheManager::pages_needed(bool live, int64_t id, int n_new, int cached_len, int* out) const {
    const Record* rec = live ? &record(id) : nullptr;
    int base = rec ? rec->cached_len : std::max(cached_len, 0);
    int total = pages_for(base + n_new, page_size_);
    for (int g = 0; g < n_groups(); ++g) {
        int have = rec ? static_cast<int>(rec->tables[g].size()) : 0;
        // Logical pages below `first` are never read: they need no physical page even if
        // they were never allocated (a window group joined late by a long portion).
        int first = first_needed_page(g, base);
        out[g] = std::max(0, total - std::max(have, first));
    }
}

bool CacheManager::can_reserve(bool live, int64_t id, int n_new, int cached_len) const {
    std::vector<int> need(pools_.size());
    pages_needed(live, id, n_new, cached_len, need.data());
    for (int g = 0; g < n_groups(); ++g)
        if (need[g] > pools_[g].free_pages()) return false;
    return true;
}

void CacheManager::reserve(int64_t id, int n_new) {
    Record& rec = record_mut(id);
    if (n_new < 1) fail(kCacheError, "a step must bring at least one token for a request");
    if (rec.reserved_len != rec.cached_len) fail(kCacheError, req(id) + " has an uncommitted reservation");
    std::vector<int> need(pools_.size());
    pages_needed(true, id, n_new, 0, need.data());
    for (int g = 0; g < n_groups(); ++g)
        if (need[g] > pools_[g].free_pages())
            fail(kOutOfPages, req(id) + " needs " + std::to_string(need[g]) + " pages in group " +
                                  std::to_string(g) + ", " + std::to_string(pools_[g].free_pages()) + " free");
    int total = pages_for(rec.cached_len + n_new, page_size_);
    for (int g = 0; g < n_groups(); ++g) {
        int first = first_needed_page(g, rec.cached_len);
        auto& table = rec.tables[g];
        while (static_cast<int>(table.size()) < total)
            table.push_back(static_cast<int>(table.size()) < first ? kReleased : pools_[g].allocate());
    }
    rec.reserved_len = rec.cached_len + n_new;
}

void CacheManager::cancel(int64_t id) {
    Record& rec = record_mut(id);
    size_t keep = static_cast<size_t>(pages_for(rec.cached_len, page_size_));
    ++rec.edits;
    for (size_t g = 0; g < rec.tables.size(); ++g) {
        auto& table = rec.tables[g];
        while (table.size() > keep) {
            int32_t page = table.back();
            table.pop_back();
            if (page != kReleased) pools_[g].free(page);
        }
    }
    rec.reserved_len = rec.cached_len;
}

void CacheManager::commit(int64_t id, int n_new) {
    Record& rec = record_mut(id);
    if (rec.cached_len + n_new != rec.reserved_len)
        fail(kCacheError, "commit of " + std::to_string(n_new) + " tokens does not match the reservation of " + req(id));
    rec.cached_len = rec.reserved_len;
    for (int g = 0; g < n_groups(); ++g) {
        auto& table = rec.tables[g];
        int first = std::min(first_needed_page(g, rec.cached_len), static_cast<int>(table.size()));
        for (int j = 0; j < first; ++j)
            if (table[j] != kReleased) {
                pools_[g].free(table[j]);
                table[j] = kReleased;
                ++rec.edits;
            }
    }
}

void CacheManager::check_invariants() const {
    for (int g = 0; g < n_groups(); ++g) {
        const PagePool& pool = pools_[g];
        std::unordered_map<int32_t, int> held;
        for (const auto& kv : requests_)
            for (int32_t page : kv.second.tables[g])
                if (page != kReleased) ++held[page];
        std::unordered_set<int32_t> free_set(pool.free_list().begin(), pool.free_list().end());
        std::string group = "group " + std::to_string(g) + ": ";
        if (free_set.size() != pool.free_list().size()) fail(kCacheError, group + "a page is on the free list twice");
        for (const auto& kv : held)
            if (free_set.count(kv.first)) fail(kCacheError, group + "a page is both free and held");
        if (static_cast<int>(free_set.size() + held.size()) != pool.capacity())
            fail(kCacheError, group + std::to_string(pool.capacity() - static_cast<int>(free_set.size() + held.size())) +
                                  " pages are lost");
        for (const auto& kv : held)
            if (pool.ref_count(kv.first) != kv.second)
                fail(kCacheError, group + "page " + std::to_string(kv.first) + " is held " + std::to_string(kv.second) +
                                      " times, count says " + std::to_string(pool.ref_count(kv.first)));
    }
    std::unordered_set<int> slots;
    for (const auto& kv : requests_)
        if (!slots.insert(kv.second.slot).second) fail(kCacheError, "a request slot is held twice");
    for (int s : free_slots_)
        if (!slots.insert(s).second) fail(kCacheError, "a request slot is held twice");
    if (static_cast<int>(slots.size()) != n_slots_) fail(kCacheError, "a request slot is lost");
}

}  // namespace llmrs_host
