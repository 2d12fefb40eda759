#include "scheduler.hpp"

#include <algorithm>
#include <string>

namespace llmrs_host {

namespace {
[[noreturn]] void fail(Status s, std::string msg) { throw Failure{s, std::move(msg)}; }
}

Scheduler::Scheduler(const CacheManager* cm, int max_positions, const int32_t* eos, int n_eos,
                     int max_tokens_per_step, int prefill_chunk, int max_requests_per_step)
    : cm_(cm), max_positions_(max_positions), max_tokens_per_step_(max_tokens_per_step),
      prefill_chunk_(prefill_chunk), max_requests_per_step_(max_requests_per_step) {
    if (cm == nullptr) fail(kBadArgument, "the scheduler needs a cache manager");
    if (max_tokens_per_step < 1 || prefill_chunk < 1 || max_requests_per_step < 1)
        fail(kBadArgument, "token budget, portion size and requests per step must be positive");
    for (int i = 0; i < n_eos; ++i) eos_.insert(eos[i]);
}

SchedRequest& Scheduler::req(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) fail(kBadArgument, "the scheduler does not know request #" + std::to_string(id));
    return it->second;
}

const SchedRequest& Scheduler::request(int64_t id) const { return const_cast<Scheduler*>(this)->req(id); }

void Scheduler::add(int64_t id, int prompt_len, int max_new_tokens, bool ignore_eos) {
    if (prompt_len < 1) fail(kBadArgument, "a request needs at least one prompt token");
    if (prompt_len >= max_positions_)
        fail(kBadArgument, "prompt of " + std::to_string(prompt_len) + " tokens leaves no room under the limit of " +
                               std::to_string(max_positions_) + " positions");
    if (requests_.count(id) && requests_[id].status != kFinished)
        fail(kBadArgument, "request #" + std::to_string(id) + " is already scheduled");
    SchedRequest r;
    r.id = id;
    r.prompt_len = prompt_len;
    r.max_new_tokens = max_new_tokens;
    r.ignore_eos = ignore_eos;
    requests_[id] = r;
    waiting_.push_back(id);
}

void Scheduler::forget(int64_t id) {
    auto it = requests_.find(id);
    if (it != requests_.end() && it->second.status == kFinished && it->second.n_inflight == 0) requests_.erase(it);
}

void Scheduler::stats(int64_t* steps, int64_t* preemptions, int64_t* tokens) const {
    *steps = stat_steps_;
    *preemptions = stat_preemptions_;
    *tokens = stat_tokens_;
}

void Scheduler::take_releases(std::vector<int64_t>* ids) {
    ids->swap(to_release_);
    to_release_.clear();
    released_.clear();   // the caller releases them before it calls again
}

void Scheduler::take_changed(std::vector<int64_t>* ids) {
    ids->swap(changed_);
    changed_.clear();
}

// -- pages ----------------------------------------------------------------------------------
bool Scheduler::fits(const SchedRequest& r, int n_new, std::vector<int>* free_pages) const {
    std::vector<int> need(free_pages->size());
    cm_->pages_needed(live(r.id), r.id, n_new, 0, need.data());
    for (size_t g = 0; g < need.size(); ++g)
        if (need[g] > (*free_pages)[g]) return false;
    for (size_t g = 0; g < need.size(); ++g) (*free_pages)[g] -= need[g];
    return true;
}

// Sends the request admitted last back to the front of the waiting queue; its pages count as free.
void Scheduler::preempt_last(std::vector<int>* free_pages) {
    if (running_.empty()) return;
    SchedRequest& victim = req(running_.back());
    running_.pop_back();
    if (live(victim.id)) {
        const Record& rec = cm_->record(victim.id);
        for (size_t g = 0; g < rec.tables.size() && g < free_pages->size(); ++g)
            for (int32_t page : rec.tables[g])
                if (page != kReleased) ++(*free_pages)[g];
        to_release_.push_back(victim.id);
        released_.insert(victim.id);
    }
    victim.n_computed = 0;
    victim.status = kWaiting;
    ++victim.preemptions;
    ++stat_preemptions_;
    waiting_.push_front(victim.id);
    changed_.push_back(victim.id);
}

void Scheduler::finish(SchedRequest& r, int reason) {
    r.status = kFinished;
    r.finish_reason = reason;
    auto in_running = std::find(running_.begin(), running_.end(), r.id);
    if (in_running != running_.end()) {
        running_.erase(in_running);
    } else {
        // it was preempted while its last token was in flight
        auto in_waiting = std::find(waiting_.begin(), waiting_.end(), r.id);
        if (in_waiting != waiting_.end()) waiting_.erase(in_waiting);
    }
    if (live(r.id)) {
        to_release_.push_back(r.id);
        released_.insert(r.id);
    }
    changed_.push_back(r.id);
}

// True when the tokens already sampled (read or not) complete the request.
bool Scheduler::ends_by_length(const SchedRequest& r) const {
    const int n_out = r.n_output + r.n_inflight;
    return n_out >= r.max_new_tokens || r.prompt_len + n_out >= max_positions_;
}

// -- one step -------------------------------------------------------------------------------
int64_t Scheduler::schedule(std::vector<SchedEntry>* entries) {
    entries->clear();
    while (true) {
        try_schedule(entries);
        if (!entries->empty() || running_.empty()) break;
        // Nothing to run. Either every running request only waits for tokens that are in flight,
        // or requests are running and none could get its pages.
        bool stuck = false;
        for (int64_t id : running_) {
            const SchedRequest& r = req(id);
            if (r.remaining() >= 1 && !ends_by_length(r)) stuck = true;
        }
        if (!stuck) break;
        if (running_.size() == 1) {
            SchedRequest& r = req(running_[0]);
            finish(r, kTooLong);
            finished_early_.push_back({r.id, -1, true, kTooLong});
        } else {
            std::vector<int> none(cm_->n_groups(), 0);
            preempt_last(&none);
        }
    }
    if (entries->empty()) return 0;
    const int64_t handle = next_batch_++;
    batches_[handle] = *entries;
    return handle;
}

void Scheduler::try_schedule(std::vector<SchedEntry>* batch) {
    batch->clear();
    std::vector<int> free_pages(cm_->n_groups());
    for (int g = 0; g < cm_->n_groups(); ++g) free_pages[g] = cm_->pool(g).free_pages();
    // Pages of requests that were reported for release in this call are free for the plan.
    for (int64_t id : released_) {
        if (!cm_->is_live(id)) continue;
        const Record& rec = cm_->record(id);
        for (size_t g = 0; g < rec.tables.size(); ++g)
            for (int32_t page : rec.tables[g])
                if (page != kReleased) ++free_pages[g];
    }
    int budget = max_tokens_per_step_;

    // 1. decoding requests, in order of admission; make room by preempting from the back
    size_t i = 0;
    while (i < running_.size() && budget >= 1 && static_cast<int>(batch->size()) < max_requests_per_step_) {
        SchedRequest& r = req(running_[i]);
        if (r.remaining() != 1 || ends_by_length(r)) {
            ++i;
            continue;
        }
        bool ok = fits(r, 1, &free_pages);
        while (!ok && running_.back() != r.id) {
            preempt_last(&free_pages);
            ok = fits(r, 1, &free_pages);
        }
        if (!ok) break;   // r is the last one running; schedule() decides what becomes of it
        if (r.n_inflight)
            batch->push_back({r.id, -1, 1, true, true});
        else
            batch->push_back({r.id, r.n_known() - 1, 1, true, false});
        --budget;
        ++i;
    }

    // 2. running requests that still have prompt left, in order of admission
    for (int64_t id : running_) {
        SchedRequest& r = req(id);
        if (r.remaining() > 1 && budget >= 1 && static_cast<int>(batch->size()) < max_requests_per_step_) {
            const int n = std::min({r.n_known() - r.n_computed, prefill_chunk_, budget});   // known tokens only
            if (n >= 1 && fits(r, n, &free_pages)) {
                batch->push_back({r.id, r.n_computed, n, r.n_computed + n == r.n_known() && !r.n_inflight, false});
                budget -= n;
            }
        }
    }

    // 3. admit from the front of the waiting queue while a slot, budget and pages last
    // Slots that are free, those of requests reported for release in this call among them.
    int slots = cm_->n_slots() - cm_->n_live() + static_cast<int>(std::count_if(
        released_.begin(), released_.end(), [&](int64_t id) { return cm_->is_live(id); }));
    while (!waiting_.empty() && budget >= 1 && slots > 0 && static_cast<int>(batch->size()) < max_requests_per_step_) {
        SchedRequest& r = req(waiting_.front());
        const int n = std::min({r.n_known() - r.n_computed, prefill_chunk_, budget});
        if (!fits(r, n, &free_pages)) {
            if (running_.empty() && batch->empty()) {
                // Nothing else holds pages: this request can never start.
                waiting_.pop_front();
                finish(r, kTooLong);
                finished_early_.push_back({r.id, -1, true, kTooLong});
                continue;
            }
            break;   // the queue waits behind its head (llm-scheduler/src/scheduler.rs:86-89)
        }
        waiting_.pop_front();
        r.status = kRunning;
        running_.push_back(r.id);
        changed_.push_back(r.id);
        --slots;
        batch->push_back({r.id, r.n_computed, n, r.n_computed + n == r.n_known() && !r.n_inflight, false});
        budget -= n;
    }
}

// The step is queued on the GPU: its tokens count as computed, its samples as in flight.
void Scheduler::on_launched(int64_t batch) {
    auto it = batches_.find(batch);
    if (it == batches_.end()) fail(kBadArgument, "unknown batch " + std::to_string(batch));
    ++stat_steps_;
    for (const SchedEntry& e : it->second) {
        SchedRequest& r = req(e.id);
        r.n_computed += e.n_tokens;
        stat_tokens_ += e.n_tokens;
        if (e.sample) ++r.n_inflight;
        changed_.push_back(e.id);
    }
}

void Scheduler::cancel(int64_t batch) { batches_.erase(batch); }

void Scheduler::on_result(int64_t batch, const int32_t* tokens, int n_tokens, std::vector<SchedOutput>* outs) {
    outs->clear();
    outs->swap(finished_early_);
    finished_early_.clear();
    if (batch == 0) return;
    auto it = batches_.find(batch);
    if (it == batches_.end()) fail(kBadArgument, "unknown batch " + std::to_string(batch));
    int at = 0;
    for (const SchedEntry& e : it->second) {
        if (!e.sample) continue;
        if (at >= n_tokens) fail(kBadArgument, "fewer tokens than entries that sample");
        const int token = tokens[at++];
        SchedRequest& r = req(e.id);
        --r.n_inflight;
        changed_.push_back(e.id);
        if (r.status == kFinished) continue;   // it had ended at EOS one step earlier: this token is one too many
        ++r.n_output;
        int reason = kNone;
        if (eos_.count(token) && !r.ignore_eos)
            reason = kStop;            // the EOS token is emitted (scheduler.rs:150-156)
        else if (r.n_output >= r.max_new_tokens)
            reason = kLength;
        else if (r.prompt_len + r.n_output >= max_positions_)
            reason = kLength;
        if (reason != kNone) finish(r, reason);
        outs->push_back({r.id, token, reason != kNone, reason});
    }
    batches_.erase(it);
}

// A step failed: every running request ends and gives its pages back
// (llm-scheduler/src/engine.rs:92-99, scheduler.rs:193-200).
void Scheduler::abort_all(int reason, std::vector<SchedOutput>* outs) {
    outs->clear();
    const std::vector<int64_t> ids = running_;
    for (int64_t id : ids) {
        SchedRequest& r = req(id);
        finish(r, reason);
        outs->push_back({id, -1, true, reason});
    }
    // No step that was scheduled or queued before the failure will be reported any more: close their
    // batches and count nothing as in flight, so that the finished requests can be forgotten.
    batches_.clear();
    for (auto& kv : requests_) {
        if (kv.second.n_inflight) changed_.push_back(kv.first);
        kv.second.n_inflight = 0;
    }
}

}  // namespace llmrs_host
