// The scheduler's decisions: which requests run in the next step and with how many tokens.
// It knows requests by their lengths only (the tokens stay with the caller) and reads the cache
// manager without changing it: a request whose pages must go back is reported to the caller, who
// releases it, and counts as released here from that moment on.
//
// The reference (llm-scheduler/src/scheduler.rs:51-190) admits a request when pages for its whole
// prompt are free, runs every sequence in every step (whole prompt or one token) and drops a
// sequence without a word when a page is missing while it decodes (:168-171). Here: a token budget
// per step, decoded tokens first, then prompt portions in order of arrival; admission needs pages
// for the first portion only; when pages run out the request admitted last is preempted (it goes
// back to the front of the queue and is recomputed later); results may come back one step late.
#pragma once

#include <cstdint>
#include <deque>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "cache_manager.hpp"

namespace llmrs_host {

enum RequestStatus : int { kWaiting = 0, kRunning = 1, kFinished = 2 };
enum FinishReason : int { kNone = 0, kStop = 1, kLength = 2, kTooLong = 3, kStepFailed = 4 };

struct SchedRequest {
    int64_t id = 0;
    int prompt_len = 0;
    int n_output = 0;        // tokens generated and read back
    int n_computed = 0;      // tokens of prompt + output whose keys and values are cached (or queued)
    int n_inflight = 0;      // tokens sampled on the device that the caller has not read yet (0 or 1)
    int max_new_tokens = 0;
    bool ignore_eos = false;
    int status = kWaiting;
    int finish_reason = kNone;
    int preemptions = 0;
    int n_known() const { return prompt_len + n_output; }
    int remaining() const { return n_known() + n_inflight - n_computed; }
};

// One request's share of a step: tokens start .. start + n_tokens - 1 of prompt + output. `pending`:
// the single token is the one still in flight (start is -1).
struct SchedEntry {
    int64_t id;
    int start;
    int n_tokens;
    bool sample;     // the last of these tokens yields the request's next token
    bool pending;
};

struct SchedOutput {
    int64_t id;
    int token;       // -1: none (a request that ended without a token)
    bool finished;
    int reason;
};

class Scheduler {
public:
    Scheduler(const CacheManager* cm, int max_positions, const int32_t* eos, int n_eos, int max_tokens_per_step,
              int prefill_chunk, int max_requests_per_step);

    void add(int64_t id, int prompt_len, int max_new_tokens, bool ignore_eos);
    bool has_work() const { return !waiting_.empty() || !running_.empty() || !finished_early_.empty(); }
    // Decides the next step. Returns a handle for on_launched / on_result (0: nothing to run).
    int64_t schedule(std::vector<SchedEntry>* entries);
    void on_launched(int64_t batch);
    // The batch was decided but never queued (its pages were gone): forget it; its requests stay as they were.
    void cancel(int64_t batch);
    // `tokens`: one per entry with `sample`, in the batch's order. batch 0: only what ended without a step.
    void on_result(int64_t batch, const int32_t* tokens, int n_tokens, std::vector<SchedOutput>* outs);
    void abort_all(int reason, std::vector<SchedOutput>* outs);

    const SchedRequest& request(int64_t id) const;
    const std::deque<int64_t>& waiting() const { return waiting_; }
    const std::vector<int64_t>& running() const { return running_; }
    void stats(int64_t* steps, int64_t* preemptions, int64_t* tokens) const;
    // Requests whose pages the caller must give back now / whose state changed since the last call.
    void take_releases(std::vector<int64_t>* ids);
    void take_changed(std::vector<int64_t>* ids);
    void forget(int64_t id);   // drop a finished request's record

private:
    bool live(int64_t id) const { return cm_->is_live(id) && !released_.count(id); }
    bool fits(const SchedRequest& r, int n_new, std::vector<int>* free_pages) const;
    bool ends_by_length(const SchedRequest& r) const;
    void preempt_last(std::vector<int>* free_pages);
    void finish(SchedRequest& r, int reason);
    void try_schedule(std::vector<SchedEntry>* batch);
    SchedRequest& req(int64_t id);

    const CacheManager* cm_;
    int max_positions_, max_tokens_per_step_, prefill_chunk_, max_requests_per_step_;
    std::unordered_set<int32_t> eos_;
    std::unordered_map<int64_t, SchedRequest> requests_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;          // in order of admission
    std::vector<SchedOutput> finished_early_;
    std::vector<int64_t> to_release_, changed_;
    std::unordered_set<int64_t> released_;  // reported for release, still live in the manager
    std::unordered_map<int64_t, std::vector<SchedEntry>> batches_;
    int64_t next_batch_ = 1;
    int64_t stat_steps_ = 0, stat_preemptions_ = 0, stat_tokens_ = 0;
};

}  // namespace llmrs_host
