// Continuous batching: which requests run which tokens in the next step (host side only).
//
// Every step is one batch under a token budget: first one row for each running request that
// is decoding, then portions of running prompts, then newly admitted requests, in order of
// arrival.  A prompt is cut into portions of at most `prefill_chunk` tokens and whatever the
// budget leaves.  A request's last scheduled row yields logits (and a sampled token) only
// when the step completes everything the request holds so far.
//
// When pages run out: a row that cannot get its page makes the scheduler preempt the running
// request that arrived last (possibly the one asking): its pages and state slot are given
// back, and it returns to the head of the waiting queue to be recomputed later with the
// tokens it has already produced kept as part of its prompt.  A prompt portion that does not
// fit is shortened to the pages that are free, or waits.  A request that could never fit in
// an empty pool is refused when it is added, so one request can always run to its end.
//
// The scheduler knows requests by the number the cache manager knows them by; it never sees
// token values except the one sampled per finished row, which it compares with the request's
// stop tokens.
//
// Role in the reference: admission in begin_request with a hard cap and no queue
// (crates/allpaca-core/src/engine.rs:3198), one prefill chunk per tick (:4717, :4756), the
// fair pick of pick_runnable (crates/allpaca-core/src/scheduler.rs:647-664), batched decode of
// all plain decoders (engine.rs:5451-5560) and finish reasons (:4607-4621).  The reference
// never mixes a prompt chunk with decode rows (engine.rs:5430) and never preempts (it spills
// pages to slower tiers, crates/allpaca-core/src/kv_tier.rs:1939-1961).
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "cache_manager.hpp"

namespace allpaca {

enum FinishReason : int { kNotFinished = 0, kStop = 1, kLength = 2 };

struct SchedRequest {
    int64_t id = 0;
    int64_t prompt_len = 0;      // tokens given with the request
    int64_t output_len = 0;      // tokens sampled so far
    int64_t num_computed = 0;    // tokens whose keys and values are in the cache
    int64_t max_tokens = 0;
    int64_t arrival = 0;
    int preemptions = 0;
    bool closing = false;        // reached its length limit; waits for the value of its last token
    std::vector<int> stop_ids;
    int64_t num_tokens() const { return prompt_len + output_len; }
};

struct ScheduledRows {
    int64_t id;
    int64_t start;               // index of the first scheduled token among the request's tokens
    int64_t count;
    int samples;                 // the last row completes the request's tokens: sample from it
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, int max_num_seqs, int64_t token_budget, int64_t prefill_chunk,
              int64_t max_model_len);

    // kOk, or kMisuse with error() set when the request can never run (or the id is in use)
    int add(int64_t id, int64_t prompt_len, int64_t max_tokens, const int* stop_ids, int num_stop);
    // a request that already holds `num_computed` tokens of cache joins the running ones
    int adopt_running(int64_t id, int64_t prompt_len, int64_t max_tokens, int64_t num_computed);
    bool has_unfinished() const { return !waiting_.empty() || !running_.empty() || !unresolved_.empty(); }

    // Plans the next step.  kOk, or kMisuse when nothing can run although requests are pending.
    int schedule();
    const std::vector<ScheduledRows>& rows() const { return rows_; }
    const std::vector<int64_t>& preempted() const { return preempted_; }     // in the order it happened
    const std::vector<int64_t>& admitted() const { return admitted_; }

    // Records the planned step: its rows are now cached; `sampled` holds one token per row with
    // `samples`, in the order of rows().  finished()/reasons() name the requests that are done;
    // their cache is the caller's to free.  It is advance_counts() followed by resolve().
    int advance(const int* sampled, int num_sampled);
    // The same in two halves, for a caller that launches the next step before the tokens of
    // this one have reached the host.  advance_counts(): the planned step has been launched;
    // its rows count as cached and every sampled row's request as one token longer.  Requests
    // that thereby reach their length limit are planned no more.  resolve(): the token values
    // of the oldest step not yet resolved, one per sampled row in order; decides who is done
    // (a stop token ends a request, also one that a later step has already been planned for:
    // that row is then run for nothing and its token must be dropped by the caller).
    int advance_counts();
    int resolve(const int* sampled, int num_sampled);
    int unresolved_steps() const { return (int)unresolved_.size(); }
    const std::vector<int64_t>& finished() const { return finished_; }
    const std::vector<int>& reasons() const { return reasons_; }

    // 1 when the request was running or waiting and is now gone (its cache is the caller's to free)
    int abort(int64_t id);
    // running (which = 0) or waiting (1) requests in their order
    std::vector<int64_t> list(int which) const;
    const SchedRequest* find(int64_t id) const;

    const std::string& error() const { return error_; }

private:
    bool fits(const SchedRequest& r, int64_t count) const;
    bool admission_fits(int64_t left) const;
    void reserve(const SchedRequest& r, int64_t count);
    int64_t largest_fit(const SchedRequest& r, int64_t want) const;
    void preempt(int64_t id);
    int64_t youngest_running() const;
    int64_t key(const SchedRequest& r) const { return cache_->has(r.id) ? r.id : -1; }

    CacheManager* cache_;
    int max_num_seqs_;
    int64_t token_budget_, prefill_chunk_, max_model_len_;
    std::unordered_map<int64_t, SchedRequest> reqs_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;
    int64_t arrivals_ = 0;
    std::vector<int> reserved_;
    std::vector<ScheduledRows> rows_;
    std::vector<int64_t> preempted_, admitted_, finished_;
    std::vector<int> reasons_;
    std::deque<std::vector<int64_t>> unresolved_;     // per launched step: the requests of its sampled rows
    std::string error_;
};

}  // namespace allpaca
