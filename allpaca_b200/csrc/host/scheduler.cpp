#include "scheduler.hpp"

#include <algorithm>
#include <vector>

namespace allpaca {

Scheduler::Scheduler(CacheManager* cache, int max_num_seqs, int64_t token_budget, int64_t prefill_chunk,
                     int64_t max_model_len)
    : cache_(cache), max_num_seqs_(max_num_seqs), token_budget_(token_budget), prefill_chunk_(prefill_chunk),
      max_model_len_(max_model_len), reserved_(cache->num_groups(), 0) {}

const SchedRequest* Scheduler::find(int64_t id) const {
    auto it = reqs_.find(id);
    return it == reqs_.end() ? nullptr : &it->second;
}

int Scheduler::add(int64_t id, int64_t prompt_len, int64_t max_tokens, const int* stop_ids, int num_stop) {
    if (reqs_.count(id)) {
        error_ = "request " + std::to_string(id) + " is already known to the scheduler";
        return kMisuse;
    }
    if (prompt_len <= 0) {
        error_ = "a request needs at least one prompt token";
        return kMisuse;
    }
    if (prompt_len >= max_model_len_) {
        error_ = "a prompt of " + std::to_string(prompt_len) + " tokens leaves no room under the model's length limit " +
                 std::to_string(max_model_len_);
        return kMisuse;
    }
    const int64_t longest = std::min(prompt_len + max_tokens, max_model_len_);
    for (int g = 0; g < cache_->num_groups(); ++g) {
        const GroupLayout& layout = cache_->group(g);
        int64_t need = (longest + layout.page_size - 1) / layout.page_size;
        if (layout.window > 0) {
            // a windowed group keeps at most the window plus one step's rows alive
            const int64_t span = layout.window + std::min(prefill_chunk_, token_budget_) + layout.page_size;
            need = std::min(need, (span + layout.page_size - 1) / layout.page_size + 1);
        }
        if (need > layout.num_pages) {
            error_ = "the request may hold " + std::to_string(longest) + " tokens = " + std::to_string(need) +
                     " pages of cache group " + std::to_string(g) + ", whose pool has " +
                     std::to_string(layout.num_pages);
            return kMisuse;
        }
    }
    SchedRequest r;
    r.id = id;
    r.prompt_len = prompt_len;
    r.max_tokens = max_tokens;
    r.arrival = arrivals_++;
    r.stop_ids.assign(stop_ids, stop_ids + (num_stop > 0 ? num_stop : 0));
    reqs_[id] = r;
    waiting_.push_back(id);
    return kOk;
}

int Scheduler::adopt_running(int64_t id, int64_t prompt_len, int64_t max_tokens, int64_t num_computed) {
    if (reqs_.count(id) || prompt_len <= 0 || num_computed < 0 || num_computed >= prompt_len) {
        error_ = "adopt_running: bad request " + std::to_string(id);
        return kMisuse;
    }
    SchedRequest r;
    r.id = id;
    r.prompt_len = prompt_len;
    r.max_tokens = max_tokens;
    r.num_computed = num_computed;
    r.arrival = arrivals_++;
    reqs_[id] = r;
    running_.push_back(id);
    return kOk;
}

bool Scheduler::fits(const SchedRequest& r, int64_t count) const {
    return cache_->can_append(key(r), count, reserved_.data());
}

void Scheduler::reserve(const SchedRequest& r, int64_t count) {
    std::vector<int> missing(cache_->num_groups(), 0);
    cache_->pages_missing(key(r), count, missing.data());
    for (int g = 0; g < cache_->num_groups(); ++g) reserved_[g] += missing[g];
}

// Whether a request that has not begun may be admitted with `left` tokens still to run: a group
// that keeps every key must have room for all of them now (else the request would be admitted
// only to be preempted); a group with a window needs room for the most it ever holds at once,
// the same bound add() checks, since pages the window has passed come back after every step.
bool Scheduler::admission_fits(int64_t left) const {
    for (int g = 0; g < cache_->num_groups(); ++g) {
        const GroupLayout& layout = cache_->group(g);
        int64_t tokens = left;
        if (layout.window > 0)
            tokens = std::min(left, (int64_t)layout.window + std::min(prefill_chunk_, token_budget_) + layout.page_size);
        const int64_t pages = (tokens + layout.page_size - 1) / layout.page_size;
        if (pages > cache_->num_free_pages(g) - reserved_[g]) return false;
    }
    return true;
}

// The most tokens up to `want` whose pages are free (0 if not even one).
int64_t Scheduler::largest_fit(const SchedRequest& r, int64_t want) const {
    if (want <= 0) return 0;
    if (fits(r, want)) return want;
    int64_t lo = 0, hi = want;              // fits(lo) holds or lo == 0
    while (lo < hi) {
        const int64_t mid = (lo + hi + 1) / 2;
        if (fits(r, mid)) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

int64_t Scheduler::youngest_running() const {
    int64_t best = running_.front();
    for (int64_t id : running_)
        if (reqs_.at(id).arrival > reqs_.at(best).arrival) best = id;
    return best;
}

void Scheduler::preempt(int64_t id) {
    running_.erase(std::find(running_.begin(), running_.end(), id));
    if (cache_->has(id)) cache_->free(id);
    SchedRequest& r = reqs_[id];
    r.num_computed = 0;
    r.preemptions += 1;
    waiting_.push_front(id);
    preempted_.push_back(id);
}

int Scheduler::schedule() {
    int64_t budget = token_budget_;
    rows_.clear();
    preempted_.clear();
    admitted_.clear();
    std::fill(reserved_.begin(), reserved_.end(), 0);

    // 1. decode rows of running requests, oldest first; preempt the youngest on shortage
    std::stable_sort(running_.begin(), running_.end(),
                     [&](int64_t a, int64_t b) { return reqs_.at(a).arrival < reqs_.at(b).arrival; });
    std::vector<int64_t> decoding;
    for (int64_t id : running_) {
        const SchedRequest& r = reqs_.at(id);
        if (r.num_tokens() - r.num_computed == 1) decoding.push_back(id);
    }
    size_t i = 0;
    while (i < decoding.size()) {
        if (budget <= 0) break;
        const int64_t id = decoding[i];
        const SchedRequest& r = reqs_.at(id);
        if (fits(r, 1)) {
            reserve(r, 1);
            rows_.push_back({id, r.num_computed, 1, 1});
            budget -= 1;
            ++i;
            continue;
        }
        const int64_t victim = youngest_running();
        preempt(victim);
        // drop rows already planned for the victim and what they had reserved
        bool had_rows = false;
        for (const ScheduledRows& row : rows_) had_rows = had_rows || row.id == victim;
        if (had_rows) {
            rows_.erase(std::remove_if(rows_.begin(), rows_.end(), [&](const ScheduledRows& row) { return row.id == victim; }),
                        rows_.end());
            budget = token_budget_;
            std::fill(reserved_.begin(), reserved_.end(), 0);
            for (const ScheduledRows& row : rows_) {
                budget -= row.count;
                reserve(reqs_.at(row.id), row.count);
            }
        }
        // the victim, being the youngest of all, lies at or after i: the rows before i stay put,
        // and if it was the one asking, the next request moves into its place
        decoding.erase(std::remove(decoding.begin(), decoding.end(), victim), decoding.end());
    }

    // 2. portions of running prompts; if every running request is starved of pages, preempt the
    //    youngest and try again
    while (true) {
        for (int64_t id : running_) {
            if (budget <= 0) break;
            const SchedRequest& r = reqs_.at(id);
            const int64_t left = r.num_tokens() - r.num_computed;
            if (left <= 1) continue;
            const int64_t count = largest_fit(r, std::min(std::min(left, budget), prefill_chunk_));
            if (count <= 0) continue;
            reserve(r, count);
            rows_.push_back({id, r.num_computed, count, count == left ? 1 : 0});
            budget -= count;
        }
        if (!rows_.empty() || running_.empty()) break;
        preempt(youngest_running());
    }

    // 3. admit waiting requests in order while all the tokens they hold would fit; stop at the
    //    first that does not
    while (!waiting_.empty() && budget > 0 && (int)running_.size() < max_num_seqs_ && cache_->can_begin()) {
        const int64_t id = waiting_.front();
        SchedRequest& r = reqs_[id];
        const int64_t left = r.num_tokens() - r.num_computed;
        if (!admission_fits(left)) break;
        const int64_t count = std::min(std::min(left, budget), prefill_chunk_);
        waiting_.pop_front();
        running_.push_back(id);
        admitted_.push_back(id);
        reserve(r, count);
        rows_.push_back({id, r.num_computed, count, count == left ? 1 : 0});
        budget -= count;
    }

    if (rows_.empty() && (!waiting_.empty() || !running_.empty()) && preempted_.empty()) {
        error_ = "the scheduler found nothing to run although requests are pending";
        return kMisuse;
    }
    return kOk;
}

int Scheduler::advance(const int* sampled, int num_sampled) {
    int need = 0;
    for (const ScheduledRows& row : rows_) need += row.samples;
    if (need != num_sampled) {
        error_ = "advance: " + std::to_string(need) + " rows were to be sampled, " + std::to_string(num_sampled) +
                 " tokens were given";
        return kMisuse;
    }
    if (!unresolved_.empty()) {
        error_ = "advance: an earlier step is not resolved yet";
        return kMisuse;
    }
    const int rc = advance_counts();
    return rc != kOk ? rc : resolve(sampled, num_sampled);
}

int Scheduler::advance_counts() {
    std::vector<int64_t> sampled_ids;
    for (const ScheduledRows& row : rows_) {
        auto it = reqs_.find(row.id);
        if (row.samples) sampled_ids.push_back(row.id);
        if (it == reqs_.end()) continue;          // ended by a stop token after this step was planned
        SchedRequest& r = it->second;
        r.num_computed += row.count;
        if (!row.samples) continue;
        r.output_len += 1;
        if (r.output_len >= r.max_tokens || r.num_tokens() >= max_model_len_) {
            r.closing = true;                     // no further step; its last token's value is still to come
            auto at = std::find(running_.begin(), running_.end(), row.id);
            if (at != running_.end()) running_.erase(at);
        }
    }
    unresolved_.push_back(std::move(sampled_ids));
    rows_.clear();
    return kOk;
}

int Scheduler::resolve(const int* sampled, int num_sampled) {
    finished_.clear();
    reasons_.clear();
    if (unresolved_.empty()) {
        error_ = "resolve: no step is waiting for its tokens";
        return kMisuse;
    }
    const std::vector<int64_t>& ids = unresolved_.front();
    if ((int)ids.size() != num_sampled) {
        error_ = "resolve: " + std::to_string(ids.size()) + " rows were sampled, " + std::to_string(num_sampled) +
                 " tokens were given";
        return kMisuse;
    }
    for (int k = 0; k < num_sampled; ++k) {
        auto it = reqs_.find(ids[k]);
        if (it == reqs_.end()) continue;          // already ended (a stop token one step earlier, or aborted)
        SchedRequest& r = it->second;
        // stop wins over length (crates/allpaca-core/src/engine.rs:4607-4621)
        int reason = kNotFinished;
        if (std::find(r.stop_ids.begin(), r.stop_ids.end(), sampled[k]) != r.stop_ids.end()) reason = kStop;
        else if (r.closing) reason = kLength;
        if (reason == kNotFinished) continue;
        finished_.push_back(ids[k]);
        reasons_.push_back(reason);
    }
    for (int64_t id : finished_) {
        auto at = std::find(running_.begin(), running_.end(), id);
        if (at != running_.end()) running_.erase(at);
        auto w = std::find(waiting_.begin(), waiting_.end(), id);
        if (w != waiting_.end()) waiting_.erase(w);
        reqs_.erase(id);
    }
    unresolved_.pop_front();
    return kOk;
}

int Scheduler::abort(int64_t id) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return 0;
    auto r = std::find(running_.begin(), running_.end(), id);
    if (r != running_.end()) running_.erase(r);
    auto w = std::find(waiting_.begin(), waiting_.end(), id);
    if (w != waiting_.end()) waiting_.erase(w);
    reqs_.erase(it);
    return 1;
}

std::vector<int64_t> Scheduler::list(int which) const {
    if (which == 0) return running_;
    return std::vector<int64_t>(waiting_.begin(), waiting_.end());
}

}  // namespace allpaca
