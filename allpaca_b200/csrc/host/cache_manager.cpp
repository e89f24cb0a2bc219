#include "cache_manager.hpp"

#include <algorithm>
#include <set>

namespace allpaca {

PagePool::PagePool(int num_pages) : held_((size_t)std::max(num_pages, 0), 0) {
    free_.reserve(held_.size());
    for (int p = (int)held_.size() - 1; p >= 0; --p) free_.push_back(p);
}

int PagePool::alloc() {
    if (free_.empty()) return -1;
    const int p = free_.back();
    free_.pop_back();
    held_[p] = 1;
    return p;
}

int PagePool::free(int page, std::string* error) {
    if (page < 0 || page >= num_pages()) {
        if (error) *error = "page " + std::to_string(page) + " is outside the pool of " + std::to_string(num_pages());
        return kMisuse;
    }
    if (!held_[page]) {
        if (error) *error = "page " + std::to_string(page) + " is freed twice";
        return kMisuse;
    }
    held_[page] = 0;
    free_.push_back(page);
    return kOk;
}

CacheManager::CacheManager(const std::vector<GroupLayout>& groups, int max_seqs)
    : groups_(groups), max_seqs_(max_seqs) {
    for (const auto& g : groups_) pools_.emplace_back(g.num_pages);
    for (int s = max_seqs - 1; s >= 0; --s) free_slots_.push_back(s);
}

int CacheManager::fail(int status, const std::string& what) const {
    error_ = what;
    return status;
}

const Sequence* CacheManager::find(int64_t req) const {
    auto it = seqs_.find(req);
    return it == seqs_.end() ? nullptr : &it->second;
}

int CacheManager::begin(int64_t req, int* slot) {
    if (seqs_.count(req)) return fail(kMisuse, "the request already holds a cache");
    if (free_slots_.empty()) return fail(kOutOfPages, "every state slot is taken");
    Sequence s;
    s.tables.resize(groups_.size());
    s.state_slot = free_slots_.back();
    free_slots_.pop_back();
    if (slot) *slot = s.state_slot;
    seqs_.emplace(req, std::move(s));
    return kOk;
}

int CacheManager::free(int64_t req) {
    auto it = seqs_.find(req);
    if (it == seqs_.end()) return fail(kMisuse, "the request holds no cache (freed twice?)");
    Sequence& s = it->second;
    for (size_t g = 0; g < s.tables.size(); ++g) {
        for (auto p = s.tables[g].rbegin(); p != s.tables[g].rend(); ++p) {
            if (*p == kFreed) continue;
            std::string why;
            if (pools_[g].free(*p, &why) != kOk) return fail(kMisuse, why);
        }
    }
    free_slots_.push_back(s.state_slot);
    seqs_.erase(it);
    return kOk;
}

int CacheManager::pages_missing(int64_t req, int64_t num_new, int* out) const {
    const Sequence* s = nullptr;
    if (req >= 0) {
        s = find(req);
        if (!s) return fail(kMisuse, "the request holds no cache");
    }
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int64_t have = s ? (int64_t)s->tables[g].size() : 0;
        const int64_t total = (s ? s->num_tokens : 0) + num_new;
        const int64_t need = (total + groups_[g].page_size - 1) / groups_[g].page_size;
        out[g] = (int)std::max<int64_t>(0, need - have);
    }
    return kOk;
}

bool CacheManager::can_append(int64_t req, int64_t num_new, const int* reserve) const {
    std::vector<int> miss(groups_.size());
    if (pages_missing(req, num_new, miss.data()) != kOk) return false;
    for (size_t g = 0; g < groups_.size(); ++g)
        if (miss[g] > pools_[g].num_free() - (reserve ? reserve[g] : 0)) return false;
    return true;
}

int CacheManager::append(int64_t req, int64_t num_new, int64_t* first_position) {
    if (num_new <= 0) return fail(kMisuse, "append needs at least one token");
    auto it = seqs_.find(req);
    if (it == seqs_.end()) return fail(kMisuse, "the request holds no cache");
    Sequence& s = it->second;
    std::vector<int> miss(groups_.size());
    pages_missing(req, num_new, miss.data());
    for (size_t g = 0; g < groups_.size(); ++g) {
        if (miss[g] > pools_[g].num_free())
            return fail(kOutOfPages, "group " + std::to_string(g) + " needs " + std::to_string(miss[g]) +
                                         " more pages, " + std::to_string(pools_[g].num_free()) + " are free");
    }
    for (size_t g = 0; g < groups_.size(); ++g)
        for (int i = 0; i < miss[g]; ++i) s.tables[g].push_back(pools_[g].alloc());
    if (first_position) *first_position = s.num_tokens;
    s.num_tokens += num_new;
    return kOk;
}

int CacheManager::release_passed(int64_t req, int* freed) {
    auto it = seqs_.find(req);
    if (it == seqs_.end()) return fail(kMisuse, "the request holds no cache");
    Sequence& s = it->second;
    int n = 0;
    for (size_t g = 0; g < groups_.size(); ++g) {
        const GroupLayout& l = groups_[g];
        if (l.window <= 0) continue;
        // the next row sits at position num_tokens and sees keys > num_tokens - window
        const int64_t first_visible = s.num_tokens - l.window + 1;
        if (first_visible <= 0) continue;
        const int64_t dead = std::min<int64_t>(first_visible / l.page_size, (int64_t)s.tables[g].size());
        for (int64_t j = 0; j < dead; ++j) {
            if (s.tables[g][j] == kFreed) continue;
            std::string why;
            if (pools_[g].free(s.tables[g][j], &why) != kOk) return fail(kMisuse, why);
            s.tables[g][j] = kFreed;
            ++n;
        }
    }
    if (freed) *freed = n;
    return kOk;
}

int CacheManager::check() {
    for (size_t g = 0; g < groups_.size(); ++g) {
        std::set<int> owned;
        for (const auto& kv : seqs_) {
            for (int p : kv.second.tables[g]) {
                if (p == kFreed) continue;
                if (!owned.insert(p).second)
                    return fail(kMisuse, "page " + std::to_string(p) + " of group " + std::to_string(g) + " is held twice");
                if (!pools_[g].held(p))
                    return fail(kMisuse, "page " + std::to_string(p) + " of group " + std::to_string(g) +
                                             " is in a block table but free in the pool");
            }
        }
        if ((int)owned.size() + pools_[g].num_free() != pools_[g].num_pages())
            return fail(kMisuse, "group " + std::to_string(g) + ": " + std::to_string(owned.size()) + " held + " +
                                     std::to_string(pools_[g].num_free()) + " free != " +
                                     std::to_string(pools_[g].num_pages()));
    }
    std::set<int> slots;
    for (const auto& kv : seqs_)
        if (!slots.insert(kv.second.state_slot).second) return fail(kMisuse, "a state slot is held twice");
    if ((int)slots.size() + (int)free_slots_.size() != max_seqs_) return fail(kMisuse, "state slots are lost");
    return kOk;
}

}  // namespace allpaca
