// Host-side bookkeeping of cache pages, block tables and state slots (no device memory).
//
// Keys and values live in fixed-size pages.  Layers with the same need form a group with a
// page pool of its own: a group keeps every key of a request, or only a trailing window of
// them, in which case pages the window has passed go back to the pool while the request is
// still running.  Each request has, per group, a block table: logical page index -> page id
// (FREED where the page was given back).  Beside the pages there are slots for per-request
// state of fixed size, one per running request.
//
// Role in the reference: KvTierManager page allocation and release
// (crates/allpaca-core/src/kv_tier.rs:341-474, :498-532), the per-request page lists of
// ActiveRequest (crates/allpaca-core/src/engine.rs:97) released on drop (engine.rs:409-432),
// growth by ensure_pages (crates/allpaca-core/src/model.rs:13452-13480) and the per-request
// recurrent state (crates/allpaca-core/src/anchors.rs:16-56).  The reference allocates a page
// per layer and evicts to slower tiers; here one page id addresses the same page in every
// layer of its group, there is one tier, and running out of pages is reported to the caller.
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace allpaca {

constexpr int kFreed = -1;

// status codes of the C interface
enum Status : int { kOk = 0, kMisuse = 1, kOutOfPages = 2 };

class PagePool {
public:
    explicit PagePool(int num_pages);
    int num_pages() const { return (int)held_.size(); }
    int num_free() const { return (int)free_.size(); }
    // page id, or -1 when the pool is empty
    int alloc();
    // kOk, or kMisuse with `error` set (outside the pool, freed twice)
    int free(int page, std::string* error);
    bool held(int page) const { return page >= 0 && page < num_pages() && held_[page]; }

private:
    std::vector<int> free_;       // last in, first out: a page just given back is handed out next
    std::vector<char> held_;
};

struct GroupLayout {
    int page_size;
    int num_pages;
    int window;                   // <= 0: keep everything
};

struct Sequence {
    std::vector<std::vector<int>> tables;
    int64_t num_tokens = 0;
    int state_slot = -1;
};

class CacheManager {
public:
    CacheManager(const std::vector<GroupLayout>& groups, int max_seqs);

    int num_groups() const { return (int)groups_.size(); }
    const GroupLayout& group(int g) const { return groups_[g]; }
    int num_free_pages(int g) const { return pools_[g].num_free(); }
    int num_running() const { return (int)seqs_.size(); }
    bool can_begin() const { return !free_slots_.empty(); }
    int free_state_slots() const { return (int)free_slots_.size(); }
    bool has(int64_t req) const { return seqs_.count(req) != 0; }
    const Sequence* find(int64_t req) const;

    // Every call returns a Status; on anything but kOk nothing has changed and error() tells why.
    int begin(int64_t req, int* slot);
    int free(int64_t req);
    // pages each group still has to allocate so that num_new more tokens fit (req < 0: a request
    // that has not begun)
    int pages_missing(int64_t req, int64_t num_new, int* out) const;
    bool can_append(int64_t req, int64_t num_new, const int* reserve) const;
    int append(int64_t req, int64_t num_new, int64_t* first_position);
    int release_passed(int64_t req, int* freed);
    // every page is free or held by exactly one request; slots likewise
    int check();

    const std::string& error() const { return error_; }

private:
    int fail(int status, const std::string& what) const;
    std::vector<GroupLayout> groups_;
    std::vector<PagePool> pools_;
    int max_seqs_;
    std::vector<int> free_slots_;
    std::unordered_map<int64_t, Sequence> seqs_;
    mutable std::string error_;
};

}  // namespace allpaca
