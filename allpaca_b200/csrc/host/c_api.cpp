// Flat C interface of the host library (called from Python through ctypes).  Handles are
// opaque pointers; every function returns a status (0 ok, 1 misuse, 2 out of pages) unless it
// says otherwise, and apc_last_error() gives the text of the last failure on this thread.
#include <cstring>
#include <string>
#include <vector>

#include "cache_manager.hpp"
#include "step_builder.hpp"

#define APC_EXPORT extern "C" __attribute__((visibility("default")))

using namespace allpaca;

static thread_local std::string g_error;

APC_EXPORT const char* apc_last_error() { return g_error.c_str(); }
APC_EXPORT int apc_abi_version() { return 1; }

// ---- page pool (exposed for tests of the pool alone) -----------------------------------
APC_EXPORT void* apc_pool_create(int num_pages) { return num_pages > 0 ? new PagePool(num_pages) : nullptr; }
APC_EXPORT void apc_pool_destroy(void* p) { delete (PagePool*)p; }
APC_EXPORT int apc_pool_alloc(void* p) { return ((PagePool*)p)->alloc(); }
APC_EXPORT int apc_pool_free(void* p, int page) { return ((PagePool*)p)->free(page, &g_error); }
APC_EXPORT int apc_pool_num_free(void* p) { return ((PagePool*)p)->num_free(); }
APC_EXPORT int apc_pool_held(void* p, int page) { return ((PagePool*)p)->held(page) ? 1 : 0; }

// ---- cache manager -----------------------------------------------------------------------
APC_EXPORT void* apc_cache_create(int ngroups, const int* page_size, const int* num_pages, const int* window,
                                  int max_seqs) {
    if (ngroups < 0 || ngroups > 8 || max_seqs <= 0) return nullptr;
    std::vector<GroupLayout> groups;
    for (int g = 0; g < ngroups; ++g) {
        if (page_size[g] <= 0 || num_pages[g] <= 0) return nullptr;
        groups.push_back({page_size[g], num_pages[g], window[g]});
    }
    return new CacheManager(groups, max_seqs);
}
APC_EXPORT void apc_cache_destroy(void* c) { delete (CacheManager*)c; }

static int done(CacheManager* c, int rc) {
    if (rc != kOk) g_error = c->error();
    return rc;
}
APC_EXPORT int apc_cache_begin(void* c, int64_t req, int* slot) { return done((CacheManager*)c, ((CacheManager*)c)->begin(req, slot)); }
APC_EXPORT int apc_cache_free(void* c, int64_t req) { return done((CacheManager*)c, ((CacheManager*)c)->free(req)); }
APC_EXPORT int apc_cache_has(void* c, int64_t req) { return ((CacheManager*)c)->has(req) ? 1 : 0; }
APC_EXPORT int apc_cache_num_running(void* c) { return ((CacheManager*)c)->num_running(); }
APC_EXPORT int apc_cache_can_begin(void* c) { return ((CacheManager*)c)->can_begin() ? 1 : 0; }
APC_EXPORT int apc_cache_num_free_pages(void* c, int g) { return ((CacheManager*)c)->num_free_pages(g); }
APC_EXPORT int64_t apc_cache_num_tokens(void* c, int64_t req) {
    const Sequence* s = ((CacheManager*)c)->find(req);
    return s ? s->num_tokens : -1;
}
APC_EXPORT int apc_cache_state_slot(void* c, int64_t req) {
    const Sequence* s = ((CacheManager*)c)->find(req);
    return s ? s->state_slot : -1;
}
APC_EXPORT int apc_cache_pages_missing(void* c, int64_t req, int64_t num_new, int* out) {
    return done((CacheManager*)c, ((CacheManager*)c)->pages_missing(req, num_new, out));
}
APC_EXPORT int apc_cache_can_append(void* c, int64_t req, int64_t num_new, const int* reserve) {
    return ((CacheManager*)c)->can_append(req, num_new, reserve) ? 1 : 0;
}
APC_EXPORT int apc_cache_append(void* c, int64_t req, int64_t num_new, int64_t* first) {
    return done((CacheManager*)c, ((CacheManager*)c)->append(req, num_new, first));
}
APC_EXPORT int apc_cache_release_passed(void* c, int64_t req, int* freed) {
    return done((CacheManager*)c, ((CacheManager*)c)->release_passed(req, freed));
}
APC_EXPORT int apc_cache_check(void* c) { return done((CacheManager*)c, ((CacheManager*)c)->check()); }
// length of the request's block table in group g (or -1); copies up to `cap` entries into out
APC_EXPORT int apc_cache_table(void* c, int64_t req, int g, int* out, int cap) {
    const Sequence* s = ((CacheManager*)c)->find(req);
    if (!s || g < 0 || g >= (int)s->tables.size()) return -1;
    const int n = (int)s->tables[g].size();
    if (out && cap > 0) std::memcpy(out, s->tables[g].data(), sizeof(int) * (size_t)(n < cap ? n : cap));
    return n;
}

// ---- one step's batch ----------------------------------------------------------------------
// layout_out: 5 int32 (T, nseq, R, max query, max context) then 8 + 8 int64 (total, 7 offsets,
// 8 table offsets) then 8 int32 widths, as the struct below.
struct ApcStepLayout {
    int32_t num_tokens, num_seqs, num_logit_rows, max_query_len, max_context_len, pad;
    int64_t total, off_tokens, off_positions, off_seq, off_start, off_context, off_slot, off_rows;
    int64_t off_table[8];
    int32_t width[8];
};
APC_EXPORT int apc_prepare_step(void* c, int vocab, int64_t max_model_len, int64_t max_batched_tokens, int nseq,
                                const int64_t* reqs, const int32_t* tok_off, const int32_t* tokens,
                                const int32_t* want_off, const int32_t* want, const int32_t* fixed_widths,
                                int32_t* buf, int64_t cap, ApcStepLayout* layout, int64_t* first_position,
                                int32_t* state_slot) {
    StepLimits lim{vocab, max_model_len, max_batched_tokens};
    StepLayout L;
    const int rc = prepare_step(*(CacheManager*)c, lim, nseq, reqs, tok_off, tokens, want_off, want, fixed_widths,
                                buf, cap, &L, first_position, state_slot, &g_error);
    if (rc != kOk) return rc;
    layout->num_tokens = L.num_tokens; layout->num_seqs = L.num_seqs; layout->num_logit_rows = L.num_logit_rows;
    layout->max_query_len = L.max_query_len; layout->max_context_len = L.max_context_len; layout->pad = 0;
    layout->total = L.total; layout->off_tokens = L.off_tokens; layout->off_positions = L.off_positions;
    layout->off_seq = L.off_seq; layout->off_start = L.off_start; layout->off_context = L.off_context;
    layout->off_slot = L.off_slot; layout->off_rows = L.off_rows;
    for (int g = 0; g < 8; ++g) { layout->off_table[g] = L.off_table[g]; layout->width[g] = L.width[g]; }
    return kOk;
}
