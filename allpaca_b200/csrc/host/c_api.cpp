// Flat C interface of the host library (called from Python through ctypes).  Handles are
// opaque pointers; every function returns a status (0 ok, 1 misuse, 2 out of pages) unless it
// says otherwise, and apc_last_error() gives the text of the last failure on this thread.
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "cache_manager.hpp"
#include "safetensors.hpp"
#include "scheduler.hpp"
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
    if (ngroups < 0 || max_seqs <= 0) return nullptr;
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
// layout: as the struct below; the block tables of the groups follow one another from off_tables,
// [nseq, widths[g]] each.  widths: [groups] output.
struct ApcStepLayout {
    int32_t num_tokens, num_seqs, num_logit_rows, max_query_len, max_context_len, pad;
    int64_t total, off_tokens, off_positions, off_seq, off_start, off_context, off_slot, off_rows;
    int64_t off_tables;
};
APC_EXPORT int apc_prepare_step(void* c, int vocab, int64_t max_model_len, int64_t max_batched_tokens, int nseq,
                                const int64_t* reqs, const int32_t* tok_off, const int32_t* tokens,
                                const int32_t* want_off, const int32_t* want, const int32_t* fixed_widths,
                                int32_t* buf, int64_t cap, ApcStepLayout* layout, int32_t* widths,
                                int64_t* first_position, int32_t* state_slot) {
    StepLimits lim{vocab, max_model_len, max_batched_tokens};
    StepLayout L;
    const int rc = prepare_step(*(CacheManager*)c, lim, nseq, reqs, tok_off, tokens, want_off, want, fixed_widths,
                                buf, cap, &L, widths, first_position, state_slot, &g_error);
    if (rc != kOk) return rc;
    layout->num_tokens = L.num_tokens; layout->num_seqs = L.num_seqs; layout->num_logit_rows = L.num_logit_rows;
    layout->max_query_len = L.max_query_len; layout->max_context_len = L.max_context_len; layout->pad = 0;
    layout->total = L.total; layout->off_tokens = L.off_tokens; layout->off_positions = L.off_positions;
    layout->off_seq = L.off_seq; layout->off_start = L.off_start; layout->off_context = L.off_context;
    layout->off_slot = L.off_slot; layout->off_rows = L.off_rows;
    layout->off_tables = L.off_tables;
    return kOk;
}

// ---- scheduler -----------------------------------------------------------------------------
APC_EXPORT void* aps_create(void* cache, int max_num_seqs, int64_t token_budget, int64_t prefill_chunk,
                            int64_t max_model_len) {
    if (!cache || max_num_seqs <= 0 || token_budget <= 0 || prefill_chunk <= 0 || max_model_len <= 0) return nullptr;
    return new Scheduler((CacheManager*)cache, max_num_seqs, token_budget, prefill_chunk, max_model_len);
}
APC_EXPORT void aps_destroy(void* s) { delete (Scheduler*)s; }
static int sdone(Scheduler* s, int rc) {
    if (rc != kOk) g_error = s->error();
    return rc;
}
APC_EXPORT int aps_add(void* s, int64_t id, int64_t prompt_len, int64_t max_tokens, const int* stop_ids, int num_stop) {
    return sdone((Scheduler*)s, ((Scheduler*)s)->add(id, prompt_len, max_tokens, stop_ids, num_stop));
}
APC_EXPORT int aps_adopt_running(void* s, int64_t id, int64_t prompt_len, int64_t max_tokens, int64_t num_computed) {
    return sdone((Scheduler*)s, ((Scheduler*)s)->adopt_running(id, prompt_len, max_tokens, num_computed));
}
APC_EXPORT int aps_has_unfinished(void* s) { return ((Scheduler*)s)->has_unfinished() ? 1 : 0; }
// Plans a step.  counts[0..2] receive the numbers of rows, preempted and admitted requests.
APC_EXPORT int aps_schedule(void* s, int* counts) {
    Scheduler* sc = (Scheduler*)s;
    const int rc = sdone(sc, sc->schedule());
    counts[0] = (int)sc->rows().size();
    counts[1] = (int)sc->preempted().size();
    counts[2] = (int)sc->admitted().size();
    return rc;
}
// The planned step: rows as (id, start, count, samples) quadruples, then the ids preempted and admitted.
APC_EXPORT void aps_planned(void* s, int64_t* rows, int64_t* preempted, int64_t* admitted) {
    Scheduler* sc = (Scheduler*)s;
    size_t k = 0;
    for (const ScheduledRows& r : sc->rows()) {
        rows[k++] = r.id;
        rows[k++] = r.start;
        rows[k++] = r.count;
        rows[k++] = r.samples;
    }
    std::copy(sc->preempted().begin(), sc->preempted().end(), preempted);
    std::copy(sc->admitted().begin(), sc->admitted().end(), admitted);
}
// Records the step; *num_finished receives how many requests are done.
APC_EXPORT int aps_advance(void* s, const int* sampled, int num_sampled, int* num_finished) {
    Scheduler* sc = (Scheduler*)s;
    const int rc = sdone(sc, sc->advance(sampled, num_sampled));
    *num_finished = rc == kOk ? (int)sc->finished().size() : 0;
    return rc;
}
// The two halves of aps_advance (see Scheduler::advance_counts and Scheduler::resolve).
APC_EXPORT int aps_advance_counts(void* s) { return sdone((Scheduler*)s, ((Scheduler*)s)->advance_counts()); }
APC_EXPORT int aps_resolve(void* s, const int* sampled, int num_sampled, int* num_finished) {
    Scheduler* sc = (Scheduler*)s;
    const int rc = sdone(sc, sc->resolve(sampled, num_sampled));
    *num_finished = rc == kOk ? (int)sc->finished().size() : 0;
    return rc;
}
APC_EXPORT int aps_unresolved_steps(void* s) { return ((Scheduler*)s)->unresolved_steps(); }
APC_EXPORT void aps_finished(void* s, int64_t* ids, int* reasons) {
    Scheduler* sc = (Scheduler*)s;
    std::copy(sc->finished().begin(), sc->finished().end(), ids);
    std::copy(sc->reasons().begin(), sc->reasons().end(), reasons);
}
APC_EXPORT int aps_abort(void* s, int64_t id) { return ((Scheduler*)s)->abort(id); }
// running (which = 0) or waiting (1) ids in their order; returns how many there are
APC_EXPORT int aps_list(void* s, int which, int64_t* out, int cap) {
    const std::vector<int64_t> v = ((Scheduler*)s)->list(which);
    for (int i = 0; i < (int)v.size() && i < cap; ++i) out[i] = v[i];
    return (int)v.size();
}

// ---- safetensors files ---------------------------------------------------------------------
// apst_open gives a handle, or null with the reason in apc_last_error(); the pointers handed out
// (names, types, the data) live as long as the handle.
APC_EXPORT void* apst_open(const char* path) {
    std::string why;
    SafetensorsFile* f = SafetensorsFile::open(path ? path : "", &why);
    if (!f) g_error = why;
    return f;
}
APC_EXPORT void apst_close(void* h) { delete (SafetensorsFile*)h; }
APC_EXPORT int apst_num_tensors(void* h) { return (int)((SafetensorsFile*)h)->tensors().size(); }
static const TensorEntry* entry(void* h, int i) {
    const auto& t = ((SafetensorsFile*)h)->tensors();
    return i >= 0 && (size_t)i < t.size() ? &t[(size_t)i] : nullptr;
}
APC_EXPORT const char* apst_name(void* h, int i) { const TensorEntry* e = entry(h, i); return e ? e->name.c_str() : nullptr; }
APC_EXPORT const char* apst_dtype(void* h, int i) { const TensorEntry* e = entry(h, i); return e ? e->dtype.c_str() : nullptr; }
APC_EXPORT int apst_ndim(void* h, int i) { const TensorEntry* e = entry(h, i); return e ? (int)e->shape.size() : -1; }
APC_EXPORT int apst_shape(void* h, int i, int64_t* out, int cap) {
    const TensorEntry* e = entry(h, i);
    if (!e || (int)e->shape.size() > cap) return -1;
    std::copy(e->shape.begin(), e->shape.end(), out);
    return (int)e->shape.size();
}
APC_EXPORT int64_t apst_begin(void* h, int i) { const TensorEntry* e = entry(h, i); return e ? e->begin : -1; }
APC_EXPORT int64_t apst_end(void* h, int i) { const TensorEntry* e = entry(h, i); return e ? e->end : -1; }
APC_EXPORT const void* apst_data(void* h) { return ((SafetensorsFile*)h)->data(); }
APC_EXPORT int64_t apst_data_len(void* h) { return ((SafetensorsFile*)h)->data_len(); }
APC_EXPORT int apst_num_metadata(void* h) { return (int)((SafetensorsFile*)h)->metadata().size(); }
APC_EXPORT const char* apst_metadata_key(void* h, int i) {
    const auto& m = ((SafetensorsFile*)h)->metadata();
    return i >= 0 && (size_t)i < m.size() ? m[(size_t)i].first.c_str() : nullptr;
}
APC_EXPORT const char* apst_metadata_value(void* h, int i) {
    const auto& m = ((SafetensorsFile*)h)->metadata();
    return i >= 0 && (size_t)i < m.size() ? m[(size_t)i].second.c_str() : nullptr;
}
