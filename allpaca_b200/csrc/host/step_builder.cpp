// Builds one step's batch on the host: checks the rows, makes room for them in the cache and
// fills the metadata buffer the kernels read (one block of 32-bit integers, copied to the
// device in one go).
//
// Layout of the block, in this order: token ids [T], positions [T], sequence index of each row
// [T], first row of each sequence [nseq+1], tokens held after the step [nseq], state slot [nseq],
// rows whose logits are wanted [R], then per cache group a block table [nseq, width_g].
//
// Role in the reference: SeqRows and the concatenated token list of forward_batch
// (crates/allpaca-core/src/model.rs:36-42, :8839-8848, :10865-10885) with the token check of
// :8215-8219 and page growth by ensure_pages (:13452-13480).
#include <algorithm>
#include <cstring>
#include <string>
#include <unordered_set>
#include <vector>

#include "cache_manager.hpp"
#include "step_builder.hpp"

namespace allpaca {

// fixed_widths: block-table widths to use (graph replay keeps them constant) or nullptr for the
// narrowest that fits.  widths: [groups] output, the width used for each group's table.
// first_position / state_slot: [nseq] outputs.
int prepare_step(CacheManager& cache, const StepLimits& lim, int nseq, const int64_t* reqs,
                 const int32_t* tok_off, const int32_t* tokens, const int32_t* want_off, const int32_t* want,
                 const int32_t* fixed_widths, int32_t* buf, int64_t cap, StepLayout* out, int32_t* widths,
                 int64_t* first_position, int32_t* state_slot, std::string* error) {
    auto fail = [&](int status, const std::string& what) {
        *error = what;
        return status;
    };
    if (nseq <= 0) return fail(kMisuse, "a step needs at least one entry");
    const int G = cache.num_groups();
    std::unordered_set<int64_t> seen;
    int64_t T = 0, R = 0;
    int fresh = 0;
    std::vector<int> reserve(G, 0), miss(G);
    for (int s = 0; s < nseq; ++s) {
        if (!seen.insert(reqs[s]).second) return fail(kMisuse, "a request appears twice in one step");
        const int n = tok_off[s + 1] - tok_off[s];
        if (n <= 0) return fail(kMisuse, "a request brings no tokens");
        for (int i = tok_off[s]; i < tok_off[s + 1]; ++i)
            if (tokens[i] < 0 || tokens[i] >= lim.vocab_size)
                return fail(kMisuse, "token " + std::to_string(tokens[i]) + " out of vocab " +
                                         std::to_string(lim.vocab_size));
        for (int i = want_off[s]; i < want_off[s + 1]; ++i)
            if (want[i] < 0 || want[i] >= n)
                return fail(kMisuse, "a request wants row " + std::to_string(want[i]) + " of " + std::to_string(n));
        const Sequence* seq = cache.find(reqs[s]);
        const int64_t held = seq ? seq->num_tokens : 0;
        if (held + n > lim.max_model_len)
            return fail(kMisuse, "a request would hold " + std::to_string(held + n) + " tokens, the model takes " +
                                     std::to_string(lim.max_model_len));
        if (!seq) ++fresh;
        cache.pages_missing(seq ? reqs[s] : -1, n, miss.data());
        for (int g = 0; g < G; ++g) reserve[g] += miss[g];
        T += n;
        R += want_off[s + 1] - want_off[s];
    }
    if (T > lim.max_batched_tokens)
        return fail(kMisuse, std::to_string(T) + " rows exceed max_num_batched_tokens " +
                                 std::to_string(lim.max_batched_tokens));
    // nothing is changed unless everything fits
    for (int g = 0; g < G; ++g)
        if (reserve[g] > cache.num_free_pages(g))
            return fail(kOutOfPages, "the cache pools cannot hold this step's tokens");
    if (fresh > cache.free_state_slots())
        return fail(kOutOfPages, std::to_string(fresh) + " new requests beside " + std::to_string(cache.num_running()) +
                                     " running ones exceed the state slots");

    for (int s = 0; s < nseq; ++s) {
        int slot = -1;
        if (!cache.has(reqs[s])) {
            const int rc = cache.begin(reqs[s], &slot);
            if (rc != kOk) return fail(rc, cache.error());
        }
        const int rc = cache.append(reqs[s], tok_off[s + 1] - tok_off[s], &first_position[s]);
        if (rc != kOk) return fail(rc, cache.error());
        state_slot[s] = cache.find(reqs[s])->state_slot;
    }

    StepLayout L;
    std::memset(&L, 0, sizeof(L));
    L.num_tokens = (int32_t)T;
    L.num_seqs = nseq;
    L.num_logit_rows = (int32_t)R;
    std::vector<int32_t> width(G);
    std::vector<int64_t> off_table(G);
    for (int g = 0; g < G; ++g) {
        int w = 0;
        if (fixed_widths) {
            w = fixed_widths[g];
        } else {
            for (int s = 0; s < nseq; ++s) w = std::max(w, (int)cache.find(reqs[s])->tables[g].size());
        }
        width[g] = w;
    }
    int64_t o = 0;
    L.off_tokens = o; o += T;
    L.off_positions = o; o += T;
    L.off_seq = o; o += T;
    L.off_start = o; o += nseq + 1;
    L.off_context = o; o += nseq;
    L.off_slot = o; o += nseq;
    L.off_rows = o; o += R;
    L.off_tables = o;
    for (int g = 0; g < G; ++g) {
        off_table[g] = o;
        o += (int64_t)nseq * width[g];
    }
    L.total = o;
    if (o > cap) return fail(kMisuse, "the staging buffer of " + std::to_string(cap) + " integers is too small for " +
                                          std::to_string(o));
    int64_t row = 0, out_row = 0;
    for (int s = 0; s < nseq; ++s) {
        const int n = tok_off[s + 1] - tok_off[s];
        const Sequence* seq = cache.find(reqs[s]);
        std::memcpy(buf + L.off_tokens + row, tokens + tok_off[s], sizeof(int32_t) * n);
        for (int i = 0; i < n; ++i) {
            buf[L.off_positions + row + i] = (int32_t)(first_position[s] + i);
            buf[L.off_seq + row + i] = s;
        }
        for (int i = want_off[s]; i < want_off[s + 1]; ++i) buf[L.off_rows + out_row++] = (int32_t)(row + want[i]);
        buf[L.off_start + s] = (int32_t)row;
        buf[L.off_context + s] = (int32_t)(first_position[s] + n);
        buf[L.off_slot + s] = seq->state_slot;
        for (int g = 0; g < G; ++g) {
            const auto& table = seq->tables[g];
            int32_t* dst = buf + off_table[g] + (int64_t)s * width[g];
            const int have = std::min((int)table.size(), (int)width[g]);
            if ((int)table.size() > width[g]) return fail(kMisuse, "a block table is wider than the fixed width");
            std::memcpy(dst, table.data(), sizeof(int32_t) * have);
            for (int j = have; j < width[g]; ++j) dst[j] = kFreed;
        }
        row += n;
        L.max_query_len = std::max(L.max_query_len, (int32_t)n);
        L.max_context_len = std::max(L.max_context_len, (int32_t)(first_position[s] + n));
    }
    buf[L.off_start + nseq] = (int32_t)row;
    std::copy(width.begin(), width.end(), widths);
    *out = L;
    return kOk;
}

}  // namespace allpaca
