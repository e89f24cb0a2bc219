// One step's batch: limits, the layout of the metadata block, and the function that checks a
// step's rows, makes room for them in the cache and fills the block (see step_builder.cpp).
#pragma once
#include <cstdint>
#include <string>

#include "cache_manager.hpp"

namespace allpaca {

struct StepLimits {
    int vocab_size;
    int64_t max_model_len;
    int64_t max_batched_tokens;
};

struct StepLayout {
    int32_t num_tokens, num_seqs, num_logit_rows;
    int32_t max_query_len, max_context_len;
    int64_t total;                       // integers used
    int64_t off_tokens, off_positions, off_seq, off_start, off_context, off_slot, off_rows;
    int64_t off_tables;                  // the block tables follow one another from here: [nseq, width_g] each
};

int prepare_step(CacheManager& cache, const StepLimits& lim, int nseq, const int64_t* reqs,
                 const int32_t* tok_off, const int32_t* tokens, const int32_t* want_off, const int32_t* want,
                 const int32_t* fixed_widths, int32_t* buf, int64_t cap, StepLayout* out, int32_t* widths,
                 int64_t* first_position, int32_t* state_slot, std::string* error);

}  // namespace allpaca
