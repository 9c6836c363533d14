// Argument block of the beam-search kernel (passed by value as a grid constant).
#pragma once

#include "tann_common.cuh"

namespace tann {

struct BeamArgs {
    TannIndexView ix;
    TannBeamParams p;
    const float* lut;        // [Q][M][256] or nullptr (build in kernel)
    const void* queries;     // [Q][dim] of query_kind (needed when lut == nullptr)
    uint32_t query_kind;
    uint32_t frontier_capacity;  // F = nextpow2(W * degree)
    uint64_t num_queries;
    const uint32_t* entry_offsets;
    const uint32_t* entry_ids;
    Cand* out_cand;
    uint32_t* out_stats;
    uint32_t* status;
};

}  // namespace tann
