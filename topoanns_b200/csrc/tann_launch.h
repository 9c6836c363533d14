// Host-side launch functions of the kernels (internal to the library).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "topoanns_b200.h"

namespace tann {

struct Cand;
struct BeamArgs;

size_t BeamSmemBytes(uint32_t M, uint32_t C, uint32_t F, uint32_t L, uint32_t d);
cudaError_t LaunchBeam(const BeamArgs& a, size_t smem, uint32_t grid, cudaStream_t stream);
cudaError_t BeamOccupancy(uint32_t M, uint32_t slots, size_t smem, int* blocks_per_sm);

cudaError_t LaunchLutBuild(const float* tables_col_major, const float* centroid,
                           const uint32_t* chunk_offsets, uint32_t dim, uint32_t M,
                           const void* queries, uint32_t query_kind, uint64_t Q, float* out,
                           cudaStream_t stream);

cudaError_t LaunchRvqNorms(const float* rows, uint32_t count, uint32_t dim, float* out,
                           cudaStream_t stream);
cudaError_t LaunchRvqEntries(const float* queries, uint64_t Q, uint32_t dim, const float* coarse,
                             const float* coarse_t, const float* coarse_norms, uint32_t nc,
                             const float* fine_t, const float* fine_norms, uint32_t nf,
                             const int32_t* bucket_sizes, const uint32_t* cluster_offsets,
                             const uint32_t* cluster_ids, uint32_t entry_count, uint32_t fallback,
                             int32_t* out_clusters, uint32_t* out_entry_ids,
                             uint32_t* out_entry_offsets, cudaStream_t stream,
                             uint32_t* status = nullptr /* dev: TANN_STATUS_* bits are or-ed in */);

cudaError_t LaunchPq2Refine(const void* cand, const uint32_t* stats, uint64_t Q, uint32_t capacity,
                            uint32_t refine_top_l, const TannShards* base_codes,
                            const TannShards& pq2_codes, uint32_t M, const float* lut2,
                            const float* cross_terms, void* out, cudaStream_t stream,
                            /* with lut2 == nullptr the table entries are computed from these instead */
                            const float* t2_col_major = nullptr, const float* mu2 = nullptr,
                            const uint32_t* chunk_offsets = nullptr, const float* queries_f32 = nullptr,
                            uint32_t dim = 0,
                            /* hybrid PQ: bit m of a node's selector row picks lut_outlier for chunk m */
                            const uint8_t* selector_bits = nullptr, uint32_t selector_stride = 0,
                            const float* lut_outlier = nullptr);
cudaError_t LaunchCrossTerms(uint32_t dim, uint32_t M, const uint32_t* chunk_offsets, const float* t1,
                             const float* mu1, const float* t2, const float* mu2, float* out,
                             cudaStream_t stream);

cudaError_t LaunchRerank(const TannIndexView& ix, const TannRerankParams& p, const void* cand,
                         uint32_t capacity, uint64_t Q, const void* queries, uint32_t query_kind,
                         const float* error_bounds, float* out_dists, uint32_t* out_ids,
                         unsigned long long* out_counts, cudaStream_t stream,
                         const uint8_t* queries_u8 = nullptr, const uint32_t* not_u8_flag = nullptr,
                         uint32_t final_ranks = 0 /* > 0: only the first final_ranks (<= 32) entries of every
                                                     output list are produced (the smallest, in order) */,
                         uint32_t* status = nullptr /* dev: TANN_STATUS_* bits are or-ed in */);
// Rerank with the learned stop / stage schedule / stop-prefix replay; out lists are [Q][top_k].
cudaError_t LaunchRerankLearned(const TannIndexView& ix, const TannRerankParams& p, const TannRerankLearnedStop& model,
                                bool use_schedule, bool evaluate, const void* cand, uint32_t capacity, uint64_t Q,
                                const void* queries, uint32_t query_kind, const float* error_bounds,
                                const uint32_t* replay_stop_prefixes, float* out_dists, uint32_t* out_ids,
                                unsigned long long* out_counts, uint32_t* out_stop_prefixes,
                                uint32_t* out_checkpoint_counts, uint32_t* out_stop_flags, cudaStream_t stream,
                                uint32_t* status = nullptr);
cudaError_t LaunchF32ToU8Checked(const float* src, uint64_t n, uint8_t* dst, uint32_t* not_u8_flag,
                                 cudaStream_t stream);
cudaError_t LaunchTopkPack(const float* dists, const uint32_t* ids, uint64_t Q, uint32_t top_n,
                           uint32_t top_k, float* out_dists, uint32_t* out_ids, cudaStream_t stream);

cudaError_t LaunchNeighborCodes(const TannIndexView& ix, uint64_t first_node, uint64_t num_rows, uint8_t* out,
                                cudaStream_t stream);

int SmCount();

// Argument checks shared by the rerank entry points (messages start with `who`); they set tann_last_error.
TannStatus CheckShards(const TannShards& s, uint64_t rows, const char* name);
TannStatus CheckRerank(const char* who, const TannIndexView* index, const TannRerankParams* params,
                       const float* error_bounds);

}  // namespace tann
