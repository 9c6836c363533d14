// C ABI of the library: argument checks, launches, and the searcher that chains the whole path.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <cmath>
#include <fstream>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "beam_args.h"
#include "tann_launch.h"
#include "topoanns_b200.h"

namespace {

thread_local char g_error[512] = "";

TannStatus Fail(TannStatus st, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return st;
}

TannStatus CudaFail(cudaError_t e, const char* what) {
    return Fail(TANN_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define TANN_CUDA(call)                                   \
    do {                                                  \
        cudaError_t e__ = (call);                         \
        if (e__ != cudaSuccess) return CudaFail(e__, #call); \
    } while (0)

// True for host memory the driver knows as page-locked (cudaHostAlloc, cudaHostRegister).
bool IsPageLocked(const void* p) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return attr.type == cudaMemoryTypeHost;
}

uint32_t NextPow2(uint32_t v) {
    uint32_t p = 1;
    while (p < v) p <<= 1;
    return p;
}

}  // namespace
namespace tann {
TannStatus CheckShards(const TannShards& s, uint64_t rows, const char* name) {
    if (s.num_shards == 0 || s.num_shards > TANN_MAX_SHARDS)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: num_shards must be 1..%d.", name, TANN_MAX_SHARDS);
    for (uint32_t i = 0; i < s.num_shards; ++i)
        if (s.base[i] == nullptr) return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: shard %u has no base pointer.", name, i);
    if (s.num_shards > 1 && (s.rows_per_shard == 0 || s.rows_per_shard * s.num_shards < rows))
        return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: shards do not cover all rows.", name);
    return TANN_OK;
}
}  // namespace tann
namespace {
using tann::CheckShards;

// Rows that the kernels read with 16-byte loads must start on 16-byte boundaries.
TannStatus CheckShardAlignment(const TannShards& s, const char* name) {
    for (uint32_t i = 0; i < s.num_shards && i < TANN_MAX_SHARDS; ++i)
        if ((reinterpret_cast<uintptr_t>(s.base[i]) & 15u) != 0)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: %s shard %u must be 16-byte aligned.", name, i);
    return TANN_OK;
}

// Parameter rules of the reference: src/search/topology_search.cpp:16-35,
// src/search/topology_search_kernel.cu:3193-3206.
TannStatus CheckBeam(const TannIndexView* ix, const TannBeamParams* p) {
    if (ix == nullptr || p == nullptr) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: null index or params.");
    if (p->top_l == 0) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: top_l must be positive.");
    if (p->search_width == 0) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: search_width must be positive.");
    if (p->search_width > TANN_MAX_SEARCH_WIDTH)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: search_width must be at most 32.");
    if (p->max_expansions == 0) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: max_expansions must be positive.");
    if (ix->num_nodes >= 0x7fffffffull)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: packed node_id requires num_nodes < 2^31 - 1.");
    if (p->candidate_capacity < p->top_l || (p->candidate_capacity & (p->candidate_capacity - 1)) != 0)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: candidate_capacity must be a power of two >= top_l.");
    if (ix->degree == 0 || ix->num_chunks == 0)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: degree and num_chunks must be positive.");
    if ((uint64_t)p->search_width * ix->degree > 2048)
        return Fail(TANN_ERR_UNSUPPORTED, "tann_beam_search: search_width * degree must be at most 2048.");
    if (p->learned_stop.enabled && (p->learned_stop.top_k == 0 || p->learned_stop.top_k > 32 ||
                                    p->learned_stop.num_stages > TANN_MAX_STOP_STAGES))
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: learned stop needs 1 <= top_k <= 32 and at most 32 stages.");
    TannStatus st = CheckShards(ix->adjacency, ix->num_nodes, "adjacency");
    if (st != TANN_OK) return st;
    return CheckShards(ix->codes, ix->num_nodes, "codes");
}

struct BeamPlan {
    uint32_t F;
    size_t smem;
    int blocks_per_sm;
    uint32_t grid;
};

TannStatus PlanBeam(const TannIndexView* ix, const TannBeamParams* p, bool lut_in_kernel, uint64_t Q,
                    BeamPlan* plan) {
    (void)lut_in_kernel;
    const uint32_t slots = p->search_width * ix->degree;
    plan->F = NextPow2(slots == 0 ? 1 : slots);
    plan->smem = tann::BeamSmemBytes(ix->num_chunks, p->candidate_capacity, plan->F, p->top_l, ix->dim);
    int dev = 0, max_optin = 0;
    TANN_CUDA(cudaGetDevice(&dev));
    TANN_CUDA(cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    if (plan->smem > (size_t)max_optin)
        return Fail(TANN_ERR_UNSUPPORTED,
                    "tann_beam_search: shared memory requirement (%zu bytes) is too large for this device (%d).",
                    plan->smem, max_optin);
    TANN_CUDA(tann::BeamOccupancy(ix->num_chunks, slots, plan->smem, &plan->blocks_per_sm));
    if (plan->blocks_per_sm < 1) plan->blocks_per_sm = 1;
    const uint64_t resident = (uint64_t)tann::SmCount() * plan->blocks_per_sm;
    // One block per query: queries differ in length, and the hardware block scheduler starts the next
    // one wherever a block retires (measured 4-5 % faster than a resident grid with a query stride).
    // An occupancy query (Q == ~0) reports the resident grid.
    if (Q == ~0ull) plan->grid = (uint32_t)resident;
    else plan->grid = (uint32_t)(Q == 0 ? 1 : (Q < 0x7fffffffull ? Q : 0x7fffffffull));
    return TANN_OK;
}

}  // namespace

namespace tann {
void SetLastError(const char* message) { Fail(TANN_OK, "%s", message); }

int SmCount() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}
}  // namespace tann

extern "C" {

const char* tann_version(void) { return "topoanns_b200 0.1 (sm_100a)"; }
const char* tann_last_error(void) { return g_error; }

TannStatus tann_lut_build(const float* tables_col_major, const float* centroid,
                          const uint32_t* chunk_offsets, uint32_t dim, uint32_t num_chunks,
                          const void* queries, uint32_t query_kind, uint64_t num_queries,
                          float* out_tables, tann_stream_t stream) {
    if (dim == 0 || num_chunks == 0) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_lut_build: PQ index is empty.");
    if (query_kind > TANN_KIND_FLOAT32) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_lut_build: unknown query kind.");
    if (num_queries == 0) return TANN_OK;
    if (!tables_col_major || !centroid || !chunk_offsets || !queries || !out_tables)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_lut_build: null pointer.");
    if (((reinterpret_cast<uintptr_t>(tables_col_major) | reinterpret_cast<uintptr_t>(out_tables)) & 15u) != 0)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_lut_build: pivots and output tables must be 16-byte aligned.");
    TANN_CUDA(tann::LaunchLutBuild(tables_col_major, centroid, chunk_offsets, dim, num_chunks, queries,
                                   query_kind, num_queries, out_tables, (cudaStream_t)stream));
    return TANN_OK;
}

TannStatus tann_beam_search(const TannIndexView* index, const TannBeamParams* params, const float* lut,
                            const void* queries, uint32_t query_kind, uint64_t num_queries,
                            const uint32_t* entry_offsets, const uint32_t* entry_ids,
                            void* out_candidates, uint32_t* out_stats, uint32_t* status,
                            tann_stream_t stream) {
    TannStatus st = CheckBeam(index, params);
    if (st != TANN_OK) return st;
    if (num_queries == 0) return TANN_OK;
    if (lut == nullptr) {
        if (queries == nullptr || query_kind > TANN_KIND_FLOAT32)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: queries are needed when no table is given.");
        if (!index->pq_tables_col_major || !index->pq_centroid || !index->pq_chunk_offsets)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: PQ index must be loaded before search.");
        if ((reinterpret_cast<uintptr_t>(index->pq_tables_col_major) & 15u) != 0)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: PQ pivots must be 16-byte aligned.");
    }
    if (!entry_offsets || !entry_ids || !out_candidates || !out_stats)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: null pointer.");
    if (lut != nullptr && (reinterpret_cast<uintptr_t>(lut) & 15u) != 0)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_beam_search: the query tables must be 16-byte aligned.");
    if (index->num_chunks % 16 == 0) {   // chunk counts with a 16-byte code row take 16-byte loads
        st = CheckShardAlignment(index->codes, "codes");
        if (st != TANN_OK) return st;
        if (index->neighbor_codes.base[0] != nullptr) {
            if (index->neighbor_codes.num_shards == 0 || index->neighbor_codes.num_shards > TANN_MAX_SHARDS)
                return Fail(TANN_ERR_INVALID_ARGUMENT, "neighbor_codes: num_shards must be 1..%d.", TANN_MAX_SHARDS);
            st = CheckShardAlignment(index->neighbor_codes, "neighbor_codes");
            if (st != TANN_OK) return st;
        }
    }
    BeamPlan plan;
    st = PlanBeam(index, params, lut == nullptr, num_queries, &plan);
    if (st != TANN_OK) return st;
    tann::BeamArgs a;
    memset(&a, 0, sizeof(a));
    a.ix = *index;
    a.p = *params;
    a.lut = lut;
    a.queries = queries;
    a.query_kind = query_kind;
    a.frontier_capacity = plan.F;
    a.num_queries = num_queries;
    a.entry_offsets = entry_offsets;
    a.entry_ids = entry_ids;
    a.out_cand = static_cast<tann::Cand*>(out_candidates);
    a.out_stats = out_stats;
    a.status = status;
    TANN_CUDA(tann::LaunchBeam(a, plan.smem, plan.grid, (cudaStream_t)stream));
    return TANN_OK;
}

TannStatus tann_beam_search_occupancy(const TannIndexView* index, const TannBeamParams* params,
                                      int lut_in_kernel, uint32_t* smem_bytes, uint32_t* blocks_per_sm,
                                      uint32_t* grid_blocks) {
    TannStatus st = CheckBeam(index, params);
    if (st != TANN_OK) return st;
    BeamPlan plan;
    st = PlanBeam(index, params, lut_in_kernel != 0, ~0ull, &plan);
    if (st != TANN_OK) return st;
    if (smem_bytes) *smem_bytes = (uint32_t)plan.smem;
    if (blocks_per_sm) *blocks_per_sm = (uint32_t)plan.blocks_per_sm;
    if (grid_blocks) *grid_blocks = plan.grid;
    return TANN_OK;
}

TannStatus tann_rvq_norms(const float* rows, uint32_t count, uint32_t dim, float* out_norms,
                          tann_stream_t stream) {
    if (count == 0) return TANN_OK;
    if (!rows || !out_norms || dim == 0) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_rvq_norms: null pointer or zero dim.");
    TANN_CUDA(tann::LaunchRvqNorms(rows, count, dim, out_norms, (cudaStream_t)stream));
    return TANN_OK;
}

TannStatus tann_rvq_entries(const float* queries, uint64_t num_queries, uint32_t dim, const float* coarse,
                            const float* coarse_t, const float* coarse_norms, uint32_t num_coarse,
                            const float* fine_t, const float* fine_norms, uint32_t num_fine,
                            const int32_t* bucket_sizes, const uint32_t* cluster_offsets,
                            const uint32_t* cluster_ids, uint32_t entry_count, uint32_t fallback_entry,
                            int32_t* out_clusters, uint32_t* out_entry_ids, uint32_t* out_entry_offsets,
                            tann_stream_t stream) {
    if (entry_count == 0) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_rvq_entries: entry_count must be positive.");
    if (num_queries == 0) return TANN_OK;
    if (!queries || !coarse || !coarse_t || !coarse_norms || !fine_t || !fine_norms || !bucket_sizes ||
        !cluster_offsets || !cluster_ids || !out_entry_ids || dim == 0 || num_coarse == 0 || num_fine == 0)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_rvq_entries: model is not loaded.");
    if (num_queries * entry_count > 0xffffffffull)
        return Fail(TANN_ERR_UNSUPPORTED, "tann_rvq_entries: entry offsets overflow uint32.");
    TANN_CUDA(tann::LaunchRvqEntries(queries, num_queries, dim, coarse, coarse_t, coarse_norms, num_coarse,
                                     fine_t, fine_norms, num_fine, bucket_sizes, cluster_offsets,
                                     cluster_ids, entry_count, fallback_entry, out_clusters, out_entry_ids,
                                     out_entry_offsets, (cudaStream_t)stream));
    return TANN_OK;
}

TannStatus tann_pq2_refine(const void* candidates, const uint32_t* stats, uint64_t num_queries,
                           uint32_t capacity, uint32_t refine_top_l, const TannShards* base_codes,
                           const TannShards* pq2_codes, uint32_t num_chunks, const float* lut2,
                           const float* cross_terms, void* out_candidates, uint32_t* status,
                           tann_stream_t stream) {
    (void)status;
    if (num_queries == 0 || refine_top_l == 0) return TANN_OK;
    if (!candidates || !stats || !pq2_codes || !lut2 || !out_candidates)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_pq2_refine: PQ2 index must be loaded.");
    // src/search/rerank_exact.cu:2285-2296
    if (num_chunks > 256) return Fail(TANN_ERR_UNSUPPORTED, "tann_pq2_refine: PQ2 num_chunks exceeds kernel specialization limit.");
    if (refine_top_l > capacity) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_pq2_refine: refine_top_l exceeds topology candidate capacity.");
    if (refine_top_l > 2048) return Fail(TANN_ERR_UNSUPPORTED, "tann_pq2_refine: refine_top_l exceeds device bitonic sort limit.");
    if (base_codes != nullptr && cross_terms == nullptr)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_pq2_refine: residual refine needs cross terms.");
    TANN_CUDA(tann::LaunchPq2Refine(candidates, stats, num_queries, capacity, refine_top_l, base_codes,
                                    *pq2_codes, num_chunks, lut2, cross_terms, out_candidates,
                                    (cudaStream_t)stream));
    return TANN_OK;
}

TannStatus tann_hpq_refine(const void* candidates, const uint32_t* stats, uint64_t num_queries, uint32_t capacity,
                           uint32_t refine_top_l, const TannShards* hybrid_codes, const uint8_t* selector_bits,
                           uint32_t num_chunks, const float* base_lut, const float* outlier_lut, void* out_candidates,
                           uint32_t* status, tann_stream_t stream) {
    (void)status;
    if (num_queries == 0 || refine_top_l == 0) return TANN_OK;
    if (!candidates || !stats || !hybrid_codes || !selector_bits || !base_lut || !outlier_lut || !out_candidates)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_hpq_refine: HPQ index must be loaded.");
    // src/search/rerank_exact.cu:2483-2492
    if (num_chunks > 256) return Fail(TANN_ERR_UNSUPPORTED, "tann_hpq_refine: HPQ layout exceeds kernel limits.");
    if (refine_top_l > capacity || refine_top_l > 2048)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_hpq_refine: HPQ refine size exceeds candidate limits.");
    TANN_CUDA(tann::LaunchPq2Refine(candidates, stats, num_queries, capacity, refine_top_l, nullptr, *hybrid_codes,
                                    num_chunks, base_lut, nullptr, out_candidates, (cudaStream_t)stream, nullptr, nullptr,
                                    nullptr, nullptr, 0, selector_bits, (num_chunks + 7u) / 8u, outlier_lut));
    return TANN_OK;
}

TannStatus tann_pq2_cross_terms(uint32_t dim, uint32_t num_chunks, const uint32_t* chunk_offsets,
                                const float* tables1_row_major, const float* centroid1,
                                const float* tables2_row_major, const float* centroid2, float* out,
                                tann_stream_t stream) {
    if (!chunk_offsets || !tables1_row_major || !centroid1 || !tables2_row_major || !centroid2 || !out)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_pq2_cross_terms: null pointer.");
    TANN_CUDA(tann::LaunchCrossTerms(dim, num_chunks, chunk_offsets, tables1_row_major, centroid1,
                                     tables2_row_major, centroid2, out, (cudaStream_t)stream));
    return TANN_OK;
}

// Parameter rules of the rerank (src/search/rerank_exact.cu:2181-2190, :2564-2585), shared by
// tann_rerank_exact and the searcher.
}  // extern "C"
namespace tann {
TannStatus CheckRerank(const char* who, const TannIndexView* index, const TannRerankParams* params,
                       const float* error_bounds) {
    if (index->vectors.base[0] == nullptr || index->vector_bytes == 0 || index->vectors_per_page == 0)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: Vector store must be loaded before rerank.", who);
    if (params->top_n > 2048) return Fail(TANN_ERR_UNSUPPORTED, "%s: top_n must be at most 2048.", who);
    if (params->use_bound_filter) {
        if (params->top_k == 0 || params->top_k > 128)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: PQ2 bound filter requires 1 <= top_k <= 128.", who);
        if (error_bounds == nullptr)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: PQ2 bound filter requires residual PQ2 error bounds.", who);
    }
    if (params->use_early_stop) {
        if (params->top_k == 0 || params->top_k > 128)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: early stop requires 1 <= top_k <= 128.", who);
        if (params->early_stop_patience_tiles == 0)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: early stop requires early_stop_patience_tiles >= 1.", who);
    }
    return CheckShards(index->vectors, index->num_nodes, "vectors");
}
}  // namespace tann
static TannStatus CheckRerank(const TannIndexView* index, const TannRerankParams* params, const float* error_bounds) {
    return tann::CheckRerank("tann_rerank_exact", index, params, error_bounds);
}
extern "C" {

TannStatus tann_rerank_exact(const TannIndexView* index, const TannRerankParams* params,
                             const void* candidates, uint32_t capacity, uint64_t num_queries,
                             const void* queries, uint32_t query_kind, const float* error_bounds,
                             float* out_dists, uint32_t* out_ids, unsigned long long* out_counts,
                             uint32_t* status, tann_stream_t stream) {
    if (!index || !params) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_rerank_exact: null index or params.");
    if (num_queries == 0 || params->top_n == 0) return TANN_OK;
    if (!candidates || !queries || !out_dists || !out_ids || query_kind > TANN_KIND_FLOAT32)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_rerank_exact: null pointer.");
    TannStatus st = CheckRerank(index, params, error_bounds);
    if (st != TANN_OK) return st;
    TANN_CUDA(tann::LaunchRerank(*index, *params, candidates, capacity, num_queries, queries, query_kind,
                                 error_bounds, out_dists, out_ids, out_counts, (cudaStream_t)stream, nullptr, nullptr, 0,
                                 status));
    return TANN_OK;
}

// ---- learned rerank stop -----------------------------------------------------------------------

extern "C++" {
namespace {

std::string TrimmedCopy(const std::string& text) {
    size_t a = 0, b = text.size();
    while (a < b && isspace((unsigned char)text[a])) ++a;
    while (b > a && isspace((unsigned char)text[b - 1])) --b;
    return text.substr(a, b - a);
}

// Comma-separated values, blanks around tokens and empty tokens dropped.
template <typename T, typename Parse>
bool ParseList(const std::string& text, Parse parse, std::vector<T>* out) {
    out->clear();
    size_t start = 0;
    while (start <= text.size()) {
        size_t comma = text.find(',', start);
        if (comma == std::string::npos) comma = text.size();
        const std::string token = TrimmedCopy(text.substr(start, comma - start));
        if (!token.empty()) {
            try {
                out->push_back(parse(token));
            } catch (...) {
                return false;
            }
        }
        start = comma + 1;
    }
    return true;
}

}  // namespace
}  // extern "C++"

TannStatus tann_rerank_learned_stop_load(const char* path, uint32_t budget_top_n, uint32_t top_k,
                                         TannRerankLearnedStop* out) {
    const char* ctx = "LoadRerankLearnedStopConfigFromFile";
    if (!path || !out) return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: null pointer.", ctx);
    std::ifstream in(path);
    if (!in.is_open()) return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: Failed to open %s", ctx, path);
    std::vector<uint32_t> stages, mask;
    std::vector<float> means, inv_stds, weights;
    std::map<uint32_t, float> threshold_of_budget;
    uint32_t file_top_k = 0, bootstrap = 0;
    float bias = 0.0f, threshold = 0.0f;
    const auto to_u32 = [](const std::string& t) { return (uint32_t)std::stoul(t); };
    const auto to_f32 = [](const std::string& t) { return std::stof(t); };
    const std::string per_budget_key = "threshold_logit_top_l_";
    std::string raw;
    while (std::getline(in, raw)) {
        const std::string line = TrimmedCopy(raw);
        if (line.empty() || line[0] == '#') continue;
        const size_t eq = line.find('=');
        if (eq == std::string::npos)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: Invalid learned-stop config line: %s", ctx, line.c_str());
        const std::string key = TrimmedCopy(line.substr(0, eq)), value = TrimmedCopy(line.substr(eq + 1));
        bool ok = true;
        try {
            if (key == "stage_prefixes") ok = ParseList(value, to_u32, &stages);
            else if (key == "feature_means") ok = ParseList(value, to_f32, &means);
            else if (key == "feature_inv_stds") ok = ParseList(value, to_f32, &inv_stds);
            else if (key == "weights") ok = ParseList(value, to_f32, &weights);
            else if (key == "feature_mask") ok = ParseList(value, to_u32, &mask);
            else if (key == "bias") bias = std::stof(value);
            else if (key == "threshold_logit") threshold = std::stof(value);
            else if (key == "top_k") file_top_k = (uint32_t)std::stoul(value);
            else if (key == "bootstrap_prefix") bootstrap = (uint32_t)std::stoul(value);
            else if (key.compare(0, per_budget_key.size(), per_budget_key) == 0 && key.size() > per_budget_key.size())
                threshold_of_budget.emplace((uint32_t)std::stoul(key.substr(per_budget_key.size())), std::stof(value));
        } catch (...) {
            ok = false;
        }
        if (!ok) return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: Invalid learned-stop config value: %s", ctx, line.c_str());
    }
    const size_t kNow = TANN_RERANK_STOP_FEATURES, kOlder = 12;
    const bool older = means.size() == kOlder && inv_stds.size() == kOlder && weights.size() == kOlder;
    const bool now = means.size() == kNow && inv_stds.size() == kNow && weights.size() == kNow;
    if (!older && !now)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: learned-stop feature vectors must all have length 13 or 12.", ctx);
    if (!mask.empty() && mask.size() != (older ? kOlder : kNow))
        return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: feature_mask must have length %zu.", ctx, older ? kOlder : kNow);

    TannRerankLearnedStop c;
    memset(&c, 0, sizeof(c));
    static const uint32_t kSixFeatureMask[TANN_RERANK_STOP_FEATURES] = {1, 1, 1, 0, 0, 1, 0, 1, 0, 1, 0, 0, 0};
    if (now && mask.size() == kNow && memcmp(mask.data(), kSixFeatureMask, sizeof(kSixFeatureMask)) == 0)
        c.feature_variant = 1;
    c.top_k = file_top_k != 0 ? file_top_k : top_k;
    c.bootstrap_prefix = bootstrap;
    const auto it = threshold_of_budget.find(budget_top_n);
    c.threshold_logit = it != threshold_of_budget.end() ? it->second : threshold;
    c.budget_log2 = std::log2(std::max(1.0f, (float)budget_top_n));
    c.inv_budget_top_n = budget_top_n == 0 ? 0.0f : 1.0f / (float)budget_top_n;
    c.inv_top_k = c.top_k == 0 ? 0.0f : 1.0f / (float)c.top_k;
    // Standardisation folded into the weights: w' = w / std, bias' = bias - sum(mean * w').
    // The older 12-feature layout has one top-k churn ratio where the kernel has a flag (5) and a ratio (6).
    float folded_bias = bias;
    for (size_t src = 0; src < weights.size(); ++src) {
        const size_t dst = (older && src >= 5) ? src + 1 : src;
        const float w = (mask.empty() || mask[src] != 0u) ? weights[src] : 0.0f;
        c.linear_weights[dst] = w * inv_stds[src];
        folded_bias -= means[src] * c.linear_weights[dst];
    }
    c.bias = folded_bias;
    for (uint32_t prefix : stages) {
        if (prefix == 0 || prefix > budget_top_n) continue;
        if (c.num_stages >= TANN_RERANK_STOP_MAX_STAGES) break;
        c.stage_prefixes[c.num_stages++] = prefix;
    }
    while (c.initial_stage_index < c.num_stages && c.stage_prefixes[c.initial_stage_index] <= c.bootstrap_prefix)
        ++c.initial_stage_index;
    c.enabled = (c.num_stages == 0 || c.bootstrap_prefix == 0) ? 0u : 1u;
    if (c.top_k == 0 || c.top_k > 128) c.enabled = 0;
    *out = c;
    return TANN_OK;
}

TannStatus tann_rerank_exact_learned_stop(const TannIndexView* index, const TannRerankParams* params,
                                          const TannRerankLearnedStop* model, const void* candidates,
                                          uint32_t capacity, uint64_t num_queries, const void* queries,
                                          uint32_t query_kind, const float* error_bounds,
                                          const uint32_t* replay_stop_prefixes, float* out_dists, uint32_t* out_ids,
                                          unsigned long long* out_counts, uint32_t* out_stop_prefixes,
                                          uint32_t* out_checkpoint_counts, uint32_t* out_stop_flags, uint32_t* status,
                                          tann_stream_t stream) {
    const char* ctx = "tann_rerank_exact_learned_stop";
    if (!index || !params) return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: null index or params.", ctx);
    if (num_queries == 0 || params->top_n == 0 || capacity == 0) return TANN_OK;
    if (!candidates || !queries || !out_dists || !out_ids || query_kind > TANN_KIND_FLOAT32)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: null pointer.", ctx);
    if (params->top_k == 0 || params->top_k > 128 || params->top_k > params->top_n)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: Persistent rerank requires 1 <= top_k <= min(top_n, 128).", ctx);
    TannStatus st = CheckRerank(index, params, error_bounds);
    if (st != TANN_OK) return st;
    TannRerankLearnedStop m;
    memset(&m, 0, sizeof(m));
    if (model) m = *model;
    const bool use_schedule = m.enabled != 0;
    if (use_schedule) {
        if (m.num_stages > TANN_RERANK_STOP_MAX_STAGES || m.initial_stage_index > m.num_stages)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: bad stage count in the model.", ctx);
        // The kernel walks the stages in order; a prefix that does not grow would give an empty or
        // negative window (the reference's kernel reads out of bounds there).
        uint32_t last = m.bootstrap_prefix;
        if (last == 0) return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: an enabled model needs bootstrap_prefix >= 1.", ctx);
        for (uint32_t i = m.initial_stage_index; i < m.num_stages; ++i) {
            if (m.stage_prefixes[i] <= last)
                return Fail(TANN_ERR_INVALID_ARGUMENT, "%s: stage prefixes must increase and exceed bootstrap_prefix.", ctx);
            last = m.stage_prefixes[i];
        }
        if ((m.linear_weights[8] != 0.0f || m.linear_weights[9] != 0.0f) && !params->use_bound_filter)
            return Fail(TANN_ERR_INVALID_ARGUMENT,
                        "%s: a model with next-window features needs the PQ2 bound filter (lower bounds).", ctx);
    }
    TANN_CUDA(tann::LaunchRerankLearned(*index, *params, m, use_schedule, use_schedule && replay_stop_prefixes == nullptr,
                                        candidates, capacity, num_queries, queries, query_kind, error_bounds,
                                        replay_stop_prefixes, out_dists, out_ids, out_counts, out_stop_prefixes,
                                        out_checkpoint_counts, out_stop_flags, (cudaStream_t)stream, status));
    return TANN_OK;
}

TannStatus tann_topk_pack(const float* dists, const uint32_t* ids, uint64_t num_queries, uint32_t top_n,
                          uint32_t top_k, float* out_dists, uint32_t* out_ids, tann_stream_t stream) {
    if (num_queries == 0 || top_k == 0) return TANN_OK;
    if (!dists || !ids || !out_dists || !out_ids) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_topk_pack: null pointer.");
    TANN_CUDA(tann::LaunchTopkPack(dists, ids, num_queries, top_n, top_k, out_dists, out_ids, (cudaStream_t)stream));
    return TANN_OK;
}

TannStatus tann_neighbor_codes_build(const TannIndexView* index, uint64_t first_node, uint64_t num_rows,
                                     void* out, tann_stream_t stream) {
    if (!index || !out) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_neighbor_codes_build: null pointer.");
    if (index->degree == 0 || index->num_chunks == 0)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_neighbor_codes_build: topology and PQ index must be loaded.");
    if (first_node + num_rows > index->num_nodes)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_neighbor_codes_build: rows beyond the index.");
    if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_neighbor_codes_build: output must be 16-byte aligned.");
    TannStatus st = CheckShards(index->adjacency, index->num_nodes, "adjacency");
    if (st != TANN_OK) return st;
    st = CheckShards(index->codes, index->num_nodes, "codes");
    if (st != TANN_OK) return st;
    TANN_CUDA(tann::LaunchNeighborCodes(*index, first_node, num_rows, static_cast<uint8_t*>(out), (cudaStream_t)stream));
    return TANN_OK;
}

// ---- memory helpers ---------------------------------------------------------------------------

TannStatus tann_device_alloc(uint64_t bytes, void** out_dev) {
    if (!out_dev) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_device_alloc: null out pointer.");
    *out_dev = nullptr;
    if (bytes == 0) return TANN_OK;
    TANN_CUDA(cudaMalloc(out_dev, bytes));
    return TANN_OK;
}
TannStatus tann_device_free(void* dev) {
    if (dev) TANN_CUDA(cudaFree(dev));
    return TANN_OK;
}
TannStatus tann_host_alloc_mapped(uint64_t bytes, void** out_host, void** out_dev) {
    if (!out_host || !out_dev) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_host_alloc_mapped: null out pointer.");
    *out_host = *out_dev = nullptr;
    if (bytes == 0) return TANN_OK;
    TANN_CUDA(cudaHostAlloc(out_host, bytes, cudaHostAllocMapped | cudaHostAllocPortable));
    cudaError_t e = cudaHostGetDevicePointer(out_dev, *out_host, 0);
    if (e != cudaSuccess) {
        cudaFreeHost(*out_host);
        *out_host = nullptr;
        return CudaFail(e, "cudaHostGetDevicePointer");
    }
    return TANN_OK;
}
TannStatus tann_host_free(void* host) {
    if (host) TANN_CUDA(cudaFreeHost(host));
    return TANN_OK;
}
TannStatus tann_ipc_export(void* dev, unsigned char handle[TANN_IPC_HANDLE_BYTES]) {
    static_assert(sizeof(cudaIpcMemHandle_t) <= TANN_IPC_HANDLE_BYTES, "handle size");
    if (!dev || !handle) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_ipc_export: null pointer.");
    cudaIpcMemHandle_t h;
    TANN_CUDA(cudaIpcGetMemHandle(&h, dev));
    memset(handle, 0, TANN_IPC_HANDLE_BYTES);
    memcpy(handle, &h, sizeof(h));
    return TANN_OK;
}
TannStatus tann_ipc_open(const unsigned char handle[TANN_IPC_HANDLE_BYTES], void** out_dev) {
    if (!handle || !out_dev) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_ipc_open: null pointer.");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    TANN_CUDA(cudaIpcOpenMemHandle(out_dev, h, cudaIpcMemLazyEnablePeerAccess));
    return TANN_OK;
}
TannStatus tann_ipc_close(void* dev) {
    if (dev) TANN_CUDA(cudaIpcCloseMemHandle(dev));
    return TANN_OK;
}
TannStatus tann_enable_peer_access(int peer_device) {
    cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return TANN_OK;
    }
    if (e != cudaSuccess) return CudaFail(e, "cudaDeviceEnablePeerAccess");
    return TANN_OK;
}

// ---- measurement aid: one dependent random load after another ----------------------------------------
__global__ void dependent_load_kernel(const uint32_t* base, uint64_t words, uint32_t steps, float* out_ns) {
    uint64_t pos = 0x9e3779b97f4a7c15ull % words;
    uint32_t acc = 0;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (uint32_t i = 0; i < steps; ++i) {
        const uint32_t v = __ldcg(base + pos);   // the next address depends on the value just read
        acc += v;
        pos = ((pos + v) * 6364136223846793005ull + 1442695040888963407ull + i) % words;
    }
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    out_ns[0] = steps ? (float)((double)(t1 - t0) / (double)steps) : 0.0f;
    out_ns[1] = __uint_as_float(acc);   // keeps the loads alive
}

TannStatus tann_dependent_load_ns(const void* base, uint64_t bytes, uint32_t steps, float* out_ns, tann_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!base || !out_ns || bytes < 4 || steps == 0)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_dependent_load_ns: null pointer or empty range.");
    if (steps > (1u << 20)) return Fail(TANN_ERR_UNSUPPORTED, "tann_dependent_load_ns: at most 2^20 steps.");
    float* d_out = nullptr;
    TANN_CUDA(cudaMalloc((void**)&d_out, 2 * sizeof(float)));
    dependent_load_kernel<<<1, 1, 0, stream>>>(static_cast<const uint32_t*>(base), bytes / 4, steps, d_out);
    cudaError_t e = cudaGetLastError();
    float host[2] = {0.0f, 0.0f};
    if (e == cudaSuccess) e = cudaMemcpyAsync(host, d_out, sizeof(host), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    cudaFree(d_out);
    if (e != cudaSuccess) return CudaFail(e, "tann_dependent_load_ns");
    *out_ns = host[0];
    return TANN_OK;
}

// ---- searcher -----------------------------------------------------------------------------------

struct TannSearcher {
    TannIndexView ix;
    uint64_t max_queries;
    uint32_t max_capacity, max_top_n, max_entries;
    bool has_rvq, has_pq2;
    bool has_rerank_stop = false;
    TannRerankLearnedStop rerank_stop;
    TannRvqModelView rvq;
    TannPq2View pq2;
    // device work space
    void* d_queries;          // max_queries * dim * 4
    float* d_queries_f32;     // float copy of the queries for RVQ / pq2 when the kind is not float
    uint8_t* d_queries_u8;    // uint8 copy of integer-valued float queries (integer rerank path)
    uint32_t* d_not_u8;       // set by the conversion kernel when a value is not an integer in [0, 255]
    uint32_t* d_entry_offsets;
    uint32_t* d_entry_ids;
    void* d_cand;
    void* d_cand_refined;
    uint32_t* d_stats;
    float* d_lut2;
    float* d_dists;
    uint32_t* d_ids;
    float* d_topk_dists;
    uint32_t* d_topk_ids;
    unsigned long long* d_counts;
    uint32_t* d_fixed_entries;   // max_entries ids: the fixed entry list before it is expanded per query
    uint32_t* d_status;          // TANN_STATUS_* bits of the last run
    uint32_t* h_status;
    // pinned staging
    // a batch that tann_searcher_submit enqueued and tann_searcher_wait has not collected yet
    struct Pending {
        bool active = false;
        cudaStream_t stream = nullptr;
        uint32_t* out_ids = nullptr;     // non-null: copy from the staging buffer after the stream drains
        float* out_dists = nullptr;
        uint32_t* out_stats = nullptr;
        size_t kbytes = 0, stats_bytes = 0;
    } pending;
    void* h_queries;
    uint32_t* h_topk_ids;
    float* h_topk_dists;
    uint32_t* h_stats;
    uint32_t* h_entries;
};

static void FreeSearcher(TannSearcher* s) {
    if (!s) return;
    cudaFree(s->d_queries); cudaFree(s->d_queries_f32); cudaFree(s->d_queries_u8); cudaFree(s->d_not_u8); cudaFree(s->d_entry_offsets);
    cudaFree(s->d_entry_ids); cudaFree(s->d_cand); cudaFree(s->d_cand_refined); cudaFree(s->d_stats);
    cudaFree(s->d_lut2); cudaFree(s->d_dists); cudaFree(s->d_ids); cudaFree(s->d_topk_dists);
    cudaFree(s->d_topk_ids); cudaFree(s->d_counts); cudaFree(s->d_fixed_entries); cudaFree(s->d_status);
    cudaFreeHost(s->h_status);
    cudaFreeHost(s->h_queries); cudaFreeHost(s->h_topk_ids); cudaFreeHost(s->h_topk_dists);
    cudaFreeHost(s->h_stats); cudaFreeHost(s->h_entries);
    cudaGetLastError();
    delete s;
}

TannStatus tann_searcher_create(const TannIndexView* index, uint64_t max_queries,
                                uint32_t max_candidate_capacity, uint32_t max_top_n,
                                uint32_t max_entries_per_query, TannSearcher** out) {
    if (!index || !out) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_create: null pointer.");
    *out = nullptr;
    if (max_queries == 0 || max_candidate_capacity == 0 || max_top_n == 0 || max_entries_per_query == 0)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_create: sizes must be positive.");
    if (max_queries * max_entries_per_query > 0xffffffffull)
        return Fail(TANN_ERR_UNSUPPORTED, "tann_searcher_create: entry offsets overflow uint32.");
    TannSearcher* s = new (std::nothrow) TannSearcher();
    if (!s) return Fail(TANN_ERR_CUDA, "tann_searcher_create: out of host memory.");
    memset(s, 0, sizeof(*s));
    s->ix = *index;
    s->max_queries = max_queries;
    s->max_capacity = NextPow2(max_candidate_capacity);
    s->max_top_n = max_top_n;
    s->max_entries = max_entries_per_query;
    const size_t Q = max_queries, d = index->dim;
    cudaError_t e = cudaSuccess;
    auto dev = [&](void** p, size_t bytes) { if (e == cudaSuccess) e = cudaMalloc(p, bytes ? bytes : 16); };
    auto host = [&](void** p, size_t bytes) { if (e == cudaSuccess) e = cudaHostAlloc(p, bytes ? bytes : 16, cudaHostAllocDefault); };
    dev(&s->d_queries, Q * d * 4);
    dev((void**)&s->d_queries_f32, Q * d * 4);
    dev((void**)&s->d_queries_u8, Q * d);
    dev((void**)&s->d_not_u8, 16);
    dev((void**)&s->d_entry_offsets, (Q + 1) * 4);
    dev((void**)&s->d_entry_ids, Q * max_entries_per_query * 4);
    dev(&s->d_cand, Q * s->max_capacity * 8);
    dev(&s->d_cand_refined, Q * s->max_capacity * 8);
    dev((void**)&s->d_stats, Q * 8 * 4);
    dev((void**)&s->d_dists, Q * max_top_n * 4);
    dev((void**)&s->d_ids, Q * max_top_n * 4);
    dev((void**)&s->d_topk_dists, Q * max_top_n * 4);
    dev((void**)&s->d_topk_ids, Q * max_top_n * 4);
    dev((void**)&s->d_counts, 16);
    dev((void**)&s->d_fixed_entries, (size_t)max_entries_per_query * 4);
    dev((void**)&s->d_status, 16);
    host((void**)&s->h_status, 16);
    host(&s->h_queries, Q * d * 4);
    host((void**)&s->h_topk_ids, Q * max_top_n * 4);
    host((void**)&s->h_topk_dists, Q * max_top_n * 4);
    host((void**)&s->h_stats, Q * 8 * 4);
    host((void**)&s->h_entries, (size_t)max_entries_per_query * 4);
    if (e != cudaSuccess) {
        FreeSearcher(s);
        return CudaFail(e, "tann_searcher_create");
    }
    *out = s;
    return TANN_OK;
}

TannStatus tann_searcher_set_rvq(TannSearcher* s, const TannRvqModelView* rvq) {
    if (!s) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_set_rvq: null searcher.");
    if (!rvq) { s->has_rvq = false; return TANN_OK; }
    if (rvq->dim != s->ix.dim) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_set_rvq: model dim differs from the index dim.");
    if (rvq->entry_count == 0 || rvq->entry_count > s->max_entries)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_set_rvq: entry_count must be 1..max_entries_per_query.");
    s->rvq = *rvq;
    s->has_rvq = true;
    return TANN_OK;
}

TannStatus tann_searcher_set_pq2(TannSearcher* s, const TannPq2View* pq2) {
    if (!s) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_set_pq2: null searcher.");
    if (!pq2 || !pq2->enabled) { s->has_pq2 = false; return TANN_OK; }
    s->pq2 = *pq2;   // no second-level table buffer: the refine kernel computes the entries it reads
    s->has_pq2 = true;
    return TANN_OK;
}

TannStatus tann_searcher_set_rerank_learned_stop(TannSearcher* s, const TannRerankLearnedStop* model) {
    if (!s) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_set_rerank_learned_stop: null searcher.");
    s->has_rerank_stop = model != nullptr;
    if (model) s->rerank_stop = *model;
    return TANN_OK;
}

__global__ void to_float_kernel(const void* src, uint32_t kind, uint64_t n, float* dst) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        dst[i] = kind == TANN_KIND_UINT8 ? (float)static_cast<const uint8_t*>(src)[i]
                                          : (float)static_cast<const int8_t*>(src)[i];
}
__global__ void fixed_entries_kernel(const uint32_t* entries, uint32_t n, uint64_t Q, uint32_t* offsets,
                                     uint32_t* ids) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < Q * n; i += (uint64_t)gridDim.x * blockDim.x)
        ids[i] = entries[i % n];
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i <= Q; i += (uint64_t)gridDim.x * blockDim.x)
        offsets[i] = (uint32_t)(i * n);
}

TannStatus tann_searcher_run_device(TannSearcher* s, const TannBeamParams* beam,
                                    const TannRerankParams* rerank, const void* queries_dev,
                                    uint32_t query_kind, uint64_t Q, const uint32_t* entry_offsets_dev,
                                    const uint32_t* entry_ids_dev, const uint32_t** out_ids_dev,
                                    const float** out_dists_dev, const uint32_t** out_stats_dev,
                                    tann_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!s || !beam || !rerank) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_run: null pointer.");
    if (Q > s->max_queries) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_run: batch exceeds max_queries.");
    if (beam->candidate_capacity > s->max_capacity) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_run: candidate capacity exceeds the searcher's.");
    if (rerank->top_n > s->max_top_n || rerank->top_k > rerank->top_n)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_run: need top_k <= top_n <= max_top_n.");
    if (rerank->top_n > beam->candidate_capacity)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_run: top_n exceeds the candidate capacity.");
    if (Q == 0) return TANN_OK;
    TANN_CUDA(cudaMemsetAsync(s->d_status, 0, sizeof(uint32_t), stream));
    const uint32_t d = s->ix.dim;
    const float* qf32 = static_cast<const float*>(queries_dev);
    const bool need_f32 = (s->has_rvq && entry_offsets_dev == nullptr) || s->has_pq2;
    if (query_kind != TANN_KIND_FLOAT32 && need_f32) {
        to_float_kernel<<<tann::SmCount() * 4, 256, 0, stream>>>(queries_dev, query_kind, Q * d, s->d_queries_f32);
        TANN_CUDA(cudaGetLastError());
        qf32 = s->d_queries_f32;
    }
    // entries
    const uint32_t* eo = entry_offsets_dev;
    const uint32_t* ei = entry_ids_dev;
    if (eo == nullptr) {
        if (!s->has_rvq) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_run: no entries and no RVQ model.");
        const TannRvqModelView& r = s->rvq;
        if (!r.coarse || !r.coarse_t || !r.coarse_norms || !r.fine_t || !r.fine_norms || !r.bucket_sizes ||
            !r.cluster_offsets || !r.cluster_ids || r.num_coarse == 0 || r.num_fine == 0)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_rvq_entries: model is not loaded.");
        TANN_CUDA(tann::LaunchRvqEntries(qf32, Q, d, r.coarse, r.coarse_t, r.coarse_norms, r.num_coarse, r.fine_t,
                                         r.fine_norms, r.num_fine, r.bucket_sizes, r.cluster_offsets, r.cluster_ids,
                                         r.entry_count, r.fallback_entry, nullptr, s->d_entry_ids, s->d_entry_offsets,
                                         stream, s->d_status));
        eo = s->d_entry_offsets;
        ei = s->d_entry_ids;
    }
    // traversal, table built in the kernel
    TannStatus st = tann_beam_search(&s->ix, beam, nullptr, queries_dev, query_kind, Q, eo, ei, s->d_cand,
                                     s->d_stats, s->d_status, stream);
    if (st != TANN_OK) return st;
    const void* cand = s->d_cand;
    uint32_t capacity = beam->candidate_capacity;
    const float* err = nullptr;
    if (s->has_pq2) {
        const TannPq2View& p2 = s->pq2;
        // src/search/rerank_exact.cu:2610-2615
        const uint32_t lr = p2.refine_top_l == 0 ? capacity : (p2.refine_top_l < capacity ? p2.refine_top_l : capacity);
        // Same checks as tann_pq2_refine (src/search/rerank_exact.cu:2285-2296); the second-level table
        // entries are computed inside the refine kernel, so no Q x M x 256 table is built here.
        if (s->ix.num_chunks > 256) return Fail(TANN_ERR_UNSUPPORTED, "tann_pq2_refine: PQ2 num_chunks exceeds kernel specialization limit.");
        if (lr > 2048) return Fail(TANN_ERR_UNSUPPORTED, "tann_pq2_refine: refine_top_l exceeds device bitonic sort limit.");
        if (p2.residual && p2.cross_terms == nullptr)
            return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_pq2_refine: residual refine needs cross terms.");
        TANN_CUDA(tann::LaunchPq2Refine(s->d_cand, s->d_stats, Q, capacity, lr, p2.residual ? &s->ix.codes : nullptr,
                                        p2.codes, s->ix.num_chunks, /*lut2=*/nullptr, p2.cross_terms, s->d_cand_refined,
                                        stream, p2.tables_col_major, p2.centroid, p2.chunk_offsets, qf32, d));
        cand = s->d_cand_refined;
        capacity = lr;
        err = p2.error_bounds;
    }
    if (s->has_rerank_stop && rerank->top_n != 0) {
        // persistent rerank with the learned stop: keeps the top_k list itself, nothing to pack
        st = tann_rerank_exact_learned_stop(&s->ix, rerank, &s->rerank_stop, cand, capacity, Q, queries_dev, query_kind, err,
                                            nullptr, s->d_topk_dists, s->d_topk_ids, nullptr, nullptr, nullptr, nullptr,
                                            s->d_status, stream);
        if (st != TANN_OK) return st;
        if (out_ids_dev) *out_ids_dev = s->d_topk_ids;
        if (out_dists_dev) *out_dists_dev = s->d_topk_dists;
        if (out_stats_dev) *out_stats_dev = s->d_stats;
        return TANN_OK;
    }
    if (rerank->top_n != 0) {
        st = CheckRerank(&s->ix, rerank, err);
        if (st != TANN_OK) return st;
        const bool u8_copy = query_kind == TANN_KIND_FLOAT32 && s->ix.vector_kind == TANN_KIND_UINT8 && !rerank->use_bound_filter;
        if (u8_copy)   // integer-valued float queries (the usual case for uint8 data) can use the integer distance path
            TANN_CUDA(tann::LaunchF32ToU8Checked(static_cast<const float*>(queries_dev), Q * d, s->d_queries_u8,
                                                 s->d_not_u8, stream));
        // only the first top_k ranks are packed below: a top-k tournament replaces the full sort when k <= 32
        TANN_CUDA(tann::LaunchRerank(s->ix, *rerank, cand, capacity, Q, queries_dev, query_kind, err, s->d_dists,
                                     s->d_ids, nullptr, stream, u8_copy ? s->d_queries_u8 : nullptr,
                                     u8_copy ? s->d_not_u8 : nullptr, rerank->top_k <= 32 ? rerank->top_k : 0,
                                     s->d_status));
    }
    st = tann_topk_pack(s->d_dists, s->d_ids, Q, rerank->top_n, rerank->top_k, s->d_topk_dists,
                        s->d_topk_ids, stream);
    if (st != TANN_OK) return st;
    if (out_ids_dev) *out_ids_dev = s->d_topk_ids;
    if (out_dists_dev) *out_dists_dev = s->d_topk_dists;
    if (out_stats_dev) *out_stats_dev = s->d_stats;
    return TANN_OK;
}

TannStatus tann_searcher_submit(TannSearcher* s, const TannBeamParams* beam, const TannRerankParams* rerank,
                                const void* queries_host, uint32_t query_kind, uint64_t Q,
                                const uint32_t* fixed_entries_host, uint32_t num_fixed_entries,
                                uint32_t* out_ids_host, float* out_dists_host, uint32_t* out_stats_host,
                                tann_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!s || !beam || !rerank || !queries_host || !out_ids_host || !out_dists_host)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_run: null pointer.");
    if (s->pending.active) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_submit: the previous batch has not been waited for.");
    if (Q > s->max_queries) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_run: batch exceeds max_queries.");
    if (query_kind > TANN_KIND_FLOAT32) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_run: unknown query kind.");
    if (Q == 0) return TANN_OK;
    const size_t qbytes = Q * (size_t)s->ix.dim * (query_kind == TANN_KIND_FLOAT32 ? 4 : 1);
    // Pageable memory goes through one pinned staging copy so that the H2D stays asynchronous;
    // page-locked memory (cudaHostAlloc / cudaHostRegister) is copied from where it is.
    const void* h2d_src = queries_host;
    if (!IsPageLocked(queries_host)) {
        memcpy(s->h_queries, queries_host, qbytes);
        h2d_src = s->h_queries;
    }
    if (fixed_entries_host != nullptr && num_fixed_entries > s->max_entries)
        return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_run: too many fixed entries.");
    // From here on work is enqueued on the stream: an error return first lets it drain, so that the caller's
    // buffers are no longer in use when the call comes back.
    const auto drained = [&](TannStatus st) {
        cudaStreamSynchronize(stream);
        return st;
    };
    cudaError_t ce = cudaMemcpyAsync(s->d_queries, h2d_src, qbytes, cudaMemcpyHostToDevice, stream);
    if (ce != cudaSuccess) return drained(CudaFail(ce, "cudaMemcpyAsync(queries)"));
    const uint32_t* eo = nullptr;
    const uint32_t* ei = nullptr;
    if (fixed_entries_host != nullptr && num_fixed_entries != 0) {
        memcpy(s->h_entries, fixed_entries_host, (size_t)num_fixed_entries * 4);
        // the list goes to its own max_entries-sized buffer, then is expanded per query on the device
        ce = cudaMemcpyAsync(s->d_fixed_entries, s->h_entries, (size_t)num_fixed_entries * 4, cudaMemcpyHostToDevice, stream);
        if (ce != cudaSuccess) return drained(CudaFail(ce, "cudaMemcpyAsync(fixed entries)"));
        fixed_entries_kernel<<<tann::SmCount() * 2, 256, 0, stream>>>(s->d_fixed_entries, num_fixed_entries, Q,
                                                                      s->d_entry_offsets, s->d_entry_ids);
        ce = cudaGetLastError();
        if (ce != cudaSuccess) return drained(CudaFail(ce, "fixed_entries_kernel"));
        eo = s->d_entry_offsets;
        ei = s->d_entry_ids;
    }
    TannStatus st = tann_searcher_run_device(s, beam, rerank, s->d_queries, query_kind, Q, eo, ei, nullptr,
                                             nullptr, nullptr, stream);
    if (st != TANN_OK) return drained(st);
    const size_t kbytes = Q * (size_t)rerank->top_k * 4;
    const bool ids_direct = IsPageLocked(out_ids_host), dists_direct = IsPageLocked(out_dists_host);
    ce = cudaMemcpyAsync(ids_direct ? (void*)out_ids_host : (void*)s->h_topk_ids, s->d_topk_ids, kbytes,
                         cudaMemcpyDeviceToHost, stream);
    if (ce == cudaSuccess)
        ce = cudaMemcpyAsync(dists_direct ? (void*)out_dists_host : (void*)s->h_topk_dists, s->d_topk_dists, kbytes,
                             cudaMemcpyDeviceToHost, stream);
    if (ce == cudaSuccess && out_stats_host)
        ce = cudaMemcpyAsync(s->h_stats, s->d_stats, Q * 32, cudaMemcpyDeviceToHost, stream);
    if (ce == cudaSuccess)
        ce = cudaMemcpyAsync(s->h_status, s->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
    if (ce != cudaSuccess) return drained(CudaFail(ce, "cudaMemcpyAsync(results)"));
    s->pending.active = true;
    s->pending.stream = stream;
    s->pending.out_ids = ids_direct ? nullptr : out_ids_host;
    s->pending.out_dists = dists_direct ? nullptr : out_dists_host;
    s->pending.out_stats = out_stats_host;
    s->pending.kbytes = kbytes;
    s->pending.stats_bytes = Q * 32;
    return TANN_OK;
}

TannStatus tann_searcher_wait(TannSearcher* s) {
    if (!s) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_wait: null searcher.");
    if (!s->pending.active) return TANN_OK;
    s->pending.active = false;
    TANN_CUDA(cudaStreamSynchronize(s->pending.stream));
    if (s->pending.out_ids) memcpy(s->pending.out_ids, s->h_topk_ids, s->pending.kbytes);
    if (s->pending.out_dists) memcpy(s->pending.out_dists, s->h_topk_dists, s->pending.kbytes);
    if (s->pending.out_stats) memcpy(s->pending.out_stats, s->h_stats, s->pending.stats_bytes);
    if (*s->h_status != 0u)
        return Fail(TANN_ERR_DEVICE_CHECK,
                    "tann_searcher_run: a kernel skipped an index outside the index view (status bits 0x%x: 1 = entry or "
                    "adjacency id, 2 = rerank candidate id, 4 = shared-memory copy timeout); results cover the rest.",
                    *s->h_status);
    return TANN_OK;
}

TannStatus tann_searcher_run(TannSearcher* s, const TannBeamParams* beam, const TannRerankParams* rerank,
                             const void* queries_host, uint32_t query_kind, uint64_t Q,
                             const uint32_t* fixed_entries_host, uint32_t num_fixed_entries,
                             uint32_t* out_ids_host, float* out_dists_host, uint32_t* out_stats_host,
                             tann_stream_t stream) {
    const TannStatus st = tann_searcher_submit(s, beam, rerank, queries_host, query_kind, Q, fixed_entries_host,
                                               num_fixed_entries, out_ids_host, out_dists_host, out_stats_host, stream);
    if (st != TANN_OK) {
        if (s) s->pending.active = false;
        return st;
    }
    return tann_searcher_wait(s);
}

TannStatus tann_searcher_status_device(TannSearcher* s, const uint32_t** out_status_dev) {
    if (!s || !out_status_dev) return Fail(TANN_ERR_INVALID_ARGUMENT, "tann_searcher_status_device: null pointer.");
    *out_status_dev = s->d_status;
    return TANN_OK;
}

TannStatus tann_searcher_destroy(TannSearcher* s) {
    if (s && s->pending.active) {   // a submitted batch still uses the buffers: let it drain first
        cudaStreamSynchronize(s->pending.stream);
        s->pending.active = false;
    }
    FreeSearcher(s);
    return TANN_OK;
}

}  // extern "C"
