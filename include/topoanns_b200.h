/*
 * C ABI of the B200 batched graph-search path (libtopoanns_b200.so).
 *
 * Every entry point takes plain pointers and sizes, enqueues its work on the given CUDA stream of
 * the current device and returns a TannStatus; nothing throws and nothing falls back to the CPU.
 * Device pointers are marked "dev". Each entry point names the reference (szrr/TopoANNS) interface
 * it replaces, by file:line inside that project.
 *
 * Candidate records are the reference's 8-byte DeviceTopologyCandidate
 * (src/search/topology_search_kernel.hpp:37-54): { float distance; uint32 node_id } with bit 31
 * of node_id = "expanded" and 0xffffffff = invalid. Per-query statistics are the reference's
 * DeviceTopologySearchStats (:56-65): 8 x uint32 { visited, expanded, topology_io_pages,
 * iterations, valid_candidates, first_full_prefix_iteration, 0, 0 }.
 */
#ifndef TOPOANNS_B200_H_
#define TOPOANNS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* tann_stream_t; /* a cudaStream_t; NULL = the default stream */

typedef enum TannStatus {
    TANN_OK = 0,
    TANN_ERR_INVALID_ARGUMENT = 1, /* a parameter check failed; see tann_last_error() */
    TANN_ERR_CUDA = 2,             /* a CUDA runtime call failed; see tann_last_error() */
    TANN_ERR_UNSUPPORTED = 3,      /* sizes beyond what the kernels are built for */
    TANN_ERR_DEVICE_CHECK = 4      /* a kernel recorded an out-of-range index (status word) */
} TannStatus;

/* Bits a kernel ors into the caller's device status word (the `status` arguments below; the searcher keeps its
 * own word and turns a non-zero value into TANN_ERR_DEVICE_CHECK). The check always precedes the access: the
 * offending id is skipped, exactly as the reference skips it (src/search/topology_search_kernel.cu:2556-2559,
 * src/search/rerank_exact.cu:344-386), and the results are those of the remaining ids. */
#define TANN_STATUS_BEAM_ID_RANGE 1u     /* an entry or adjacency id that is neither 0xffffffff nor < num_nodes */
#define TANN_STATUS_RERANK_ID_RANGE 2u   /* a candidate id >= num_nodes reached the rerank */
#define TANN_STATUS_COPY_TIMEOUT 4u      /* a bulk shared-memory copy did not complete within its poll limit; the
                                            block wrote no results for its remaining queries */

/* include/topoanns/common.hpp:17-21 (ScalarKind) */
enum { TANN_KIND_INT8 = 0, TANN_KIND_UINT8 = 1, TANN_KIND_FLOAT32 = 2 };

#define TANN_INVALID_NODE 0xffffffffu
#define TANN_MAX_SHARDS 8
#define TANN_MAX_SEARCH_WIDTH 32   /* src/search/topology_search_kernel.cu:58 */
#define TANN_MAX_STOP_STAGES 32    /* :65 */
#define TANN_STOP_FEATURES 12      /* :64 */

/*
 * Where the rows of one index array live. Replaces the opaque BaM handle returned by
 * VectorPageProvider::DeviceReadHandle() (include/topoanns/vector_page_provider.hpp:22) and the
 * single pinned-host pointer of PinnedTopology::device_data() (include/topoanns/pinned_topology.hpp:34).
 * Row n is in shard n / rows_per_shard at local row n % rows_per_shard. One shard = HBM-resident
 * (or pinned-host / UVA, the pointer being a mapped host pointer); several shards = node-id-range
 * sharding over the GPUs of one box, base[s] being a peer-mapped pointer.
 */
typedef struct TannShards {
    uint32_t num_shards;
    uint32_t reserved;
    uint64_t rows_per_shard;
    const void* base[TANN_MAX_SHARDS]; /* dev (local, peer or mapped host) */
} TannShards;

/* The index as the kernels see it. Replaces what the reference pulls out of SearchResources
 * (include/topoanns/search_resources.hpp:24-101) before a launch. */
typedef struct TannIndexView {
    uint64_t num_nodes;
    uint32_t degree;      /* adjacency slots per node (64 in topology.bin; any value in memory) */
    uint32_t num_chunks;  /* PQ chunks M */
    uint32_t dim;
    uint32_t vector_kind; /* TANN_KIND_* of the stored vectors */
    /* vector page layout, src/io/vector_page_layout.cpp:15-57; offsets are relative to the first
     * page (the 4 KB file header is not part of the array) and, with several shards, to the
     * shard's first page with the node's local row number. */
    uint64_t vector_bytes;
    uint64_t vectors_per_page;
    uint64_t page_bytes;
    TannShards adjacency; /* rows of `degree` uint32 */
    TannShards codes;     /* rows of `num_chunks` uint8 */
    TannShards vectors;   /* pages */
    /* Optional HBM cache in front of a slow adjacency tier: rows [0, adjacency_cached_rows) are
     * read from here instead (prefix semantics of TopologySearchParams::topology_cached_node_count,
     * include/topoanns/topology_search.hpp:23). NULL / 0 = no cache. */
    const uint32_t* adjacency_cache; /* dev */
    uint64_t adjacency_cached_rows;
    /* PQ pivots as loaded by src/io/pq_index.cpp:116-173 */
    const float* pq_tables_col_major; /* dev, [dim][256] */
    const float* pq_centroid;         /* dev, [dim] */
    const uint32_t* pq_chunk_offsets; /* dev, [M + 1] */
    /* Optional (base[0] == NULL = absent): the PQ codes of every node's neighbours stored next to each
     * other in adjacency order, rows of degree * num_chunks bytes sharded like `adjacency`. With it an
     * expansion reads its neighbours' codes from one contiguous row whose address is known together
     * with the adjacency row's, so both arrive in one memory round trip instead of two dependent ones.
     * Costs degree * num_chunks bytes per node of HBM (2 KB at R = 64, M = 32); results are identical.
     * No counterpart in the reference's resident layout (its disk layout co-locates node data,
     * include/topoanns/topology_search.hpp:27-28 combined_node_bytes). */
    TannShards neighbor_codes;
} TannIndexView;

/* Folded learned traversal-stop model, src/search/topology_search_kernel.cu:98-112,327-380. */
typedef struct TannLearnedStop {
    uint32_t enabled;
    uint32_t num_stages;
    uint32_t top_k;
    uint32_t shadow_mode;
    uint32_t topk_churn_flag_mode; /* 1 = "flag", 0 = ratio */
    uint32_t next64_flag_mode;     /* 1 = "flag", 0 = fraction */
    uint32_t stage_prefixes[TANN_MAX_STOP_STAGES];
    uint32_t feature_mask[TANN_STOP_FEATURES];
    float weights[TANN_STOP_FEATURES];
    float bias;
    float threshold_logit;
    float inv_top_l;
} TannLearnedStop;

/* TopologySearchParams (include/topoanns/topology_search.hpp:17-32) as the kernel needs them. */
typedef struct TannBeamParams {
    uint32_t top_l;
    uint32_t search_width;       /* 1..32 */
    uint32_t max_expansions;
    uint32_t candidate_capacity; /* power of two >= top_l; src/search/topology_search_kernel.cu:3207-3210 */
    uint32_t stop_prefix;        /* top_l, or the TOPOANNS_CANDIDATE_STOP_* prefix (:3445-3473) */
    uint32_t stop_use_expanded;  /* TOPOANNS_CANDIDATE_STOP_USE_EXPANDED (:3474-3480) */
    uint32_t reserved0;
    uint32_t reserved1;
    TannLearnedStop learned_stop;
} TannBeamParams;

const char* tann_version(void);
/* Message of the last non-OK status returned on this thread. */
const char* tann_last_error(void);

/*
 * ADC look-up tables: out[q][m][c] = sum over the dims of chunk m of
 * (table[c][dim] - (float(query[q][dim]) - centroid[dim]))^2, FMA-accumulated in ascending dim.
 * Replaces PqQueryDistanceTables::BuildFromQueries / FromFloatQueriesDeviceBufferAsync
 * (src/search/pq_query_tables.cu:13-158): same values, written once (no zero-fill pass).
 */
TannStatus tann_lut_build(const float* tables_col_major /*dev [dim][256]*/,
                          const float* centroid /*dev*/, const uint32_t* chunk_offsets /*dev*/,
                          uint32_t dim, uint32_t num_chunks, const void* queries /*dev*/,
                          uint32_t query_kind, uint64_t num_queries, float* out_tables /*dev*/,
                          tann_stream_t stream);

/*
 * Batched Bloom-filtered beam search, one query per thread block. Replaces
 * detail::RunTopologySearchKernelBatchDevice (src/search/topology_search_kernel.hpp:158-220;
 * kernel src/search/topology_search_kernel.cu:2190-2664).
 *   lut       dev [Q][M][256], or NULL to build each query's table inside the kernel from
 *             `queries` (then queries / query_kind must be given);
 *   entries   CSR as in DeviceEntryBatch (include/topoanns/device_entry_batch.hpp:10-23);
 *   out_candidates dev [Q][candidate_capacity] records, out_stats dev [Q][8] uint32;
 *   status    dev uint32 or NULL; TANN_STATUS_* bits are or-ed into it (clear it before the call).
 * Alignment: `lut`, every base pointer of `index->codes` and of `index->neighbor_codes`, and the PQ pivots must
 * be 16-byte aligned (rows are read with 16-byte loads); anything else is rejected before the launch.
 */
TannStatus tann_beam_search(const TannIndexView* index, const TannBeamParams* params,
                            const float* lut /*dev or NULL*/, const void* queries /*dev or NULL*/,
                            uint32_t query_kind, uint64_t num_queries,
                            const uint32_t* entry_offsets /*dev [Q+1]*/,
                            const uint32_t* entry_ids /*dev*/, void* out_candidates /*dev*/,
                            uint32_t* out_stats /*dev*/, uint32_t* status /*dev or NULL*/,
                            tann_stream_t stream);

/* Shared-memory bytes and resident blocks per SM the beam-search kernel gets for these sizes
 * (for reports; returns TANN_ERR_UNSUPPORTED when the sizes do not fit one block). */
TannStatus tann_beam_search_occupancy(const TannIndexView* index, const TannBeamParams* params,
                                      int lut_in_kernel, uint32_t* smem_bytes,
                                      uint32_t* blocks_per_sm, uint32_t* grid_blocks);

/*
 * RVQ entry selection: nearest coarse centroid, nearest non-empty fine bucket of the residual,
 * then the first `entry_count` ids of that bucket (else `fallback_entry`), unused slots
 * 0xffffffff. Replaces RVQ::search + gather_rvq_entries_kernel
 * (src/legacy_rvq/gas_legacy/anns/RVQ/RVQ.cu:792-882, src/search/rvq_device_entries.cu:15-52).
 *   coarse_t / fine_t   dev, codebooks transposed to [dim][count];
 *   coarse_norms / fine_norms dev, from tann_rvq_norms;
 *   bucket_sizes dev int32 [coarse*fine] (uncapped sizes), cluster_offsets / cluster_ids the CSR of
 *   posting lists capped at 256 ids (src/search/rvq_entry_provider.cpp:21,115-144);
 *   out_clusters dev int32 [Q] (optional), out_entry_ids dev [Q][entry_count],
 *   out_entry_offsets dev [Q+1] = q * entry_count (optional).
 */
TannStatus tann_rvq_norms(const float* rows /*dev [count][dim]*/, uint32_t count, uint32_t dim,
                          float* out_norms /*dev*/, tann_stream_t stream);
TannStatus tann_rvq_entries(const float* queries /*dev [Q][dim]*/, uint64_t num_queries,
                            uint32_t dim, const float* coarse /*dev [nc][dim]*/,
                            const float* coarse_t, const float* coarse_norms, uint32_t num_coarse,
                            const float* fine_t, const float* fine_norms, uint32_t num_fine,
                            const int32_t* bucket_sizes, const uint32_t* cluster_offsets,
                            const uint32_t* cluster_ids, uint32_t entry_count,
                            uint32_t fallback_entry, int32_t* out_clusters,
                            uint32_t* out_entry_ids, uint32_t* out_entry_offsets,
                            tann_stream_t stream);

/*
 * pq2 refine and re-sort of the first refine_top_l candidates of every query. Replaces
 * RunPq2RefineBatchDevice (src/search/rerank_exact.cu:2263-2455; kernels :573-665 plain,
 * :773-879 residual). base_codes == NULL selects the plain form. Output: dev
 * [Q][refine_top_l] records sorted by (distance, id), expanded flags cleared. `status` is accepted for
 * symmetry and not written: the ids come out of tann_beam_search, which has range-checked them.
 */
TannStatus tann_pq2_refine(const void* candidates /*dev [Q][capacity]*/,
                           const uint32_t* stats /*dev [Q][8]*/, uint64_t num_queries,
                           uint32_t capacity, uint32_t refine_top_l, const TannShards* base_codes,
                           const TannShards* pq2_codes, uint32_t num_chunks,
                           const float* lut2 /*dev [Q][M][256]*/,
                           const float* cross_terms /*dev [M][256][256] or NULL*/,
                           void* out_candidates /*dev*/, uint32_t* status, tann_stream_t stream);

/*
 * Hybrid-PQ (HPQ) refine and re-sort of the first refine_top_l candidates of every query. Replaces
 * detail::RunHpqRefineBatchDevice (src/search/rerank_exact.cu:2457-2531; kernel :667-771): every node has one
 * code per chunk and one selector bit per chunk (row of (M + 7) / 8 bytes, bit m & 7 of byte m >> 3); the bit
 * picks the base or the outlier codebook's query table for that chunk; distance = lane-strided sums + shuffle
 * tree. hybrid_codes and selector_bits may live in device memory or mapped pinned host memory (the reference:
 * mapped host memory only). Output as tann_pq2_refine.
 */
TannStatus tann_hpq_refine(const void* candidates /*dev [Q][capacity]*/, const uint32_t* stats /*dev [Q][8]*/,
                           uint64_t num_queries, uint32_t capacity, uint32_t refine_top_l,
                           const TannShards* hybrid_codes, const uint8_t* selector_bits /*[N][(M+7)/8]*/,
                           uint32_t num_chunks, const float* base_lut /*dev [Q][M][256]*/,
                           const float* outlier_lut /*dev [Q][M][256]*/, void* out_candidates /*dev*/,
                           uint32_t* status, tann_stream_t stream);

/* X[m][b][r] = 2 * sum_dim (T1[b][dim]+mu1[dim]) * (T2[r][dim]+mu2[dim]); replaces the host loop
 * BuildPq2CrossTerms (src/search/search_resources.cpp:52-91), same order, no FMA. */
TannStatus tann_pq2_cross_terms(uint32_t dim, uint32_t num_chunks,
                                const uint32_t* chunk_offsets /*dev*/,
                                const float* tables1_row_major /*dev [256][dim]*/,
                                const float* centroid1 /*dev*/,
                                const float* tables2_row_major /*dev*/,
                                const float* centroid2 /*dev*/, float* out /*dev*/,
                                tann_stream_t stream);

typedef struct TannRerankParams {
    uint32_t top_n;           /* ranks [0, top_n) of each candidate list are scored */
    uint32_t top_k;
    uint32_t tile;            /* rank tile for the bound filter and the early stop; 0 = one tile */
    uint32_t use_bound_filter;
    /* Early stop of the reference's persistent rerank (src/io/bam_vector_provider.cu:1124-1135): after a
     * tile that ends at rank >= early_stop_min_prefix, with a finite k-th best exact distance, a tile
     * that does not improve the k-th distance counts as stable (an improving one resets the count);
     * early_stop_patience_tiles stable tiles end the query's rerank, later ranks are not scored. */
    uint32_t use_early_stop;
    uint32_t early_stop_min_prefix;
    uint32_t early_stop_patience_tiles;
    uint32_t reserved;
} TannRerankParams;

/*
 * Exact rerank: exact distances of ranks [0, top_n), optional pq2 lower-bound filter in rank
 * tiles, sort by (distance, id), top-k. Replaces RerankExact::RunBatch* and
 * detail::RunBatchFloat32FromDeviceTopology (src/search/rerank_exact.cu:242-311 distance,
 * :434-571 bound filter, :153-204 sort, :1426-1737 and :1743-2165 drivers). uint8 queries on
 * uint8 vectors are computed in integers (dp4a) and converted once; every other pair of kinds
 * uses the reference's float order (lane-strided FMA partials + shuffle tree).
 *   out_dists / out_ids dev [Q][top_n] sorted, skipped or invalid ranks = (+inf, 0xffffffff);
 *   out_counts dev uint64[2] += { exact distances computed, candidates filtered } (optional);
 *   status dev uint32 or NULL: TANN_STATUS_RERANK_ID_RANGE is or-ed in when a candidate id >= num_nodes is skipped.
 */
TannStatus tann_rerank_exact(const TannIndexView* index, const TannRerankParams* params,
                             const void* candidates /*dev [Q][capacity]*/, uint32_t capacity,
                             uint64_t num_queries, const void* queries /*dev [Q][dim]*/,
                             uint32_t query_kind, const float* error_bounds /*dev [N] or NULL*/,
                             float* out_dists /*dev*/, uint32_t* out_ids /*dev*/,
                             unsigned long long* out_counts /*dev or NULL*/, uint32_t* status,
                             tann_stream_t stream);

/* ---- learned rerank stop (the reference's persistent rerank, src/io/bam_vector_provider.cu) ----
 * The folded linear model and stage schedule, field for field DeviceRerankLearnedStopConfig
 * (src/io/bam_vector_provider.cu:65-79). */
#define TANN_RERANK_STOP_FEATURES 13
#define TANN_RERANK_STOP_MAX_STAGES 64
#define TANN_RERANK_STOP_HEAD_PROBE 8 /* ranks of the next window that are looked at (:56) */
typedef struct TannRerankLearnedStop {
    uint32_t enabled;
    uint32_t feature_variant; /* 0 = all 13 features, 1 = the six-feature variant (:59-63) */
    uint32_t num_stages;
    uint32_t top_k;
    uint32_t bootstrap_prefix;
    uint32_t initial_stage_index;
    uint32_t stage_prefixes[TANN_RERANK_STOP_MAX_STAGES];
    float linear_weights[TANN_RERANK_STOP_FEATURES];
    float bias;
    float threshold_logit;
    float budget_log2;
    float inv_budget_top_n;
    float inv_top_k;
} TannRerankLearnedStop;

/* Reads a model file ("key = value" lines: stage_prefixes, feature_means, feature_inv_stds, weights,
 * feature_mask, bias, threshold_logit, threshold_logit_top_l_<n>, top_k, bootstrap_prefix; 13 features or
 * the older 12) and folds it for a rerank budget of budget_top_n ranks, as
 * LoadRerankLearnedStopConfigFromFile does (src/io/bam_vector_provider.cu:125-279). Host only. */
TannStatus tann_rerank_learned_stop_load(const char* path, uint32_t budget_top_n, uint32_t top_k,
                                         TannRerankLearnedStop* out);

/*
 * Exact rerank with the reference's learned stop, stage schedule and stop-prefix replay
 * (persistent_bam_rerank_kernel_float32_dim, src/io/bam_vector_provider.cu:721-1323, with the vectors
 * read from the index view instead of the NVMe page cache). Per query a sorted list of the top_k best
 * (distance, id) is kept; ranks [0, min(top_n, capacity)) are scored window by window: up to
 * model->bootstrap_prefix, then from stage prefix to stage prefix (plain tiles of params->tile ranks when
 * the model is NULL or not enabled, and after the last stage). At a stage boundary the 13 features
 * are taken (:542-596, :976-1019) and the query stops when the logit falls below threshold_logit. With
 * replay_stop_prefixes the model is not evaluated; query q stops at the first window end >= its
 * recorded prefix (:1111-1122). params->use_early_stop applies at window ends where no stage is due
 * (:1123-1135); params->use_bound_filter as in tann_rerank_exact. The next-window features (weights 8
 * and 9) read the candidates' lower bounds, so a model that uses them needs error_bounds.
 *   out_dists / out_ids     dev [Q][top_k], sorted, unfilled = (+inf, 0xffffffff);
 *   out_stop_prefixes       dev [Q] ranks scored when the query stopped (min(top_n, capacity) if it never did);
 *   out_checkpoint_counts   dev [Q] model evaluations; out_stop_flags dev [Q] 1 = stopped by the model / replay /
 *                           early stop. All three optional.
 */
TannStatus tann_rerank_exact_learned_stop(const TannIndexView* index, const TannRerankParams* params,
                                          const TannRerankLearnedStop* model /*host or NULL*/,
                                          const void* candidates /*dev [Q][capacity]*/, uint32_t capacity,
                                          uint64_t num_queries, const void* queries /*dev [Q][dim]*/,
                                          uint32_t query_kind, const float* error_bounds /*dev [N] or NULL*/,
                                          const uint32_t* replay_stop_prefixes /*dev [Q] or NULL*/,
                                          float* out_dists /*dev*/, uint32_t* out_ids /*dev*/,
                                          unsigned long long* out_counts /*dev or NULL*/,
                                          uint32_t* out_stop_prefixes, uint32_t* out_checkpoint_counts,
                                          uint32_t* out_stop_flags, uint32_t* status, tann_stream_t stream);

/* Copies the first top_k (distance, id) pairs of every sorted list into dense [Q][top_k] arrays
 * (one small D2H copy instead of the reference's per-query host loops,
 * src/search/rerank_exact.cu:1310-1374). */
TannStatus tann_topk_pack(const float* dists /*dev [Q][top_n]*/, const uint32_t* ids, uint64_t num_queries,
                          uint32_t top_n, uint32_t top_k, float* out_dists /*dev [Q][top_k]*/,
                          uint32_t* out_ids, tann_stream_t stream);

/* ---- exact rerank by the owner of the rows (indexes sharded by node-id range over several GPUs) ----
 * NO COUNTERPART IN THE REFERENCE (single GPU). Instead of reading candidates' vectors from other GPUs'
 * shards, the GPU that ran the traversal splits every query's candidate list by owner, the lists are
 * exchanged (one all-to-all), every owner scores what it received against its own shard with
 * tann_rerank_exact + tann_topk_pack on a view of that shard alone, the [Q][top_k] lists travel back (a
 * second all-to-all) and are merged. Exact distances and the (distance, id) order do not depend on where a
 * row is scored: the result is the unsharded one, bit for bit.
 *
 * tann_partition_candidates: ranks [0, min(top_n, capacity)) of every list; owner = id / rows_per_shard.
 *   out       dev [num_owners][Q][slot] records (id = row number inside the owner's shard, distance kept);
 *             unused tail = (0xffffffff, 0); ids beyond the last owner are dropped;
 *   overflow  dev uint32, or-ed with 1 when some (query, owner) list had more than `slot` records (the
 *             excess is dropped: rerun with a larger slot; slot = top_n can never overflow).
 * tann_merge_topk_lists: dists / ids dev [num_lists][Q][top_k] sorted lists (top_k <= 32), list l holding
 *   row numbers of shard l; out dev [Q][top_k]: the top_k smallest by (distance, l * rows_per_shard + id),
 *   ids global; unfilled = (+inf, 0xffffffff). */
TannStatus tann_partition_candidates(const void* candidates /*dev [Q][capacity]*/, uint32_t capacity, uint32_t top_n,
                                     uint64_t num_queries, uint64_t rows_per_shard, uint32_t num_owners,
                                     uint32_t slot, void* out, uint32_t* overflow, tann_stream_t stream);
TannStatus tann_merge_topk_lists(const float* dists, const uint32_t* ids, uint32_t num_lists, uint64_t num_queries,
                                 uint32_t top_k, uint64_t rows_per_shard, float* out_dists, uint32_t* out_ids,
                                 tann_stream_t stream);

/* Exact rerank + top-k of one batch (tann_rerank_exact followed by tann_topk_pack, same results)
 * that allocates nothing: its work space is a fixed device array of TANN_STATIC_SCRATCH_BYTES inside
 * the library. NO COUNTERPART IN THE REFERENCE. It is for callers that may not call cudaMalloc /
 * cudaFree where they rerank (both synchronise the whole device, which stalls every other stream of a
 * serving process) and that hold no pre-allocated work space.
 *   - needs 256 + align256(Q*dim) [float queries on uint8 vectors] + 2*align256(Q*top_n*4) bytes;
 *     larger batches return TANN_ERR_UNSUPPORTED with the sizes in tann_last_error();
 *   - the first call on a device looks up the array's address with that device current: make that
 *     call before any stream capture;
 *   - calls that overlap on the GPU (other streams or threads) share the array and race: serialise them. */
#define TANN_STATIC_SCRATCH_BYTES (8u << 20)
TannStatus tann_rerank_topk_static(const TannIndexView* index, const TannRerankParams* params,
                                   const void* candidates /*dev [Q][capacity]*/, uint32_t candidate_capacity,
                                   uint64_t num_queries, const void* queries /*dev [Q][dim]*/,
                                   uint32_t query_kind, const float* error_bounds /*dev [N] or NULL*/,
                                   float* out_dists /*dev [Q][top_k]*/, uint32_t* out_ids /*dev [Q][top_k]*/,
                                   tann_stream_t stream);

/* Fills rows [first_node, first_node + num_rows) of the optional neighbour-code layout
 * (TannIndexView::neighbor_codes): out[row][j][0..M) = codes[adjacency[first_node + row][j]], zeros for padding
 * slots. `out` is dev, num_rows * degree * num_chunks bytes, 16-byte aligned; a rank of a sharded index builds its
 * own node range (peer code rows are read over NVLink). No counterpart in the reference. */
TannStatus tann_neighbor_codes_build(const TannIndexView* index, uint64_t first_node, uint64_t num_rows,
                                     void* out /*dev*/, tann_stream_t stream);

/* ---- memory helpers for the providers (HBM-resident, NVLink-peer, pinned-host / UVA) -------- */
TannStatus tann_device_alloc(uint64_t bytes, void** out_dev);
TannStatus tann_device_free(void* dev);
/* Pinned, device-mapped host memory (stands in for the SSD tier): returns host and device views. */
TannStatus tann_host_alloc_mapped(uint64_t bytes, void** out_host, void** out_dev);
TannStatus tann_host_free(void* host);
/* Cross-process sharing of a tann_device_alloc'd buffer between the ranks of one box. */
#define TANN_IPC_HANDLE_BYTES 64
TannStatus tann_ipc_export(void* dev, unsigned char handle[TANN_IPC_HANDLE_BYTES]);
TannStatus tann_ipc_open(const unsigned char handle[TANN_IPC_HANDLE_BYTES], void** out_dev);
TannStatus tann_ipc_close(void* dev);
TannStatus tann_enable_peer_access(int peer_device);

/* ---- whole path behind one call, host buffers in and out ------------------------------------
 * A searcher owns the device work space for batches of up to max_queries queries, so that a call
 * allocates nothing. tann_searcher_run copies the queries host -> device, runs entry selection
 * (RVQ model if one is attached, else the given fixed entries), table build, beam search,
 * optional pq2 refine / bound filter, exact rerank and top-k packing, and copies ids and
 * distances back. It is what TopoAnnsSearch::RunBatchFloat32Fused does
 * (src/search/topoanns_search.cpp:330-344) minus the per-query host materialisation.
 * Page-locked caller buffers (cudaHostAlloc / cudaHostRegister) are copied from and to directly,
 * pageable ones go through the searcher's pinned staging buffers. With a pq2 view attached the
 * second-level table entries are computed inside the refine kernel (no Q x M x 256 table is built).
 */
typedef struct TannRvqModelView {
    uint32_t dim, num_coarse, num_fine, entry_count;
    uint32_t fallback_entry, reserved;
    const float* coarse;       /* dev [nc][dim] */
    const float* coarse_t;     /* dev [dim][nc] */
    const float* coarse_norms; /* dev */
    const float* fine_t;       /* dev [dim][nf] */
    const float* fine_norms;   /* dev */
    const int32_t* bucket_sizes;
    const uint32_t* cluster_offsets;
    const uint32_t* cluster_ids;
} TannRvqModelView;

typedef struct TannPq2View {
    uint32_t enabled, residual;
    uint32_t refine_top_l, reserved;
    TannShards codes;                 /* pq2 codes, rows of M uint8 */
    const float* tables_col_major;    /* dev [dim][256] */
    const float* centroid;            /* dev */
    const uint32_t* chunk_offsets;    /* dev */
    const float* cross_terms;         /* dev or NULL */
    const float* error_bounds;        /* dev [N] or NULL */
} TannPq2View;

typedef struct TannSearcher TannSearcher;

TannStatus tann_searcher_create(const TannIndexView* index, uint64_t max_queries,
                                uint32_t max_candidate_capacity, uint32_t max_top_n,
                                uint32_t max_entries_per_query, TannSearcher** out);
TannStatus tann_searcher_set_rvq(TannSearcher* s, const TannRvqModelView* rvq);
TannStatus tann_searcher_set_pq2(TannSearcher* s, const TannPq2View* pq2);
/* Reranks of this searcher run the persistent rerank with this learned-stop model (folded for the top_n the
 * runs will use, see tann_rerank_learned_stop_load); NULL switches back to the plain rerank. */
TannStatus tann_searcher_set_rerank_learned_stop(TannSearcher* s, const TannRerankLearnedStop* model);
/* queries_host: [Q][dim] of query_kind. fixed_entries_host may be NULL when an RVQ model is set.
 * out_ids_host / out_dists_host: [Q][top_k]. out_stats_host: [Q][8] or NULL. */
TannStatus tann_searcher_run(TannSearcher* s, const TannBeamParams* beam,
                             const TannRerankParams* rerank, const void* queries_host,
                             uint32_t query_kind, uint64_t num_queries,
                             const uint32_t* fixed_entries_host, uint32_t num_fixed_entries,
                             uint32_t* out_ids_host, float* out_dists_host,
                             uint32_t* out_stats_host, tann_stream_t stream);
/* tann_searcher_run in two halves, for pipelining: submit enqueues the H2D copy, the kernels and the D2H copy
 * on `stream` and returns without waiting; wait blocks until that batch's results are in the host buffers. Two
 * searchers on two streams, submitted alternately, overlap one batch's copies with the other's kernels. One
 * batch per searcher may be in flight; host buffers must stay valid until wait returns. An early return of
 * submit (Q == 0 or an error) leaves nothing pending. */
TannStatus tann_searcher_submit(TannSearcher* s, const TannBeamParams* beam,
                                const TannRerankParams* rerank, const void* queries_host,
                                uint32_t query_kind, uint64_t num_queries,
                                const uint32_t* fixed_entries_host, uint32_t num_fixed_entries,
                                uint32_t* out_ids_host, float* out_dists_host,
                                uint32_t* out_stats_host, tann_stream_t stream);
TannStatus tann_searcher_wait(TannSearcher* s);
/* Same, device buffers in and out, nothing copied; results stay in the searcher's buffers until
 * the next call. Pointers returned through out_* are device pointers owned by the searcher. */
TannStatus tann_searcher_run_device(TannSearcher* s, const TannBeamParams* beam,
                                    const TannRerankParams* rerank, const void* queries_dev,
                                    uint32_t query_kind, uint64_t num_queries,
                                    const uint32_t* entry_offsets_dev, const uint32_t* entry_ids_dev,
                                    const uint32_t** out_ids_dev, const float** out_dists_dev,
                                    const uint32_t** out_stats_dev, tann_stream_t stream);
TannStatus tann_searcher_destroy(TannSearcher* s);
/* The searcher's device status word (TANN_STATUS_* bits of its last run; cleared when a run starts).
 * tann_searcher_wait / tann_searcher_run read it back and return TANN_ERR_DEVICE_CHECK when it is non-zero (the
 * results are still delivered); callers of tann_searcher_run_device read it themselves. */
TannStatus tann_searcher_status_device(TannSearcher* s, const uint32_t** out_status_dev);

/* Mean time in nanoseconds of one dependent random 4-byte load out of `bytes` bytes of device memory at `base`
 * (one thread chasing `steps` loads, each address derived from the value just read): the memory round trip that
 * one expansion of the beam search cannot go below. A measurement aid for reports; synchronises `stream`.
 * No counterpart in the reference. */
TannStatus tann_dependent_load_ns(const void* base /*dev*/, uint64_t bytes, uint32_t steps, float* out_ns /*host*/,
                                  tann_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TOPOANNS_B200_H_ */
