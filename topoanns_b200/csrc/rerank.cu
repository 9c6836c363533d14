// Exact rerank fused per query: exact distances of ranks [0, top_n) of the candidate list, the
// optional pq2 lower-bound filter in rank tiles, the final (distance, id) sort and the top-k
// copy, all in one persistent kernel with no host round trip between tiles.
//
// Values follow the reference: distance = lane-strided FMA partial sums of
// (float(v) - float(q))^2 and the 16/8/4/2/1 shuffle tree (src/search/rerank_exact.cu:242-276);
// lower bound (:137-142) against the running k-th smallest exact distance of the ranks handled so
// far (:434-497,541-571); |q|^2 summed in double and rounded once (:1892-1899); sort order
// (distance, id) (:92-100,153-204). uint8 queries on uint8 vectors with dim <= 256 take an integer
// path (|a-b| per byte, dp4a square-accumulate): every partial sum of the reference's float
// accumulation is then an integer below 2^24, so both give the same bits.
//
// Work split: one thread per rank reads the candidate record, applies the bound filter and works
// out the vector's address; then 8 lanes per candidate ("octet") read the row with 16-byte loads,
// several candidates per octet in flight. For float rows octet lane p owns the reference's lanes
// 4p..4p+3 (dims 32k+4p..32k+4p+3, ascending k), so every partial sum and every tree step is the
// reference's. Rows that do not start on 16-byte boundaries take a warp-per-candidate path.
#include "tann_common.cuh"
#include "tann_launch.h"

namespace tann {

constexpr int kRerankThreads = 128;
constexpr unsigned long long kInvalidKey64 = 0xff800000ffffffffull;

__device__ __forceinline__ const uint8_t* VectorPtr(const TannIndexView& ix, uint32_t id) {
    uint32_t local = id;
    const uint8_t* base = static_cast<const uint8_t*>(ix.vectors.base[0]);
    if (ix.vectors.num_shards > 1) {
        const uint64_t shard = id / ix.vectors.rows_per_shard;
        local = (uint32_t)(id - shard * ix.vectors.rows_per_shard);
        base = static_cast<const uint8_t*>(ix.vectors.base[shard]);
    }
    // src/io/vector_page_layout.cpp:50-57
    const uint32_t page = local / ix.vectors_per_page;
    const uint32_t slot = local - page * ix.vectors_per_page;
    return base + (uint64_t)page * ix.page_bytes + (uint64_t)slot * ix.vector_bytes;
}

__device__ __forceinline__ float LowerBoundSq(float approx_sq, float err) {
    const float a = sqrtf(fmaxf(approx_sq, 0.0f));
    const float lo = fmaxf(0.0f, a - err);
    return lo * lo;
}

__device__ __forceinline__ uint32_t SqDiffBytes(uint32_t a, uint32_t b, uint32_t acc) {
    const uint32_t ad = __vabsdiffu4(a, b);
    return __dp4a(ad, ad, acc);
}

// Integer rows: kStep candidates per octet and step; dim / 16 sixteen-byte pieces per row.
template <uint32_t kStep, uint32_t kOctets>
__device__ __forceinline__ void OctetRanksInt(unsigned long long* keys, const uint32_t* rank_ids,
                                              const uint8_t* qrow, uint32_t dim, uint32_t begin, uint32_t end,
                                              uint32_t octet, uint32_t ol) {
    const uint32_t pieces = dim / 16;
    // The loop bound is the warp's first octet, so all 32 lanes make the same number of trips (the
    // shuffles below need every lane); octets past the end carry invalid slots and write nothing.
    for (uint32_t w0 = begin + (octet & ~3u) * kStep; w0 < end; w0 += kOctets * kStep) {
        const uint32_t r0 = w0 + (octet & 3u) * kStep;
        unsigned long long ptr[kStep];
        uint32_t acc[kStep];
        bool live = false;
#pragma unroll
        for (uint32_t g = 0; g < kStep; ++g) {
            ptr[g] = (r0 + g < end) ? keys[r0 + g] : kInvalidKey64;
            acc[g] = 0;
            live = live || ptr[g] != kInvalidKey64;
        }
        if (!__any_sync(kFull, live)) continue;   // every slot of this step is empty (filtered or past the list)
        for (uint32_t j = ol; j < pieces; j += 8) {
            uint4 v[kStep];
#pragma unroll
            for (uint32_t g = 0; g < kStep; ++g)
                v[g] = ptr[g] != kInvalidKey64 ? __ldg(reinterpret_cast<const uint4*>(ptr[g]) + j)
                                               : make_uint4(0, 0, 0, 0);
            const uint4 qv = reinterpret_cast<const uint4*>(qrow)[j];
#pragma unroll
            for (uint32_t g = 0; g < kStep; ++g) {
                acc[g] = SqDiffBytes(v[g].x, qv.x, acc[g]);
                acc[g] = SqDiffBytes(v[g].y, qv.y, acc[g]);
                acc[g] = SqDiffBytes(v[g].z, qv.z, acc[g]);
                acc[g] = SqDiffBytes(v[g].w, qv.w, acc[g]);
            }
        }
#pragma unroll
        for (uint32_t g = 0; g < kStep; ++g) {
            acc[g] += __shfl_xor_sync(kFull, acc[g], 4);
            acc[g] += __shfl_xor_sync(kFull, acc[g], 2);
            acc[g] += __shfl_xor_sync(kFull, acc[g], 1);
        }
        if (ol == 0) {
#pragma unroll
            for (uint32_t g = 0; g < kStep; ++g)
                if (ptr[g] != kInvalidKey64) keys[r0 + g] = KeyOf(static_cast<float>(acc[g]), rank_ids[r0 + g]);
        }
    }
}

// Float rows with float queries, dim a multiple of 4.
template <uint32_t kStep, uint32_t kOctets>
__device__ __forceinline__ void OctetRanksF32(unsigned long long* keys, const uint32_t* rank_ids,
                                              const uint8_t* qrow, uint32_t dim, uint32_t begin, uint32_t end,
                                              uint32_t octet, uint32_t ol) {
    // The loop bound is the warp's first octet, so all 32 lanes make the same number of trips (the
    // shuffles below need every lane); octets past the end carry invalid slots and write nothing.
    for (uint32_t w0 = begin + (octet & ~3u) * kStep; w0 < end; w0 += kOctets * kStep) {
        const uint32_t r0 = w0 + (octet & 3u) * kStep;
        unsigned long long ptr[kStep];
        float acc[kStep][4];
        bool live = false;
#pragma unroll
        for (uint32_t g = 0; g < kStep; ++g) {
            ptr[g] = (r0 + g < end) ? keys[r0 + g] : kInvalidKey64;
            acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.0f;
            live = live || ptr[g] != kInvalidKey64;
        }
        if (!__any_sync(kFull, live)) continue;   // every slot of this step is empty (filtered or past the list)
        for (uint32_t d0 = 4 * ol; d0 < dim; d0 += 32) {
            float4 v[kStep];
#pragma unroll
            for (uint32_t g = 0; g < kStep; ++g)
                v[g] = ptr[g] != kInvalidKey64 ? __ldg(reinterpret_cast<const float4*>(ptr[g] + 4ull * d0))
                                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const float4 qv = *reinterpret_cast<const float4*>(qrow + 4u * d0);
#pragma unroll
            for (uint32_t g = 0; g < kStep; ++g) {
                float df = v[g].x - qv.x; acc[g][0] = fmaf(df, df, acc[g][0]);
                df = v[g].y - qv.y; acc[g][1] = fmaf(df, df, acc[g][1]);
                df = v[g].z - qv.z; acc[g][2] = fmaf(df, df, acc[g][2]);
                df = v[g].w - qv.w; acc[g][3] = fmaf(df, df, acc[g][3]);
            }
        }
#pragma unroll
        for (uint32_t g = 0; g < kStep; ++g) {
            // tree steps 16, 8, 4 of the reference's 32 lanes = octet lanes +4, +2, +1
#pragma unroll
            for (int off = 4; off >= 1; off >>= 1) {
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[g][i] += __shfl_down_sync(kFull, acc[g][i], off, 8);
            }
            acc[g][0] += acc[g][2];   // step 2
            acc[g][1] += acc[g][3];
            acc[g][0] += acc[g][1];   // step 1
        }
        if (ol == 0) {
#pragma unroll
            for (uint32_t g = 0; g < kStep; ++g)
                if (ptr[g] != kInvalidKey64) keys[r0 + g] = KeyOf(acc[g][0], rank_ids[r0 + g]);
        }
    }
}

// uint8 rows with float queries that are not uint8-valued: the same lane ownership as the float
// rows, four bytes per lane and 32 dims.
template <uint32_t kStep, uint32_t kOctets>
__device__ __forceinline__ void OctetRanksU8F32(unsigned long long* keys, const uint32_t* rank_ids,
                                                const uint8_t* qrow, uint32_t dim, uint32_t begin, uint32_t end,
                                                uint32_t octet, uint32_t ol) {
    for (uint32_t w0 = begin + (octet & ~3u) * kStep; w0 < end; w0 += kOctets * kStep) {
        const uint32_t r0 = w0 + (octet & 3u) * kStep;
        unsigned long long ptr[kStep];
        float acc[kStep][4];
        bool live = false;
#pragma unroll
        for (uint32_t g = 0; g < kStep; ++g) {
            ptr[g] = (r0 + g < end) ? keys[r0 + g] : kInvalidKey64;
            acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.0f;
            live = live || ptr[g] != kInvalidKey64;
        }
        if (!__any_sync(kFull, live)) continue;   // every slot of this step is empty (filtered or past the list)
        for (uint32_t d0 = 4 * ol; d0 < dim; d0 += 32) {
            uint32_t v[kStep];
#pragma unroll
            for (uint32_t g = 0; g < kStep; ++g)
                v[g] = ptr[g] != kInvalidKey64 ? __ldg(reinterpret_cast<const uint32_t*>(ptr[g] + d0)) : 0u;
            const float4 qv = *reinterpret_cast<const float4*>(qrow + 4u * d0);
#pragma unroll
            for (uint32_t g = 0; g < kStep; ++g) {
                float df = static_cast<float>(v[g] & 0xffu) - qv.x; acc[g][0] = fmaf(df, df, acc[g][0]);
                df = static_cast<float>((v[g] >> 8) & 0xffu) - qv.y; acc[g][1] = fmaf(df, df, acc[g][1]);
                df = static_cast<float>((v[g] >> 16) & 0xffu) - qv.z; acc[g][2] = fmaf(df, df, acc[g][2]);
                df = static_cast<float>(v[g] >> 24) - qv.w; acc[g][3] = fmaf(df, df, acc[g][3]);
            }
        }
#pragma unroll
        for (uint32_t g = 0; g < kStep; ++g) {
#pragma unroll
            for (int off = 4; off >= 1; off >>= 1) {
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[g][i] += __shfl_down_sync(kFull, acc[g][i], off, 8);
            }
            acc[g][0] += acc[g][2];
            acc[g][1] += acc[g][3];
            acc[g][0] += acc[g][1];
        }
        if (ol == 0) {
#pragma unroll
            for (uint32_t g = 0; g < kStep; ++g)
                if (ptr[g] != kInvalidKey64) keys[r0 + g] = KeyOf(acc[g][0], rank_ids[r0 + g]);
        }
    }
}

// How a block scores its ranks; the same for every tile of a query.
struct ScoreMode {
    bool int_path;      // uint8 rows and uint8 queries: integer arithmetic
    bool octet_int;     // ... with rows on 16-byte boundaries and dim a multiple of 16
    bool octet_f32;     // float rows, float queries, rows on 16-byte boundaries
    bool octet_u8f32;   // uint8 rows, float queries
    uint32_t qkind;
};

// Exact distances of ranks [rb, end): keys[r] holds the address of rank r's vector (or the invalid
// key) on entry and its (distance, id) sort key on return. Called by all kGroupThreads threads that
// share the range (a block of kRerankThreads, or one warp); tid is the thread's number among them.
template <uint32_t kGroupThreads>
__device__ __forceinline__ void ScoreRanks(const TannIndexView& ix, const ScoreMode& m, unsigned long long* keys,
                                           const uint32_t* rank_ids, const uint8_t* qrow, uint32_t rb, uint32_t end,
                                           uint32_t tid) {
    constexpr uint32_t kOct = kGroupThreads / 8;
    const uint32_t lane = tid & 31, warp = tid >> 5;
    const uint32_t dim = ix.dim, rc = end - rb, qkind = m.qkind;
    const bool int_path = m.int_path, octet_int = m.octet_int, octet_f32 = m.octet_f32, octet_u8f32 = m.octet_u8f32;
    if (octet_int) {
        if (rc >= 64) OctetRanksInt<4, kOct>(keys, rank_ids, qrow, dim, rb, end, tid >> 3, lane & 7);
        else OctetRanksInt<2, kOct>(keys, rank_ids, qrow, dim, rb, end, tid >> 3, lane & 7);
    } else if (octet_f32) {
        if (rc >= 64) OctetRanksF32<4, kOct>(keys, rank_ids, qrow, dim, rb, end, tid >> 3, lane & 7);
        else OctetRanksF32<2, kOct>(keys, rank_ids, qrow, dim, rb, end, tid >> 3, lane & 7);
    } else if (octet_u8f32) {
        if (rc >= 64) OctetRanksU8F32<4, kOct>(keys, rank_ids, qrow, dim, rb, end, tid >> 3, lane & 7);
        else OctetRanksU8F32<2, kOct>(keys, rank_ids, qrow, dim, rb, end, tid >> 3, lane & 7);
    } else {
        // A warp scores kGroup candidates per step: all their row loads are issued before any
        // reduction, so several random reads are in flight per lane.
        constexpr uint32_t kGroup = 4;
        for (uint32_t r0 = rb + warp * kGroup; r0 < end; r0 += (kGroupThreads / 32) * kGroup) {
            const uint8_t* vptr[kGroup];
            bool act[kGroup];
#pragma unroll
            for (uint32_t g = 0; g < kGroup; ++g) {
                const unsigned long long slot = (r0 + g < end) ? keys[r0 + g] : kInvalidKey64;
                act[g] = slot != kInvalidKey64;
                vptr[g] = reinterpret_cast<const uint8_t*>(slot);
            }
            bool live = false;
#pragma unroll
            for (uint32_t g = 0; g < kGroup; ++g) live = live || act[g];
            if (!live) continue;   // the same for every lane of the warp
            float dist[kGroup];
            if (int_path) {
                uint32_t acc[kGroup];
#pragma unroll
                for (uint32_t g = 0; g < kGroup; ++g) acc[g] = 0;
                const uint32_t* q4 = reinterpret_cast<const uint32_t*>(qrow);
                for (uint32_t i = lane; i < dim / 4; i += 32) {
                    uint32_t w[kGroup];
#pragma unroll
                    for (uint32_t g = 0; g < kGroup; ++g)
                        w[g] = act[g] ? __ldg(reinterpret_cast<const uint32_t*>(vptr[g]) + i) : 0u;
                    const uint32_t qw = q4[i];
#pragma unroll
                    for (uint32_t g = 0; g < kGroup; ++g) acc[g] = SqDiffBytes(w[g], qw, acc[g]);
                }
#pragma unroll
                for (uint32_t g = 0; g < kGroup; ++g) {
#pragma unroll
                    for (int off = 16; off >= 1; off >>= 1) acc[g] += __shfl_xor_sync(kFull, acc[g], off);
                    dist[g] = static_cast<float>(acc[g]);
                }
            } else {
                float acc[kGroup];
#pragma unroll
                for (uint32_t g = 0; g < kGroup; ++g) acc[g] = 0.0f;
                for (uint32_t i = lane; i < dim; i += 32) {
                    float v[kGroup];
#pragma unroll
                    for (uint32_t g = 0; g < kGroup; ++g)
                        v[g] = act[g] ? LoadAsFloat<float>(vptr[g], ix.vector_kind, i) : 0.0f;
                    const float qv = LoadAsFloat<float>(qrow, qkind, i);
#pragma unroll
                    for (uint32_t g = 0; g < kGroup; ++g) {
                        const float diff = v[g] - qv;
                        acc[g] = fmaf(diff, diff, acc[g]);
                    }
                }
#pragma unroll
                for (uint32_t g = 0; g < kGroup; ++g) dist[g] = WarpTreeSum(acc[g]);
            }
            if (lane == 0) {
#pragma unroll
                for (uint32_t g = 0; g < kGroup; ++g)
                    if (act[g]) keys[r0 + g] = KeyOf(dist[g], rank_ids[r0 + g]);
            }
        }
    }
}

__global__ void __launch_bounds__(kRerankThreads)
rerank_kernel(const __grid_constant__ TannIndexView ix, TannRerankParams p, const Cand* __restrict__ cand,
              uint32_t capacity, uint64_t Q, const void* __restrict__ queries, uint32_t qkind,
              const float* __restrict__ error_bounds, uint32_t padded, float* __restrict__ out_dists,
              uint32_t* __restrict__ out_ids, unsigned long long* __restrict__ out_counts,
              const uint8_t* __restrict__ queries_u8, const uint32_t* __restrict__ not_u8_flag,
              uint32_t final_ranks, uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char rr_smem[];
    // keys[r] first holds the address of candidate r's vector (or the invalid key when the rank is
    // empty or filtered), then its (distance, id) sort key.
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(rr_smem);   // [padded]
    uint32_t* rank_ids = reinterpret_cast<uint32_t*>(keys + padded);              // [padded]
    uint8_t* qrow = rr_smem + (((size_t)padded * 12 + 15) & ~(size_t)15);          // query row copy, 16-byte aligned
    __shared__ float s_threshold, s_qnorm, s_prev_kth;
    __shared__ unsigned int s_exact, s_filtered, s_stable, s_stop;
    __shared__ float s_best[128];   // the top_k <= 128 smallest exact distances so far (bound filter, early stop)
    __shared__ float s_tile[128], s_merged[128];   // a tile's distances, and the merged list under construction
    const bool track_kth = p.use_bound_filter || p.use_early_stop;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t dim = ix.dim;
    // Float queries whose values are all integers in [0, 255] (checked on the device by the caller,
    // which then passes their uint8 copy) take the integer path too: same bits, 4 bytes per load.
    const bool as_u8 = qkind == TANN_KIND_UINT8 || (queries_u8 != nullptr && not_u8_flag != nullptr && *not_u8_flag == 0u);
    const bool int_path = as_u8 && ix.vector_kind == TANN_KIND_UINT8 && (dim % 4 == 0) && dim <= 256 &&
                          (ix.vector_bytes % 4 == 0) && (ix.page_bytes % 4 == 0);
    const bool swap_queries = int_path && qkind != TANN_KIND_UINT8;
    if (swap_queries) { queries = queries_u8; qkind = TANN_KIND_UINT8; }
    const uint32_t qbytes = dim * (qkind == TANN_KIND_FLOAT32 ? 4u : 1u);
    const uint32_t tile = p.tile == 0 ? p.top_n : p.tile;
    // Rows that start on 16-byte boundaries are read with 16-byte loads by 8 lanes per candidate.
    const bool rows16 = (ix.vector_bytes % 16 == 0) && (ix.page_bytes % 16 == 0);
    const bool octet_int = int_path && rows16 && (dim % 16 == 0);
    const bool octet_f32 = !int_path && rows16 && ix.vector_kind == TANN_KIND_FLOAT32 &&
                           qkind == TANN_KIND_FLOAT32 && (dim % 4 == 0);
    const bool octet_u8f32 = !int_path && ix.vector_kind == TANN_KIND_UINT8 && qkind == TANN_KIND_FLOAT32 &&
                             (ix.vector_bytes % 4 == 0) && (ix.page_bytes % 4 == 0) && (dim % 4 == 0);
    const ScoreMode mode{int_path, octet_int, octet_f32, octet_u8f32, qkind};
    unsigned long long tot_exact = 0, tot_filtered = 0;

    for (uint64_t q = blockIdx.x; q < Q; q += gridDim.x) {
        const uint8_t* qsrc = static_cast<const uint8_t*>(queries) + q * qbytes;
        if (qbytes % 16 == 0) {
            for (uint32_t i = tid; i < qbytes / 16; i += kRerankThreads)
                reinterpret_cast<uint4*>(qrow)[i] = __ldg(reinterpret_cast<const uint4*>(qsrc) + i);
        } else {
            for (uint32_t i = tid; i < qbytes; i += kRerankThreads) qrow[i] = qsrc[i];
        }
        for (uint32_t i = tid; i < padded; i += kRerankThreads) keys[i] = kInvalidKey64;
        if (tid == 0) {
            s_threshold = __int_as_float(0x7f800000);
            s_prev_kth = __int_as_float(0x7f800000);
            s_exact = 0; s_filtered = 0; s_stable = 0; s_stop = 0;
        }
        if (track_kth) s_best[tid] = __int_as_float(0x7f800000);   // 128 threads, 128 slots
        __syncthreads();
        if (p.use_bound_filter && tid == 0) {
            double s = 0.0;
            for (uint32_t i = 0; i < dim; ++i) {
                const double v = (double)LoadAsFloat<float>(qrow, qkind, i);
                s += v * v;
            }
            s_qnorm = (float)s;
        }
        if (p.use_bound_filter) __syncthreads();
        for (uint32_t rb = 0; rb < p.top_n; rb += tile) {
            const uint32_t rc = min(tile, p.top_n - rb);
            const float threshold = s_threshold;
            // ---- one thread per rank: candidate record, bound filter, vector address ----------
            uint32_t n_act = 0, n_flt = 0;
            for (uint32_t r = rb + tid; r < rb + rc; r += kRerankThreads) {
                unsigned long long slot = kInvalidKey64;
                if (r < capacity) {
                    const Cand c = cand[q * capacity + r];
                    const uint32_t id = c.id & kRawMask;
                    if (c.id != kInvalid && id >= ix.num_nodes && status != nullptr)
                        atomicOr(status, TANN_STATUS_RERANK_ID_RANGE);   // skipped, and reported
                    if (c.id != kInvalid && id < ix.num_nodes) {
                        bool keep = true;
                        if (p.use_bound_filter && isfinite(threshold))
                            keep = !(LowerBoundSq(c.dist - s_qnorm, __ldg(error_bounds + id)) > threshold);
                        if (keep) {
                            slot = reinterpret_cast<unsigned long long>(VectorPtr(ix, id));
                            rank_ids[r] = id;
                            ++n_act;
                        } else {
                            ++n_flt;
                        }
                    }
                }
                keys[r] = slot;
            }
            n_act = __reduce_add_sync(kFull, n_act);   // one shared-memory atomic per warp, not per thread
            n_flt = __reduce_add_sync(kFull, n_flt);
            if (lane == 0 && n_act) atomicAdd(&s_exact, n_act);
            if (lane == 0 && n_flt) atomicAdd(&s_filtered, n_flt);
            __syncthreads();
            // ---- distances --------------------------------------------------------------------
            ScoreRanks<kRerankThreads>(ix, mode, keys, rank_ids, qrow, rb, rb + rc, tid);
            __syncthreads();
            if (track_kth) {
                // k-th smallest exact distance over ranks [0, rb + rc) (:541-571): the sorted best-k list is
                // kept across tiles. A tile of up to 128 distances is merged in by counting: thread t places old
                // entry t behind the tile's distances below it, and the tile's distance t behind the old entries
                // not above it and the tile's distances in front of it (ties: the lower rank first). Only the
                // values matter, so the order among equal values is free.
                const uint32_t k = p.top_k;
                if (rc <= (uint32_t)kRerankThreads) {
                    const float inf = __int_as_float(0x7f800000);
                    const float oldv = tid < k ? s_best[tid] : inf;
                    const float newv = tid < rc ? FromOrderedBits((uint32_t)(keys[rb + tid] >> 32)) : inf;
                    s_tile[tid] = newv;
                    __syncthreads();
                    uint32_t c_old = 0, c_new = 0;
#pragma unroll 4
                    for (uint32_t l = 0; l < rc; ++l) {
                        const float x = s_tile[l];
                        c_old += x < oldv ? 1u : 0u;
                        c_new += (x < newv || (x == newv && l < tid)) ? 1u : 0u;
                    }
                    uint32_t lo = 0;   // old entries <= newv (fixed-trip binary search over the k sorted values)
#pragma unroll
                    for (uint32_t b = 128; b > 0; b >>= 1) {
                        const uint32_t t = lo + b;
                        if (t <= k && s_best[t - 1] <= newv) lo = t;
                    }
                    if (tid < k && tid + c_old < k) s_merged[tid + c_old] = oldv;
                    if (tid < rc && lo + c_new < k) s_merged[lo + c_new] = newv;
                    __syncthreads();
                    if (tid < k) s_best[tid] = s_merged[tid];
                    if (tid == 0) {
                        const float kth = s_merged[k - 1];
                        s_threshold = kth;
                        if (p.use_early_stop) {   // src/io/bam_vector_provider.cu:1124-1135
                            if (rb + rc >= p.early_stop_min_prefix && isfinite(kth)) {
                                if (kth < s_prev_kth) s_stable = 0; else ++s_stable;
                                if (s_stable >= p.early_stop_patience_tiles) s_stop = 1;
                            }
                            s_prev_kth = kth;
                        }
                    }
                } else if (tid == 0) {
                    // wider tiles: insertion by one thread
                    for (uint32_t r = rb; r < rb + rc; ++r) {
                        const float x = FromOrderedBits((uint32_t)(keys[r] >> 32));
                        if (!(x < s_best[k - 1])) continue;
                        uint32_t ins = k - 1;
                        while (ins > 0 && x < s_best[ins - 1]) { s_best[ins] = s_best[ins - 1]; --ins; }
                        s_best[ins] = x;
                    }
                    const float kth = s_best[k - 1];
                    s_threshold = kth;
                    if (p.use_early_stop) {   // src/io/bam_vector_provider.cu:1124-1135
                        if (rb + rc >= p.early_stop_min_prefix && isfinite(kth)) {
                            if (kth < s_prev_kth) s_stable = 0; else ++s_stable;
                            if (s_stable >= p.early_stop_patience_tiles) s_stop = 1;
                        }
                        s_prev_kth = kth;
                    }
                }
                __syncthreads();
                if (s_stop) break;
            }
        }
        // final sort and output: bitonic network; the stages inside runs of 32 keys are done by one
        // warp per run with shuffles (no barriers), the wider stages in shared memory
        uint32_t first_k = 2;
        uint32_t out_n = p.top_n;
        if (final_ranks != 0 && final_ranks <= 32 && padded >= 64) {
            // The caller consumes only the first final_ranks <= 32 entries: sort every run of 32 keys,
            // then a tournament keeps the 32 smallest of two runs (element-wise minimum of one run and
            // the other reversed is a bitonic sequence of exactly those) and re-sorts them with five
            // shuffle stages, halving the number of runs per round.
            const uint32_t runs = padded / 32;
            for (uint32_t c = warp; c < runs; c += kRerankThreads / 32)
                keys[c * 32 + lane] = WarpSortKey(keys[c * 32 + lane], lane);
            __syncthreads();
            for (uint32_t stride = 1; stride < runs; stride <<= 1) {
                for (uint32_t a = warp * 2 * stride; a + stride < runs; a += (kRerankThreads / 32) * 2 * stride) {
                    const unsigned long long ka = keys[a * 32 + lane];
                    const unsigned long long kb = keys[(a + stride) * 32 + (31 - lane)];
                    unsigned long long m = ka < kb ? ka : kb;
#pragma unroll
                    for (uint32_t sft = 16; sft > 0; sft >>= 1) {
                        const unsigned long long o = __shfl_xor_sync(kFull, m, sft);
                        const bool upper = (lane & sft) != 0;
                        m = upper ? (o > m ? o : m) : (o < m ? o : m);
                    }
                    keys[a * 32 + lane] = m;
                }
                __syncthreads();
            }
            first_k = padded * 2;   // skips the network below
            out_n = min(p.top_n, 32u);
        } else if (padded >= 64) {
            for (uint32_t c = warp; c < padded / 32; c += kRerankThreads / 32) {
                unsigned long long k = WarpSortKey(keys[c * 32 + lane], lane);
                if (c & 1u) k = __shfl_sync(kFull, k, 31 - lane);   // odd runs descending, as the network expects
                keys[c * 32 + lane] = k;
            }
            __syncthreads();
            first_k = 64;
        }
        for (uint32_t k = first_k; k <= padded; k <<= 1) {
            for (uint32_t j = k >> 1; j > 0; j >>= 1) {
                for (uint32_t t = tid; t < padded / 2; t += kRerankThreads) {
                    const uint32_t lo = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                    const uint32_t hi = lo | j;
                    const bool asc = (lo & k) == 0;
                    const unsigned long long a = keys[lo], b = keys[hi];
                    if ((a > b) == asc) { keys[lo] = b; keys[hi] = a; }
                }
                __syncthreads();
            }
        }
        for (uint32_t i = tid; i < out_n; i += kRerankThreads) {
            const unsigned long long k = keys[i];
            out_dists[q * p.top_n + i] = FromOrderedBits((uint32_t)(k >> 32));
            out_ids[q * p.top_n + i] = (uint32_t)k;
        }
        if (tid == 0) { tot_exact += s_exact; tot_filtered += s_filtered; }
        __syncthreads();
    }
    if (tid == 0 && out_counts != nullptr) {
        if (tot_exact) atomicAdd(out_counts, tot_exact);
        if (tot_filtered) atomicAdd(out_counts + 1, tot_filtered);
    }
}

// ---- rerank with the learned stop ------------------------------------------------------------
// The reference's persistent rerank (src/io/bam_vector_provider.cu:721-1323) with the vectors read
// from the index view: per query a sorted list of the top_k best (distance, id); ranks are scored
// window by window (bootstrap prefix, then stage prefix to stage prefix, then plain tiles); at a stage
// boundary thread 0 takes the features and evaluates the folded linear model. The reference sorts a
// window and inserts it in ascending order into the list with one thread; here every thread places
// one window entry and one list entry by counting (a parallel merge). An entry enters exactly when
// fewer than top_k entries of (list + earlier window entries) are <= it, which is the reference's
// test against the list's last element at its turn, so the list and the entered count are the same.

__device__ __forceinline__ float KeyDist(unsigned long long k) { return FromOrderedBits((uint32_t)(k >> 32)); }

// src/io/bam_vector_provider.cu:542-596 (all 13 features) and :598-617 (six-feature variant)
__device__ __forceinline__ float RerankStopLogit(const TannRerankLearnedStop& c, uint32_t processed_prefix,
                                                 float current_kth, float delta_kth_last, float delta_kth_prev,
                                                 float topk_changed_flag, uint32_t entered_topk_count, float topk_spread,
                                                 uint32_t next_live, uint32_t next_count, float best_live_lb,
                                                 uint32_t window_exact, uint32_t window_count, uint32_t cumulative_exact) {
    const float prefix_frac = static_cast<float>(processed_prefix) * c.inv_budget_top_n;
    const float lb_gap = isfinite(best_live_lb) ? (best_live_lb - current_kth) : 0.0f;
    float logit = c.bias;
    logit = fmaf(c.budget_log2, c.linear_weights[0], logit);
    logit = fmaf(prefix_frac, c.linear_weights[1], logit);
    logit = fmaf(current_kth, c.linear_weights[2], logit);
    if (c.feature_variant == 1u) {
        logit = fmaf(topk_changed_flag, c.linear_weights[5], logit);
        logit = fmaf(topk_spread, c.linear_weights[7], logit);
        return fmaf(lb_gap, c.linear_weights[9], logit);
    }
    const float entered_ratio = static_cast<float>(entered_topk_count) * c.inv_top_k;
    const float live_ratio = next_count == 0u ? 0.0f : static_cast<float>(next_live) / static_cast<float>(next_count);
    const float inv_window = window_count == 0u ? 0.0f : 1.0f / static_cast<float>(window_count);
    const float exact_ratio = static_cast<float>(window_exact) * inv_window;
    const float filtered_ratio = static_cast<float>(window_count - window_exact) * inv_window;
    const float exact_frac =
        processed_prefix == 0u ? 0.0f : static_cast<float>(cumulative_exact) / static_cast<float>(processed_prefix);
    logit = fmaf(delta_kth_last, c.linear_weights[3], logit);
    logit = fmaf(delta_kth_prev, c.linear_weights[4], logit);
    logit = fmaf(topk_changed_flag, c.linear_weights[5], logit);
    logit = fmaf(entered_ratio, c.linear_weights[6], logit);
    logit = fmaf(topk_spread, c.linear_weights[7], logit);
    logit = fmaf(live_ratio, c.linear_weights[8], logit);
    logit = fmaf(lb_gap, c.linear_weights[9], logit);
    logit = fmaf(exact_ratio, c.linear_weights[10], logit);
    logit = fmaf(filtered_ratio, c.linear_weights[11], logit);
    return fmaf(exact_frac, c.linear_weights[12], logit);
}

__global__ void __launch_bounds__(kRerankThreads)
rerank_learned_kernel(const __grid_constant__ TannIndexView ix, TannRerankParams p,
                      const __grid_constant__ TannRerankLearnedStop ls, uint32_t use_schedule, uint32_t evaluate,
                      const Cand* __restrict__ cand, uint32_t capacity, uint64_t Q, const void* __restrict__ queries,
                      uint32_t qkind, const float* __restrict__ error_bounds, const uint32_t* __restrict__ replay,
                      uint32_t padded, float* __restrict__ out_dists, uint32_t* __restrict__ out_ids,
                      unsigned long long* __restrict__ out_counts, uint32_t* __restrict__ out_stop_prefixes,
                      uint32_t* __restrict__ out_checkpoints, uint32_t* __restrict__ out_stop_flags,
                      uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char rr_smem[];
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(rr_smem);   // [padded]
    uint32_t* rank_ids = reinterpret_cast<uint32_t*>(keys + padded);              // [padded]
    uint8_t* qrow = rr_smem + (((size_t)padded * 12 + 15) & ~(size_t)15);
    __shared__ unsigned long long s_top[2][kRerankThreads];   // the sorted top_k list, double-buffered
    __shared__ float s_kth, s_qnorm, s_prev_ckpt_kth, s_prev_delta;
    __shared__ unsigned int s_exact, s_filtered, s_entered, s_stable, s_stop, s_stage, s_next, s_ckpt, s_stop_prefix,
        s_has_prev;
    const uint32_t tid = threadIdx.x, lane = tid & 31;
    const uint32_t dim = ix.dim, k = p.top_k;
    const uint32_t budget = min(p.top_n, capacity);
    const uint32_t tile = p.tile == 0 ? budget : p.tile;
    const float kInf = __int_as_float(0x7f800000);
    ScoreMode mode;
    mode.qkind = qkind;
    mode.int_path = qkind == TANN_KIND_UINT8 && ix.vector_kind == TANN_KIND_UINT8 && (dim % 4 == 0) && dim <= 256 &&
                    (ix.vector_bytes % 4 == 0) && (ix.page_bytes % 4 == 0);
    const bool rows16 = (ix.vector_bytes % 16 == 0) && (ix.page_bytes % 16 == 0);
    mode.octet_int = mode.int_path && rows16 && (dim % 16 == 0);
    mode.octet_f32 = !mode.int_path && rows16 && ix.vector_kind == TANN_KIND_FLOAT32 && qkind == TANN_KIND_FLOAT32 &&
                     (dim % 4 == 0);
    mode.octet_u8f32 = !mode.int_path && ix.vector_kind == TANN_KIND_UINT8 && qkind == TANN_KIND_FLOAT32 &&
                       (ix.vector_bytes % 4 == 0) && (ix.page_bytes % 4 == 0) && (dim % 4 == 0);
    const uint32_t qbytes = dim * (qkind == TANN_KIND_FLOAT32 ? 4u : 1u);
    unsigned long long tot_exact = 0, tot_filtered = 0;

    for (uint64_t q = blockIdx.x; q < Q; q += gridDim.x) {
        const uint8_t* qsrc = static_cast<const uint8_t*>(queries) + q * qbytes;
        for (uint32_t i = tid; i < qbytes; i += kRerankThreads) qrow[i] = qsrc[i];
        s_top[0][tid] = kInvalidKey64;
        if (tid == 0) {
            s_kth = kInf;
            s_exact = 0; s_filtered = 0; s_entered = 0; s_stable = 0; s_stop = 0;
            s_stage = ls.initial_stage_index;
            s_next = use_schedule ? min(budget, ls.bootstrap_prefix) : min(budget, tile);
            s_ckpt = 0; s_stop_prefix = budget; s_has_prev = 0;
            s_prev_ckpt_kth = kInf; s_prev_delta = 0.0f;
        }
        __syncthreads();
        if (p.use_bound_filter && tid == 0) {
            double sum = 0.0;
            for (uint32_t i = 0; i < dim; ++i) {
                const double v = (double)LoadAsFloat<float>(qrow, qkind, i);
                sum += v * v;
            }
            s_qnorm = (float)sum;
        }
        __syncthreads();
        uint32_t cur = 0, exact_before = 0;
        for (uint32_t rb = 0; rb < budget;) {
            if (s_stop) break;
            const uint32_t re = use_schedule ? s_next : min(budget, rb + tile);
            const uint32_t rc = re - rb;
            const float threshold = s_kth;
            // ---- one thread per rank: candidate record, bound filter, vector address ----------
            uint32_t n_act = 0, n_flt = 0;
            for (uint32_t r = rb + tid; r < re; r += kRerankThreads) {
                unsigned long long slot = kInvalidKey64;
                const Cand c = cand[q * capacity + r];
                const uint32_t id = c.id & kRawMask;
                if (c.id != kInvalid && id >= ix.num_nodes && status != nullptr)
                    atomicOr(status, TANN_STATUS_RERANK_ID_RANGE);   // skipped, and reported
                if (c.id != kInvalid && id < ix.num_nodes) {
                    bool keep = true;
                    if (p.use_bound_filter && isfinite(threshold))
                        keep = !(LowerBoundSq(c.dist - s_qnorm, __ldg(error_bounds + id)) > threshold);
                    if (keep) {
                        slot = reinterpret_cast<unsigned long long>(VectorPtr(ix, id));
                        rank_ids[r] = id;
                        ++n_act;
                    } else {
                        ++n_flt;
                    }
                }
                keys[r] = slot;
            }
            n_act = __reduce_add_sync(kFull, n_act);
            n_flt = __reduce_add_sync(kFull, n_flt);
            if (lane == 0 && n_act) atomicAdd(&s_exact, n_act);
            if (lane == 0 && n_flt) atomicAdd(&s_filtered, n_flt);
            s_top[cur ^ 1][tid] = kInvalidKey64;
            __syncthreads();
            ScoreRanks<kRerankThreads>(ix, mode, keys, rank_ids, qrow, rb, re, tid);
            __syncthreads();
            // ---- merge the window into the top_k list (:945-965) ---------------------------------
            {
                const unsigned long long* old_list = s_top[cur];
                unsigned long long* new_list = s_top[cur ^ 1];
                uint32_t entered = 0;
                for (uint32_t t = tid; t < rc; t += kRerankThreads) {
                    const unsigned long long e = keys[rb + t];
                    if (e == kInvalidKey64) continue;
                    uint32_t cnt = 0;
                    for (uint32_t u = 0; u < rc; ++u) {
                        const unsigned long long x = keys[rb + u];
                        cnt += (x < e || (x == e && u < t)) ? 1u : 0u;
                    }
                    for (uint32_t j = 0; j < k; ++j) cnt += old_list[j] <= e ? 1u : 0u;
                    if (cnt < k) {
                        new_list[cnt] = e;
                        ++entered;
                    }
                }
                if (tid < k) {
                    const unsigned long long x = old_list[tid];
                    if (x != kInvalidKey64) {
                        uint32_t pos = tid;
                        for (uint32_t u = 0; u < rc; ++u) pos += keys[rb + u] < x ? 1u : 0u;
                        if (pos < k) new_list[pos] = x;
                    }
                }
                entered = __reduce_add_sync(kFull, entered);
                if (lane == 0 && entered) atomicAdd(&s_entered, entered);
            }
            __syncthreads();
            cur ^= 1;
            if (tid == 0) {
                const unsigned long long* list = s_top[cur];
                const float previous_window_kth = KeyDist(s_top[cur ^ 1][k - 1]);
                const uint32_t processed = re;
                const float kth = KeyDist(list[k - 1]);
                const uint32_t entered = s_entered;
                const uint32_t window_exact = s_exact - exact_before;
                exact_before = s_exact;
                s_entered = 0;
                s_kth = kth;
                uint32_t stage = s_stage;
                uint32_t stop = 0;
                if (evaluate && ls.enabled != 0u && isfinite(kth) && stage < ls.num_stages &&
                    processed >= ls.stage_prefixes[stage]) {   // :981-1110, :1213-1276
                    const float delta_last = s_has_prev ? (s_prev_ckpt_kth - kth) : 0.0f;
                    const float spread = kth - KeyDist(list[0]);
                    uint32_t nwe = (stage + 1u < ls.num_stages) ? min(budget, ls.stage_prefixes[stage + 1u])
                                                                : min(budget, re + tile);
                    if (nwe < re) nwe = re;
                    nwe = min(nwe, re + (uint32_t)TANN_RERANK_STOP_HEAD_PROBE);
                    uint32_t live = 0;
                    float best_lb = kInf;
                    if (ls.linear_weights[8] != 0.0f || ls.linear_weights[9] != 0.0f) {
                        for (uint32_t r = re; r < nwe; ++r) {
                            const Cand c = cand[q * capacity + r];
                            const uint32_t id = c.id & kRawMask;
                            float lb = kInf;
                            if (c.id != kInvalid && id < ix.num_nodes)
                                lb = LowerBoundSq(c.dist - s_qnorm, __ldg(error_bounds + id));
                            if (lb <= kth) {
                                ++live;
                                best_lb = fminf(best_lb, lb);
                            }
                        }
                    }
                    const float logit = RerankStopLogit(ls, processed, kth, delta_last, s_prev_delta,
                                                        entered == 0u ? 0.0f : 1.0f, entered, spread, live, nwe - re,
                                                        best_lb, window_exact, rc, s_exact);
                    ++s_ckpt;
                    if (logit < ls.threshold_logit) stop = 1;
                    s_prev_ckpt_kth = kth;
                    s_prev_delta = delta_last;
                    s_has_prev = 1;
                    ++stage;
                } else if (replay != nullptr) {   // :1111-1122
                    while (stage < ls.num_stages && ls.stage_prefixes[stage] <= processed) ++stage;
                    if (processed >= replay[q]) stop = 1;
                } else if (p.use_early_stop && processed >= p.early_stop_min_prefix && isfinite(kth)) {   // :1123-1135
                    if (kth < previous_window_kth) s_stable = 0; else ++s_stable;
                    if (s_stable >= p.early_stop_patience_tiles) stop = 1;
                }
                s_stage = stage;
                if (stop) {
                    s_stop = 1;
                    s_stop_prefix = processed;
                } else if (use_schedule) {
                    s_next = stage < ls.num_stages ? min(budget, ls.stage_prefixes[stage]) : min(budget, processed + tile);
                }
            }
            __syncthreads();
            rb = re;
        }
        if (tid < k) {
            const unsigned long long key = s_top[cur][tid];
            out_dists[q * k + tid] = KeyDist(key);
            out_ids[q * k + tid] = (uint32_t)key;
        }
        if (tid == 0) {
            tot_exact += s_exact;
            tot_filtered += s_filtered;
            if (out_stop_prefixes != nullptr) out_stop_prefixes[q] = s_stop_prefix;
            if (out_checkpoints != nullptr) out_checkpoints[q] = s_ckpt;
            if (out_stop_flags != nullptr) out_stop_flags[q] = s_stop;
        }
        __syncthreads();
    }
    if (tid == 0 && out_counts != nullptr) {
        if (tot_exact) atomicAdd(out_counts, tot_exact);
        if (tot_filtered) atomicAdd(out_counts + 1, tot_filtered);
    }
}

// The same rerank with one WARP per query (top_k <= 32, lists of at most kWarpFormMaxRanks ranks): the windows of
// the schedule are 16 to 64 ranks wide, which leaves three warps of a block waiting at every barrier of the
// block-per-query form; here the four warps of a block work on four queries and meet at no barrier. Every lane
// holds the query's control state (all lanes compute it from the same values); the head probe of the next window
// is spread over the lanes (a count and a minimum, both independent of the order).
constexpr uint32_t kWarpFormWarps = 4;
constexpr uint32_t kWarpFormMaxRanks = 512;

__host__ __device__ inline size_t WarpFormBytes(uint32_t padded, size_t qbytes) {
    return (((size_t)padded * 12 + 15) & ~(size_t)15) + ((qbytes + 15) & ~(size_t)15) + 2 * 32 * 8;
}

__global__ void __launch_bounds__(kWarpFormWarps * 32, 8)
rerank_learned_warp_kernel(const __grid_constant__ TannIndexView ix, TannRerankParams p,
                           const __grid_constant__ TannRerankLearnedStop ls, uint32_t use_schedule, uint32_t evaluate,
                           const Cand* __restrict__ cand, uint32_t capacity, uint64_t Q, const void* __restrict__ queries,
                           uint32_t qkind, const float* __restrict__ error_bounds, const uint32_t* __restrict__ replay,
                           uint32_t padded, float* __restrict__ out_dists, uint32_t* __restrict__ out_ids,
                           unsigned long long* __restrict__ out_counts, uint32_t* __restrict__ out_stop_prefixes,
                           uint32_t* __restrict__ out_checkpoints, uint32_t* __restrict__ out_stop_flags,
                           uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char rr_smem[];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t dim = ix.dim, k = p.top_k;
    const uint32_t qbytes = dim * (qkind == TANN_KIND_FLOAT32 ? 4u : 1u);
    unsigned char* mine = rr_smem + (size_t)warp * WarpFormBytes(padded, qbytes);
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(mine);      // [padded]
    uint32_t* rank_ids = reinterpret_cast<uint32_t*>(keys + padded);              // [padded]
    uint8_t* qrow = mine + (((size_t)padded * 12 + 15) & ~(size_t)15);
    unsigned long long* top = reinterpret_cast<unsigned long long*>(qrow + ((qbytes + 15) & ~15u));   // [2][32]
    const uint32_t budget = min(p.top_n, capacity);
    const uint32_t tile = p.tile == 0 ? budget : p.tile;
    const float kInf = __int_as_float(0x7f800000);
    ScoreMode mode;
    mode.qkind = qkind;
    mode.int_path = qkind == TANN_KIND_UINT8 && ix.vector_kind == TANN_KIND_UINT8 && (dim % 4 == 0) && dim <= 256 &&
                    (ix.vector_bytes % 4 == 0) && (ix.page_bytes % 4 == 0);
    const bool rows16 = (ix.vector_bytes % 16 == 0) && (ix.page_bytes % 16 == 0);
    mode.octet_int = mode.int_path && rows16 && (dim % 16 == 0);
    mode.octet_f32 = !mode.int_path && rows16 && ix.vector_kind == TANN_KIND_FLOAT32 && qkind == TANN_KIND_FLOAT32 &&
                     (dim % 4 == 0);
    mode.octet_u8f32 = !mode.int_path && ix.vector_kind == TANN_KIND_UINT8 && qkind == TANN_KIND_FLOAT32 &&
                       (ix.vector_bytes % 4 == 0) && (ix.page_bytes % 4 == 0) && (dim % 4 == 0);
    unsigned long long tot_exact = 0, tot_filtered = 0;

    for (uint64_t q = (uint64_t)blockIdx.x * kWarpFormWarps + warp; q < Q; q += (uint64_t)gridDim.x * kWarpFormWarps) {
        const uint8_t* qsrc = static_cast<const uint8_t*>(queries) + q * qbytes;
        __syncwarp();   // the previous query's reads of this warp's buffers are done
        if (qbytes % 16 == 0) {
            for (uint32_t i = lane; i < qbytes / 16; i += 32)
                reinterpret_cast<uint4*>(qrow)[i] = __ldg(reinterpret_cast<const uint4*>(qsrc) + i);
        } else {
            for (uint32_t i = lane; i < qbytes; i += 32) qrow[i] = qsrc[i];
        }
        top[lane] = kInvalidKey64;
        float kth_now = kInf, prev_ckpt_kth = kInf, prev_delta = 0.0f, qnorm = 0.0f;
        uint32_t n_exact = 0, n_filtered = 0, stable = 0, stop = 0, stage = ls.initial_stage_index;
        uint32_t next = use_schedule ? min(budget, ls.bootstrap_prefix) : min(budget, tile);
        uint32_t ckpt = 0, stop_prefix = budget, has_prev = 0;
        __syncwarp();
        if (p.use_bound_filter) {
            double sum = 0.0;
            if (lane == 0) {
                for (uint32_t i = 0; i < dim; ++i) {
                    const double v = (double)LoadAsFloat<float>(qrow, qkind, i);
                    sum += v * v;
                }
            }
            qnorm = __shfl_sync(kFull, (float)sum, 0);
        }
        uint32_t cur = 0, exact_before = 0;
        for (uint32_t rb = 0; rb < budget;) {
            if (stop) break;
            const uint32_t re = use_schedule ? next : min(budget, rb + tile);
            const uint32_t rc = re - rb;
            const float threshold = kth_now;
            // ---- one lane per rank: candidate record, bound filter, vector address -----------------
            uint32_t n_act = 0, n_flt = 0;
            for (uint32_t r = rb + lane; r < re; r += 32) {
                unsigned long long slot = kInvalidKey64;
                const Cand c = cand[q * capacity + r];
                const uint32_t id = c.id & kRawMask;
                if (c.id != kInvalid && id >= ix.num_nodes && status != nullptr)
                    atomicOr(status, TANN_STATUS_RERANK_ID_RANGE);   // skipped, and reported
                if (c.id != kInvalid && id < ix.num_nodes) {
                    bool keep = true;
                    if (p.use_bound_filter && isfinite(threshold))
                        keep = !(LowerBoundSq(c.dist - qnorm, __ldg(error_bounds + id)) > threshold);
                    if (keep) {
                        slot = reinterpret_cast<unsigned long long>(VectorPtr(ix, id));
                        rank_ids[r] = id;
                        ++n_act;
                    } else {
                        ++n_flt;
                    }
                }
                keys[r] = slot;
            }
            n_exact += __reduce_add_sync(kFull, n_act);
            n_filtered += __reduce_add_sync(kFull, n_flt);
            unsigned long long* old_list = top + cur * 32;
            unsigned long long* new_list = top + (cur ^ 1) * 32;
            new_list[lane] = kInvalidKey64;
            __syncwarp();
            ScoreRanks<32>(ix, mode, keys, rank_ids, qrow, rb, re, lane);
            __syncwarp();
            // ---- merge the window into the top_k list by counting ------------------------------------
            uint32_t entered = 0;
            for (uint32_t t = lane; t < rc; t += 32) {
                const unsigned long long e = keys[rb + t];
                if (e == kInvalidKey64) continue;
                uint32_t cnt = 0;
                for (uint32_t u = 0; u < rc; ++u) {
                    const unsigned long long x = keys[rb + u];
                    cnt += (x < e || (x == e && u < t)) ? 1u : 0u;
                }
                for (uint32_t j = 0; j < k; ++j) cnt += old_list[j] <= e ? 1u : 0u;
                if (cnt < k) {
                    new_list[cnt] = e;
                    ++entered;
                }
            }
            if (lane < k) {
                const unsigned long long x = old_list[lane];
                if (x != kInvalidKey64) {
                    uint32_t pos = lane;
                    for (uint32_t u = 0; u < rc; ++u) pos += keys[rb + u] < x ? 1u : 0u;
                    if (pos < k) new_list[pos] = x;
                }
            }
            entered = __reduce_add_sync(kFull, entered);
            __syncwarp();
            cur ^= 1;
            // ---- the stage boundary, by every lane alike -----------------------------------------------
            {
                const float previous_window_kth = KeyDist(old_list[k - 1]);
                const uint32_t processed = re;
                const float kth = KeyDist(new_list[k - 1]);
                const uint32_t window_exact = n_exact - exact_before;
                exact_before = n_exact;
                kth_now = kth;
                uint32_t stop_here = 0;
                if (evaluate && ls.enabled != 0u && isfinite(kth) && stage < ls.num_stages &&
                    processed >= ls.stage_prefixes[stage]) {
                    const float delta_last = has_prev ? (prev_ckpt_kth - kth) : 0.0f;
                    const float spread = kth - KeyDist(new_list[0]);
                    uint32_t nwe = (stage + 1u < ls.num_stages) ? min(budget, ls.stage_prefixes[stage + 1u])
                                                                : min(budget, re + tile);
                    if (nwe < re) nwe = re;
                    nwe = min(nwe, re + (uint32_t)TANN_RERANK_STOP_HEAD_PROBE);
                    uint32_t live = 0;
                    float best_lb = kInf;
                    if (ls.linear_weights[8] != 0.0f || ls.linear_weights[9] != 0.0f) {
                        for (uint32_t r = re + lane; r < nwe; r += 32) {
                            const Cand c = cand[q * capacity + r];
                            const uint32_t id = c.id & kRawMask;
                            float lb = kInf;
                            if (c.id != kInvalid && id < ix.num_nodes)
                                lb = LowerBoundSq(c.dist - qnorm, __ldg(error_bounds + id));
                            if (lb <= kth) {
                                ++live;
                                best_lb = fminf(best_lb, lb);
                            }
                        }
                        live = __reduce_add_sync(kFull, live);
#pragma unroll
                        for (int off = 16; off >= 1; off >>= 1) best_lb = fminf(best_lb, __shfl_xor_sync(kFull, best_lb, off));
                    }
                    const float logit = RerankStopLogit(ls, processed, kth, delta_last, prev_delta,
                                                        entered == 0u ? 0.0f : 1.0f, entered, spread, live, nwe - re,
                                                        best_lb, window_exact, rc, n_exact);
                    ++ckpt;
                    if (logit < ls.threshold_logit) stop_here = 1;
                    prev_ckpt_kth = kth;
                    prev_delta = delta_last;
                    has_prev = 1;
                    ++stage;
                } else if (replay != nullptr) {
                    while (stage < ls.num_stages && ls.stage_prefixes[stage] <= processed) ++stage;
                    if (processed >= replay[q]) stop_here = 1;
                } else if (p.use_early_stop && processed >= p.early_stop_min_prefix && isfinite(kth)) {
                    if (kth < previous_window_kth) stable = 0; else ++stable;
                    if (stable >= p.early_stop_patience_tiles) stop_here = 1;
                }
                if (stop_here) {
                    stop = 1;
                    stop_prefix = processed;
                } else if (use_schedule) {
                    next = stage < ls.num_stages ? min(budget, ls.stage_prefixes[stage]) : min(budget, processed + tile);
                }
            }
            __syncwarp();   // the old list is the next window's new list
            rb = re;
        }
        if (lane < k) {
            const unsigned long long key = top[cur * 32 + lane];
            out_dists[q * k + lane] = KeyDist(key);
            out_ids[q * k + lane] = (uint32_t)key;
        }
        if (lane == 0) {
            tot_exact += n_exact;
            tot_filtered += n_filtered;
            if (out_stop_prefixes != nullptr) out_stop_prefixes[q] = stop_prefix;
            if (out_checkpoints != nullptr) out_checkpoints[q] = ckpt;
            if (out_stop_flags != nullptr) out_stop_flags[q] = stop;
        }
    }
    if (lane == 0 && out_counts != nullptr) {
        if (tot_exact) atomicAdd(out_counts, tot_exact);
        if (tot_filtered) atomicAdd(out_counts + 1, tot_filtered);
    }
}

// rerank_kernel's tiled form (bound filter and/or early stop, tiles of at most kWarpFormMaxTile ranks, top_k <= 32)
// with one warp per query: a 16-rank tile keeps half a warp busy and a block of four warps would spend its time at
// the five barriers of every tile. Same values as the block form: the tile is merged into the sorted best-k
// distances by counting, the threshold of the next tile is their k-th, the final order is (distance, id).
constexpr uint32_t kWarpFormMaxTile = 64;

__global__ void __launch_bounds__(kWarpFormWarps * 32, 8)
rerank_warp_kernel(const __grid_constant__ TannIndexView ix, TannRerankParams p, const Cand* __restrict__ cand,
                   uint32_t capacity, uint64_t Q, const void* __restrict__ queries, uint32_t qkind,
                   const float* __restrict__ error_bounds, uint32_t padded, float* __restrict__ out_dists,
                   uint32_t* __restrict__ out_ids, unsigned long long* __restrict__ out_counts,
                   const uint8_t* __restrict__ queries_u8, const uint32_t* __restrict__ not_u8_flag,
                   uint32_t final_ranks, uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char rr_smem[];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t dim = ix.dim, k = p.top_k;
    const bool as_u8 = qkind == TANN_KIND_UINT8 || (queries_u8 != nullptr && not_u8_flag != nullptr && *not_u8_flag == 0u);
    const bool int_path = as_u8 && ix.vector_kind == TANN_KIND_UINT8 && (dim % 4 == 0) && dim <= 256 &&
                          (ix.vector_bytes % 4 == 0) && (ix.page_bytes % 4 == 0);
    // the buffers are laid out for the caller's query kind; the uint8 copy is never the larger one
    const uint32_t qbytes_layout = dim * (qkind == TANN_KIND_FLOAT32 ? 4u : 1u);
    if (int_path && qkind != TANN_KIND_UINT8) { queries = queries_u8; qkind = TANN_KIND_UINT8; }
    const uint32_t qbytes = dim * (qkind == TANN_KIND_FLOAT32 ? 4u : 1u);
    unsigned char* mine = rr_smem + (size_t)warp * WarpFormBytes(padded, qbytes_layout);
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(mine);      // [padded]
    uint32_t* rank_ids = reinterpret_cast<uint32_t*>(keys + padded);              // [padded]
    uint8_t* qrow = mine + (((size_t)padded * 12 + 15) & ~(size_t)15);
    float* best = reinterpret_cast<float*>(qrow + ((qbytes_layout + 15) & ~15u));   // [2][32] sorted best-k distances
    float* tl = best + 64;                                                          // [64] a tile's distances
    const uint32_t tile = p.tile;
    const float kInf = __int_as_float(0x7f800000);
    const bool rows16 = (ix.vector_bytes % 16 == 0) && (ix.page_bytes % 16 == 0);
    const bool octet_int = int_path && rows16 && (dim % 16 == 0);
    const bool octet_f32 = !int_path && rows16 && ix.vector_kind == TANN_KIND_FLOAT32 &&
                           qkind == TANN_KIND_FLOAT32 && (dim % 4 == 0);
    const bool octet_u8f32 = !int_path && ix.vector_kind == TANN_KIND_UINT8 && qkind == TANN_KIND_FLOAT32 &&
                             (ix.vector_bytes % 4 == 0) && (ix.page_bytes % 4 == 0) && (dim % 4 == 0);
    const ScoreMode mode{int_path, octet_int, octet_f32, octet_u8f32, qkind};
    unsigned long long tot_exact = 0, tot_filtered = 0;

    for (uint64_t q = (uint64_t)blockIdx.x * kWarpFormWarps + warp; q < Q; q += (uint64_t)gridDim.x * kWarpFormWarps) {
        const uint8_t* qsrc = static_cast<const uint8_t*>(queries) + q * qbytes;
        __syncwarp();   // the previous query's reads of this warp's buffers are done
        if (qbytes % 16 == 0) {
            for (uint32_t i = lane; i < qbytes / 16; i += 32)
                reinterpret_cast<uint4*>(qrow)[i] = __ldg(reinterpret_cast<const uint4*>(qsrc) + i);
        } else {
            for (uint32_t i = lane; i < qbytes; i += 32) qrow[i] = qsrc[i];
        }
        for (uint32_t i = lane; i < padded; i += 32) keys[i] = kInvalidKey64;
        best[lane] = kInf;
        float threshold = kInf, prev_kth = kInf, qnorm = 0.0f;
        uint32_t n_exact = 0, n_filtered = 0, stable = 0, cur = 0;
        __syncwarp();
        if (p.use_bound_filter) {
            double sum = 0.0;
            if (lane == 0) {
                for (uint32_t i = 0; i < dim; ++i) {
                    const double v = (double)LoadAsFloat<float>(qrow, qkind, i);
                    sum += v * v;
                }
            }
            qnorm = __shfl_sync(kFull, (float)sum, 0);
        }
        for (uint32_t rb = 0; rb < p.top_n; rb += tile) {
            const uint32_t rc = min(tile, p.top_n - rb);
            uint32_t n_act = 0, n_flt = 0;
            for (uint32_t r = rb + lane; r < rb + rc; r += 32) {
                unsigned long long slot = kInvalidKey64;
                if (r < capacity) {
                    const Cand c = cand[q * capacity + r];
                    const uint32_t id = c.id & kRawMask;
                    if (c.id != kInvalid && id >= ix.num_nodes && status != nullptr)
                        atomicOr(status, TANN_STATUS_RERANK_ID_RANGE);   // skipped, and reported
                    if (c.id != kInvalid && id < ix.num_nodes) {
                        bool keep = true;
                        if (p.use_bound_filter && isfinite(threshold))
                            keep = !(LowerBoundSq(c.dist - qnorm, __ldg(error_bounds + id)) > threshold);
                        if (keep) {
                            slot = reinterpret_cast<unsigned long long>(VectorPtr(ix, id));
                            rank_ids[r] = id;
                            ++n_act;
                        } else {
                            ++n_flt;
                        }
                    }
                }
                keys[r] = slot;
            }
            n_exact += __reduce_add_sync(kFull, n_act);
            n_filtered += __reduce_add_sync(kFull, n_flt);
            __syncwarp();
            ScoreRanks<32>(ix, mode, keys, rank_ids, qrow, rb, rb + rc, lane);
            __syncwarp();
            // ---- the tile's distances merged into the best-k list by counting ---------------------------
            const float* old_best = best + cur * 32;
            float* new_best = best + (cur ^ 1) * 32;
            for (uint32_t t = lane; t < rc; t += 32) tl[t] = FromOrderedBits((uint32_t)(keys[rb + t] >> 32));
            __syncwarp();
            if (lane < k) {
                const float oldv = old_best[lane];
                uint32_t c_old = 0;
                for (uint32_t l = 0; l < rc; ++l) c_old += tl[l] < oldv ? 1u : 0u;
                if (lane + c_old < k) new_best[lane + c_old] = oldv;
            }
            for (uint32_t t = lane; t < rc; t += 32) {
                const float newv = tl[t];
                uint32_t c_new = 0;
                for (uint32_t l = 0; l < rc; ++l) {
                    const float x = tl[l];
                    c_new += (x < newv || (x == newv && l < t)) ? 1u : 0u;
                }
                uint32_t lo = 0;   // old entries <= newv
#pragma unroll
                for (uint32_t b = 32; b > 0; b >>= 1) {
                    const uint32_t u = lo + b;
                    if (u <= k && old_best[u - 1] <= newv) lo = u;
                }
                if (lo + c_new < k) new_best[lo + c_new] = newv;
            }
            __syncwarp();
            cur ^= 1;
            const float kth = new_best[k - 1];
            threshold = kth;
            bool stop = false;
            if (p.use_early_stop) {   // src/io/bam_vector_provider.cu:1124-1135
                if (rb + rc >= p.early_stop_min_prefix && isfinite(kth)) {
                    if (kth < prev_kth) stable = 0; else ++stable;
                    if (stable >= p.early_stop_patience_tiles) stop = true;
                }
                prev_kth = kth;
            }
            __syncwarp();   // the old list is the next tile's new list
            if (stop) break;
        }
        // ---- final order ---------------------------------------------------------------------------------
        uint32_t out_n = p.top_n;
        if (final_ranks != 0 && final_ranks <= 32 && padded >= 64) {
            // the 32 smallest keys: every run of 32 sorted, then folded one after another into the running best 32
            unsigned long long m = WarpSortKey(keys[lane], lane);
            for (uint32_t c = 1; c < padded / 32; ++c) {
                unsigned long long kb = WarpSortKey(keys[c * 32 + lane], lane);
                kb = __shfl_sync(kFull, kb, 31 - lane);
                m = m < kb ? m : kb;
#pragma unroll
                for (uint32_t sft = 16; sft > 0; sft >>= 1) {
                    const unsigned long long o = __shfl_xor_sync(kFull, m, sft);
                    const bool upper = (lane & sft) != 0;
                    m = upper ? (o > m ? o : m) : (o < m ? o : m);
                }
            }
            keys[lane] = m;
            out_n = min(p.top_n, 32u);
        } else {
            uint32_t first_k = 2;
            if (padded >= 64) {
                for (uint32_t c = 0; c < padded / 32; ++c) {
                    unsigned long long key = WarpSortKey(keys[c * 32 + lane], lane);
                    if (c & 1u) key = __shfl_sync(kFull, key, 31 - lane);   // odd runs descending, as the network expects
                    keys[c * 32 + lane] = key;
                }
                first_k = 64;
                __syncwarp();
            }
            for (uint32_t kk = first_k; kk <= padded; kk <<= 1) {
                for (uint32_t j = kk >> 1; j > 0; j >>= 1) {
                    for (uint32_t t = lane; t < padded / 2; t += 32) {
                        const uint32_t lo = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                        const uint32_t hi = lo | j;
                        const bool asc = (lo & kk) == 0;
                        const unsigned long long a = keys[lo], b = keys[hi];
                        if ((a > b) == asc) { keys[lo] = b; keys[hi] = a; }
                    }
                    __syncwarp();
                }
            }
        }
        __syncwarp();
        for (uint32_t i = lane; i < out_n; i += 32) {
            const unsigned long long key = keys[i];
            out_dists[q * p.top_n + i] = FromOrderedBits((uint32_t)(key >> 32));
            out_ids[q * p.top_n + i] = (uint32_t)key;
        }
        tot_exact += n_exact;
        tot_filtered += n_filtered;
    }
    if (lane == 0 && out_counts != nullptr) {
        if (tot_exact) atomicAdd(out_counts, tot_exact);
        if (tot_filtered) atomicAdd(out_counts + 1, tot_filtered);
    }
}

__global__ void topk_pack_kernel(const float* __restrict__ dists, const uint32_t* __restrict__ ids,
                                 uint64_t Q, uint32_t top_n, uint32_t top_k,
                                 float* __restrict__ out_dists, uint32_t* __restrict__ out_ids) {
    const uint64_t total = Q * top_k;
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t q = e / top_k;
        const uint32_t r = (uint32_t)(e - q * top_k);
        const bool in = r < top_n;
        out_dists[e] = in ? dists[q * top_n + r] : __int_as_float(0x7f800000);
        out_ids[e] = in ? ids[q * top_n + r] : kInvalid;
    }
}

cudaError_t LaunchRerank(const TannIndexView& ix, const TannRerankParams& p, const void* cand,
                         uint32_t capacity, uint64_t Q, const void* queries, uint32_t query_kind,
                         const float* error_bounds, float* out_dists, uint32_t* out_ids,
                         unsigned long long* out_counts, cudaStream_t stream, const uint8_t* queries_u8,
                         const uint32_t* not_u8_flag, uint32_t final_ranks, uint32_t* status) {
    if (Q == 0 || p.top_n == 0) return cudaSuccess;
    uint32_t padded = 1;
    while (padded < p.top_n) padded <<= 1;
    const size_t qbytes = (size_t)ix.dim * (query_kind == TANN_KIND_FLOAT32 ? 4 : 1);
    if ((p.use_bound_filter || p.use_early_stop) && p.tile != 0 && p.tile <= kWarpFormMaxTile && p.top_k <= 32 &&
        p.top_k != 0 && padded <= kWarpFormMaxRanks) {   // short tiles: one warp per query
        const size_t smem_w = WarpFormBytes(padded, qbytes) * kWarpFormWarps;
        if (smem_w > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(rerank_warp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem_w);
            if (e != cudaSuccess) return e;
        }
        const uint64_t blocks = (Q + kWarpFormWarps - 1) / kWarpFormWarps;
        const uint64_t cap_w = (uint64_t)SmCount() * 8;
        rerank_warp_kernel<<<(unsigned)(blocks < cap_w ? blocks : cap_w), kWarpFormWarps * 32, smem_w, stream>>>(
            ix, p, static_cast<const Cand*>(cand), capacity, Q, queries, query_kind, error_bounds, padded,
            out_dists, out_ids, out_counts, queries_u8, not_u8_flag, final_ranks, status);
        return cudaGetLastError();
    }
    const size_t smem = (((size_t)padded * 12 + 15) & ~(size_t)15) + ((qbytes + 15) & ~(size_t)15);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(rerank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
    }
    const uint64_t cap = (uint64_t)SmCount() * 8;
    rerank_kernel<<<(unsigned)(Q < cap ? Q : cap), kRerankThreads, smem, stream>>>(
        ix, p, static_cast<const Cand*>(cand), capacity, Q, queries, query_kind, error_bounds, padded,
        out_dists, out_ids, out_counts, queries_u8, not_u8_flag, final_ranks, status);
    return cudaGetLastError();
}

cudaError_t LaunchRerankLearned(const TannIndexView& ix, const TannRerankParams& p, const TannRerankLearnedStop& model,
                                bool use_schedule, bool evaluate, const void* cand, uint32_t capacity, uint64_t Q,
                                const void* queries, uint32_t query_kind, const float* error_bounds,
                                const uint32_t* replay_stop_prefixes, float* out_dists, uint32_t* out_ids,
                                unsigned long long* out_counts, uint32_t* out_stop_prefixes,
                                uint32_t* out_checkpoint_counts, uint32_t* out_stop_flags, cudaStream_t stream,
                                uint32_t* status) {
    if (Q == 0 || p.top_n == 0 || capacity == 0) return cudaSuccess;
    const uint32_t budget = p.top_n < capacity ? p.top_n : capacity;
    uint32_t padded = 1;
    while (padded < budget) padded <<= 1;
    const size_t qbytes = (size_t)ix.dim * (query_kind == TANN_KIND_FLOAT32 ? 4 : 1);
    if (p.top_k <= 32 && padded <= kWarpFormMaxRanks) {   // one warp per query
        const size_t smem = WarpFormBytes(padded, qbytes) * kWarpFormWarps;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(rerank_learned_warp_kernel,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
        }
        const uint64_t blocks = (Q + kWarpFormWarps - 1) / kWarpFormWarps;
        const uint64_t cap = (uint64_t)SmCount() * 8;
        rerank_learned_warp_kernel<<<(unsigned)(blocks < cap ? blocks : cap), kWarpFormWarps * 32, smem, stream>>>(
            ix, p, model, use_schedule ? 1u : 0u, evaluate ? 1u : 0u, static_cast<const Cand*>(cand), capacity, Q,
            queries, query_kind, error_bounds, replay_stop_prefixes, padded, out_dists, out_ids, out_counts,
            out_stop_prefixes, out_checkpoint_counts, out_stop_flags, status);
        return cudaGetLastError();
    }
    const size_t smem = (((size_t)padded * 12 + 15) & ~(size_t)15) + ((qbytes + 15) & ~(size_t)15);
    if (smem > 40 * 1024) {   // the kernel also has 2 KB of static shared memory
        cudaError_t e = cudaFuncSetAttribute(rerank_learned_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
    }
    const uint64_t cap = (uint64_t)SmCount() * 9;   // 56 registers: nine blocks per SM are resident
    rerank_learned_kernel<<<(unsigned)(Q < cap ? Q : cap), kRerankThreads, smem, stream>>>(
        ix, p, model, use_schedule ? 1u : 0u, evaluate ? 1u : 0u, static_cast<const Cand*>(cand), capacity, Q, queries,
        query_kind, error_bounds, replay_stop_prefixes, padded, out_dists, out_ids, out_counts, out_stop_prefixes,
        out_checkpoint_counts, out_stop_flags, status);
    return cudaGetLastError();
}

cudaError_t LaunchTopkPack(const float* dists, const uint32_t* ids, uint64_t Q, uint32_t top_n,
                           uint32_t top_k, float* out_dists, uint32_t* out_ids, cudaStream_t stream) {
    if (Q == 0 || top_k == 0) return cudaSuccess;
    const uint64_t total = Q * top_k;
    const uint64_t blocks = (total + 255) / 256;
    const uint64_t cap = (uint64_t)SmCount() * 16;
    topk_pack_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, stream>>>(
        dists, ids, Q, top_n, top_k, out_dists, out_ids);
    return cudaGetLastError();
}

}  // namespace tann

namespace tann {

// float -> uint8 copy of a query batch; *not_u8_flag becomes non-zero if any value is not an
// integer in [0, 255] (the flag must be zero on entry).
__global__ void f32_to_u8_checked_kernel(const float* __restrict__ src, uint64_t n, uint8_t* __restrict__ dst,
                                         uint32_t* __restrict__ not_u8_flag) {
    bool bad = false;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const float v = src[i];
        const bool ok = v >= 0.0f && v <= 255.0f && v == truncf(v);
        bad |= !ok;
        dst[i] = ok ? (uint8_t)v : 0;
    }
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(not_u8_flag, 1u);
}

cudaError_t LaunchF32ToU8Checked(const float* src, uint64_t n, uint8_t* dst, uint32_t* not_u8_flag, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(not_u8_flag, 0, sizeof(uint32_t), stream);
    if (e != cudaSuccess || n == 0) return e;
    const uint64_t blocks = (n + 255) / 256;
    const uint64_t cap = (uint64_t)SmCount() * 8;
    f32_to_u8_checked_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, stream>>>(src, n, dst, not_u8_flag);
    return cudaGetLastError();
}

}  // namespace tann
