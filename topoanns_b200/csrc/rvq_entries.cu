// RVQ entry selection fused into one kernel: coarse scores + argmin, residual, fine scores +
// argmin over non-empty buckets, posting-list gather. The reference does this with a cuBLAS
// SGEMM and about a dozen small launches that materialise two Q x 256 score matrices
// (src/legacy_rvq/gas_legacy/anns/RVQ/RVQ.cu:792-882, functions/distance_kernel.cu:229-323,
// functions/selectMin1.cu:9-23,66-81, src/search/rvq_device_entries.cu:15-52); here the scores
// never leave registers. Scores are FP32 FMA dot products: the argmin decides which bucket a
// query enters, so reduced-precision tensor-core products are not used.
#include <float.h>

#include "tann_common.cuh"
#include "tann_launch.h"

namespace tann {

constexpr int kRvqThreads = 256;
constexpr int kRvqQueriesPerBlock = 8;

// |x|^2 in the order of the reference's L2NormKernel (distance_kernel.cu:25-111): 128 "threads"
// take columns t, t+128, ... with FMA, each warp runs the shuffle tree, and the four warp sums
// are added as (w0 + w2) + (w1 + w3). Called by the first 128 threads of a block; the result is
// valid in thread 0.
__device__ __forceinline__ float NormBy128(const float* x, uint32_t dim, float* warp_sums /*[4]*/) {
    const uint32_t t = threadIdx.x;
    float acc = 0.0f;
    for (uint32_t col = t; col < dim; col += 128) acc = fmaf(x[col], x[col], acc);
    acc = WarpTreeSum(acc);
    if ((t & 31) == 0) warp_sums[t >> 5] = acc;
    return acc;
}

__global__ void __launch_bounds__(128) rvq_norms_kernel(const float* __restrict__ rows, uint32_t count,
                                                       uint32_t dim, float* __restrict__ out) {
    __shared__ float ws[4];
    for (uint32_t r = blockIdx.x; r < count; r += gridDim.x) {
        NormBy128(rows + (size_t)r * dim, dim, ws);
        __syncthreads();
        if (threadIdx.x == 0) out[r] = (ws[0] + ws[2]) + (ws[1] + ws[3]);
        __syncthreads();
    }
}

struct ArgMin {
    float d;
    int idx;
};
__device__ __forceinline__ ArgMin Better(ArgMin a, ArgMin b) {
    // first strict minimum in ascending index order == lexicographic minimum of (value, index)
    if (b.d < a.d || (b.d == a.d && b.idx < a.idx)) return b;
    return a;
}

// The same sum as NormBy128 by ONE warp: lane l plays threads l, 32 + l, 64 + l, 96 + l of the
// 128 in turn (x is read with stride `stride`). All lanes return the result.
__device__ __forceinline__ float NormByWarp(const float* x, uint32_t stride, uint32_t dim, uint32_t lane) {
    float s[4];
#pragma unroll
    for (uint32_t v = 0; v < 4; ++v) {
        float acc = 0.0f;
        for (uint32_t col = v * 32 + lane; col < dim; col += 128) {
            const float xv = x[(size_t)col * stride];
            acc = fmaf(xv, xv, acc);
        }
        s[v] = __shfl_sync(kFull, WarpTreeSum(acc), 0);
    }
    return (s[0] + s[2]) + (s[1] + s[3]);
}

// One block scores kRvqQueriesPerBlock queries against a 256-entry codebook level: thread c owns
// centroid c (codebooks are stored transposed, so a warp reads 128 contiguous bytes per dim), the
// queries sit transposed in shared memory so that one 16-byte broadcast load feeds four FMAs.
__global__ void __launch_bounds__(kRvqThreads)
rvq_entries_kernel(const float* __restrict__ queries, uint64_t Q, uint32_t dim,
                   const float* __restrict__ coarse, const float* __restrict__ coarse_t,
                   const float* __restrict__ coarse_norms, uint32_t nc,
                   const float* __restrict__ fine_t, const float* __restrict__ fine_norms, uint32_t nf,
                   const int32_t* __restrict__ bucket_sizes, const uint32_t* __restrict__ cluster_offsets,
                   const uint32_t* __restrict__ cluster_ids, uint32_t entry_count, uint32_t fallback,
                   int32_t* __restrict__ out_clusters, uint32_t* __restrict__ out_entry_ids,
                   uint32_t* __restrict__ out_entry_offsets) {
    constexpr int QB = kRvqQueriesPerBlock;
    constexpr int kWarps = kRvqThreads / 32;
    extern __shared__ __align__(16) float rvq_smem[];
    float* x = rvq_smem;  // [dim][QB]: queries, then residuals
    __shared__ float norms[QB];
    __shared__ ArgMin scratch[kWarps][QB];
    __shared__ int best_coarse[QB];
    __shared__ int best_cluster[QB];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (blockIdx.x == 0 && out_entry_offsets != nullptr)
        for (uint64_t i = tid; i <= Q; i += kRvqThreads) out_entry_offsets[i] = (uint32_t)(i * entry_count);

    for (uint64_t q0 = (uint64_t)blockIdx.x * QB; q0 < Q; q0 += (uint64_t)gridDim.x * QB) {
        const int nq = (int)min((uint64_t)QB, Q - q0);
        for (uint32_t i = tid; i < (uint32_t)QB * dim; i += kRvqThreads) {
            const uint32_t qi = i / dim, k = i - qi * dim;
            x[k * QB + qi] = (int)qi < nq ? queries[q0 * dim + i] : 0.0f;
        }
        __syncthreads();
        for (int level = 0; level < 2; ++level) {
            // norms of the (residual) queries, one warp per query
            for (int qi = warp; qi < nq; qi += kWarps) {
                const float n2 = NormByWarp(x + qi, QB, dim, lane);
                if (lane == 0) norms[qi] = n2;
            }
            __syncthreads();
            const float* book_t = level == 0 ? coarse_t : fine_t;
            const float* book_norms = level == 0 ? coarse_norms : fine_norms;
            const uint32_t count = level == 0 ? nc : nf;
            ArgMin best[QB];
#pragma unroll
            for (int qi = 0; qi < QB; ++qi) { best[qi].d = __int_as_float(0x7f800000); best[qi].idx = 0x7fffffff; }
            for (uint32_t c = tid; c < count; c += kRvqThreads) {
                float dot[QB];
#pragma unroll
                for (int qi = 0; qi < QB; ++qi) dot[qi] = 0.0f;
                // 16 codebook values per step are requested before the first is used (the FMA order per
                // query stays ascending k)
                constexpr uint32_t kAhead = 16;
                uint32_t k0 = 0;
                for (; k0 + kAhead <= dim; k0 += kAhead) {
                    float w[kAhead];
#pragma unroll
                    for (uint32_t u = 0; u < kAhead; ++u) w[u] = __ldg(book_t + (size_t)(k0 + u) * count + c);
#pragma unroll
                    for (uint32_t u = 0; u < kAhead; ++u) {
#pragma unroll
                        for (int g = 0; g < QB / 4; ++g) {
                            const float4 xv = *reinterpret_cast<const float4*>(x + (k0 + u) * QB + 4 * g);
                            dot[4 * g + 0] = fmaf(xv.x, w[u], dot[4 * g + 0]);
                            dot[4 * g + 1] = fmaf(xv.y, w[u], dot[4 * g + 1]);
                            dot[4 * g + 2] = fmaf(xv.z, w[u], dot[4 * g + 2]);
                            dot[4 * g + 3] = fmaf(xv.w, w[u], dot[4 * g + 3]);
                        }
                    }
                }
                for (uint32_t k = k0; k < dim; ++k) {
                    const float w = __ldg(book_t + (size_t)k * count + c);
#pragma unroll
                    for (int g = 0; g < QB / 4; ++g) {
                        const float4 xv = *reinterpret_cast<const float4*>(x + k * QB + 4 * g);
                        dot[4 * g + 0] = fmaf(xv.x, w, dot[4 * g + 0]);
                        dot[4 * g + 1] = fmaf(xv.y, w, dot[4 * g + 1]);
                        dot[4 * g + 2] = fmaf(xv.z, w, dot[4 * g + 2]);
                        dot[4 * g + 3] = fmaf(xv.w, w, dot[4 * g + 3]);
                    }
                }
                const float cn = book_norms[c];
#pragma unroll
                for (int qi = 0; qi < QB; ++qi) {
                    if (qi >= nq) continue;
                    const float D = (-2.0f * dot[qi] + norms[qi]) + cn;
                    bool ok;
                    if (level == 0) {
                        // selectMin1.cu:9-23: starts from element 0, strict "<" afterwards
                        ok = true;
                    } else {
                        // :66-81: starts from FLT_MAX and skips empty buckets
                        ok = D < FLT_MAX && bucket_sizes[(size_t)best_coarse[qi] * nf + c] > 0;
                    }
                    if (ok) best[qi] = Better(best[qi], ArgMin{D, (int)c});
                }
            }
            // block argmin of all queries at once: warp shuffles, then one thread per query
#pragma unroll
            for (int qi = 0; qi < QB; ++qi) {
                ArgMin v = best[qi];
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
                    ArgMin o;
                    o.d = __shfl_xor_sync(kFull, v.d, off);
                    o.idx = __shfl_xor_sync(kFull, v.idx, off);
                    v = Better(v, o);
                }
                if (lane == 0) scratch[warp][qi] = v;
            }
            __syncthreads();
            if ((int)tid < nq) {
                ArgMin r = scratch[0][tid];
#pragma unroll
                for (int w = 1; w < kWarps; ++w) r = Better(r, scratch[w][tid]);
                const int idx = r.idx == 0x7fffffff ? 0 : r.idx;
                if (level == 0) best_coarse[tid] = idx;
                else best_cluster[tid] = best_coarse[tid] * (int)nf + idx;
            }
            __syncthreads();
            if (level == 0) {
                // residual, RVQ.cu:180-188
                for (uint32_t i = tid; i < (uint32_t)nq * dim; i += kRvqThreads) {
                    const uint32_t qi = i / dim, k = i - qi * dim;
                    x[k * QB + qi] = x[k * QB + qi] - coarse[(size_t)best_coarse[qi] * dim + k];
                }
                __syncthreads();
            }
        }
        // gather, rvq_device_entries.cu:15-52
        for (int qi = 0; qi < nq; ++qi) {
            const int cluster = best_cluster[qi];
            uint32_t* o = out_entry_ids + (q0 + qi) * entry_count;
            if (tid == 0 && out_clusters != nullptr) out_clusters[q0 + qi] = cluster;
            uint32_t begin = 0, n = 0;
            if (cluster >= 0) {
                begin = cluster_offsets[cluster];
                n = min(cluster_offsets[cluster + 1] - begin, entry_count);
            }
            for (uint32_t i = tid; i < entry_count; i += kRvqThreads) {
                uint32_t v = kInvalid;
                if (i < n) v = cluster_ids[begin + i];
                else if (n == 0 && i == 0) v = fallback;
                o[i] = v;
            }
        }
        __syncthreads();
    }
}

// Tiled variant for codebook sizes that are multiples of 4: one block scores kTileQueries queries;
// thread (qg, cg) owns queries 8 qg .. 8 qg + 7 and centroids 4 cg .. 4 cg + 3 (+ 256 per further pass),
// i.e. 32 FMA chains fed by one 16-byte codebook load and two 16-byte broadcast loads per dim. Every
// chain is still the ascending-k FMA dot product, so the scores equal the one-centroid form bit for bit.
constexpr int kTileQueries = 32;

__global__ void __launch_bounds__(kRvqThreads)
rvq_entries_tile_kernel(const float* __restrict__ queries, uint64_t Q, uint32_t dim,
                        const float* __restrict__ coarse, const float* __restrict__ coarse_t,
                        const float* __restrict__ coarse_norms, uint32_t nc,
                        const float* __restrict__ fine_t, const float* __restrict__ fine_norms, uint32_t nf,
                        const int32_t* __restrict__ bucket_sizes, const uint32_t* __restrict__ cluster_offsets,
                        const uint32_t* __restrict__ cluster_ids, uint32_t entry_count, uint32_t fallback,
                        int32_t* __restrict__ out_clusters, uint32_t* __restrict__ out_entry_ids,
                        uint32_t* __restrict__ out_entry_offsets) {
    constexpr int QB = kTileQueries;
    constexpr int kWarps = kRvqThreads / 32;
    extern __shared__ __align__(16) float rvq_smem[];
    float* x = rvq_smem;  // [dim][QB]: queries, then residuals
    __shared__ float norms[QB];
    __shared__ ArgMin scratch[kWarps][8];
    __shared__ int best_coarse[QB];
    __shared__ int best_cluster[QB];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t cg = tid & 63, qg = tid >> 6;

    if (blockIdx.x == 0 && out_entry_offsets != nullptr)
        for (uint64_t i = tid; i <= Q; i += kRvqThreads) out_entry_offsets[i] = (uint32_t)(i * entry_count);

    for (uint64_t q0 = (uint64_t)blockIdx.x * QB; q0 < Q; q0 += (uint64_t)gridDim.x * QB) {
        const int nq = (int)min((uint64_t)QB, Q - q0);
        for (uint32_t i = tid; i < (uint32_t)QB * dim; i += kRvqThreads) {
            const uint32_t qi = i / dim, k = i - qi * dim;
            x[k * QB + qi] = (int)qi < nq ? queries[q0 * dim + i] : 0.0f;
        }
        __syncthreads();
        for (int level = 0; level < 2; ++level) {
            for (int qi = warp; qi < nq; qi += kWarps) {
                const float n2 = NormByWarp(x + qi, QB, dim, lane);
                if (lane == 0) norms[qi] = n2;
            }
            __syncthreads();
            const float* book_t = level == 0 ? coarse_t : fine_t;
            const float* book_norms = level == 0 ? coarse_norms : fine_norms;
            const uint32_t count = level == 0 ? nc : nf;
            ArgMin best[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { best[j].d = __int_as_float(0x7f800000); best[j].idx = 0x7fffffff; }
            for (uint32_t c0 = 4 * cg; c0 < count; c0 += 4 * 64) {
                float dot[8][4];
#pragma unroll
                for (int j = 0; j < 8; ++j) dot[j][0] = dot[j][1] = dot[j][2] = dot[j][3] = 0.0f;
                const float* col = book_t + c0;
                const float* xq = x + qg * 8;
#pragma unroll 4
                for (uint32_t k = 0; k < dim; ++k) {
                    const float4 w = __ldg(reinterpret_cast<const float4*>(col + (size_t)k * count));
                    const float4 xa = *reinterpret_cast<const float4*>(xq + k * QB);
                    const float4 xb = *reinterpret_cast<const float4*>(xq + k * QB + 4);
                    const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        dot[j][0] = fmaf(xv[j], w.x, dot[j][0]);
                        dot[j][1] = fmaf(xv[j], w.y, dot[j][1]);
                        dot[j][2] = fmaf(xv[j], w.z, dot[j][2]);
                        dot[j][3] = fmaf(xv[j], w.w, dot[j][3]);
                    }
                }
                const float4 cn4 = __ldg(reinterpret_cast<const float4*>(book_norms + c0));
                const float cn[4] = {cn4.x, cn4.y, cn4.z, cn4.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int qi = (int)qg * 8 + j;
                    if (qi >= nq) continue;
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float D = (-2.0f * dot[j][u] + norms[qi]) + cn[u];
                        bool ok = true;   // level 0, selectMin1.cu:9-23
                        if (level == 1)   // :66-81: starts from FLT_MAX and skips empty buckets
                            ok = D < FLT_MAX && bucket_sizes[(size_t)best_coarse[qi] * nf + c0 + u] > 0;
                        if (ok) best[j] = Better(best[j], ArgMin{D, (int)(c0 + u)});
                    }
                }
            }
            // argmin over the 64 threads (two warps) that share a query group
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                ArgMin v = best[j];
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
                    ArgMin o;
                    o.d = __shfl_xor_sync(kFull, v.d, off);
                    o.idx = __shfl_xor_sync(kFull, v.idx, off);
                    v = Better(v, o);
                }
                if (lane == 0) scratch[warp][j] = v;
            }
            __syncthreads();
            if ((int)tid < nq) {
                const uint32_t g = tid >> 3, j = tid & 7;      // query tid = 8 g + j, scored by warps 2 g and 2 g + 1
                const ArgMin r = Better(scratch[2 * g][j], scratch[2 * g + 1][j]);
                const int idx = r.idx == 0x7fffffff ? 0 : r.idx;
                if (level == 0) best_coarse[tid] = idx;
                else best_cluster[tid] = best_coarse[tid] * (int)nf + idx;
            }
            __syncthreads();
            if (level == 0) {
                // residual, RVQ.cu:180-188
                for (uint32_t i = tid; i < (uint32_t)nq * dim; i += kRvqThreads) {
                    const uint32_t qi = i / dim, k = i - qi * dim;
                    x[k * QB + qi] = x[k * QB + qi] - coarse[(size_t)best_coarse[qi] * dim + k];
                }
                __syncthreads();
            }
        }
        // gather, rvq_device_entries.cu:15-52
        for (uint32_t e = tid; e < (uint32_t)nq * entry_count; e += kRvqThreads) {
            const uint32_t qi = e / entry_count, i = e - qi * entry_count;
            const int cluster = best_cluster[qi];
            uint32_t begin = 0, n = 0;
            if (cluster >= 0) {
                begin = cluster_offsets[cluster];
                n = min(cluster_offsets[cluster + 1] - begin, entry_count);
            }
            uint32_t v = kInvalid;
            if (i < n) v = cluster_ids[begin + i];
            else if (n == 0 && i == 0) v = fallback;
            out_entry_ids[(q0 + qi) * entry_count + i] = v;
        }
        if (out_clusters != nullptr && (int)tid < nq) out_clusters[q0 + tid] = best_cluster[tid];
        __syncthreads();
    }
}

// Codebook-in-shared-memory variant: one 576-thread block per SM keeps one level's transposed codebook
// (count x dim floats, 128 KB at 256 x 128) in shared memory and scores all of its queries against it,
// level 0 for every query first, then level 1 (the residual is recomputed from the query and the chosen
// coarse centroid). All blocks of the other variants stream the same codebook rows from L2 at the same
// moment, which serialises on the L2 slices that hold them; here a row crosses L2 once per SM and level.
// Thread (qg, cg) owns queries 8 qg .. 8 qg + 7 of a 72-query tile and centroids 4 cg .. 4 cg + 3
// (+ 256 per further pass); every dot product is the ascending-k FMA chain of the other variants.
constexpr int kSmemThreads = 576;      // 9 query groups x 64 centroid groups
constexpr int kSmemTile = 72;          // queries per tile: 10 000 queries over 148 SMs are one tile per block
constexpr int kSmemMaxPerBlock = 1024; // queries per block

__global__ void __launch_bounds__(kSmemThreads, 1)
rvq_entries_smem_kernel(const float* __restrict__ queries, uint64_t Q, uint32_t dim,
                        const float* __restrict__ coarse, const float* __restrict__ coarse_t,
                        const float* __restrict__ coarse_norms, uint32_t nc,
                        const float* __restrict__ fine_t, const float* __restrict__ fine_norms, uint32_t nf,
                        const int32_t* __restrict__ bucket_sizes, const uint32_t* __restrict__ cluster_offsets,
                        const uint32_t* __restrict__ cluster_ids, uint32_t entry_count, uint32_t fallback,
                        int32_t* __restrict__ out_clusters, uint32_t* __restrict__ out_entry_ids,
                        uint32_t* __restrict__ out_entry_offsets, uint32_t per_block, uint32_t* __restrict__ status) {
    constexpr int QB = kSmemTile;
    constexpr int XS = kSmemTile + 4;   // row stride of x: keeps 16-byte alignment, spreads a column over 8 banks
    constexpr int kWarps = kSmemThreads / 32;
    extern __shared__ __align__(16) float rvq_smem[];
    const uint32_t max_count = max(nc, nf);
    float* cb = rvq_smem;                              // [dim][count] of the current level
    float* x = cb + (size_t)max_count * dim;           // [dim][XS], QB used
    __shared__ float norms[QB];
    __shared__ ArgMin scratch[kWarps][8];
    __shared__ int best_coarse[kSmemMaxPerBlock];
    __shared__ int best_cluster[kSmemMaxPerBlock];
    __shared__ __align__(8) unsigned long long copy_barrier;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t cg = tid & 63, qg = tid >> 6;

    if (blockIdx.x == 0 && out_entry_offsets != nullptr)
        for (uint64_t i = tid; i <= Q; i += kSmemThreads) out_entry_offsets[i] = (uint32_t)(i * entry_count);
    const uint64_t q_begin = (uint64_t)blockIdx.x * per_block;
    if (q_begin >= Q) return;
    const uint32_t n_mine = (uint32_t)min((uint64_t)per_block, Q - q_begin);
    if (tid == 0) BarrierInit(&copy_barrier, 1);
    const bool bulk_ok = true;   // the level's codebook arrives by one bulk copy

    for (int level = 0; level < 2; ++level) {
        const float* book_t = level == 0 ? coarse_t : fine_t;
        const float* book_norms = level == 0 ? coarse_norms : fine_norms;
        const uint32_t count = level == 0 ? nc : nf;
        __syncthreads();   // the previous level's readers are done with cb (and the barrier is initialised)
        const uint32_t book_bytes = count * dim * 4;
        const bool bulk = bulk_ok;
        if (bulk) {
            // one bulk copy stages the level's codebook while the block fills and norms its first tile
            if (tid == 0) BulkLoadToShared(cb, book_t, book_bytes, &copy_barrier);
        } else {
#pragma unroll 8
            for (uint32_t i = tid; i < book_bytes / 16; i += kSmemThreads)
                reinterpret_cast<float4*>(cb)[i] = __ldg(reinterpret_cast<const float4*>(book_t) + i);
        }
        for (uint32_t t0 = 0; t0 < n_mine; t0 += QB) {
            const int nq = (int)min((uint32_t)QB, n_mine - t0);
            __syncthreads();   // cb is loaded; the previous tile's readers are done with x
            const uint32_t dim4 = dim / 4;
            // A warp takes 16 queries x 2 groups of four dims: its transposed stores then fall on 32 different
            // banks (row stride XS = 76 words = 12 banks, 4 rows apart = 16 banks), and every query row is read
            // in whole 32-byte sectors.
            constexpr uint32_t kQ16 = (QB + 15) / 16;
#pragma unroll 2
            for (uint32_t i = tid; i < kQ16 * 16u * ((dim4 + 1u) & ~1u); i += kSmemThreads) {
                const uint32_t l = i & 31u, wi = i >> 5;
                const uint32_t qi = (wi % kQ16) * 16u + (l & 15u);
                const uint32_t kg = (wi / kQ16) * 2u + (l >> 4);
                if (qi >= (uint32_t)QB || kg >= dim4) continue;
                const uint32_t k = kg * 4u;
                float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if ((int)qi < nq) {
                    v = __ldg(reinterpret_cast<const float4*>(queries + (q_begin + t0 + qi) * dim + k));
                    if (level == 1) {   // residual, RVQ.cu:180-188
                        const float4 c = __ldg(reinterpret_cast<const float4*>(coarse + (size_t)best_coarse[t0 + qi] * dim + k));
                        v.x = v.x - c.x; v.y = v.y - c.y; v.z = v.z - c.z; v.w = v.w - c.w;
                    }
                }
                x[(k + 0) * XS + qi] = v.x;
                x[(k + 1) * XS + qi] = v.y;
                x[(k + 2) * XS + qi] = v.z;
                x[(k + 3) * XS + qi] = v.w;
            }
            __syncthreads();
            {   // four queries per warp at a time, so that their shuffle trees overlap
                float n2[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int qi = (int)warp + u * kWarps;
                    n2[u] = qi < nq ? NormByWarp(x + qi, XS, dim, lane) : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int qi = (int)warp + u * kWarps;
                    if (lane == 0 && qi < nq) norms[qi] = n2[u];
                }
            }
            __syncthreads();
            if (bulk && t0 == 0) {
                const bool arrived = BarrierWaitBounded(&copy_barrier, (uint32_t)level & 1u);
                if (!__syncthreads_and(arrived)) {
                    // Never seen. The copy may still land in `cb` later, so the block must not use that memory
                    // again: it reports the timeout, gives the copy one more bounded wait and ends without
                    // entries for its queries.
                    if (tid == 0 && status != nullptr) atomicOr(status, TANN_STATUS_COPY_TIMEOUT);
                    BarrierWaitBounded(&copy_barrier, (uint32_t)level & 1u);
                    return;
                }
            }
            ArgMin best[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { best[j].d = __int_as_float(0x7f800000); best[j].idx = 0x7fffffff; }
            if ((int)(qg * 8) < nq) {   // warp-uniform: a warp holds one query group
                for (uint32_t c0 = 4 * cg; c0 < count; c0 += 4 * 64) {
                    float dot[8][4];
#pragma unroll
                    for (int j = 0; j < 8; ++j) dot[j][0] = dot[j][1] = dot[j][2] = dot[j][3] = 0.0f;
                    // level 1: sizes of the four buckets per query, requested before the FMA loop
                    int4 sizes[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        sizes[j] = make_int4(1, 1, 1, 1);
                        const int qi = (int)qg * 8 + j;
                        if (level == 1 && qi < nq)
                            sizes[j] = __ldg(reinterpret_cast<const int4*>(bucket_sizes + (size_t)best_coarse[t0 + qi] * nf + c0));
                    }
                    const float* col = cb + c0;
                    const float* xq = x + qg * 8;
#pragma unroll 4
                    for (uint32_t k = 0; k < dim; ++k) {
                        const float4 w = *reinterpret_cast<const float4*>(col + (size_t)k * count);
                        const float4 xa = *reinterpret_cast<const float4*>(xq + k * XS);
                        const float4 xb = *reinterpret_cast<const float4*>(xq + k * XS + 4);
                        const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            dot[j][0] = fmaf(xv[j], w.x, dot[j][0]);
                            dot[j][1] = fmaf(xv[j], w.y, dot[j][1]);
                            dot[j][2] = fmaf(xv[j], w.z, dot[j][2]);
                            dot[j][3] = fmaf(xv[j], w.w, dot[j][3]);
                        }
                    }
                    const float4 cn4 = __ldg(reinterpret_cast<const float4*>(book_norms + c0));
                    const float cn[4] = {cn4.x, cn4.y, cn4.z, cn4.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int qi = (int)qg * 8 + j;
                        if (qi >= nq) continue;
                        const int sz[4] = {sizes[j].x, sizes[j].y, sizes[j].z, sizes[j].w};
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float D = (-2.0f * dot[j][u] + norms[qi]) + cn[u];
                            // level 0: selectMin1.cu:9-23; level 1 (:66-81) starts from FLT_MAX and skips empty buckets
                            const bool ok = level == 0 || (D < FLT_MAX && sz[u] > 0);
                            if (ok) best[j] = Better(best[j], ArgMin{D, (int)(c0 + u)});
                        }
                    }
                }
            }
            if ((int)(qg * 8) < nq) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    ArgMin v = best[j];
#pragma unroll
                    for (int off = 16; off >= 1; off >>= 1) {
                        ArgMin o;
                        o.d = __shfl_xor_sync(kFull, v.d, off);
                        o.idx = __shfl_xor_sync(kFull, v.idx, off);
                        v = Better(v, o);
                    }
                    if (lane == 0) scratch[warp][j] = v;
                }
            }
            __syncthreads();
            if ((int)tid < nq) {
                const uint32_t g = tid >> 3, j = tid & 7;      // query 8 g + j was scored by warps 2 g and 2 g + 1
                const ArgMin r = Better(scratch[2 * g][j], scratch[2 * g + 1][j]);
                const int idx = r.idx == 0x7fffffff ? 0 : r.idx;
                if (level == 0) best_coarse[t0 + tid] = idx;
                else best_cluster[t0 + tid] = best_coarse[t0 + tid] * (int)nf + idx;
            }
        }
    }
    __syncthreads();
    // gather, rvq_device_entries.cu:15-52
    for (uint32_t qi = warp; qi < n_mine; qi += kWarps) {   // one warp per query: no index division
        const int cluster = best_cluster[qi];
        uint32_t begin = 0, n = 0;
        if (cluster >= 0) {
            begin = cluster_offsets[cluster];
            n = min(cluster_offsets[cluster + 1] - begin, entry_count);
        }
        uint32_t* o = out_entry_ids + (q_begin + qi) * entry_count;
        for (uint32_t i = lane; i < entry_count; i += 32) {
            uint32_t v = kInvalid;
            if (i < n) v = cluster_ids[begin + i];
            else if (n == 0 && i == 0) v = fallback;
            o[i] = v;
        }
    }
    if (out_clusters != nullptr)
        for (uint32_t qi = tid; qi < n_mine; qi += kSmemThreads) out_clusters[q_begin + qi] = best_cluster[qi];
}

cudaError_t LaunchRvqNorms(const float* rows, uint32_t count, uint32_t dim, float* out,
                           cudaStream_t stream) {
    if (count == 0) return cudaSuccess;
    rvq_norms_kernel<<<count < 4096u ? count : 4096u, 128, 0, stream>>>(rows, count, dim, out);
    return cudaGetLastError();
}

cudaError_t LaunchRvqEntries(const float* queries, uint64_t Q, uint32_t dim, const float* coarse,
                             const float* coarse_t, const float* coarse_norms, uint32_t nc,
                             const float* fine_t, const float* fine_norms, uint32_t nf,
                             const int32_t* bucket_sizes, const uint32_t* cluster_offsets,
                             const uint32_t* cluster_ids, uint32_t entry_count, uint32_t fallback,
                             int32_t* out_clusters, uint32_t* out_entry_ids,
                             uint32_t* out_entry_offsets, cudaStream_t stream, uint32_t* status) {
    if (Q == 0) return cudaSuccess;
    // codebooks that fit shared memory next to a 64-query tile: one resident block per SM
    {
        const bool aligned = nc % 4 == 0 && nf % 4 == 0 && dim % 4 == 0 &&
                             ((reinterpret_cast<uintptr_t>(coarse_t) | reinterpret_cast<uintptr_t>(fine_t) |
                               reinterpret_cast<uintptr_t>(coarse_norms) | reinterpret_cast<uintptr_t>(fine_norms) |
                               reinterpret_cast<uintptr_t>(bucket_sizes) | reinterpret_cast<uintptr_t>(queries) |
                               reinterpret_cast<uintptr_t>(coarse)) & 15u) == 0;
        const size_t max_count = nc > nf ? nc : nf;
        const size_t smem = (max_count + kSmemTile + 4) * (size_t)dim * 4;
        const uint64_t grid = (uint64_t)SmCount();
        const uint64_t per = (Q + grid - 1) / grid;   // an even share per SM; a share need not be a multiple of 8
        if (aligned && smem <= 200 * 1024 && per <= (uint64_t)kSmemMaxPerBlock) {
            cudaError_t e = cudaFuncSetAttribute(rvq_entries_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
            const uint64_t blocks = (Q + per - 1) / per;
            rvq_entries_smem_kernel<<<(unsigned)blocks, kSmemThreads, smem, stream>>>(
                queries, Q, dim, coarse, coarse_t, coarse_norms, nc, fine_t, fine_norms, nf, bucket_sizes,
                cluster_offsets, cluster_ids, entry_count, fallback, out_clusters, out_entry_ids,
                out_entry_offsets, (uint32_t)per, status);
            return cudaGetLastError();
        }
    }
    // codebooks whose sizes are multiples of 4 (and 16-byte aligned) take the tiled kernel
    const bool tiled = nc % 4 == 0 && nf % 4 == 0 &&
                       ((reinterpret_cast<uintptr_t>(coarse_t) | reinterpret_cast<uintptr_t>(fine_t) |
                         reinterpret_cast<uintptr_t>(coarse_norms) | reinterpret_cast<uintptr_t>(fine_norms)) & 15u) == 0;
    const int qb = tiled ? kTileQueries : kRvqQueriesPerBlock;
    const size_t smem = (size_t)qb * dim * 4;
    const uint64_t blocks = (Q + qb - 1) / qb;
    const uint64_t cap = (uint64_t)SmCount() * 8;
    auto kernel = tiled ? rvq_entries_tile_kernel : rvq_entries_kernel;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    kernel<<<(unsigned)(blocks < cap ? blocks : cap), kRvqThreads, smem, stream>>>(
        queries, Q, dim, coarse, coarse_t, coarse_norms, nc, fine_t, fine_norms, nf, bucket_sizes,
        cluster_offsets, cluster_ids, entry_count, fallback, out_clusters, out_entry_ids,
        out_entry_offsets);
    return cudaGetLastError();
}

}  // namespace tann
