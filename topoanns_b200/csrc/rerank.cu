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
#include "tann_common.cuh"
#include "tann_launch.h"

namespace tann {

constexpr int kRerankThreads = 128;
constexpr unsigned long long kInvalidKey64 = 0xff800000ffffffffull;

__device__ __forceinline__ const uint8_t* VectorPtr(const TannIndexView& ix, uint32_t id) {
    uint64_t local = id;
    const uint8_t* base = static_cast<const uint8_t*>(ix.vectors.base[0]);
    if (ix.vectors.num_shards > 1) {
        const uint64_t shard = id / ix.vectors.rows_per_shard;
        local = id - shard * ix.vectors.rows_per_shard;
        base = static_cast<const uint8_t*>(ix.vectors.base[shard]);
    }
    // src/io/vector_page_layout.cpp:50-57
    return base + (local / ix.vectors_per_page) * ix.page_bytes + (local % ix.vectors_per_page) * ix.vector_bytes;
}

__device__ __forceinline__ float LowerBoundSq(float approx_sq, float err) {
    const float a = sqrtf(fmaxf(approx_sq, 0.0f));
    const float lo = fmaxf(0.0f, a - err);
    return lo * lo;
}

__global__ void __launch_bounds__(kRerankThreads)
rerank_kernel(const __grid_constant__ TannIndexView ix, TannRerankParams p, const Cand* __restrict__ cand,
              uint32_t capacity, uint64_t Q, const void* __restrict__ queries, uint32_t qkind,
              const float* __restrict__ error_bounds, uint32_t padded, float* __restrict__ out_dists,
              uint32_t* __restrict__ out_ids, unsigned long long* __restrict__ out_counts,
              const uint8_t* __restrict__ queries_u8, const uint32_t* __restrict__ not_u8_flag) {
    extern __shared__ __align__(16) unsigned char rr_smem[];
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(rr_smem);   // [padded]
    uint8_t* qrow = reinterpret_cast<uint8_t*>(keys + padded);                   // query row copy
    __shared__ float s_threshold, s_qnorm;
    __shared__ unsigned int s_exact, s_filtered;
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
    unsigned long long tot_exact = 0, tot_filtered = 0;

    for (uint64_t q = blockIdx.x; q < Q; q += gridDim.x) {
        const uint8_t* qsrc = static_cast<const uint8_t*>(queries) + q * qbytes;
        for (uint32_t i = tid; i < qbytes; i += kRerankThreads) qrow[i] = qsrc[i];
        for (uint32_t i = tid; i < padded; i += kRerankThreads) keys[i] = kInvalidKey64;
        if (tid == 0) {
            s_threshold = __int_as_float(0x7f800000);
            s_exact = 0; s_filtered = 0;
        }
        __syncthreads();
        if (p.use_bound_filter && tid == 0) {
            double s = 0.0;
            for (uint32_t i = 0; i < dim; ++i) {
                const double v = (double)LoadAsFloat<float>(qrow, qkind, i);
                s += v * v;
            }
            s_qnorm = (float)s;
        }
        __syncthreads();
        for (uint32_t rb = 0; rb < p.top_n; rb += tile) {
            const uint32_t rc = min(tile, p.top_n - rb);
            const float threshold = s_threshold;
            // A warp scores kGroup candidates per step: all their row loads are issued before any
            // reduction, so several random 128-byte (or longer) reads are in flight per lane.
            constexpr uint32_t kGroup = 4;
            for (uint32_t r0 = rb + warp * kGroup; r0 < rb + rc; r0 += (kRerankThreads / 32) * kGroup) {
                const uint8_t* vptr[kGroup];
                uint32_t ids[kGroup];
                bool act[kGroup];
#pragma unroll
                for (uint32_t g = 0; g < kGroup; ++g) {
                    const uint32_t r = r0 + g;
                    act[g] = false;
                    ids[g] = kInvalid;
                    vptr[g] = nullptr;
                    if (r >= rb + rc || r >= capacity) continue;
                    const Cand c = cand[q * capacity + r];
                    if (c.id == kInvalid) continue;
                    const uint32_t id = c.id & kRawMask;
                    if (id >= ix.num_nodes) continue;
                    if (p.use_bound_filter && isfinite(threshold)) {
                        if (LowerBoundSq(c.dist - s_qnorm, __ldg(error_bounds + id)) > threshold) {
                            if (lane == 0) atomicAdd(&s_filtered, 1u);
                            continue;
                        }
                    }
                    act[g] = true;
                    ids[g] = id;
                    vptr[g] = VectorPtr(ix, id);
                }
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
                        for (uint32_t g = 0; g < kGroup; ++g) {
                            const uint32_t ad = __vabsdiffu4(w[g], qw);
                            acc[g] = __dp4a(ad, ad, acc[g]);
                        }
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
                    uint32_t n = 0;
#pragma unroll
                    for (uint32_t g = 0; g < kGroup; ++g) {
                        if (!act[g]) continue;
                        keys[r0 + g] = KeyOf(dist[g], ids[g]);
                        ++n;
                    }
                    if (n) atomicAdd(&s_exact, n);
                }
            }
            __syncthreads();
            if (p.use_bound_filter) {
                if (tid == 0) {  // :541-571, k-th smallest over ranks [0, rb + rc)
                    float best[128];
                    const uint32_t k = p.top_k;
                    for (uint32_t i = 0; i < k; ++i) best[i] = __int_as_float(0x7f800000);
                    const uint32_t prefix = min(p.top_n, rb + rc);
                    for (uint32_t r = 0; r < prefix; ++r) {
                        const float x = FromOrderedBits((uint32_t)(keys[r] >> 32));
                        if (!(x < best[k - 1])) continue;
                        uint32_t ins = k - 1;
                        while (ins > 0 && x < best[ins - 1]) { best[ins] = best[ins - 1]; --ins; }
                        best[ins] = x;
                    }
                    s_threshold = best[k - 1];
                }
                __syncthreads();
            }
        }
        // final sort and output
        for (uint32_t k = 2; k <= padded; k <<= 1) {
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
        for (uint32_t i = tid; i < p.top_n; i += kRerankThreads) {
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
                         const uint32_t* not_u8_flag) {
    if (Q == 0 || p.top_n == 0) return cudaSuccess;
    uint32_t padded = 1;
    while (padded < p.top_n) padded <<= 1;
    const size_t qbytes = (size_t)ix.dim * (query_kind == TANN_KIND_FLOAT32 ? 4 : 1);
    const size_t smem = (size_t)padded * 8 + ((qbytes + 15) & ~(size_t)15);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(rerank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
    }
    const uint64_t cap = (uint64_t)SmCount() * 8;
    rerank_kernel<<<(unsigned)(Q < cap ? Q : cap), kRerankThreads, smem, stream>>>(
        ix, p, static_cast<const Cand*>(cand), capacity, Q, queries, query_kind, error_bounds, padded,
        out_dists, out_ids, out_counts, queries_u8, not_u8_flag);
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
