// pq2 refine: re-score the first refine_top_l candidates of every query with the second-level
// PQ and re-sort them. Values follow the reference kernels (src/search/rerank_exact.cu:573-665
// plain, :773-879 residual): lane l sums chunks l, l+32, ... then the shuffle tree; the residual
// form adds (LUT2 + cross term) per chunk and the base distance once at the end. One block per
// query (persistent), one warp per rank, 64-bit keys sorted in shared memory.
//
// The second-level table entries can come from a table built beforehand (tann_lut_build, what the
// reference does) or be computed where they are needed: a refine reads refine_top_l x M of the M x 256
// entries of a query, so summing the chunk's dims on the spot - the same ascending-dim FMA chain as
// the table build (src/search/pq_query_tables.cu:33-52), hence the same bits - saves writing and
// reading Q x M x 1 KB of tables.
#include "tann_common.cuh"
#include "tann_launch.h"

namespace tann {

constexpr int kPq2Threads = 256;

__device__ inline void BlockSortKeys(unsigned long long* keys, uint32_t n_pow2, int threads) {
    for (uint32_t k = 2; k <= n_pow2; k <<= 1) {
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
            for (uint32_t t = threadIdx.x; t < n_pow2 / 2; t += threads) {
                const uint32_t lo = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                const uint32_t hi = lo | j;
                const bool asc = (lo & k) == 0;
                const unsigned long long a = keys[lo], b = keys[hi];
                if ((a > b) == asc) { keys[lo] = b; keys[hi] = a; }
            }
            __syncthreads();
        }
    }
}

__global__ void __launch_bounds__(kPq2Threads)
pq2_refine_kernel(const Cand* __restrict__ cand, const uint32_t* __restrict__ stats, uint64_t Q,
                  uint32_t capacity, uint32_t Lr, uint32_t padded, int has_base, TannShards base_codes,
                  TannShards pq2_codes, uint32_t M, const float* __restrict__ lut2,
                  const float* __restrict__ cross, Cand* __restrict__ out,
                  const float* __restrict__ t2_col_major, const float* __restrict__ mu2,
                  const uint32_t* __restrict__ chunk_offsets, const float* __restrict__ queries_f32, uint32_t dim,
                  const uint8_t* __restrict__ selector_bits, uint32_t selector_stride,
                  const float* __restrict__ lut_outlier) {
    extern __shared__ unsigned long long pq2_keys[];
    float* sq = reinterpret_cast<float*>(pq2_keys + padded);   // [dim] query minus centroid (table-free form)
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr unsigned long long kInvalidKey = 0xff800000ffffffffull;
    for (uint64_t q = blockIdx.x; q < Q; q += gridDim.x) {
        const uint32_t valid = min(stats[q * 8 + 4], Lr);
        const float* lut = lut2 != nullptr ? lut2 + q * (uint64_t)M * kCentroids : nullptr;
        const float* lut_out = lut_outlier != nullptr ? lut_outlier + q * (uint64_t)M * kCentroids : nullptr;
        if (lut == nullptr) {
            for (uint32_t i = threadIdx.x; i < dim; i += kPq2Threads) sq[i] = queries_f32[q * dim + i] - __ldg(mu2 + i);
            __syncthreads();
        }
        for (uint32_t rank = warp; rank < padded; rank += kPq2Threads / 32) {
            unsigned long long key = kInvalidKey;
            if (rank < valid) {
                const Cand c = cand[q * capacity + rank];
                const uint32_t id = RawId(c.id);
                if (id != kInvalid) {
                    const uint8_t* rc_row = ShardRow(pq2_codes, id, M);
                    const uint8_t* bc_row = has_base ? ShardRow(base_codes, id, M) : nullptr;
                    // hybrid PQ (src/search/rerank_exact.cu:667-771): bit m of the node's selector row picks the
                    // outlier codebook's table for chunk m
                    const uint8_t* sel_row = selector_bits != nullptr ? selector_bits + (uint64_t)id * selector_stride : nullptr;
                    float partial = 0.0f;
                    for (uint32_t m = lane; m < M; m += 32) {
                        const uint32_t rc = rc_row[m];
                        float entry;
                        if (lut != nullptr) {
                            const bool outlier = sel_row != nullptr && ((sel_row[m >> 3] >> (m & 7u)) & 1u) != 0;
                            entry = (outlier ? lut_out : lut)[m * kCentroids + rc];
                        } else {
                            entry = 0.0f;
                            for (uint32_t k = __ldg(chunk_offsets + m); k < __ldg(chunk_offsets + m + 1); ++k) {
                                const float diff = __ldg(t2_col_major + (size_t)k * kCentroids + rc) - sq[k];
                                entry = fmaf(diff, diff, entry);
                            }
                        }
                        if (has_base) {
                            const uint32_t bc = bc_row[m];
                            partial += entry + __ldg(cross + ((size_t)m * kCentroids + bc) * kCentroids + rc);
                        } else {
                            partial += entry;
                        }
                    }
                    partial = WarpTreeSum(partial);
                    const float dist = has_base ? c.dist + partial : partial;
                    key = KeyOf(dist, id);
                }
            }
            if (lane == 0) pq2_keys[rank] = key;
        }
        __syncthreads();
        BlockSortKeys(pq2_keys, padded, kPq2Threads);
        for (uint32_t i = threadIdx.x; i < Lr; i += kPq2Threads) {
            const unsigned long long k = pq2_keys[i];
            Cand c;
            c.dist = FromOrderedBits((uint32_t)(k >> 32));
            c.id = (uint32_t)k;
            out[q * Lr + i] = c;
        }
        __syncthreads();
    }
}

// X[m][b][r] = 2 * sum_dim (T1[b][dim] + mu1[dim]) * (T2[r][dim] + mu2[dim]), products and sums
// rounded separately like the host loop of the reference (src/search/search_resources.cpp:52-91).
__global__ void __launch_bounds__(256)
cross_terms_kernel(uint32_t dim, uint32_t M, const uint32_t* __restrict__ offs,
                   const float* __restrict__ t1, const float* __restrict__ mu1,
                   const float* __restrict__ t2, const float* __restrict__ mu2, float* __restrict__ out) {
    const uint64_t total = (uint64_t)M * kCentroids * kCentroids;
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = e & 255u, b = (e >> 8) & 255u, m = (uint32_t)(e >> 16);
        float dot = 0.0f;
        for (uint32_t k = offs[m]; k < offs[m + 1]; ++k) {
            const float bv = __fadd_rn(t1[(size_t)b * dim + k], mu1[k]);
            const float rv = __fadd_rn(t2[(size_t)r * dim + k], mu2[k]);
            dot = __fadd_rn(dot, __fmul_rn(bv, rv));
        }
        out[e] = __fmul_rn(2.0f, dot);
    }
}

cudaError_t LaunchPq2Refine(const void* cand, const uint32_t* stats, uint64_t Q, uint32_t capacity,
                            uint32_t refine_top_l, const TannShards* base_codes,
                            const TannShards& pq2_codes, uint32_t M, const float* lut2,
                            const float* cross_terms, void* out, cudaStream_t stream,
                            const float* t2_col_major, const float* mu2, const uint32_t* chunk_offsets,
                            const float* queries_f32, uint32_t dim, const uint8_t* selector_bits,
                            uint32_t selector_stride, const float* lut_outlier) {
    if (Q == 0 || refine_top_l == 0) return cudaSuccess;
    uint32_t padded = 1;
    while (padded < refine_top_l) padded <<= 1;
    const size_t smem = (size_t)padded * 8 + (lut2 == nullptr ? (size_t)dim * 4 : 0);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(pq2_refine_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const uint64_t cap = (uint64_t)SmCount() * 6;
    TannShards none{};
    pq2_refine_kernel<<<(unsigned)(Q < cap ? Q : cap), kPq2Threads, smem, stream>>>(
        static_cast<const Cand*>(cand), stats, Q, capacity, refine_top_l, padded,
        base_codes != nullptr ? 1 : 0, base_codes != nullptr ? *base_codes : none, pq2_codes, M, lut2,
        cross_terms, static_cast<Cand*>(out), t2_col_major, mu2, chunk_offsets, queries_f32, dim, selector_bits,
        selector_stride, lut_outlier);
    return cudaGetLastError();
}

cudaError_t LaunchCrossTerms(uint32_t dim, uint32_t M, const uint32_t* chunk_offsets, const float* t1,
                             const float* mu1, const float* t2, const float* mu2, float* out,
                             cudaStream_t stream) {
    if (M == 0) return cudaSuccess;
    cross_terms_kernel<<<SmCount() * 8, 256, 0, stream>>>(dim, M, chunk_offsets, t1, mu1, t2, mu2, out);
    return cudaGetLastError();
}

}  // namespace tann
