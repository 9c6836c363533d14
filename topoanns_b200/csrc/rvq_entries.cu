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
                             uint32_t* out_entry_offsets, cudaStream_t stream) {
    if (Q == 0) return cudaSuccess;
    const size_t smem = (size_t)kRvqQueriesPerBlock * dim * 4;
    const uint64_t blocks = (Q + kRvqQueriesPerBlock - 1) / kRvqQueriesPerBlock;
    const uint64_t cap = (uint64_t)SmCount() * 8;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(rvq_entries_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    rvq_entries_kernel<<<(unsigned)(blocks < cap ? blocks : cap), kRvqThreads, smem, stream>>>(
        queries, Q, dim, coarse, coarse_t, coarse_norms, nc, fine_t, fine_norms, nf, bucket_sizes,
        cluster_offsets, cluster_ids, entry_count, fallback, out_clusters, out_entry_ids,
        out_entry_offsets);
    return cudaGetLastError();
}

}  // namespace tann
