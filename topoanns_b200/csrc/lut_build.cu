// ADC look-up tables for a batch of queries: out[q][m][c] written once, in the accumulation
// order of the reference kernel (src/search/pq_query_tables.cu:33-52: ascending dim, one FMA per
// dim), without its zero-fill pass and global read-modify-write.
#include "tann_common.cuh"
#include "tann_launch.h"

namespace tann {

constexpr int kLutThreads = 256;

__global__ void __launch_bounds__(kLutThreads)
lut_build_kernel(const float* __restrict__ tables_col_major, const float* __restrict__ centroid,
                 const uint32_t* __restrict__ chunk_offsets, uint32_t dim, uint32_t M,
                 const void* __restrict__ queries, uint32_t query_kind, uint64_t Q,
                 float* __restrict__ out) {
    extern __shared__ float lut_smem[];
    float* sq = lut_smem;                                       // [dim]
    uint32_t* offs = reinterpret_cast<uint32_t*>(sq + dim);     // [M + 1]
    const uint32_t tid = threadIdx.x;
    for (uint32_t i = tid; i <= M; i += kLutThreads) offs[i] = chunk_offsets[i];
    // chunks of equal width (the usual case) take the unrolled build: four centroids per thread and
    // 16 sixteen-byte loads in flight; the entries are written straight to their place in the output
    const uint32_t sub0 = __ldg(chunk_offsets + 1) - __ldg(chunk_offsets);
    bool same = __ldg(chunk_offsets) == 0u;
    for (uint32_t i = tid; i < M; i += kLutThreads)
        same = same && (__ldg(chunk_offsets + i + 1) - __ldg(chunk_offsets + i)) == sub0;
    const uint32_t uniform_sub = __syncthreads_and(same) ? sub0 : 0u;
    for (uint64_t q = blockIdx.x; q < Q; q += gridDim.x) {
        __syncthreads();
        for (uint32_t i = tid; i < dim; i += kLutThreads)
            sq[i] = LoadAsFloat<float>(queries, query_kind, q * dim + i) - centroid[i];
        __syncthreads();
        float* o = out + q * (uint64_t)M * kCentroids;
        switch (uniform_sub) {
            case 1: BuildLutUniform<1, kLutThreads>(o, sq, tables_col_major, M, tid); break;
            case 2: BuildLutUniform<2, kLutThreads>(o, sq, tables_col_major, M, tid); break;
            case 3: BuildLutUniform<3, kLutThreads>(o, sq, tables_col_major, M, tid); break;
            case 4: BuildLutUniform<4, kLutThreads>(o, sq, tables_col_major, M, tid); break;
            case 6: BuildLutUniform<6, kLutThreads>(o, sq, tables_col_major, M, tid); break;
            case 8: BuildLutUniform<8, kLutThreads>(o, sq, tables_col_major, M, tid); break;
            default: BuildLutGeneric<kLutThreads>(o, sq, offs, tables_col_major, M, tid); break;
        }
    }
}

cudaError_t LaunchLutBuild(const float* tables_col_major, const float* centroid,
                           const uint32_t* chunk_offsets, uint32_t dim, uint32_t M,
                           const void* queries, uint32_t query_kind, uint64_t Q, float* out,
                           cudaStream_t stream) {
    if (Q == 0) return cudaSuccess;
    const size_t smem = (size_t)dim * 4 + ((size_t)M + 1) * 4;
    const uint64_t grid = Q < (uint64_t)SmCount() * 8 ? Q : (uint64_t)SmCount() * 8;
    lut_build_kernel<<<(unsigned)grid, kLutThreads, smem, stream>>>(
        tables_col_major, centroid, chunk_offsets, dim, M, queries, query_kind, Q, out);
    return cudaGetLastError();
}

}  // namespace tann
