// Builds the neighbour-code layout: out[n][j][:] = codes[adjacency[n][j]][:] for every node n and
// adjacency slot j (zeros for padding slots), so that an expansion finds its neighbours' PQ codes in one
// contiguous row. A plain gather: every thread moves one code row (16-byte pieces when M allows it).
#include "tann_common.cuh"
#include "tann_launch.h"

namespace tann {

__global__ void __launch_bounds__(256)
neighbor_codes_kernel(const __grid_constant__ TannIndexView ix, uint64_t first_node, uint64_t num_rows,
                      uint8_t* __restrict__ out) {
    const uint32_t deg = ix.degree, M = ix.num_chunks;
    const uint64_t total = num_rows * deg;
    const bool wide = (M % 16 == 0);
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = e / deg;
        const uint32_t j = (uint32_t)(e - row * deg);
        const uint64_t node = first_node + row;
        const uint32_t* adj = reinterpret_cast<const uint32_t*>(ShardRow(ix.adjacency, node, (uint64_t)deg * 4));
        const uint32_t id = __ldg(adj + j);
        uint8_t* dst = out + e * M;
        if (id != kInvalid && id < ix.num_nodes) {
            const uint8_t* src = ShardRow(ix.codes, id, M);
            if (wide) {
                for (uint32_t b = 0; b < M; b += 16)
                    *reinterpret_cast<uint4*>(dst + b) = __ldg(reinterpret_cast<const uint4*>(src + b));
            } else {
                for (uint32_t b = 0; b < M; ++b) dst[b] = __ldg(src + b);
            }
        } else {
            for (uint32_t b = 0; b < M; ++b) dst[b] = 0;
        }
    }
}

cudaError_t LaunchNeighborCodes(const TannIndexView& ix, uint64_t first_node, uint64_t num_rows, uint8_t* out,
                                cudaStream_t stream) {
    if (num_rows == 0) return cudaSuccess;
    neighbor_codes_kernel<<<SmCount() * 16, 256, 0, stream>>>(ix, first_node, num_rows, out);
    return cudaGetLastError();
}

}  // namespace tann
