// Stand-ins for the NVMe (BaM) entry points that the reference's search sources declare but that
// live in its BaM provider, which cannot be built here (its BaM submodule is not vendored). None
// of them is reached unless a BaM provider is attached, which the driver never does: the host
// stubs throw and the device stubs do nothing. TEST INFRASTRUCTURE ONLY.
#include <stdexcept>

#include "fused_rerank_device.hpp"
#include "topoanns/bam_vector_provider.hpp"
#include "topology_microbatch_io.hpp"

namespace topoanns {

double RunBamFusedExactDistanceFloatQueries(const VectorPageProvider&, ScalarKind, const CudaBuffer<float>&,
                                            const CudaBuffer<std::uint64_t>&, const CudaBuffer<std::uint32_t>&,
                                            const CudaBuffer<std::uint32_t>&, const CudaBuffer<std::uint32_t>&,
                                            std::size_t, const VectorPageLayout&, std::size_t, CudaBuffer<float>*) {
    throw std::runtime_error("ref_stub: no NVMe provider in this build");
}

namespace detail {

void LaunchBamTopologyMicrobatchReads(const void*, const DeviceTopologyIoRequest*, const std::uint32_t*, std::size_t,
                                      const TopologyMicrobatchIoConfig&, std::uint32_t*, float*, std::size_t,
                                      std::size_t, cudaStream_t) {
    throw std::runtime_error("ref_stub: no NVMe provider in this build");
}

__device__ void CopyTopologyNeighborsFromBam(const void*, std::size_t, std::size_t, std::uint32_t, std::uint32_t*,
                                             std::uint32_t, std::uint32_t) {}

__device__ float ReadCombinedNodeFromBam(const void*, std::size_t, std::size_t, std::uint32_t, std::uint32_t,
                                         std::uint64_t, std::uint32_t, const float*, std::uint32_t*, std::uint32_t,
                                         std::uint32_t) {
    return 0.0f;
}

}  // namespace detail
}  // namespace topoanns

namespace topoanns::detail {
PersistentBamRerankRunResult RunPersistentBamRerankFloat32(const SearchResources&, const CudaBuffer<float>&,
                                                           const DeviceTopologyBatchResult&, std::size_t,
                                                           const RerankExactParams&) {
    throw std::runtime_error("ref_stub: the persistent rerank needs the NVMe provider");
}
PersistentBamRerankRunResult RunPersistentBamRerankFloat32(const SearchResources&, const CudaBuffer<float>&,
                                                           const std::vector<float>&, const DeviceTopologyBatchResult&,
                                                           std::size_t, const RerankExactParams&, cudaStream_t) {
    throw std::runtime_error("ref_stub: the persistent rerank needs the NVMe provider");
}
}  // namespace topoanns::detail
