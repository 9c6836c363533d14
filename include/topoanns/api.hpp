// Host C++ API of the B200 graph-search path.
//
// The classes below carry the names, signatures, defaults and error texts of the public headers of
// szrr/TopoANNS (include/topoanns/*.hpp), so that code written against that project's batched search
// path compiles against this one; each of the per-class header names of that project exists here
// as a forwarding header. Behind them everything runs through the C ABI of libtopoanns_b200.so
// (include/topoanns_b200.h): no kernel is launched from this layer and nothing is computed on the
// host except result materialisation.
//
// Differences a caller can see:
//   * VectorPageProvider::DeviceReadHandle() points at a TannShards descriptor (HBM, NVLink-peer or
//     pinned-host pages) instead of a BaM array; the three providers are declared below and replace
//     BamVectorPageProvider.
//   * topology.bin files of any degree load (the reference accepts 64 only).
//   * RerankExecutionMode::kPersistent runs the same fused tile kernel as kTiled; the rerank early stop
//     works in the tiled and persistent modes, and the learned rerank stop (persistent mode + bound
//     filter, as in the reference) runs on every vector provider and scalar kind, not only on the
//     NVMe provider with float32 vectors.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <filesystem>
#include <limits>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "topoanns_b200.h"

namespace topoanns {

// ---- common (reference: include/topoanns/common.hpp) ---------------------------------------------
constexpr std::size_t kDefaultPageSizeBytes = 4096;
constexpr std::uint32_t kFixedTopologyDegree = 64;
constexpr std::uint32_t kInvalidNodeId = 0xffffffffu;

enum class ScalarKind { kInt8, kUint8, kFloat32 };

inline std::size_t ScalarKindBytes(ScalarKind k) {
    if (k == ScalarKind::kInt8 || k == ScalarKind::kUint8) return 1;
    if (k == ScalarKind::kFloat32) return 4;
    throw std::runtime_error("Unsupported ScalarKind.");
}
inline const char* ScalarKindName(ScalarKind k) {
    return k == ScalarKind::kInt8 ? "int8" : k == ScalarKind::kUint8 ? "uint8"
         : k == ScalarKind::kFloat32 ? "float32" : "unknown";
}
inline std::string BuildErrorMessage(const std::string& context, const std::string& detail) {
    return context + ": " + detail;
}
inline void ThrowIfCudaError(cudaError_t status, const char* context) {
    if (status != cudaSuccess) throw std::runtime_error(BuildErrorMessage(context, cudaGetErrorString(status)));
}
// Turns a non-zero C-ABI status into the reference's exception form.
void ThrowIfTannError(TannStatus status, const char* context);

// ---- CudaBuffer (reference: include/topoanns/cuda_buffer.hpp) -------------------------------------
template <typename T>
class CudaBuffer {
public:
    CudaBuffer() = default;
    ~CudaBuffer() { Reset(); }
    CudaBuffer(const CudaBuffer&) = delete;
    CudaBuffer& operator=(const CudaBuffer&) = delete;
    CudaBuffer(CudaBuffer&& o) noexcept : ptr_(o.ptr_), count_(o.count_) { o.ptr_ = nullptr; o.count_ = 0; }
    CudaBuffer& operator=(CudaBuffer&& o) noexcept {
        if (this != &o) { Reset(); ptr_ = o.ptr_; count_ = o.count_; o.ptr_ = nullptr; o.count_ = 0; }
        return *this;
    }
    static CudaBuffer Allocate(std::size_t count) {
        CudaBuffer b;
        b.count_ = count;
        if (count != 0) ThrowIfCudaError(cudaMalloc(reinterpret_cast<void**>(&b.ptr_), count * sizeof(T)), "cudaMalloc");
        return b;
    }
    static CudaBuffer CopyFromHost(const std::vector<T>& host) {
        CudaBuffer b = Allocate(host.size());
        if (!host.empty())
            ThrowIfCudaError(cudaMemcpy(b.ptr_, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice),
                             "cudaMemcpyHostToDevice");
        return b;
    }
    std::vector<T> CopyToHost() const {
        std::vector<T> host(count_);
        if (count_ != 0)
            ThrowIfCudaError(cudaMemcpy(host.data(), ptr_, count_ * sizeof(T), cudaMemcpyDeviceToHost),
                             "cudaMemcpyDeviceToHost");
        return host;
    }
    T* get() { return ptr_; }
    const T* get() const { return ptr_; }
    std::size_t size() const { return count_; }
    bool empty() const { return count_ == 0; }

private:
    void Reset() noexcept {
        if (ptr_ != nullptr) cudaFree(ptr_);
        ptr_ = nullptr;
        count_ = 0;
    }
    T* ptr_ = nullptr;
    std::size_t count_ = 0;
};

// ---- entries (reference: device_entry_batch.hpp, entry_provider.hpp) -------------------------------
struct DeviceEntryBatch {
    DeviceEntryBatch() = default;
    DeviceEntryBatch(const DeviceEntryBatch&) = delete;
    DeviceEntryBatch& operator=(const DeviceEntryBatch&) = delete;
    DeviceEntryBatch(DeviceEntryBatch&&) noexcept = default;
    DeviceEntryBatch& operator=(DeviceEntryBatch&&) noexcept = default;
    std::size_t num_queries = 0;
    std::size_t entries_per_query = 0;
    CudaBuffer<std::uint32_t> offsets;  // num_queries + 1
    CudaBuffer<std::uint32_t> ids;
};

class EntryProvider {
public:
    virtual ~EntryProvider() = default;
    virtual std::vector<std::uint32_t> GetEntryPoints(std::size_t query_id) const = 0;
};
class FixedEntryProvider final : public EntryProvider {
public:
    explicit FixedEntryProvider(std::vector<std::uint32_t> entries);
    std::vector<std::uint32_t> GetEntryPoints(std::size_t query_id) const override;
private:
    std::vector<std::uint32_t> entries_;
};
class PerQueryEntryProvider final : public EntryProvider {
public:
    explicit PerQueryEntryProvider(std::vector<std::vector<std::uint32_t>> entries_by_query);
    std::vector<std::uint32_t> GetEntryPoints(std::size_t query_id) const override;
private:
    std::vector<std::vector<std::uint32_t>> entries_by_query_;
};

// ---- candidates and the stop rule (reference: search_stop_condition.hpp) ---------------------------
struct RankedCandidate {
    float distance = 0.0f;
    std::uint32_t node_id = kInvalidNodeId;
    bool expanded = false;
    bool valid() const { return node_id != kInvalidNodeId; }
};
class SearchStopCondition {
public:
    static std::size_t CountValid(const std::vector<RankedCandidate>& candidates);
    static std::size_t BestUnexpandedRank(const std::vector<RankedCandidate>& candidates);
    static bool TopLHasNoBetterUnexpanded(const std::vector<RankedCandidate>& candidates, std::size_t top_l);
};

// ---- topology.bin (reference: topology_layout.hpp) -------------------------------------------------
struct TopologyHeader {
    char magic[8];
    std::uint32_t version, degree;
    std::uint64_t num_nodes, header_bytes, payload_bytes;
    std::uint8_t reserved[kDefaultPageSizeBytes - 40];
};
static_assert(sizeof(TopologyHeader) == kDefaultPageSizeBytes, "TopologyHeader must be exactly one 4KB page.");

struct TopologyDataset {
    std::uint64_t num_nodes = 0;
    std::uint32_t degree = kFixedTopologyDegree;
    std::vector<std::uint32_t> adjacency;
    std::size_t NodeBytes() const;
    const std::uint32_t* NodeNeighbors(std::uint64_t node_id) const;
};
class TopologyLayout {
public:
    static constexpr std::uint32_t kVersion = 1;
    static std::size_t NodeBytes();
    static std::uint64_t NodeOffsetBytes(std::uint64_t node_id);
    static TopologyHeader ReadHeader(const std::filesystem::path& path);
    static TopologyDataset MakePadded(std::uint64_t num_nodes,
                                      const std::vector<std::vector<std::uint32_t>>& adjacency_lists);
    // Same, with `degree` slots per node instead of 64 (compact records for degree-32 graphs).
    static TopologyDataset MakePaddedDegree(std::uint64_t num_nodes, std::uint32_t degree,
                                            const std::vector<std::vector<std::uint32_t>>& adjacency_lists);
    static void WriteFile(const std::filesystem::path& path, const TopologyDataset& dataset);
    static TopologyDataset ReadFile(const std::filesystem::path& path);
};

// ---- vectors.ssd (reference: vector_page_layout.hpp, vector_store_builder.hpp) ---------------------
struct VectorPageAddress {
    std::uint64_t page_id = 0;
    std::uint32_t slot_id = 0;
    std::uint64_t byte_offset = 0;
};
class VectorPageLayout {
public:
    static VectorPageLayout Create(std::uint32_t dim, ScalarKind scalar_kind,
                                   std::size_t page_size_bytes = kDefaultPageSizeBytes);
    static VectorPageLayout CreateFromVectorBytes(std::size_t vector_bytes,
                                                  std::size_t page_size_bytes = kDefaultPageSizeBytes);
    std::size_t page_size_bytes() const { return page_size_bytes_; }
    std::size_t header_bytes() const { return header_bytes_; }
    std::size_t vector_bytes() const { return vector_bytes_; }
    std::size_t vectors_per_page() const { return vectors_per_page_; }
    std::size_t payload_bytes_per_page() const { return payload_bytes_per_page_; }
    std::uint64_t PageCountForVectors(std::uint64_t num_vectors) const;
    VectorPageAddress Resolve(std::uint64_t node_id) const;
private:
    std::size_t page_size_bytes_ = kDefaultPageSizeBytes, header_bytes_ = kDefaultPageSizeBytes;
    std::size_t vector_bytes_ = 0, vectors_per_page_ = 0, payload_bytes_per_page_ = 0;
};
struct VectorStoreHeader {
    char magic[8];
    std::uint32_t version, scalar_kind, dim, reserved0;
    std::uint64_t num_vectors, page_size_bytes, vector_bytes, vectors_per_page;
    std::uint8_t reserved[kDefaultPageSizeBytes - 56];
};
static_assert(sizeof(VectorStoreHeader) == kDefaultPageSizeBytes, "VectorStoreHeader must be exactly one 4KB page.");
class VectorStoreBuilder {
public:
    static constexpr std::uint32_t kVersion = 1;
    static void WriteFile(const std::filesystem::path& path, const VectorPageLayout& layout, ScalarKind scalar_kind,
                          std::uint32_t dim, const std::vector<std::vector<std::uint8_t>>& vectors);
    static VectorStoreHeader ReadHeader(const std::filesystem::path& path);
    static std::vector<std::uint8_t> ReadVectorById(const std::filesystem::path& path, const VectorPageLayout& layout,
                                                    std::uint64_t node_id);
};

// ---- PQ index (reference: pq_index.hpp) -------------------------------------------------------------
constexpr std::size_t kPqMetadataSizeBytes = 4096;
constexpr std::size_t kNumPqBits = 8;
constexpr std::size_t kNumPqCentroids = 1ULL << kNumPqBits;

struct PqHostIndex {
    std::vector<std::uint8_t> codes;
    std::vector<float> tables_row_major, tables_col_major;
    std::vector<std::uint32_t> chunk_offsets;
    std::vector<float> centroid;
    std::uint64_t num_points = 0, ndims = 0, num_chunks = 0;
    bool codes_on_host = false;
};
struct PqDeviceIndex {
    CudaBuffer<std::uint8_t> codes;
    CudaBuffer<float> tables_col_major;
    CudaBuffer<std::uint32_t> chunk_offsets;
    CudaBuffer<float> centroid;
};
class PqIndex {
public:
    PqIndex() = default;
    ~PqIndex();
    PqIndex(PqIndex&& other) noexcept;
    PqIndex& operator=(PqIndex&& other) noexcept;
    PqIndex(const PqIndex&) = delete;
    PqIndex& operator=(const PqIndex&) = delete;
    static PqIndex LoadFromSeparatePaths(const std::filesystem::path& pivots_path,
                                         const std::filesystem::path& compressed_path);
    // Codes in pinned, device-mapped host memory (the reference's placement of pq2 codes).
    static PqIndex LoadFromSeparatePathsMapped(const std::filesystem::path& pivots_path,
                                               const std::filesystem::path& compressed_path);
    static PqIndex LoadPivotsOnly(const std::filesystem::path& pivots_path,
                                  const std::filesystem::path& compressed_path);
    const PqHostIndex& host() const { return host_; }
    const PqDeviceIndex& device() const { return device_; }
    const std::uint8_t* host_codes() const;
    const std::uint8_t* device_codes() const;
    bool codes_are_mapped() const { return mapped_device_codes_ != nullptr; }
    // Device copy of the row-major pivots (needed by the pq2 cross-term kernel).
    const CudaBuffer<float>& device_tables_row_major() const { return device_tables_row_major_; }
private:
    static PqIndex LoadImpl(const std::filesystem::path& pivots_path, const std::filesystem::path& compressed_path,
                            bool map_codes, bool load_codes);
    void Release() noexcept;
    PqHostIndex host_;
    PqDeviceIndex device_;
    CudaBuffer<float> device_tables_row_major_;
    std::uint8_t* mapped_host_codes_ = nullptr;
    std::uint8_t* mapped_device_codes_ = nullptr;
};

// ---- hybrid PQ index (reference: hpq_index.hpp) -------------------------------------------------------
// One hybrid code per chunk plus one selector bit per chunk that picks the base or the outlier codebook
// (include/topoanns/hpq_index.hpp:13-44, src/io/hpq_index.cpp). Codes and selector bits stay in pinned,
// device-mapped host memory as in the reference; tann_hpq_refine reads them from there or from HBM.
class HpqIndex {
public:
    HpqIndex() = default;
    ~HpqIndex();
    HpqIndex(HpqIndex&& other) noexcept;
    HpqIndex& operator=(HpqIndex&& other) noexcept;
    HpqIndex(const HpqIndex&) = delete;
    HpqIndex& operator=(const HpqIndex&) = delete;
    static HpqIndex Load(const std::filesystem::path& base_pivots_path, const std::filesystem::path& outlier_pivots_path,
                         const std::filesystem::path& hybrid_codes_path, const std::filesystem::path& selector_bits_path);
    const PqIndex& base_index() const { return base_index_; }
    const PqIndex& outlier_index() const { return outlier_index_; }
    std::size_t selector_stride_bytes() const { return selector_stride_bytes_; }
    const std::uint8_t* device_selector_bits() const { return mapped_device_selector_bits_; }
private:
    void Release() noexcept;
    PqIndex base_index_, outlier_index_;
    std::size_t selector_stride_bytes_ = 0;
    std::uint8_t* mapped_host_selector_bits_ = nullptr;
    std::uint8_t* mapped_device_selector_bits_ = nullptr;
};

// ---- query tables and the distance oracle (reference: pq_query_tables.hpp, pq_distance_oracle.hpp) --
struct PqQueryTablesProfile {
    double total_ms = 0.0, query_upload_ms = 0.0, zero_fill_ms = 0.0, kernel_ms = 0.0, table_download_ms = 0.0;
};
class PqQueryDistanceTables {
public:
    PqQueryDistanceTables() = default;
    PqQueryDistanceTables(PqQueryDistanceTables&&) noexcept = default;
    PqQueryDistanceTables& operator=(PqQueryDistanceTables&&) noexcept = default;
    PqQueryDistanceTables(const PqQueryDistanceTables&) = delete;
    PqQueryDistanceTables& operator=(const PqQueryDistanceTables&) = delete;
    static PqQueryDistanceTables FromFloatQueries(const PqIndex& pq_index, const std::vector<float>& queries,
                                                  std::size_t num_queries);
    static PqQueryDistanceTables FromFloatQueriesDeviceOnly(const PqIndex& pq_index, const std::vector<float>& queries,
                                                            std::size_t num_queries);
    static PqQueryDistanceTables FromFloatQueriesDeviceBufferAsync(const PqIndex& pq_index,
                                                                   const CudaBuffer<float>& device_queries,
                                                                   std::size_t num_queries, cudaStream_t stream);
    static PqQueryDistanceTables FromUint8Queries(const PqIndex& pq_index, const std::vector<std::uint8_t>& queries,
                                                  std::size_t num_queries);
    static PqQueryDistanceTables FromInt8Queries(const PqIndex& pq_index, const std::vector<std::int8_t>& queries,
                                                 std::size_t num_queries);
    std::size_t num_queries() const { return num_queries_; }
    std::size_t num_chunks() const { return num_chunks_; }
    bool has_host_tables() const { return host_tables_materialized_; }
    const std::vector<float>& host_tables() const { return host_tables_; }
    const CudaBuffer<float>& device_tables() const { return device_tables_; }
    const PqQueryTablesProfile& profile() const { return profile_; }
    float Lookup(std::size_t query_id, std::size_t chunk_id, std::uint32_t centroid_id) const;
    float Distance(std::size_t query_id, std::uint32_t node_id, const PqIndex& pq_index) const;
private:
    static PqQueryDistanceTables Build(const PqIndex& pq_index, const void* host_queries, std::uint32_t kind,
                                       std::size_t element_count, std::size_t num_queries, bool materialize,
                                       const char* context);
    std::size_t num_queries_ = 0, num_chunks_ = 0;
    bool host_tables_materialized_ = false;
    std::vector<float> host_tables_;
    CudaBuffer<float> device_tables_;
    PqQueryTablesProfile profile_;
};

class SearchResources;

class PqDistanceOracle final {
public:
    PqDistanceOracle(const PqIndex& pq_index, PqQueryDistanceTables query_tables);
    static PqDistanceOracle FromFloatQueries(const PqIndex& pq_index, const std::vector<float>& queries, std::size_t n);
    static PqDistanceOracle FromFloatQueriesDeviceOnly(const PqIndex& pq_index, const std::vector<float>& queries,
                                                       std::size_t n);
    static PqDistanceOracle FromFloatQueries(const SearchResources& resources, const std::vector<float>& queries,
                                             std::size_t n);
    static PqDistanceOracle FromFloatQueriesDeviceOnly(const SearchResources& resources,
                                                       const std::vector<float>& queries, std::size_t n);
    static PqDistanceOracle FromUint8Queries(const PqIndex& pq_index, const std::vector<std::uint8_t>& queries,
                                             std::size_t n);
    static PqDistanceOracle FromUint8Queries(const SearchResources& resources,
                                             const std::vector<std::uint8_t>& queries, std::size_t n);
    static PqDistanceOracle FromInt8Queries(const PqIndex& pq_index, const std::vector<std::int8_t>& queries,
                                            std::size_t n);
    static PqDistanceOracle FromInt8Queries(const SearchResources& resources, const std::vector<std::int8_t>& queries,
                                            std::size_t n);
    float Distance(std::size_t query_id, std::uint32_t node_id) const;
    std::size_t num_queries() const { return query_tables_.num_queries(); }
    const PqIndex& pq_index() const;
    const PqQueryDistanceTables& query_tables() const { return query_tables_; }
private:
    const PqIndex* pq_index_ = nullptr;  // must outlive the oracle
    PqQueryDistanceTables query_tables_;
};

// ---- topology in memory (reference: pinned_topology.hpp) ---------------------------------------------
// The adjacency is kept twice: in pinned host memory (host_data(), also reachable from the GPU over
// UVA) and, unless the host tier is selected, in HBM. device_data() is the pointer the kernels use.
enum class TopologyResidency { kHbm, kPinnedHost };

class PinnedTopology {
public:
    PinnedTopology() = default;
    ~PinnedTopology();
    PinnedTopology(const PinnedTopology&) = delete;
    PinnedTopology& operator=(const PinnedTopology&) = delete;
    PinnedTopology(PinnedTopology&& other) noexcept;
    PinnedTopology& operator=(PinnedTopology&& other) noexcept;
    static PinnedTopology FromDataset(const TopologyDataset& dataset);
    static PinnedTopology FromFile(const std::filesystem::path& path);
    static PinnedTopology FromRaw(std::uint64_t num_nodes, std::uint32_t degree,
                                  const std::vector<std::uint32_t>& adjacency);
    std::uint64_t num_nodes() const { return num_nodes_; }
    std::uint32_t degree() const { return degree_; }
    const std::uint32_t* host_data() const { return host_data_; }
    const std::uint32_t* device_data() const { return hbm_data_ != nullptr ? hbm_data_ : mapped_data_; }
    const std::uint32_t* mapped_host_device_pointer() const { return mapped_data_; }
    const std::uint32_t* hbm_data() const { return hbm_data_; }
    // Drops or (re)creates the HBM copy; with kPinnedHost the first `cached_rows` rows stay in HBM.
    void SetResidency(TopologyResidency residency, std::uint64_t cached_rows = 0);
    TopologyResidency residency() const { return residency_; }
    std::uint64_t cached_rows() const { return cached_rows_; }
    std::vector<std::uint32_t> ReadHostNode(std::uint64_t node_id) const;
    std::vector<std::uint32_t> CopyNodeFromDevice(std::uint64_t node_id) const;
private:
    void Release() noexcept;
    std::uint32_t* host_data_ = nullptr;
    std::uint32_t* mapped_data_ = nullptr;
    std::uint32_t* hbm_data_ = nullptr;
    std::uint64_t num_nodes_ = 0, cached_rows_ = 0;
    std::uint32_t degree_ = 0;
    std::size_t element_count_ = 0;
    TopologyResidency residency_ = TopologyResidency::kHbm;
};

// ---- providers (reference: vector_page_provider.hpp) -------------------------------------------------
struct DevicePageReadResult {
    CudaBuffer<std::uint8_t> page_bytes;
    double io_ms = 0.0;
};
class VectorPageProvider {
public:
    virtual ~VectorPageProvider() = default;
    virtual bool SupportsDeviceReads() const { return false; }
    // In this library: a `const TannShards*` describing where the pages live (never a BaM handle).
    virtual const void* DeviceReadHandle() const { return nullptr; }
    virtual std::vector<std::uint8_t> ReadPages(const std::filesystem::path& path,
                                                const std::vector<std::uint64_t>& page_ids, std::size_t header_bytes,
                                                std::size_t page_size_bytes) const = 0;
    virtual DevicePageReadResult ReadPagesToDevice(const std::filesystem::path& path,
                                                   const std::vector<std::uint64_t>& page_ids,
                                                   std::size_t header_bytes, std::size_t page_size_bytes) const;
    virtual DevicePageReadResult ReadPagesToDevice(const std::filesystem::path& path,
                                                   const CudaBuffer<std::uint64_t>& page_ids, std::size_t num_pages,
                                                   std::size_t header_bytes, std::size_t page_size_bytes) const;
};

// All pages of one vectors.ssd file resident in HBM.
class HbmVectorPageProvider final : public VectorPageProvider {
public:
    explicit HbmVectorPageProvider(const std::filesystem::path& vector_store_path);
    bool SupportsDeviceReads() const override { return true; }
    const void* DeviceReadHandle() const override { return &shards_; }
    std::vector<std::uint8_t> ReadPages(const std::filesystem::path&, const std::vector<std::uint64_t>& page_ids,
                                        std::size_t header_bytes, std::size_t page_size_bytes) const override;
    DevicePageReadResult ReadPagesToDevice(const std::filesystem::path&, const std::vector<std::uint64_t>& page_ids,
                                           std::size_t header_bytes, std::size_t page_size_bytes) const override;
private:
    CudaBuffer<std::uint8_t> pages_;
    std::vector<std::uint8_t> host_pages_;
    TannShards shards_{};
};

// All pages in pinned, device-mapped host memory: the tier that stands in for the SSD.
class PinnedHostVectorPageProvider final : public VectorPageProvider {
public:
    explicit PinnedHostVectorPageProvider(const std::filesystem::path& vector_store_path);
    ~PinnedHostVectorPageProvider() override;
    bool SupportsDeviceReads() const override { return true; }
    const void* DeviceReadHandle() const override { return &shards_; }
    std::vector<std::uint8_t> ReadPages(const std::filesystem::path&, const std::vector<std::uint64_t>& page_ids,
                                        std::size_t header_bytes, std::size_t page_size_bytes) const override;
    DevicePageReadResult ReadPagesToDevice(const std::filesystem::path&, const std::vector<std::uint64_t>& page_ids,
                                           std::size_t header_bytes, std::size_t page_size_bytes) const override;
private:
    std::uint8_t* host_ = nullptr;
    std::uint8_t* mapped_ = nullptr;
    std::size_t bytes_ = 0;
    TannShards shards_{};
};

// Pages split by node-id range over the GPUs of one box; `shards` holds peer-mapped base pointers.
class PeerVectorPageProvider final : public VectorPageProvider {
public:
    explicit PeerVectorPageProvider(const TannShards& shards) : shards_(shards) {}
    bool SupportsDeviceReads() const override { return true; }
    const void* DeviceReadHandle() const override { return &shards_; }
    std::vector<std::uint8_t> ReadPages(const std::filesystem::path&, const std::vector<std::uint64_t>&, std::size_t,
                                        std::size_t) const override;
private:
    TannShards shards_{};
};

// ---- SearchResources (reference: search_resources.hpp) -------------------------------------------------
enum class Pq2ErrorBoundStorage { kNone = 0, kFloat32 = 1 };

class SearchResources {
public:
    SearchResources() = default;
    static SearchResources FromDataset(const TopologyDataset& dataset);
    static SearchResources FromTopologyFile(const std::filesystem::path& path);

    std::uint64_t num_nodes() const;
    std::uint32_t degree() const;
    const PinnedTopology& topology() const { return *topology_; }
    PinnedTopology& mutable_topology() { return *topology_; }
    const std::uint32_t* host_topology_data() const { return topology_->host_data(); }
    const std::uint32_t* device_topology_data() const { return topology_->device_data(); }
    std::vector<std::uint32_t> ReadHostNeighbors(std::uint64_t node_id) const;

    void LoadPqIndex(const std::filesystem::path& pivots_path, const std::filesystem::path& compressed_path);
    bool has_pq_index() const { return static_cast<bool>(pq_index_); }
    const PqIndex& pq_index() const;
    void LoadPq2Index(const std::filesystem::path& pivots_path, const std::filesystem::path& compressed_path,
                      const std::filesystem::path& error_bounds_path = {});
    bool has_pq2_index() const { return static_cast<bool>(pq2_index_); }
    const PqIndex& pq2_index() const;
    bool pq2_is_residual_refine() const;
    bool has_pq2_error_bounds() const;
    Pq2ErrorBoundStorage pq2_error_bound_storage() const;
    const CudaBuffer<float>& pq2_cross_terms() const;
    const CudaBuffer<float>& pq2_error_bounds_fp32() const;

    // include/topoanns/search_resources.hpp:52-57
    void LoadHpqIndex(const std::filesystem::path& base_pivots_path, const std::filesystem::path& outlier_pivots_path,
                      const std::filesystem::path& hybrid_codes_path, const std::filesystem::path& selector_bits_path);
    bool has_hpq_index() const { return static_cast<bool>(hpq_index_); }
    const HpqIndex& hpq_index() const;

    void LoadVectorStore(const std::filesystem::path& path);
    bool has_vector_store() const { return static_cast<bool>(vector_store_); }
    const VectorStoreHeader& vector_store_header() const;
    const VectorPageLayout& vector_store_layout() const;
    const std::filesystem::path& vector_store_path() const;
    void AttachVectorPageProvider(std::shared_ptr<VectorPageProvider> provider);
    void ClearVectorPageProvider();
    const VectorPageProvider& vector_page_provider() const;
    void AttachTopologyPageProvider(std::shared_ptr<VectorPageProvider> provider);
    void ClearTopologyPageProvider();
    bool has_topology_page_provider() const { return static_cast<bool>(topology_page_provider_); }
    const VectorPageProvider& topology_page_provider() const;
    const void* topology_device_read_handle() const;

    // Node-id-range sharding over peers: replaces the local adjacency / code arrays as the kernels'
    // source (vectors are sharded through a PeerVectorPageProvider).
    void AttachTopologyShards(const TannShards& adjacency);
    void AttachPqCodeShards(const TannShards& codes);

    // Optional HBM layout with every node's neighbours' PQ codes next to each other (degree * M bytes per
    // node): an expansion then reads adjacency ids and neighbour codes in one memory round trip. Results do
    // not change. Needs the topology in HBM and the PQ index loaded; call again after either changes.
    void BuildNeighborCodeLayout();
    void DropNeighborCodeLayout() { neighbor_codes_.reset(); }
    bool has_neighbor_code_layout() const { return static_cast<bool>(neighbor_codes_); }

    // The view the C ABI takes; `need_vectors` also resolves the attached provider's pages.
    TannIndexView MakeIndexView(bool need_vectors) const;

private:
    struct Pq2Aux {
        bool residual_refine = false;
        Pq2ErrorBoundStorage storage = Pq2ErrorBoundStorage::kNone;
        CudaBuffer<float> cross_terms, error_bounds_fp32;
    };
    struct VectorStore {
        std::filesystem::path path;
        VectorStoreHeader header{};
        VectorPageLayout layout;
        std::shared_ptr<VectorPageProvider> provider;
    };
    std::shared_ptr<PinnedTopology> topology_ = std::make_shared<PinnedTopology>();
    std::shared_ptr<VectorPageProvider> topology_page_provider_;
    std::shared_ptr<PqIndex> pq_index_, pq2_index_;
    std::shared_ptr<HpqIndex> hpq_index_;
    std::shared_ptr<Pq2Aux> pq2_aux_;
    std::shared_ptr<VectorStore> vector_store_;
    bool has_adjacency_shards_ = false, has_code_shards_ = false;
    TannShards adjacency_shards_{}, code_shards_{};
    std::shared_ptr<CudaBuffer<std::uint8_t>> neighbor_codes_;
};

// ---- traversal (reference: topology_search.hpp) ---------------------------------------------------------
struct TopologySearchParams {
    std::size_t top_k = 10;
    std::size_t top_l = 32;
    std::size_t candidate_queue_size = 0;
    std::size_t search_width = 1;
    std::size_t max_expansions = 1024;
    std::uint64_t topology_cached_node_count = std::numeric_limits<std::uint64_t>::max();
    // Fields of the SSD exact-reuse cache; accepted and ignored (that cache is tied to the NVMe tier).
    bool enable_exact_reuse = false;
    const float* exact_reuse_device_queries = nullptr;
    std::size_t exact_reuse_query_dim = 0;
    std::uint32_t combined_node_bytes = 0, combined_nodes_per_page = 0;
    std::size_t exact_reuse_cache_capacity = 0;
    bool enable_occupancy_profile = false;
    bool enable_expanded_trace = false;
};
struct TopologySearchStats {
    std::size_t visited_nodes = 0, expanded_nodes = 0, topology_io_pages = 0, iterations = 0;
};
struct TopologySearchBatchProfile {
    double kernel_ms = 0.0, candidate_download_ms = 0.0, stats_download_ms = 0.0, host_postprocess_ms = 0.0;
    double candidate_materialize_ms = 0.0, topology_topk_extract_ms = 0.0;
    // Per-stage sums of in-kernel cycle counters in the reference; this kernel does not instrument itself,
    // so these stay zero (per-kernel figures come from the profiler instead).
    double sum_query_pq_distance_ms = 0.0, sum_query_pq_compute_ms = 0.0, sum_query_pq_prefetch_issue_ms = 0.0;
    double sum_query_pq_prefetch_wait_ms = 0.0, sum_query_pq_checksum_ms = 0.0, sum_query_queue_update_ms = 0.0;
    double sum_query_queue_scan_ms = 0.0, sum_query_queue_select_ms = 0.0, sum_query_frontier_sort_ms = 0.0;
    double sum_query_tail_merge_ms = 0.0, sum_query_candidate_sort_ms = 0.0;
    double sum_query_candidate_sort_before_full_prefix_ms = 0.0, sum_query_candidate_sort_after_full_prefix_ms = 0.0;
    double sum_query_hash_rebuild_ms = 0.0, sum_query_learned_stop_model_ms = 0.0;
    double sum_query_learned_stop_feature_ms = 0.0, sum_query_learned_stop_find_first_set_ms = 0.0;
    double sum_query_learned_stop_count_bits_ms = 0.0, sum_query_learned_stop_topk_churn_ms = 0.0;
    double sum_query_learned_stop_logit_eval_ms = 0.0, sum_query_combined_node_read_ms = 0.0;
    double sum_query_exact_reuse_insert_ms = 0.0;
    std::uint64_t batch_max_pq_cycles = 0, batch_max_queue_cycles = 0;
    double batch_avg_iterations = 0.0;
    std::size_t batch_p50_iterations = 0, batch_p95_iterations = 0, batch_max_iterations = 0;
    std::size_t batch_full_prefix_reached_queries = 0;
    double batch_avg_full_prefix_iteration = 0.0;
    std::size_t batch_p50_full_prefix_iteration = 0, batch_p95_full_prefix_iteration = 0;
    std::size_t batch_max_full_prefix_iteration = 0, batch_max_expanded_nodes = 0, batch_p95_expanded_nodes = 0;
};
struct TopologySearchResult {
    std::vector<RankedCandidate> sorted_candidates;
    std::vector<RankedCandidate> topk;
    TopologySearchStats stats;
};
class TopologySearch {
public:
    static TopologySearchResult Run(const SearchResources& resources, const EntryProvider& entry_provider,
                                    const PqDistanceOracle& distance_oracle, std::size_t query_id,
                                    const TopologySearchParams& params,
                                    TopologySearchBatchProfile* out_profile = nullptr);
    static std::vector<TopologySearchResult> RunBatch(const SearchResources& resources,
                                                      const EntryProvider& entry_provider,
                                                      const PqDistanceOracle& distance_oracle,
                                                      const TopologySearchParams& params,
                                                      TopologySearchBatchProfile* out_profile = nullptr);
    static std::vector<TopologySearchResult> RunBatch(const SearchResources& resources,
                                                      const DeviceEntryBatch& entry_batch,
                                                      const PqDistanceOracle& distance_oracle,
                                                      const TopologySearchParams& params,
                                                      TopologySearchBatchProfile* out_profile = nullptr);
};

// Hybrid-PQ refine of a traversal's candidate lists (the reference keeps this step in its private header
// src/search/fused_rerank_device.hpp:63 as detail::RunHpqRefineBatchDevice and reaches it from its overlap
// pipeline tool only): the traversal runs on the device, the first refine_top_l candidates of every query are
// re-scored with the hybrid codes of resources.hpq_index() and re-sorted by (distance, id).
class HpqRefine {
public:
    static std::vector<std::vector<RankedCandidate>> RunBatchFloat32(const SearchResources& resources,
                                                                    const DeviceEntryBatch& entry_batch,
                                                                    const std::vector<float>& queries,
                                                                    std::size_t num_queries,
                                                                    const TopologySearchParams& topology_params,
                                                                    std::size_t refine_top_l);
};

// ---- rerank (reference: rerank_exact.hpp) -----------------------------------------------------------------
enum class RerankExecutionMode { kLinear, kTiled, kPageByPage, kPersistent };

struct RerankExactParams {
    std::size_t top_k = 10;
    std::size_t top_n = 100;
    RerankExecutionMode mode = RerankExecutionMode::kPersistent;
    std::size_t rank_tile_size = 16;
    bool use_pq2_refine = false;
    bool use_pq2_bound_filter = false;
    std::size_t pq2_refine_top_l = 0;
    bool use_early_stop = false;
    std::size_t early_stop_min_prefix = 32;
    std::size_t early_stop_patience_tiles = 1;
    bool use_learned_stop = false;
    std::filesystem::path learned_stop_model_path;
    std::size_t ssd_records_per_page = 0;
    std::size_t ssd_record_stride_bytes = 0;
};
struct RerankQueryResult {
    std::vector<RankedCandidate> sorted_candidates;
    std::vector<RankedCandidate> topk;
};
struct RerankBatchStats {
    std::size_t io_pages = 0, exact_distance_count = 0, bound_filtered_count = 0;
};
struct RerankBatchProfile {
    double total_ms = 0.0, pq2_query_tables_ms = 0.0, pq2_query_upload_ms = 0.0, pq2_query_zero_fill_ms = 0.0;
    double pq2_query_table_kernel_ms = 0.0, pq2_query_table_download_ms = 0.0, pq2_refine_kernel_ms = 0.0;
    double pq2_bound_filter_ms = 0.0, pq2_threshold_update_ms = 0.0, learned_stop_model_ms = 0.0;
    double learned_stop_checkpoint_bookkeeping_ms = 0.0, learned_stop_topk_churn_ms = 0.0;
    double learned_stop_next_window_scan_ms = 0.0, learned_stop_logit_eval_ms = 0.0, rerank_query_block_ms = 0.0;
    double query_upload_ms = 0.0, prepare_ms = 0.0, io_ms = 0.0, unpack_ms = 0.0, exact_distance_total_ms = 0.0;
    double exact_distance_kernel_ms = 0.0, sort_ms = 0.0, result_download_ms = 0.0, rerank_topk_extract_ms = 0.0;
    double sorted_candidates_materialize_ms = 0.0;
    std::size_t pq2_refine_input_candidates = 0, pq2_refine_input_candidates_min = 0;
    std::size_t pq2_refine_input_candidates_max = 0, pq2_refine_top_l = 0, requested_top_n = 0, effective_top_n = 0;
    std::size_t exact_candidates = 0, bound_filtered_candidates = 0, rerank_batches = 0, pq2_refine_batches = 0;
    std::size_t rerank_tile_size = 0, rerank_prepare_valid_candidates = 0, rerank_prepare_valid_candidates_min = 0;
    std::size_t rerank_prepare_valid_candidates_max = 0, rerank_prepare_filtered_candidates = 0;
    std::size_t rerank_prepare_filtered_candidates_min = 0, rerank_prepare_filtered_candidates_max = 0;
    std::size_t rerank_prepare_nonzero_tiles = 0, rerank_prepare_zero_tiles = 0, pq2_residual_refine_batches = 0;
    std::size_t rerank_bam_direct_batches = 0, rerank_gpu_sort_batches = 0, rerank_host_sort_batches = 0;
    std::size_t learned_stop_checkpoints = 0, learned_stop_queries = 0, learned_stop_prefix_sum = 0;
    std::size_t learned_stop_prefix_min = 0, learned_stop_prefix_max = 0;
};
struct RerankBatchResult {
    std::vector<RerankQueryResult> queries;
    RerankBatchStats stats;
    RerankBatchProfile profile;
};
class RerankExact {
public:
    static RerankBatchResult RunBatchFloat32(const SearchResources& resources,
                                             const std::vector<TopologySearchResult>& topology_results,
                                             const std::vector<float>& queries, std::size_t num_queries,
                                             const RerankExactParams& params, RerankBatchProfile* out_profile = nullptr);
    static RerankBatchResult RunBatchUint8(const SearchResources& resources,
                                           const std::vector<TopologySearchResult>& topology_results,
                                           const std::vector<std::uint8_t>& queries, std::size_t num_queries,
                                           const RerankExactParams& params, RerankBatchProfile* out_profile = nullptr);
    static RerankBatchResult RunBatchInt8(const SearchResources& resources,
                                          const std::vector<TopologySearchResult>& topology_results,
                                          const std::vector<std::int8_t>& queries, std::size_t num_queries,
                                          const RerankExactParams& params, RerankBatchProfile* out_profile = nullptr);
};

// ---- whole path (reference: topoanns_search.hpp) ---------------------------------------------------------
struct TopoAnnsSearchParams {
    TopologySearchParams topology;
    RerankExactParams rerank;
};
struct TopoAnnsQueryResult {
    TopologySearchResult topology;
    RerankQueryResult rerank;
};
struct TopoAnnsBatchResult {
    std::vector<TopoAnnsQueryResult> queries;
    RerankBatchStats rerank_stats;
    PqQueryTablesProfile pq_profile;
    TopologySearchBatchProfile topology_profile;
    RerankBatchProfile rerank_profile;
};
class TopoAnnsSearch final {
public:
    static TopoAnnsBatchResult RunBatchFloat32(const SearchResources& resources, const EntryProvider& entry_provider,
                                               const std::vector<float>& queries, std::size_t num_queries,
                                               const TopoAnnsSearchParams& params);
    static TopoAnnsBatchResult RunBatchFloat32(const SearchResources& resources, const DeviceEntryBatch& entry_batch,
                                               const std::vector<float>& queries, std::size_t num_queries,
                                               const TopoAnnsSearchParams& params);
    static TopoAnnsBatchResult RunBatchFloat32Fused(const SearchResources& resources,
                                                    const DeviceEntryBatch& entry_batch,
                                                    const std::vector<float>& queries, std::size_t num_queries,
                                                    const TopoAnnsSearchParams& params);
    static std::vector<TopoAnnsBatchResult> RunBatchFloat32FusedRerankSweep(
        const SearchResources& resources, const DeviceEntryBatch& entry_batch, const std::vector<float>& queries,
        std::size_t num_queries, const TopologySearchParams& topology_params,
        const std::vector<RerankExactParams>& rerank_params_list);
    static TopoAnnsBatchResult RunBatchUint8(const SearchResources& resources, const EntryProvider& entry_provider,
                                             const std::vector<std::uint8_t>& queries, std::size_t num_queries,
                                             const TopoAnnsSearchParams& params);
    static TopoAnnsBatchResult RunBatchInt8(const SearchResources& resources, const EntryProvider& entry_provider,
                                            const std::vector<std::int8_t>& queries, std::size_t num_queries,
                                            const TopoAnnsSearchParams& params);
};

// ---- RVQ entries (reference: rvq_entry_provider.hpp) ------------------------------------------------------
struct RvqEntryProfile {
    double total_ms = 0.0, query_upload_ms = 0.0, search_kernel_ms = 0.0, entry_gather_ms = 0.0;
};
class RvqModel {
public:
    RvqModel();
    ~RvqModel();
    RvqModel(RvqModel&&) noexcept;
    RvqModel& operator=(RvqModel&&) noexcept;
    RvqModel(const RvqModel&) = delete;
    RvqModel& operator=(const RvqModel&) = delete;
    static RvqModel Load(const std::filesystem::path& model_path);
    std::uint32_t dim() const;
    std::uint32_t coarse_centroids() const;
    std::uint32_t fine_centroids() const;
    void WarmUp() const;
    std::vector<std::vector<std::uint32_t>> ComputeFloat32EntryPoints(const std::vector<float>& queries,
                                                                      std::size_t num_queries, std::size_t entry_count,
                                                                      std::uint32_t fallback_entry = 0,
                                                                      RvqEntryProfile* out_profile = nullptr) const;
    DeviceEntryBatch ComputeFloat32DeviceEntryBatch(const std::vector<float>& queries, std::size_t num_queries,
                                                    std::size_t entry_count, std::uint32_t fallback_entry = 0,
                                                    RvqEntryProfile* out_profile = nullptr) const;
private:
    struct Impl;
    explicit RvqModel(std::unique_ptr<Impl> impl);
    std::unique_ptr<Impl> impl_;
};
class RvqEntryProvider final : public EntryProvider {
public:
    explicit RvqEntryProvider(std::vector<std::vector<std::uint32_t>> entries_by_query);
    static RvqEntryProvider FromFloatQueries(const RvqModel& model, const std::vector<float>& queries,
                                             std::size_t num_queries, std::size_t entry_count,
                                             std::uint32_t fallback_entry = 0, RvqEntryProfile* out_profile = nullptr);
    std::vector<std::uint32_t> GetEntryPoints(std::size_t query_id) const override;
    std::size_t num_queries() const { return entries_by_query_.size(); }
private:
    std::vector<std::vector<std::uint32_t>> entries_by_query_;
};

}  // namespace topoanns
