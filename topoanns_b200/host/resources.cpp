// Index resources on the device: topology (pinned host + HBM), PQ indices, the three page providers
// and SearchResources. Loading facts follow the reference (src/providers/pinned_topology.cu,
// src/io/pq_index.cpp, src/search/search_resources.cpp); the placement is new: adjacency and codes
// default to HBM, and the BaM provider is replaced by HBM / pinned-host / peer providers.
#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <fstream>

#include "topoanns/api.hpp"

namespace topoanns {
namespace {

template <typename T>
struct BinBlock {
    std::size_t rows = 0, cols = 0;
    std::vector<T> data;
};

// DiskANN "bin" block: {int32 rows, int32 cols, rows*cols values} at a byte offset.
template <typename T>
BinBlock<T> ReadBinBlock(const std::filesystem::path& path, std::size_t offset, const char* context) {
    std::ifstream in(path, std::ios::binary);
    if (!in.is_open()) throw std::runtime_error(BuildErrorMessage(context, "Failed to open " + path.string()));
    in.seekg(static_cast<std::streamoff>(offset), std::ios::beg);
    std::int32_t r = 0, c = 0;
    in.read(reinterpret_cast<char*>(&r), 4);
    in.read(reinterpret_cast<char*>(&c), 4);
    if (!in.good() || r < 0 || c < 0) throw std::runtime_error(BuildErrorMessage(context, "Invalid bin metadata in " + path.string()));
    BinBlock<T> b;
    b.rows = static_cast<std::size_t>(r);
    b.cols = static_cast<std::size_t>(c);
    b.data.resize(b.rows * b.cols);
    if (!b.data.empty()) {
        in.read(reinterpret_cast<char*>(b.data.data()), static_cast<std::streamsize>(b.data.size() * sizeof(T)));
        if (!in.good()) throw std::runtime_error(BuildErrorMessage(context, "Short read in " + path.string()));
    }
    return b;
}

std::vector<std::uint8_t> ReadFileRange(const std::filesystem::path& path, std::uint64_t offset, std::uint64_t bytes,
                                        const char* context) {
    std::vector<std::uint8_t> out(bytes);
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) throw std::runtime_error(BuildErrorMessage(context, "Failed to open " + path.string()));
    std::uint64_t done = 0;
    while (done < bytes) {
        const ssize_t n = pread(fd, out.data() + done, bytes - done, static_cast<off_t>(offset + done));
        if (n <= 0) {
            close(fd);
            throw std::runtime_error(BuildErrorMessage(context, "Unexpected EOF in " + path.string()));
        }
        done += static_cast<std::uint64_t>(n);
    }
    close(fd);
    return out;
}

TannShards OneShard(const void* base) {
    TannShards s{};
    s.num_shards = 1;
    s.base[0] = base;
    return s;
}

std::vector<std::uint8_t> GatherHostPages(const std::uint8_t* pages, std::size_t total_bytes,
                                          const std::vector<std::uint64_t>& page_ids, std::size_t page_size,
                                          const char* context) {
    std::vector<std::uint8_t> out(page_ids.size() * page_size);
    for (std::size_t i = 0; i < page_ids.size(); ++i) {
        const std::uint64_t off = page_ids[i] * page_size;
        if (off + page_size > total_bytes) throw std::runtime_error(BuildErrorMessage(context, "page id is out of range."));
        std::memcpy(out.data() + i * page_size, pages + off, page_size);
    }
    return out;
}

}  // namespace

// ---- PinnedTopology ---------------------------------------------------------------------------------------
PinnedTopology::~PinnedTopology() { Release(); }
PinnedTopology::PinnedTopology(PinnedTopology&& o) noexcept { *this = std::move(o); }
PinnedTopology& PinnedTopology::operator=(PinnedTopology&& o) noexcept {
    if (this == &o) return *this;
    Release();
    host_data_ = o.host_data_; mapped_data_ = o.mapped_data_; hbm_data_ = o.hbm_data_;
    num_nodes_ = o.num_nodes_; cached_rows_ = o.cached_rows_; degree_ = o.degree_;
    element_count_ = o.element_count_; residency_ = o.residency_;
    o.host_data_ = o.mapped_data_ = o.hbm_data_ = nullptr;
    o.num_nodes_ = o.cached_rows_ = 0; o.degree_ = 0; o.element_count_ = 0;
    return *this;
}
void PinnedTopology::Release() noexcept {
    if (hbm_data_ != nullptr) cudaFree(hbm_data_);
    if (host_data_ != nullptr) cudaFreeHost(host_data_);
    host_data_ = mapped_data_ = hbm_data_ = nullptr;
    num_nodes_ = cached_rows_ = 0;
    degree_ = 0;
    element_count_ = 0;
}
PinnedTopology PinnedTopology::FromRaw(std::uint64_t num_nodes, std::uint32_t degree,
                                       const std::vector<std::uint32_t>& adjacency) {
    if (adjacency.size() != static_cast<std::size_t>(num_nodes) * degree)
        throw std::runtime_error(BuildErrorMessage("PinnedTopology::FromRaw", "Adjacency vector size does not match num_nodes * degree."));
    PinnedTopology t;
    t.num_nodes_ = num_nodes;
    t.degree_ = degree;
    t.element_count_ = adjacency.size();
    if (t.element_count_ == 0) return t;
    const std::size_t bytes = t.element_count_ * sizeof(std::uint32_t);
    ThrowIfCudaError(cudaHostAlloc(reinterpret_cast<void**>(&t.host_data_), bytes, cudaHostAllocMapped | cudaHostAllocPortable),
                     "cudaMallocHost");
    std::memcpy(t.host_data_, adjacency.data(), bytes);
    ThrowIfCudaError(cudaHostGetDevicePointer(reinterpret_cast<void**>(&t.mapped_data_), t.host_data_, 0),
                     "cudaHostGetDevicePointer");
    t.SetResidency(TopologyResidency::kHbm);
    return t;
}
PinnedTopology PinnedTopology::FromDataset(const TopologyDataset& d) { return FromRaw(d.num_nodes, d.degree, d.adjacency); }
PinnedTopology PinnedTopology::FromFile(const std::filesystem::path& path) {
    const TopologyDataset d = TopologyLayout::ReadFile(path);
    return FromRaw(d.num_nodes, d.degree, d.adjacency);
}
void PinnedTopology::SetResidency(TopologyResidency residency, std::uint64_t cached_rows) {
    if (hbm_data_ != nullptr) {
        cudaFree(hbm_data_);
        hbm_data_ = nullptr;
    }
    residency_ = residency;
    cached_rows_ = 0;
    if (element_count_ == 0) return;
    const std::uint64_t rows = residency == TopologyResidency::kHbm ? num_nodes_ : std::min(cached_rows, num_nodes_);
    if (rows == 0) return;
    const std::size_t bytes = static_cast<std::size_t>(rows) * degree_ * sizeof(std::uint32_t);
    ThrowIfCudaError(cudaMalloc(reinterpret_cast<void**>(&hbm_data_), bytes), "cudaMalloc");
    ThrowIfCudaError(cudaMemcpy(hbm_data_, host_data_, bytes, cudaMemcpyHostToDevice), "cudaMemcpyHostToDevice");
    cached_rows_ = residency == TopologyResidency::kHbm ? 0 : rows;
}
std::vector<std::uint32_t> PinnedTopology::ReadHostNode(std::uint64_t node_id) const {
    if (node_id >= num_nodes_) throw std::runtime_error(BuildErrorMessage("PinnedTopology::ReadHostNode", "node_id is out of range."));
    const std::uint32_t* row = host_data_ + node_id * degree_;
    return std::vector<std::uint32_t>(row, row + degree_);
}
std::vector<std::uint32_t> PinnedTopology::CopyNodeFromDevice(std::uint64_t node_id) const {
    if (node_id >= num_nodes_) throw std::runtime_error(BuildErrorMessage("PinnedTopology::CopyNodeFromDevice", "node_id is out of range."));
    std::vector<std::uint32_t> row(degree_);
    const bool in_hbm = hbm_data_ != nullptr && (residency_ == TopologyResidency::kHbm || node_id < cached_rows_);
    const std::uint32_t* src = (in_hbm ? hbm_data_ : mapped_data_) + node_id * degree_;
    ThrowIfCudaError(cudaMemcpy(row.data(), src, degree_ * sizeof(std::uint32_t), cudaMemcpyDefault), "cudaMemcpy");
    return row;
}

// ---- PqIndex ----------------------------------------------------------------------------------------------
PqIndex::~PqIndex() { Release(); }
PqIndex::PqIndex(PqIndex&& o) noexcept { *this = std::move(o); }
PqIndex& PqIndex::operator=(PqIndex&& o) noexcept {
    if (this == &o) return *this;
    Release();
    host_ = std::move(o.host_);
    device_ = std::move(o.device_);
    device_tables_row_major_ = std::move(o.device_tables_row_major_);
    mapped_host_codes_ = o.mapped_host_codes_;
    mapped_device_codes_ = o.mapped_device_codes_;
    o.mapped_host_codes_ = o.mapped_device_codes_ = nullptr;
    return *this;
}
void PqIndex::Release() noexcept {
    if (mapped_host_codes_ != nullptr) cudaFreeHost(mapped_host_codes_);
    mapped_host_codes_ = mapped_device_codes_ = nullptr;
}
const std::uint8_t* PqIndex::host_codes() const {
    return mapped_host_codes_ != nullptr ? mapped_host_codes_ : host_.codes.data();
}
const std::uint8_t* PqIndex::device_codes() const {
    return mapped_device_codes_ != nullptr ? mapped_device_codes_ : device_.codes.get();
}
PqIndex PqIndex::LoadImpl(const std::filesystem::path& pivots, const std::filesystem::path& compressed, bool map_codes,
                          bool load_codes) {
    const char* ctx = "PqIndex::LoadFromSeparatePaths";
    PqIndex ix;
    const BinBlock<std::size_t> offsets = ReadBinBlock<std::size_t>(pivots, 0, "ReadBinBlock");
    if (offsets.rows != 4 && offsets.rows != 5) throw std::runtime_error(BuildErrorMessage(ctx, "Unexpected PQ offset count."));
    const bool old_type = offsets.rows == 5;
    const BinBlock<float> tables = ReadBinBlock<float>(pivots, offsets.data[0], "ReadBinBlock");
    if (tables.rows != kNumPqCentroids) throw std::runtime_error(BuildErrorMessage(ctx, "Unexpected PQ centroid count."));
    ix.host_.ndims = tables.cols;
    {
        std::ifstream in(compressed, std::ios::binary);
        if (!in.is_open()) throw std::runtime_error(BuildErrorMessage("ReadBinMetadata", "Failed to open " + compressed.string()));
        std::int32_t r = 0, c = 0;
        in.read(reinterpret_cast<char*>(&r), 4);
        in.read(reinterpret_cast<char*>(&c), 4);
        if (!in.good() || r < 0 || c < 0) throw std::runtime_error(BuildErrorMessage("ReadBinMetadata", "Invalid metadata in " + compressed.string()));
        ix.host_.num_points = static_cast<std::uint64_t>(r);
        ix.host_.num_chunks = static_cast<std::uint64_t>(c);
    }
    ix.host_.tables_row_major = tables.data;
    ix.host_.tables_col_major.assign(tables.data.size(), 0.0f);
    for (std::size_t r = 0; r < tables.rows; ++r)
        for (std::size_t c = 0; c < tables.cols; ++c)
            ix.host_.tables_col_major[c * tables.rows + r] = tables.data[r * tables.cols + c];
    const BinBlock<float> centroid = ReadBinBlock<float>(pivots, offsets.data[1], "ReadBinBlock");
    if (centroid.rows != ix.host_.ndims || centroid.cols != 1)
        throw std::runtime_error(BuildErrorMessage(ctx, "Unexpected PQ centroid vector shape."));
    ix.host_.centroid = centroid.data;
    const BinBlock<std::uint32_t> chunk = ReadBinBlock<std::uint32_t>(pivots, offsets.data[old_type ? 3 : 2], "ReadBinBlock");
    if (chunk.cols != 1 || chunk.rows != ix.host_.num_chunks + 1)
        throw std::runtime_error(BuildErrorMessage(ctx, "Unexpected PQ chunk offsets shape."));
    ix.host_.chunk_offsets = chunk.data;

    const std::size_t code_bytes = static_cast<std::size_t>(ix.host_.num_points * ix.host_.num_chunks);
    if (load_codes && code_bytes != 0) {
        std::vector<std::uint8_t> codes = ReadFileRange(compressed, 8, code_bytes, ctx);
        if (map_codes) {
            ThrowIfCudaError(cudaHostAlloc(reinterpret_cast<void**>(&ix.mapped_host_codes_), code_bytes,
                                           cudaHostAllocMapped | cudaHostAllocPortable), "cudaMallocHost");
            std::memcpy(ix.mapped_host_codes_, codes.data(), code_bytes);
            ThrowIfCudaError(cudaHostGetDevicePointer(reinterpret_cast<void**>(&ix.mapped_device_codes_),
                                                      ix.mapped_host_codes_, 0), "cudaHostGetDevicePointer");
            ix.host_.codes_on_host = true;
        } else {
            ix.device_.codes = CudaBuffer<std::uint8_t>::CopyFromHost(codes);
            ix.host_.codes_on_host = code_bytes <= (1ULL << 30);  // the reference keeps a host copy up to 1 GiB
            if (ix.host_.codes_on_host) ix.host_.codes = std::move(codes);
        }
    }
    ix.device_.tables_col_major = CudaBuffer<float>::CopyFromHost(ix.host_.tables_col_major);
    ix.device_.chunk_offsets = CudaBuffer<std::uint32_t>::CopyFromHost(ix.host_.chunk_offsets);
    ix.device_.centroid = CudaBuffer<float>::CopyFromHost(ix.host_.centroid);
    ix.device_tables_row_major_ = CudaBuffer<float>::CopyFromHost(ix.host_.tables_row_major);
    return ix;
}
PqIndex PqIndex::LoadFromSeparatePaths(const std::filesystem::path& p, const std::filesystem::path& c) { return LoadImpl(p, c, false, true); }
PqIndex PqIndex::LoadFromSeparatePathsMapped(const std::filesystem::path& p, const std::filesystem::path& c) { return LoadImpl(p, c, true, true); }
PqIndex PqIndex::LoadPivotsOnly(const std::filesystem::path& p, const std::filesystem::path& c) { return LoadImpl(p, c, false, false); }

// ---- hybrid PQ index (src/io/hpq_index.cpp) ---------------------------------------------------------------------
HpqIndex::~HpqIndex() { Release(); }
HpqIndex::HpqIndex(HpqIndex&& other) noexcept { *this = std::move(other); }
HpqIndex& HpqIndex::operator=(HpqIndex&& other) noexcept {
    if (this != &other) {
        Release();
        base_index_ = std::move(other.base_index_);
        outlier_index_ = std::move(other.outlier_index_);
        selector_stride_bytes_ = other.selector_stride_bytes_;
        mapped_host_selector_bits_ = other.mapped_host_selector_bits_;
        mapped_device_selector_bits_ = other.mapped_device_selector_bits_;
        other.selector_stride_bytes_ = 0;
        other.mapped_host_selector_bits_ = nullptr;
        other.mapped_device_selector_bits_ = nullptr;
    }
    return *this;
}
void HpqIndex::Release() noexcept {
    if (mapped_host_selector_bits_ != nullptr) tann_host_free(mapped_host_selector_bits_);
    mapped_host_selector_bits_ = nullptr;
    mapped_device_selector_bits_ = nullptr;
    selector_stride_bytes_ = 0;
}
HpqIndex HpqIndex::Load(const std::filesystem::path& base_pivots_path, const std::filesystem::path& outlier_pivots_path,
                        const std::filesystem::path& hybrid_codes_path, const std::filesystem::path& selector_bits_path) {
    const char* ctx = "HpqIndex::Load";
    HpqIndex result;
    result.base_index_ = PqIndex::LoadPivotsOnly(base_pivots_path, hybrid_codes_path);
    result.outlier_index_ = PqIndex::LoadFromSeparatePathsMapped(outlier_pivots_path, hybrid_codes_path);
    std::ifstream in(selector_bits_path, std::ios::binary);
    std::int32_t rows = 0, cols = 0;
    in.read(reinterpret_cast<char*>(&rows), sizeof(rows));
    in.read(reinterpret_cast<char*>(&cols), sizeof(cols));
    if (!in.good() || rows < 0 || cols <= 0) throw std::runtime_error(BuildErrorMessage(ctx, "Invalid selector-bit metadata."));
    const auto& host = result.outlier_index_.host();
    const std::size_t stride = (host.num_chunks + 7U) / 8U;
    if (static_cast<std::uint64_t>(rows) != host.num_points || static_cast<std::size_t>(cols) != stride)
        throw std::runtime_error(BuildErrorMessage(ctx, "Selector-bit shape does not match HPQ codes."));
    const std::size_t total = static_cast<std::size_t>(rows) * stride;
    void* hp = nullptr;
    void* dp = nullptr;
    ThrowIfTannError(tann_host_alloc_mapped(total == 0 ? 16 : total, &hp, &dp), ctx);
    result.mapped_host_selector_bits_ = static_cast<std::uint8_t*>(hp);
    result.mapped_device_selector_bits_ = static_cast<std::uint8_t*>(dp);
    result.selector_stride_bytes_ = stride;
    in.read(reinterpret_cast<char*>(result.mapped_host_selector_bits_), static_cast<std::streamsize>(total));
    if (static_cast<std::size_t>(in.gcount()) != total) {
        result.Release();
        throw std::runtime_error(BuildErrorMessage(ctx, "Short selector-bit read."));
    }
    return result;
}

// ---- providers ----------------------------------------------------------------------------------------------
DevicePageReadResult VectorPageProvider::ReadPagesToDevice(const std::filesystem::path&, const std::vector<std::uint64_t>&,
                                                           std::size_t, std::size_t) const {
    throw std::runtime_error(BuildErrorMessage("VectorPageProvider::ReadPagesToDevice", "Device-direct reads are not supported by this provider."));
}
DevicePageReadResult VectorPageProvider::ReadPagesToDevice(const std::filesystem::path&, const CudaBuffer<std::uint64_t>&,
                                                           std::size_t, std::size_t, std::size_t) const {
    throw std::runtime_error(BuildErrorMessage("VectorPageProvider::ReadPagesToDevice", "Device-direct reads are not supported by this provider."));
}

namespace {
std::vector<std::uint8_t> LoadAllPages(const std::filesystem::path& path, const char* context) {
    const VectorStoreHeader h = VectorStoreBuilder::ReadHeader(path);
    const std::uint64_t pages = (h.num_vectors + h.vectors_per_page - 1) / h.vectors_per_page;
    return ReadFileRange(path, kDefaultPageSizeBytes, pages * h.page_size_bytes, context);
}
DevicePageReadResult UploadPages(const std::vector<std::uint8_t>& gathered) {
    const auto t0 = std::chrono::steady_clock::now();
    DevicePageReadResult r;
    r.page_bytes = CudaBuffer<std::uint8_t>::CopyFromHost(gathered);
    r.io_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    return r;
}
}  // namespace

HbmVectorPageProvider::HbmVectorPageProvider(const std::filesystem::path& path) {
    host_pages_ = LoadAllPages(path, "HbmVectorPageProvider");
    pages_ = CudaBuffer<std::uint8_t>::CopyFromHost(host_pages_);
    shards_ = OneShard(pages_.get());
}
std::vector<std::uint8_t> HbmVectorPageProvider::ReadPages(const std::filesystem::path&, const std::vector<std::uint64_t>& ids,
                                                           std::size_t, std::size_t page_size) const {
    return GatherHostPages(host_pages_.data(), host_pages_.size(), ids, page_size, "HbmVectorPageProvider::ReadPages");
}
DevicePageReadResult HbmVectorPageProvider::ReadPagesToDevice(const std::filesystem::path& p, const std::vector<std::uint64_t>& ids,
                                                              std::size_t header_bytes, std::size_t page_size) const {
    return UploadPages(ReadPages(p, ids, header_bytes, page_size));
}

PinnedHostVectorPageProvider::PinnedHostVectorPageProvider(const std::filesystem::path& path) {
    const std::vector<std::uint8_t> all = LoadAllPages(path, "PinnedHostVectorPageProvider");
    bytes_ = all.size();
    if (bytes_ != 0) {
        ThrowIfCudaError(cudaHostAlloc(reinterpret_cast<void**>(&host_), bytes_, cudaHostAllocMapped | cudaHostAllocPortable),
                         "cudaMallocHost");
        std::memcpy(host_, all.data(), bytes_);
        ThrowIfCudaError(cudaHostGetDevicePointer(reinterpret_cast<void**>(&mapped_), host_, 0), "cudaHostGetDevicePointer");
    }
    shards_ = OneShard(mapped_);
}
PinnedHostVectorPageProvider::~PinnedHostVectorPageProvider() {
    if (host_ != nullptr) cudaFreeHost(host_);
}
std::vector<std::uint8_t> PinnedHostVectorPageProvider::ReadPages(const std::filesystem::path&, const std::vector<std::uint64_t>& ids,
                                                                  std::size_t, std::size_t page_size) const {
    return GatherHostPages(host_, bytes_, ids, page_size, "PinnedHostVectorPageProvider::ReadPages");
}
DevicePageReadResult PinnedHostVectorPageProvider::ReadPagesToDevice(const std::filesystem::path& p, const std::vector<std::uint64_t>& ids,
                                                                     std::size_t header_bytes, std::size_t page_size) const {
    return UploadPages(ReadPages(p, ids, header_bytes, page_size));
}
std::vector<std::uint8_t> PeerVectorPageProvider::ReadPages(const std::filesystem::path&, const std::vector<std::uint64_t>&,
                                                            std::size_t, std::size_t) const {
    throw std::runtime_error(BuildErrorMessage("PeerVectorPageProvider::ReadPages", "peer-resident pages are read by the kernels only."));
}

// ---- SearchResources --------------------------------------------------------------------------------------------
SearchResources SearchResources::FromDataset(const TopologyDataset& dataset) {
    SearchResources r;
    r.topology_ = std::make_shared<PinnedTopology>(PinnedTopology::FromDataset(dataset));
    return r;
}
SearchResources SearchResources::FromTopologyFile(const std::filesystem::path& path) {
    SearchResources r;
    r.topology_ = std::make_shared<PinnedTopology>(PinnedTopology::FromFile(path));
    return r;
}
std::uint64_t SearchResources::num_nodes() const { return topology_->num_nodes(); }
std::uint32_t SearchResources::degree() const { return topology_->degree(); }
std::vector<std::uint32_t> SearchResources::ReadHostNeighbors(std::uint64_t node_id) const { return topology_->ReadHostNode(node_id); }

void SearchResources::LoadPqIndex(const std::filesystem::path& pivots, const std::filesystem::path& compressed) {
    pq_index_ = std::make_shared<PqIndex>(PqIndex::LoadFromSeparatePaths(pivots, compressed));
}
const PqIndex& SearchResources::pq_index() const {
    if (!pq_index_) throw std::runtime_error(BuildErrorMessage("SearchResources::pq_index", "PQ index is not loaded."));
    return *pq_index_;
}
void SearchResources::LoadPq2Index(const std::filesystem::path& pivots, const std::filesystem::path& compressed,
                                   const std::filesystem::path& error_bounds_path) {
    // pq2 codes live in HBM here (the reference maps them from pinned host memory over PCIe).
    pq2_index_ = std::make_shared<PqIndex>(PqIndex::LoadFromSeparatePaths(pivots, compressed));
    pq2_aux_.reset();
    if (error_bounds_path.empty()) return;
    if (!pq_index_)
        throw std::runtime_error(BuildErrorMessage("SearchResources::LoadPq2Index",
                                                   "Base PQ index must be loaded before residual PQ refine resources."));
    const auto& b = pq_index_->host();
    const auto& r = pq2_index_->host();
    if (b.ndims != r.ndims) throw std::runtime_error(BuildErrorMessage("BuildPq2CrossTerms", "Base PQ and residual PQ dimensions differ."));
    if (b.num_chunks != r.num_chunks) throw std::runtime_error(BuildErrorMessage("BuildPq2CrossTerms", "Base PQ and residual PQ chunk counts differ."));
    if (b.chunk_offsets != r.chunk_offsets) throw std::runtime_error(BuildErrorMessage("BuildPq2CrossTerms", "Base PQ and residual PQ chunk offsets differ."));
    auto aux = std::make_shared<Pq2Aux>();
    aux->residual_refine = true;
    aux->cross_terms = CudaBuffer<float>::Allocate(b.num_chunks * kNumPqCentroids * kNumPqCentroids);
    ThrowIfTannError(tann_pq2_cross_terms(static_cast<std::uint32_t>(b.ndims), static_cast<std::uint32_t>(b.num_chunks),
                                          pq_index_->device().chunk_offsets.get(), pq_index_->device_tables_row_major().get(),
                                          pq_index_->device().centroid.get(), pq2_index_->device_tables_row_major().get(),
                                          pq2_index_->device().centroid.get(), aux->cross_terms.get(), nullptr),
                     "BuildPq2CrossTerms");
    ThrowIfCudaError(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    const BinBlock<float> eps = ReadBinBlock<float>(error_bounds_path, 0, "ReadBinBlock");
    if (eps.cols != 1 || eps.rows != static_cast<std::size_t>(r.num_points))
        throw std::runtime_error(BuildErrorMessage("SearchResources::LoadPq2Index",
                                                   "Residual error-bound file shape does not match PQ2 point count."));
    aux->error_bounds_fp32 = CudaBuffer<float>::CopyFromHost(eps.data);
    aux->storage = Pq2ErrorBoundStorage::kFloat32;
    pq2_aux_ = std::move(aux);
}
const PqIndex& SearchResources::pq2_index() const {
    if (!pq2_index_) throw std::runtime_error(BuildErrorMessage("SearchResources::pq2_index", "PQ2 index is not loaded."));
    return *pq2_index_;
}
void SearchResources::LoadHpqIndex(const std::filesystem::path& base_pivots_path, const std::filesystem::path& outlier_pivots_path,
                                   const std::filesystem::path& hybrid_codes_path, const std::filesystem::path& selector_bits_path) {
    // src/search/search_resources.cpp:221-246
    const char* ctx = "SearchResources::LoadHpqIndex";
    if (!pq_index_) throw std::runtime_error(BuildErrorMessage(ctx, "Base PQ index must be loaded first."));
    auto hpq = std::make_shared<HpqIndex>(HpqIndex::Load(base_pivots_path, outlier_pivots_path, hybrid_codes_path, selector_bits_path));
    const auto& base = hpq->base_index().host();
    const auto& outlier = hpq->outlier_index().host();
    if (base.ndims != outlier.ndims || base.num_chunks != outlier.num_chunks || base.chunk_offsets != outlier.chunk_offsets)
        throw std::runtime_error(BuildErrorMessage(ctx, "Base and outlier HPQ layouts differ."));
    if (outlier.num_points != num_nodes()) throw std::runtime_error(BuildErrorMessage(ctx, "Graph and HPQ dataset shapes differ."));
    hpq_index_ = std::move(hpq);
}
const HpqIndex& SearchResources::hpq_index() const {
    if (!hpq_index_) throw std::runtime_error(BuildErrorMessage("SearchResources::hpq_index", "HPQ index is not loaded."));
    return *hpq_index_;
}
bool SearchResources::pq2_is_residual_refine() const { return pq2_aux_ && pq2_aux_->residual_refine; }
bool SearchResources::has_pq2_error_bounds() const { return pq2_aux_ && pq2_aux_->storage != Pq2ErrorBoundStorage::kNone; }
Pq2ErrorBoundStorage SearchResources::pq2_error_bound_storage() const { return pq2_aux_ ? pq2_aux_->storage : Pq2ErrorBoundStorage::kNone; }
const CudaBuffer<float>& SearchResources::pq2_cross_terms() const {
    if (!pq2_aux_) throw std::runtime_error(BuildErrorMessage("SearchResources::pq2_cross_terms", "Residual PQ2 resources are not loaded."));
    return pq2_aux_->cross_terms;
}
const CudaBuffer<float>& SearchResources::pq2_error_bounds_fp32() const {
    if (!pq2_aux_) throw std::runtime_error(BuildErrorMessage("SearchResources::pq2_error_bounds_fp32", "Residual PQ2 resources are not loaded."));
    return pq2_aux_->error_bounds_fp32;
}

void SearchResources::LoadVectorStore(const std::filesystem::path& path) {
    auto vs = std::make_shared<VectorStore>();
    vs->path = path;
    vs->header = VectorStoreBuilder::ReadHeader(path);
    vs->layout = VectorPageLayout::CreateFromVectorBytes(vs->header.vector_bytes, vs->header.page_size_bytes);
    if (vector_store_) vs->provider = vector_store_->provider;
    vector_store_ = std::move(vs);
}
namespace {
[[noreturn]] void NoVectorStore(const char* ctx) { throw std::runtime_error(BuildErrorMessage(ctx, "Vector store is not loaded.")); }
}
const VectorStoreHeader& SearchResources::vector_store_header() const {
    if (!vector_store_) NoVectorStore("SearchResources::vector_store_header");
    return vector_store_->header;
}
const VectorPageLayout& SearchResources::vector_store_layout() const {
    if (!vector_store_) NoVectorStore("SearchResources::vector_store_layout");
    return vector_store_->layout;
}
const std::filesystem::path& SearchResources::vector_store_path() const {
    if (!vector_store_) NoVectorStore("SearchResources::vector_store_path");
    return vector_store_->path;
}
void SearchResources::AttachVectorPageProvider(std::shared_ptr<VectorPageProvider> provider) {
    if (!vector_store_) NoVectorStore("SearchResources::AttachVectorPageProvider");
    vector_store_->provider = std::move(provider);
}
void SearchResources::ClearVectorPageProvider() {
    if (vector_store_) vector_store_->provider.reset();
}
const VectorPageProvider& SearchResources::vector_page_provider() const {
    if (!vector_store_ || !vector_store_->provider)
        throw std::runtime_error(BuildErrorMessage("SearchResources::vector_page_provider", "Vector page provider is not attached."));
    return *vector_store_->provider;
}
void SearchResources::AttachTopologyPageProvider(std::shared_ptr<VectorPageProvider> provider) { topology_page_provider_ = std::move(provider); }
void SearchResources::ClearTopologyPageProvider() { topology_page_provider_.reset(); }
const VectorPageProvider& SearchResources::topology_page_provider() const {
    if (!topology_page_provider_)
        throw std::runtime_error(BuildErrorMessage("SearchResources::topology_page_provider", "Topology page provider is not attached."));
    return *topology_page_provider_;
}
const void* SearchResources::topology_device_read_handle() const {
    return topology_page_provider_ ? topology_page_provider_->DeviceReadHandle() : nullptr;
}
void SearchResources::AttachTopologyShards(const TannShards& adjacency) {
    adjacency_shards_ = adjacency;
    has_adjacency_shards_ = true;
}
void SearchResources::AttachPqCodeShards(const TannShards& codes) {
    code_shards_ = codes;
    has_code_shards_ = true;
}

void SearchResources::BuildNeighborCodeLayout() {
    const char* ctx = "BuildNeighborCodeLayout";
    if (!pq_index_) throw std::runtime_error(BuildErrorMessage(ctx, "PQ index must be loaded first."));
    if (has_adjacency_shards_ || has_code_shards_ || topology_->residency() != TopologyResidency::kHbm)
        throw std::runtime_error(BuildErrorMessage(ctx, "the layout is built for an HBM-resident, unsharded index."));
    neighbor_codes_.reset();
    const TannIndexView view = MakeIndexView(false);
    const std::size_t bytes = static_cast<std::size_t>(view.num_nodes) * view.degree * view.num_chunks;
    auto buffer = std::make_shared<CudaBuffer<std::uint8_t>>(CudaBuffer<std::uint8_t>::Allocate(bytes));
    ThrowIfTannError(tann_neighbor_codes_build(&view, 0, view.num_nodes, buffer->get(), nullptr), ctx);
    ThrowIfCudaError(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    neighbor_codes_ = std::move(buffer);
}

TannIndexView SearchResources::MakeIndexView(bool need_vectors) const {
    TannIndexView v{};
    v.num_nodes = topology_->num_nodes();
    v.degree = topology_->degree();
    if (has_adjacency_shards_) {
        v.adjacency = adjacency_shards_;
    } else if (topology_->residency() == TopologyResidency::kPinnedHost) {
        v.adjacency = OneShard(topology_->mapped_host_device_pointer());
        v.adjacency_cache = topology_->hbm_data();
        v.adjacency_cached_rows = topology_->cached_rows();
    } else {
        v.adjacency = OneShard(topology_->device_data());
    }
    if (pq_index_) {
        const PqIndex& pq = *pq_index_;
        v.num_chunks = static_cast<std::uint32_t>(pq.host().num_chunks);
        v.dim = static_cast<std::uint32_t>(pq.host().ndims);
        v.codes = has_code_shards_ ? code_shards_ : OneShard(pq.device_codes());
        v.pq_tables_col_major = pq.device().tables_col_major.get();
        v.pq_centroid = pq.device().centroid.get();
        v.pq_chunk_offsets = pq.device().chunk_offsets.get();
        if (neighbor_codes_) v.neighbor_codes = OneShard(neighbor_codes_->get());
    }
    if (need_vectors && vector_store_) {
        const VectorStoreHeader& h = vector_store_->header;
        v.dim = h.dim;
        // ScalarKind order of the reference: 0 int8, 1 uint8, 2 float32 (same as TANN_KIND_*)
        v.vector_kind = h.scalar_kind;
        v.vector_bytes = h.vector_bytes;
        v.vectors_per_page = h.vectors_per_page;
        v.page_bytes = h.page_size_bytes;
        if (vector_store_->provider && vector_store_->provider->DeviceReadHandle() != nullptr)
            v.vectors = *static_cast<const TannShards*>(vector_store_->provider->DeviceReadHandle());
    }
    return v;
}

}  // namespace topoanns
