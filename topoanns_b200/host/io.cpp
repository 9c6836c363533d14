// Index file layouts and the small host-only classes of the API (no device work here).
// Layout facts are those of the reference's readers and writers: src/io/topology_layout.cpp,
// src/io/vector_page_layout.cpp, src/builder/vector_store_builder.cpp,
// src/search/entry_provider.cpp, src/search/search_stop_condition.cpp.
#include <cstring>
#include <fstream>

#include "topoanns/api.hpp"

namespace topoanns {

void ThrowIfTannError(TannStatus status, const char* context) {
    if (status == TANN_OK) return;
    // The C ABI prefixes its messages with its own entry-point name; callers of this API expect
    // "context: detail" with the reference's context, so the prefix is replaced.
    std::string detail = tann_last_error();
    const std::size_t colon = detail.find(": ");
    if (colon != std::string::npos && detail.compare(0, 5, "tann_") == 0) detail = detail.substr(colon + 2);
    throw std::runtime_error(BuildErrorMessage(context, detail));
}

// ---- entry providers ------------------------------------------------------------------------------
FixedEntryProvider::FixedEntryProvider(std::vector<std::uint32_t> entries) : entries_(std::move(entries)) {}
std::vector<std::uint32_t> FixedEntryProvider::GetEntryPoints(std::size_t) const { return entries_; }

PerQueryEntryProvider::PerQueryEntryProvider(std::vector<std::vector<std::uint32_t>> entries_by_query)
    : entries_by_query_(std::move(entries_by_query)) {}
std::vector<std::uint32_t> PerQueryEntryProvider::GetEntryPoints(std::size_t query_id) const {
    if (query_id >= entries_by_query_.size())
        throw std::runtime_error(BuildErrorMessage("PerQueryEntryProvider::GetEntryPoints", "query_id is out of range."));
    return entries_by_query_[query_id];
}

// ---- stop rule --------------------------------------------------------------------------------------
std::size_t SearchStopCondition::CountValid(const std::vector<RankedCandidate>& candidates) {
    std::size_t n = 0;
    for (const auto& c : candidates) n += c.valid() ? 1 : 0;
    return n;
}
std::size_t SearchStopCondition::BestUnexpandedRank(const std::vector<RankedCandidate>& candidates) {
    for (std::size_t i = 0; i < candidates.size(); ++i)
        if (candidates[i].valid() && !candidates[i].expanded) return i;
    return std::numeric_limits<std::size_t>::max();
}
bool SearchStopCondition::TopLHasNoBetterUnexpanded(const std::vector<RankedCandidate>& candidates, std::size_t top_l) {
    if (top_l == 0) return true;
    if (CountValid(candidates) < top_l) return false;
    return BestUnexpandedRank(candidates) >= top_l;
}

// ---- topology.bin -------------------------------------------------------------------------------------
namespace {
const char kTopologyMagic[8] = {'T', 'O', 'P', 'O', 'A', 'N', 'N', 'S'};
const char kVectorMagic[8] = {'T', 'P', 'V', 'E', 'C', 'T', 'O', 'R'};

TopologyHeader ReadTopologyHeader(std::ifstream& in, const char* context, std::streamsize* file_size) {
    if (!in.is_open()) throw std::runtime_error(BuildErrorMessage(context, "Failed to open topology file."));
    in.seekg(0, std::ios::end);
    *file_size = in.tellg();
    if (*file_size < static_cast<std::streamsize>(sizeof(TopologyHeader)))
        throw std::runtime_error(BuildErrorMessage(context, "Topology file is smaller than the header."));
    in.seekg(0, std::ios::beg);
    TopologyHeader h{};
    in.read(reinterpret_cast<char*>(&h), sizeof(h));
    if (!in.good()) throw std::runtime_error(BuildErrorMessage(context, "Failed to read topology header."));
    if (std::memcmp(h.magic, kTopologyMagic, 8) != 0)
        throw std::runtime_error(BuildErrorMessage(context, "Unexpected topology magic."));
    if (h.version != TopologyLayout::kVersion)
        throw std::runtime_error(BuildErrorMessage(context, "Unexpected topology version."));
    if (h.degree == 0) throw std::runtime_error(BuildErrorMessage(context, "Unexpected topology degree."));
    const std::uint64_t expect = sizeof(TopologyHeader) + h.num_nodes * h.degree * sizeof(std::uint32_t);
    if (static_cast<std::uint64_t>(*file_size) != expect)
        throw std::runtime_error(BuildErrorMessage(context, "Topology file size does not match metadata."));
    return h;
}
}  // namespace

std::size_t TopologyDataset::NodeBytes() const { return static_cast<std::size_t>(degree) * sizeof(std::uint32_t); }
const std::uint32_t* TopologyDataset::NodeNeighbors(std::uint64_t node_id) const {
    if (node_id >= num_nodes) throw std::runtime_error(BuildErrorMessage("NodeNeighbors", "node_id is out of range."));
    return adjacency.data() + node_id * degree;
}
std::size_t TopologyLayout::NodeBytes() { return kFixedTopologyDegree * sizeof(std::uint32_t); }
std::uint64_t TopologyLayout::NodeOffsetBytes(std::uint64_t node_id) { return sizeof(TopologyHeader) + node_id * NodeBytes(); }

TopologyDataset TopologyLayout::MakePaddedDegree(std::uint64_t num_nodes, std::uint32_t degree,
                                                 const std::vector<std::vector<std::uint32_t>>& lists) {
    if (lists.size() != num_nodes)
        throw std::runtime_error(BuildErrorMessage("MakePadded", "adjacency_lists size must match num_nodes."));
    TopologyDataset d;
    d.num_nodes = num_nodes;
    d.degree = degree;
    d.adjacency.assign(static_cast<std::size_t>(num_nodes) * degree, kInvalidNodeId);
    for (std::uint64_t n = 0; n < num_nodes; ++n) {
        const auto& l = lists[static_cast<std::size_t>(n)];
        if (l.size() > degree)
            throw std::runtime_error(BuildErrorMessage("MakePadded", "A node has more than " + std::to_string(degree) + " neighbors."));
        std::copy(l.begin(), l.end(), d.adjacency.begin() + static_cast<std::ptrdiff_t>(n * degree));
    }
    return d;
}
TopologyDataset TopologyLayout::MakePadded(std::uint64_t num_nodes, const std::vector<std::vector<std::uint32_t>>& lists) {
    return MakePaddedDegree(num_nodes, kFixedTopologyDegree, lists);
}
void TopologyLayout::WriteFile(const std::filesystem::path& path, const TopologyDataset& dataset) {
    if (dataset.degree == 0 || dataset.adjacency.size() != static_cast<std::size_t>(dataset.num_nodes) * dataset.degree)
        throw std::runtime_error(BuildErrorMessage("ValidateDataset", "Adjacency vector size does not match num_nodes * degree."));
    std::ofstream out(path, std::ios::binary | std::ios::trunc);
    if (!out.is_open()) throw std::runtime_error(BuildErrorMessage("WriteFile", "Failed to open output file."));
    TopologyHeader h{};
    std::memcpy(h.magic, kTopologyMagic, 8);
    h.version = kVersion;
    h.degree = dataset.degree;
    h.num_nodes = dataset.num_nodes;
    h.header_bytes = sizeof(TopologyHeader);
    h.payload_bytes = dataset.adjacency.size() * sizeof(std::uint32_t);
    out.write(reinterpret_cast<const char*>(&h), sizeof(h));
    out.write(reinterpret_cast<const char*>(dataset.adjacency.data()), static_cast<std::streamsize>(h.payload_bytes));
    if (!out.good()) throw std::runtime_error(BuildErrorMessage("WriteFile", "Failed while writing topology file."));
}
TopologyHeader TopologyLayout::ReadHeader(const std::filesystem::path& path) {
    std::ifstream in(path, std::ios::binary);
    std::streamsize size = 0;
    return ReadTopologyHeader(in, "ReadHeader", &size);
}
TopologyDataset TopologyLayout::ReadFile(const std::filesystem::path& path) {
    std::ifstream in(path, std::ios::binary);
    std::streamsize size = 0;
    const TopologyHeader h = ReadTopologyHeader(in, "ReadFile", &size);
    TopologyDataset d;
    d.num_nodes = h.num_nodes;
    d.degree = h.degree;
    d.adjacency.resize(static_cast<std::size_t>(h.num_nodes) * h.degree);
    in.read(reinterpret_cast<char*>(d.adjacency.data()), static_cast<std::streamsize>(d.adjacency.size() * sizeof(std::uint32_t)));
    if (!in.good()) throw std::runtime_error(BuildErrorMessage("ReadFile", "Failed to read adjacency payload."));
    return d;
}

// ---- vector pages -----------------------------------------------------------------------------------------
VectorPageLayout VectorPageLayout::CreateFromVectorBytes(std::size_t vector_bytes, std::size_t page_size_bytes) {
    if (vector_bytes == 0) throw std::runtime_error(BuildErrorMessage("VectorPageLayout", "vector_bytes must be positive."));
    if (vector_bytes > page_size_bytes)
        throw std::runtime_error(BuildErrorMessage("VectorPageLayout", "A vector must fit in one page."));
    VectorPageLayout l;
    l.page_size_bytes_ = page_size_bytes;
    l.header_bytes_ = kDefaultPageSizeBytes;
    l.vector_bytes_ = vector_bytes;
    l.vectors_per_page_ = page_size_bytes / vector_bytes;
    l.payload_bytes_per_page_ = l.vectors_per_page_ * vector_bytes;
    return l;
}
VectorPageLayout VectorPageLayout::Create(std::uint32_t dim, ScalarKind kind, std::size_t page_size_bytes) {
    return CreateFromVectorBytes(static_cast<std::size_t>(dim) * ScalarKindBytes(kind), page_size_bytes);
}
std::uint64_t VectorPageLayout::PageCountForVectors(std::uint64_t n) const {
    return vectors_per_page_ == 0 ? 0 : (n + vectors_per_page_ - 1) / vectors_per_page_;
}
VectorPageAddress VectorPageLayout::Resolve(std::uint64_t node_id) const {
    VectorPageAddress a;
    a.page_id = node_id / vectors_per_page_;
    a.slot_id = static_cast<std::uint32_t>(node_id % vectors_per_page_);
    a.byte_offset = header_bytes_ + a.page_id * page_size_bytes_ + static_cast<std::uint64_t>(a.slot_id) * vector_bytes_;
    return a;
}

void VectorStoreBuilder::WriteFile(const std::filesystem::path& path, const VectorPageLayout& layout, ScalarKind kind,
                                   std::uint32_t dim, const std::vector<std::vector<std::uint8_t>>& vectors) {
    const std::size_t vb = static_cast<std::size_t>(dim) * ScalarKindBytes(kind);
    if (vb != layout.vector_bytes())
        throw std::runtime_error(BuildErrorMessage("VectorStoreBuilder::WriteFile", "layout does not match dim * scalar size."));
    VectorStoreHeader h{};
    std::memcpy(h.magic, kVectorMagic, 8);
    h.version = kVersion;
    h.scalar_kind = static_cast<std::uint32_t>(kind);
    h.dim = dim;
    h.num_vectors = vectors.size();
    h.page_size_bytes = layout.page_size_bytes();
    h.vector_bytes = vb;
    h.vectors_per_page = layout.vectors_per_page();
    std::ofstream out(path, std::ios::binary | std::ios::trunc);
    if (!out.is_open()) throw std::runtime_error(BuildErrorMessage("VectorStoreBuilder::WriteFile", "Failed to open output file."));
    out.write(reinterpret_cast<const char*>(&h), sizeof(h));
    std::vector<std::uint8_t> page(layout.page_size_bytes(), 0);
    const std::uint64_t pages = layout.PageCountForVectors(vectors.size());
    for (std::uint64_t p = 0; p < pages; ++p) {
        std::fill(page.begin(), page.end(), 0);
        for (std::size_t s = 0; s < layout.vectors_per_page(); ++s) {
            const std::uint64_t id = p * layout.vectors_per_page() + s;
            if (id >= vectors.size()) break;
            if (vectors[id].size() != vb)
                throw std::runtime_error(BuildErrorMessage("VectorStoreBuilder::WriteFile", "vector byte size mismatch."));
            std::memcpy(page.data() + s * vb, vectors[id].data(), vb);
        }
        out.write(reinterpret_cast<const char*>(page.data()), static_cast<std::streamsize>(page.size()));
    }
    if (!out.good()) throw std::runtime_error(BuildErrorMessage("VectorStoreBuilder::WriteFile", "Failed while writing."));
}
VectorStoreHeader VectorStoreBuilder::ReadHeader(const std::filesystem::path& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in.is_open()) throw std::runtime_error(BuildErrorMessage("VectorStoreBuilder::ReadHeader", "Failed to open " + path.string()));
    VectorStoreHeader h{};
    in.read(reinterpret_cast<char*>(&h), sizeof(h));
    if (!in.good() || std::memcmp(h.magic, kVectorMagic, 8) != 0)
        throw std::runtime_error(BuildErrorMessage("VectorStoreBuilder::ReadHeader", "Unexpected vector store magic."));
    if (h.version != kVersion || h.scalar_kind > 2 || h.vector_bytes == 0 || h.vectors_per_page == 0)
        throw std::runtime_error(BuildErrorMessage("VectorStoreBuilder::ReadHeader", "Invalid vector store header."));
    return h;
}
std::vector<std::uint8_t> VectorStoreBuilder::ReadVectorById(const std::filesystem::path& path, const VectorPageLayout& layout,
                                                             std::uint64_t node_id) {
    std::ifstream in(path, std::ios::binary);
    if (!in.is_open()) throw std::runtime_error(BuildErrorMessage("VectorStoreBuilder::ReadVectorById", "Failed to open " + path.string()));
    std::vector<std::uint8_t> v(layout.vector_bytes());
    in.seekg(static_cast<std::streamoff>(layout.Resolve(node_id).byte_offset), std::ios::beg);
    in.read(reinterpret_cast<char*>(v.data()), static_cast<std::streamsize>(v.size()));
    if (!in.good()) throw std::runtime_error(BuildErrorMessage("VectorStoreBuilder::ReadVectorById", "Short read."));
    return v;
}

}  // namespace topoanns
