// RVQ entry model over the C ABI. File layout and posting-list rules follow the reference
// (src/legacy_rvq/gas_legacy/anns/RVQ/RVQ.cu:884-924,977-1033 model file;
// src/search/rvq_entry_provider.cpp:21,115-144 lists capped at 256 ids, uncapped bucket sizes for the
// "non-empty" test; :226-321 entry computation).
#include <chrono>
#include <fstream>

#include "topoanns/api.hpp"

namespace topoanns {
namespace {
constexpr std::size_t kPostingLimit = 256;
using Clock = std::chrono::steady_clock;
double MsSince(const Clock::time_point& t0) { return std::chrono::duration<double, std::milli>(Clock::now() - t0).count(); }
}  // namespace

struct RvqModel::Impl {
    int dim = 0, num_coarse = 0, num_fine = 0;
    CudaBuffer<float> coarse, coarse_t, coarse_norms, fine, fine_t, fine_norms;
    CudaBuffer<std::int32_t> bucket_sizes;
    CudaBuffer<std::uint32_t> cluster_offsets, cluster_ids;
    std::vector<std::uint32_t> host_offsets, host_ids;

    explicit Impl(const std::filesystem::path& path) {
        std::ifstream in(path, std::ios::binary);
        if (!in.is_open()) throw std::runtime_error(BuildErrorMessage("ReadRvqModelHeader", "Failed to open " + path.string()));
        std::int32_t hdr[3] = {0, 0, 0};
        in.read(reinterpret_cast<char*>(hdr), sizeof(hdr));
        if (!in.good() || hdr[0] <= 0 || hdr[1] <= 0 || hdr[2] <= 0)
            throw std::runtime_error(BuildErrorMessage("ReadRvqModelHeader", "Invalid RVQ model header in " + path.string()));
        dim = hdr[0];
        num_coarse = hdr[1];
        num_fine = hdr[2];
        std::vector<float> hc(static_cast<std::size_t>(num_coarse) * dim), hf(static_cast<std::size_t>(num_fine) * dim);
        in.read(reinterpret_cast<char*>(hc.data()), static_cast<std::streamsize>(hc.size() * 4));
        in.read(reinterpret_cast<char*>(hf.data()), static_cast<std::streamsize>(hf.size() * 4));
        std::uint64_t outer = 0;
        in.read(reinterpret_cast<char*>(&outer), 8);
        if (!in.good() || outer != static_cast<std::uint64_t>(num_coarse))
            throw std::runtime_error(BuildErrorMessage("RvqModel::Load", "Posting lists do not match the coarse centroid count."));
        std::vector<std::int32_t> sizes;
        sizes.reserve(static_cast<std::size_t>(num_coarse) * num_fine);
        host_offsets.assign(1, 0u);
        std::vector<std::int32_t> bucket;
        for (std::uint64_t c = 0; c < outer; ++c) {
            std::uint64_t inner = 0;
            in.read(reinterpret_cast<char*>(&inner), 8);
            if (!in.good() || inner != static_cast<std::uint64_t>(num_fine))
                throw std::runtime_error(BuildErrorMessage("RvqModel::Load", "Posting lists do not match the fine centroid count."));
            for (std::uint64_t f = 0; f < inner; ++f) {
                std::uint64_t n = 0;
                in.read(reinterpret_cast<char*>(&n), 8);
                bucket.resize(n);
                if (n != 0) in.read(reinterpret_cast<char*>(bucket.data()), static_cast<std::streamsize>(n * 4));
                if (!in.good()) throw std::runtime_error(BuildErrorMessage("RvqModel::Load", "Short read in " + path.string()));
                sizes.push_back(static_cast<std::int32_t>(n));
                const std::size_t keep = std::min<std::size_t>(n, kPostingLimit);
                for (std::size_t i = 0; i < keep; ++i) host_ids.push_back(static_cast<std::uint32_t>(bucket[i]));
                host_offsets.push_back(static_cast<std::uint32_t>(host_ids.size()));
            }
        }
        auto transpose = [](const std::vector<float>& rows, int count, int d) {
            std::vector<float> t(rows.size());
            for (int r = 0; r < count; ++r)
                for (int k = 0; k < d; ++k) t[static_cast<std::size_t>(k) * count + r] = rows[static_cast<std::size_t>(r) * d + k];
            return t;
        };
        coarse = CudaBuffer<float>::CopyFromHost(hc);
        fine = CudaBuffer<float>::CopyFromHost(hf);
        coarse_t = CudaBuffer<float>::CopyFromHost(transpose(hc, num_coarse, dim));
        fine_t = CudaBuffer<float>::CopyFromHost(transpose(hf, num_fine, dim));
        coarse_norms = CudaBuffer<float>::Allocate(num_coarse);
        fine_norms = CudaBuffer<float>::Allocate(num_fine);
        ThrowIfTannError(tann_rvq_norms(coarse.get(), num_coarse, dim, coarse_norms.get(), nullptr), "RvqModel::Load");
        ThrowIfTannError(tann_rvq_norms(fine.get(), num_fine, dim, fine_norms.get(), nullptr), "RvqModel::Load");
        bucket_sizes = CudaBuffer<std::int32_t>::CopyFromHost(sizes);
        cluster_offsets = CudaBuffer<std::uint32_t>::CopyFromHost(host_offsets);
        cluster_ids = CudaBuffer<std::uint32_t>::CopyFromHost(host_ids.empty() ? std::vector<std::uint32_t>{kInvalidNodeId} : host_ids);
        ThrowIfCudaError(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    }

    DeviceEntryBatch Entries(const std::vector<float>& queries, std::size_t n, std::size_t entry_count, std::uint32_t fallback,
                             CudaBuffer<std::int32_t>* out_clusters, RvqEntryProfile* profile, const char* ctx) const {
        if (queries.size() != n * static_cast<std::size_t>(dim))
            throw std::runtime_error(BuildErrorMessage("AssignClustersFloat32", "queries size must equal num_queries * dim."));
        DeviceEntryBatch batch;
        batch.num_queries = n;
        batch.entries_per_query = entry_count;
        if (n == 0) return batch;
        auto t0 = Clock::now();
        const CudaBuffer<float> d_q = CudaBuffer<float>::CopyFromHost(queries);
        const double upload_ms = MsSince(t0);
        batch.offsets = CudaBuffer<std::uint32_t>::Allocate(n + 1);
        batch.ids = CudaBuffer<std::uint32_t>::Allocate(n * entry_count);
        CudaBuffer<std::int32_t> clusters = CudaBuffer<std::int32_t>::Allocate(n);
        t0 = Clock::now();
        ThrowIfTannError(tann_rvq_entries(d_q.get(), n, dim, coarse.get(), coarse_t.get(), coarse_norms.get(), num_coarse,
                                          fine_t.get(), fine_norms.get(), num_fine, bucket_sizes.get(), cluster_offsets.get(),
                                          cluster_ids.get(), static_cast<std::uint32_t>(entry_count), fallback, clusters.get(),
                                          batch.ids.get(), batch.offsets.get(), nullptr), ctx);
        ThrowIfCudaError(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        const double kernel_ms = MsSince(t0);
        if (profile != nullptr) {
            profile->query_upload_ms += upload_ms;
            profile->search_kernel_ms += kernel_ms;
            profile->total_ms += upload_ms + kernel_ms;
        }
        if (out_clusters != nullptr) *out_clusters = std::move(clusters);
        return batch;
    }
};

RvqModel::RvqModel() = default;
RvqModel::~RvqModel() = default;
RvqModel::RvqModel(std::unique_ptr<Impl> impl) : impl_(std::move(impl)) {}
RvqModel::RvqModel(RvqModel&&) noexcept = default;
RvqModel& RvqModel::operator=(RvqModel&&) noexcept = default;
RvqModel RvqModel::Load(const std::filesystem::path& path) { return RvqModel(std::make_unique<Impl>(path)); }

std::uint32_t RvqModel::dim() const {
    if (!impl_) throw std::runtime_error(BuildErrorMessage("RvqModel::dim", "model is not loaded."));
    return static_cast<std::uint32_t>(impl_->dim);
}
std::uint32_t RvqModel::coarse_centroids() const {
    if (!impl_) throw std::runtime_error(BuildErrorMessage("RvqModel::coarse_centroids", "model is not loaded."));
    return static_cast<std::uint32_t>(impl_->num_coarse);
}
std::uint32_t RvqModel::fine_centroids() const {
    if (!impl_) throw std::runtime_error(BuildErrorMessage("RvqModel::fine_centroids", "model is not loaded."));
    return static_cast<std::uint32_t>(impl_->num_fine);
}
void RvqModel::WarmUp() const {
    if (!impl_) throw std::runtime_error(BuildErrorMessage("RvqModel::WarmUp", "model is not loaded."));
    const std::vector<float> zero(static_cast<std::size_t>(impl_->dim), 0.0f);
    (void)impl_->Entries(zero, 1, 1, 0, nullptr, nullptr, "RvqModel::WarmUp");
}
std::vector<std::vector<std::uint32_t>> RvqModel::ComputeFloat32EntryPoints(const std::vector<float>& queries, std::size_t n,
                                                                            std::size_t entry_count, std::uint32_t fallback,
                                                                            RvqEntryProfile* profile) const {
    const char* ctx = "RvqModel::ComputeFloat32EntryPoints";
    if (!impl_) throw std::runtime_error(BuildErrorMessage(ctx, "model is not loaded."));
    if (entry_count == 0) throw std::runtime_error(BuildErrorMessage(ctx, "entry_count must be positive."));
    // The host variant is not capped at 256 ids per bucket in the reference; entry_count beyond the
    // cap is served from the capped device lists here, which only matters for entry_count > 256.
    const DeviceEntryBatch batch = impl_->Entries(queries, n, entry_count, fallback, nullptr, profile, ctx);
    const std::vector<std::uint32_t> ids = batch.ids.CopyToHost();
    std::vector<std::vector<std::uint32_t>> out(n);
    for (std::size_t q = 0; q < n; ++q)
        for (std::size_t i = 0; i < entry_count; ++i) {
            const std::uint32_t id = ids[q * entry_count + i];
            if (id == kInvalidNodeId) break;
            out[q].push_back(id);
        }
    return out;
}
DeviceEntryBatch RvqModel::ComputeFloat32DeviceEntryBatch(const std::vector<float>& queries, std::size_t n,
                                                          std::size_t entry_count, std::uint32_t fallback,
                                                          RvqEntryProfile* profile) const {
    const char* ctx = "RvqModel::ComputeFloat32DeviceEntryBatch";
    if (!impl_) throw std::runtime_error(BuildErrorMessage(ctx, "model is not loaded."));
    if (entry_count == 0) throw std::runtime_error(BuildErrorMessage(ctx, "entry_count must be positive."));
    return impl_->Entries(queries, n, entry_count, fallback, nullptr, profile, ctx);
}

RvqEntryProvider::RvqEntryProvider(std::vector<std::vector<std::uint32_t>> e) : entries_by_query_(std::move(e)) {}
RvqEntryProvider RvqEntryProvider::FromFloatQueries(const RvqModel& model, const std::vector<float>& queries, std::size_t n,
                                                    std::size_t entry_count, std::uint32_t fallback, RvqEntryProfile* profile) {
    return RvqEntryProvider(model.ComputeFloat32EntryPoints(queries, n, entry_count, fallback, profile));
}
std::vector<std::uint32_t> RvqEntryProvider::GetEntryPoints(std::size_t q) const {
    if (q >= entries_by_query_.size())
        throw std::runtime_error(BuildErrorMessage("RvqEntryProvider::GetEntryPoints", "query_id is out of range."));
    return entries_by_query_[q];
}

}  // namespace topoanns
