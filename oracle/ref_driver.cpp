// Runs the reference's own implementation of the batched search path (compiled from its sources by
// ref_build.sh) on an index directory and dumps what it computes, so that the CPU checker and the
// CUDA path can be compared with the reference itself. TEST INFRASTRUCTURE ONLY.
//
//   ref_driver <dir> <out_prefix> <mode> top_l search_width max_expansions top_k top_n [rerank_mode tile pq2 bound repeats]
//     dir: topology.bin, _pq_pivots.bin, _pq_compressed.bin, vectors.ssd, queries.fbin, entries.bin
//          (+ _pq2_pivots.bin, _pq2_compressed.bin, _pq2_error.bin when pq2 = 1)
//     mode: lut | search | e2e_f32 | e2e_u8 | fused | pq2refine | rvq | hpq | time
//       rvq:  dir/rvq_model.bin through RvqModel::Load; dumps the device entry batch and the host entry lists
//             for <top_n> entries per query (the argument is reused as the entry count)
//       hpq:  dir/_hpq_outlier_pivots.bin, _hpq_codes.bin, _hpq_selector.bin (+ the base pivots); traversal on the
//             device, then the hybrid-PQ refine; dumps the refined lists
//       time: `repeats` passes of RunBatchFloat32Fused over the query file, prints wall and kernel times
//     The learned traversal stop is switched on as in the reference: TOPOANNS_LEARNED_STOP_MODEL=<file> in the
//     environment of the `search` mode.
//   Outputs raw little-endian arrays <out_prefix>.<name>.bin (shapes are implied by the arguments).
#include <chrono>
#include <cstdint>
#include <cstring>
#include <fstream>
#include <iostream>
#include <memory>
#include <string>
#include <vector>

#include "fused_rerank_device.hpp"
#include "topoanns/entry_provider.hpp"
#include "topoanns/pq_distance_oracle.hpp"
#include "topoanns/rerank_exact.hpp"
#include "topoanns/rvq_entry_provider.hpp"
#include "topoanns/search_resources.hpp"
#include "topoanns/topoanns_search.hpp"
#include "topoanns/topology_search.hpp"
#include "topology_search_kernel.hpp"

namespace {

using namespace topoanns;

std::vector<char> ReadAll(const std::string& path) {
    std::ifstream in(path, std::ios::binary | std::ios::ate);
    if (!in.is_open()) throw std::runtime_error("cannot open " + path);
    std::vector<char> buf(static_cast<std::size_t>(in.tellg()));
    in.seekg(0);
    in.read(buf.data(), static_cast<std::streamsize>(buf.size()));
    return buf;
}

template <typename T>
void Dump(const std::string& prefix, const std::string& name, const std::vector<T>& v) {
    std::ofstream out(prefix + "." + name + ".bin", std::ios::binary | std::ios::trunc);
    out.write(reinterpret_cast<const char*>(v.data()), static_cast<std::streamsize>(v.size() * sizeof(T)));
}

// Whole vector store in host memory; pages are gathered on the host and uploaded.
class WholeFileProvider final : public VectorPageProvider {
public:
    explicit WholeFileProvider(const std::string& path) : bytes_(ReadAll(path)) {}
    bool SupportsDeviceReads() const override { return true; }
    std::vector<std::uint8_t> ReadPages(const std::filesystem::path&, const std::vector<std::uint64_t>& ids,
                                        std::size_t header_bytes, std::size_t page) const override {
        std::vector<std::uint8_t> out(ids.size() * page);
        for (std::size_t i = 0; i < ids.size(); ++i) std::memcpy(out.data() + i * page, bytes_.data() + header_bytes + ids[i] * page, page);
        return out;
    }
    DevicePageReadResult ReadPagesToDevice(const std::filesystem::path& p, const std::vector<std::uint64_t>& ids,
                                           std::size_t header_bytes, std::size_t page) const override {
        DevicePageReadResult r;
        r.page_bytes = CudaBuffer<std::uint8_t>::CopyFromHost(ReadPages(p, ids, header_bytes, page));
        return r;
    }
    DevicePageReadResult ReadPagesToDevice(const std::filesystem::path& p, const CudaBuffer<std::uint64_t>& ids,
                                           std::size_t n, std::size_t header_bytes, std::size_t page) const override {
        std::vector<std::uint64_t> host = ids.CopyToHost();
        host.resize(n);
        return ReadPagesToDevice(p, host, header_bytes, page);
    }
private:
    std::vector<char> bytes_;
};

void DumpTopology(const std::string& prefix, const std::string& tag, const std::vector<TopologySearchResult>& res,
                  std::size_t limit) {
    std::vector<float> dist;
    std::vector<std::uint32_t> ids, counts, stats;
    for (const auto& r : res) {
        counts.push_back(static_cast<std::uint32_t>(r.sorted_candidates.size()));
        for (std::size_t i = 0; i < limit; ++i) {
            const bool have = i < r.sorted_candidates.size();
            dist.push_back(have ? r.sorted_candidates[i].distance : 0.0f);
            ids.push_back(have ? (r.sorted_candidates[i].node_id | (r.sorted_candidates[i].expanded ? 0x80000000u : 0u)) : 0xffffffffu);
        }
        stats.push_back(static_cast<std::uint32_t>(r.stats.visited_nodes));
        stats.push_back(static_cast<std::uint32_t>(r.stats.expanded_nodes));
        stats.push_back(static_cast<std::uint32_t>(r.stats.iterations));
    }
    Dump(prefix, tag + "_dist", dist);
    Dump(prefix, tag + "_ids", ids);
    Dump(prefix, tag + "_counts", counts);
    Dump(prefix, tag + "_stats", stats);
}

void DumpRerank(const std::string& prefix, const std::vector<RerankQueryResult>& res, const RerankBatchStats& st,
                std::size_t top_n) {
    std::vector<float> dist;
    std::vector<std::uint32_t> ids;
    for (const auto& r : res)
        for (std::size_t i = 0; i < top_n; ++i) {
            const bool have = i < r.sorted_candidates.size();
            dist.push_back(have ? r.sorted_candidates[i].distance : std::numeric_limits<float>::infinity());
            ids.push_back(have ? r.sorted_candidates[i].node_id : 0xffffffffu);
        }
    Dump(prefix, "rerank_dist", dist);
    Dump(prefix, "rerank_ids", ids);
    Dump(prefix, "rerank_stats", std::vector<std::uint64_t>{st.io_pages, st.exact_distance_count, st.bound_filtered_count});
}

}  // namespace

int main(int argc, char** argv) {
    if (argc < 9) {
        std::cerr << "usage: ref_driver dir out mode top_l width max_exp top_k top_n [rerank_mode tile pq2 bound repeats]\n";
        return 2;
    }
    try {
        const std::string dir = argv[1], prefix = argv[2], mode = argv[3];
        TopoAnnsSearchParams params;
        params.topology.top_l = std::stoul(argv[4]);
        params.topology.search_width = std::stoul(argv[5]);
        params.topology.max_expansions = std::stoul(argv[6]);
        params.topology.top_k = std::stoul(argv[7]);
        params.rerank.top_k = std::stoul(argv[7]);
        params.rerank.top_n = std::stoul(argv[8]);
        const std::string rerank_mode = argc > 9 ? argv[9] : "linear";
        params.rerank.rank_tile_size = argc > 10 ? std::stoul(argv[10]) : 16;
        const bool pq2 = argc > 11 && std::stoi(argv[11]) != 0;
        const bool bound = argc > 12 && std::stoi(argv[12]) != 0;
        const int repeats = argc > 13 ? std::stoi(argv[13]) : 1;
        params.rerank.mode = rerank_mode == "tiled" ? RerankExecutionMode::kTiled
                             : rerank_mode == "page" ? RerankExecutionMode::kPageByPage : RerankExecutionMode::kLinear;
        params.rerank.use_pq2_refine = pq2;
        params.rerank.use_pq2_bound_filter = bound;
        params.rerank.pq2_refine_top_l = pq2 ? params.topology.top_l : 0;

        SearchResources res = SearchResources::FromTopologyFile(dir + "/topology.bin");
        res.LoadPqIndex(dir + "/_pq_pivots.bin", dir + "/_pq_compressed.bin");
        if (pq2) res.LoadPq2Index(dir + "/_pq2_pivots.bin", dir + "/_pq2_compressed.bin", dir + "/_pq2_error.bin");
        res.LoadVectorStore(dir + "/vectors.ssd");
        res.AttachVectorPageProvider(std::make_shared<WholeFileProvider>(dir + "/vectors.ssd"));

        const std::vector<char> qraw = ReadAll(dir + "/queries.fbin");
        std::uint32_t nq = 0, dim = 0;
        std::memcpy(&nq, qraw.data(), 4);
        std::memcpy(&dim, qraw.data() + 4, 4);
        std::vector<float> queries(static_cast<std::size_t>(nq) * dim);
        std::memcpy(queries.data(), qraw.data() + 8, queries.size() * 4);
        const std::vector<char> eraw = ReadAll(dir + "/entries.bin");
        std::uint32_t eq = 0, ecount = 0;
        std::memcpy(&eq, eraw.data(), 4);
        std::memcpy(&ecount, eraw.data() + 4, 4);
        std::vector<std::vector<std::uint32_t>> entries(eq, std::vector<std::uint32_t>(ecount));
        for (std::uint32_t q = 0; q < eq; ++q) std::memcpy(entries[q].data(), eraw.data() + 8 + (static_cast<std::size_t>(q) * ecount) * 4, ecount * 4);
        const PerQueryEntryProvider provider(entries);

        if (mode == "lut") {
            const auto tables = PqQueryDistanceTables::FromFloatQueries(res.pq_index(), queries, nq);
            Dump(prefix, "lut", tables.host_tables());
        } else if (mode == "search") {
            const auto oracle = PqDistanceOracle::FromFloatQueries(res, queries, nq);
            TopologySearchParams tp = params.topology;
            tp.candidate_queue_size = std::max(tp.top_l, params.rerank.top_n);
            const std::size_t limit = tp.candidate_queue_size;
            for (int rep = 0; rep < repeats; ++rep) {
                const auto out = TopologySearch::RunBatch(res, provider, oracle, tp);
                DumpTopology(prefix, "search" + std::to_string(rep), out, limit);
            }
        } else if (mode == "e2e_f32") {
            const auto out = TopoAnnsSearch::RunBatchFloat32(res, provider, queries, nq, params);
            std::vector<TopologySearchResult> topo;
            std::vector<RerankQueryResult> rr;
            for (const auto& q : out.queries) { topo.push_back(q.topology); rr.push_back(q.rerank); }
            DumpTopology(prefix, "search0", topo, std::max(params.topology.top_l, params.rerank.top_n));
            DumpRerank(prefix, rr, out.rerank_stats, params.rerank.top_n);
        } else if (mode == "e2e_u8") {
            std::vector<std::uint8_t> q8(queries.size());
            for (std::size_t i = 0; i < queries.size(); ++i) q8[i] = static_cast<std::uint8_t>(queries[i]);
            const auto out = TopoAnnsSearch::RunBatchUint8(res, provider, q8, nq, params);
            std::vector<RerankQueryResult> rr;
            for (const auto& q : out.queries) rr.push_back(q.rerank);
            DumpRerank(prefix, rr, out.rerank_stats, params.rerank.top_n);
        } else if (mode == "fused") {
            DeviceEntryBatch batch;
            batch.num_queries = nq;
            batch.entries_per_query = ecount;
            std::vector<std::uint32_t> offsets(nq + 1), flat;
            for (std::uint32_t q = 0; q <= nq; ++q) offsets[q] = q * ecount;
            for (const auto& e : entries) flat.insert(flat.end(), e.begin(), e.end());
            batch.offsets = CudaBuffer<std::uint32_t>::CopyFromHost(offsets);
            batch.ids = CudaBuffer<std::uint32_t>::CopyFromHost(flat);
            const auto out = TopoAnnsSearch::RunBatchFloat32Fused(res, batch, queries, nq, params);
            std::vector<RerankQueryResult> rr;
            std::vector<std::uint32_t> stats;
            for (const auto& q : out.queries) {
                rr.push_back(q.rerank);
                stats.push_back(static_cast<std::uint32_t>(q.topology.stats.visited_nodes));
                stats.push_back(static_cast<std::uint32_t>(q.topology.stats.expanded_nodes));
                stats.push_back(static_cast<std::uint32_t>(q.topology.stats.iterations));
            }
            DumpRerank(prefix, rr, out.rerank_stats, params.rerank.top_n);
            Dump(prefix, "search0_stats", stats);
        } else if (mode == "pq2refine") {
            // traversal on the device, then the pq2 refine stage alone; dumps the refined lists
            DeviceEntryBatch batch;
            batch.num_queries = nq;
            batch.entries_per_query = ecount;
            std::vector<std::uint32_t> offsets(nq + 1), flat;
            for (std::uint32_t q = 0; q <= nq; ++q) offsets[q] = q * ecount;
            for (const auto& e : entries) flat.insert(flat.end(), e.begin(), e.end());
            batch.offsets = CudaBuffer<std::uint32_t>::CopyFromHost(offsets);
            batch.ids = CudaBuffer<std::uint32_t>::CopyFromHost(flat);
            const auto oracle = PqDistanceOracle::FromFloatQueries(res, queries, nq);
            TopologySearchParams tp = params.topology;
            tp.candidate_queue_size = std::max(tp.top_l, params.rerank.top_n);
            const auto topo = detail::RunTopologySearchKernelBatchDevice(res, oracle, batch, tp);
            const auto refined = detail::RunPq2RefineBatchDevice(res, topo, queries, nq, params.topology.top_l);
            const auto host = refined.candidate_buffer.CopyToHost();
            std::vector<float> dist;
            std::vector<std::uint32_t> ids;
            for (const auto& c : host) { dist.push_back(c.distance); ids.push_back(c.node_id); }
            Dump(prefix, "refined_dist", dist);
            Dump(prefix, "refined_ids", ids);
            std::cout << "traversal_kernel_ms=" << topo.kernel_ms << " pq2_refine_kernel_ms=" << refined.kernel_ms << "\n";
        } else if (mode == "rvq") {
            // RVQ entry selection by the reference's own RVQ::search (cuBLAS scores + its argmin kernels)
            const std::size_t entry_count = params.rerank.top_n;
            const RvqModel model = RvqModel::Load(dir + "/rvq_model.bin");
            const auto lists = model.ComputeFloat32EntryPoints(queries, nq, entry_count, 0);
            std::vector<std::uint32_t> flat(static_cast<std::size_t>(nq) * entry_count, 0xffffffffu), counts(nq);
            for (std::uint32_t q = 0; q < nq; ++q) {
                counts[q] = static_cast<std::uint32_t>(lists[q].size());
                for (std::size_t i = 0; i < lists[q].size() && i < entry_count; ++i) flat[q * entry_count + i] = lists[q][i];
            }
            Dump(prefix, "rvq_host_ids", flat);
            Dump(prefix, "rvq_host_counts", counts);
            const DeviceEntryBatch dev = model.ComputeFloat32DeviceEntryBatch(queries, nq, entry_count, 0);
            Dump(prefix, "rvq_dev_offsets", dev.offsets.CopyToHost());
            Dump(prefix, "rvq_dev_ids", dev.ids.CopyToHost());
        } else if (mode == "hpq") {
            res.LoadHpqIndex(dir + "/_pq_pivots.bin", dir + "/_hpq_outlier_pivots.bin", dir + "/_hpq_codes.bin",
                             dir + "/_hpq_selector.bin");
            DeviceEntryBatch batch;
            batch.num_queries = nq;
            batch.entries_per_query = ecount;
            std::vector<std::uint32_t> offsets(nq + 1), flat;
            for (std::uint32_t q = 0; q <= nq; ++q) offsets[q] = q * ecount;
            for (const auto& e : entries) flat.insert(flat.end(), e.begin(), e.end());
            batch.offsets = CudaBuffer<std::uint32_t>::CopyFromHost(offsets);
            batch.ids = CudaBuffer<std::uint32_t>::CopyFromHost(flat);
            const auto oracle = PqDistanceOracle::FromFloatQueries(res, queries, nq);
            TopologySearchParams tp = params.topology;
            tp.candidate_queue_size = std::max(tp.top_l, params.rerank.top_n);
            const auto topo = detail::RunTopologySearchKernelBatchDevice(res, oracle, batch, tp);
            const CudaBuffer<float> dq = CudaBuffer<float>::CopyFromHost(queries);
            const auto refined = detail::RunHpqRefineBatchDevice(res, topo, dq, nq, params.topology.top_l, nullptr);
            const auto host = refined.candidate_buffer.CopyToHost();
            std::vector<float> dist;
            std::vector<std::uint32_t> ids;
            for (const auto& c : host) { dist.push_back(c.distance); ids.push_back(c.node_id); }
            Dump(prefix, "refined_dist", dist);
            Dump(prefix, "refined_ids", ids);
        } else if (mode == "time") {
            // the reference's fused path (device entries given), timed as a caller sees it
            DeviceEntryBatch batch;
            batch.num_queries = nq;
            batch.entries_per_query = ecount;
            std::vector<std::uint32_t> offsets(nq + 1), flat;
            for (std::uint32_t q = 0; q <= nq; ++q) offsets[q] = q * ecount;
            for (const auto& e : entries) flat.insert(flat.end(), e.begin(), e.end());
            batch.offsets = CudaBuffer<std::uint32_t>::CopyFromHost(offsets);
            batch.ids = CudaBuffer<std::uint32_t>::CopyFromHost(flat);
            TopoAnnsSearch::RunBatchFloat32Fused(res, batch, queries, nq, params);   // warm-up
            double best_ms = 1e30, sum_ms = 0.0, traversal_ms = 0.0;
            std::vector<std::uint32_t> ids;
            for (int rep = 0; rep < repeats; ++rep) {
                const auto t0 = std::chrono::steady_clock::now();
                const auto out = TopoAnnsSearch::RunBatchFloat32Fused(res, batch, queries, nq, params);
                const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
                best_ms = std::min(best_ms, ms);
                sum_ms += ms;
                traversal_ms = out.topology_profile.kernel_ms;
                if (rep + 1 == repeats) {
                    for (const auto& q : out.queries)
                        for (std::size_t i = 0; i < params.rerank.top_k; ++i)
                            ids.push_back(i < q.rerank.topk.size() ? q.rerank.topk[i].node_id : 0xffffffffu);
                }
            }
            Dump(prefix, "time_topk_ids", ids);
            std::cout << "ref_time queries=" << nq << " repeats=" << repeats << " best_ms=" << best_ms
                      << " mean_ms=" << sum_ms / repeats << " traversal_kernel_ms=" << traversal_ms << "\n";
        } else {
            std::cerr << "unknown mode " << mode << "\n";
            return 2;
        }
        std::cout << "ref_driver ok\n";
        return 0;
    } catch (const std::exception& e) {
        std::cerr << "ref_driver failed: " << e.what() << "\n";
        return 1;
    }
}
