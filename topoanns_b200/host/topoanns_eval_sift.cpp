// Evaluation driver on the C++ API: sweeps top_l (and optionally rerank_top_n) over an index directory,
// prints one summary line per point and the QPS / recall Pareto frontier. It takes the flags and prints
// the "[topoanns_eval] ... qps= ... recall@10= ..." and "[topoanns_pareto] ..." lines of the reference's
// tools/topoanns_eval_sift.cpp (usage :221-259, summary line :613-658, frontier :1068-1102, main loop
// :1209-1325), so scripts that parse that output keep working. Flags that configure the reference's NVMe
// backend are accepted and ignored; --vector-residency and --topology-residency choose among the providers
// of this library instead.
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <iostream>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "topoanns/topoanns_search.hpp"

namespace {

struct Args {
    std::filesystem::path index_dir, rvq_model, query_bin, gt_bin;
    std::filesystem::path pq2_pivots, pq2_codes, pq2_error_bounds;
    bool has_gt = false;
    std::size_t num_queries = 0;
    std::vector<std::size_t> eval_query_counts, top_l_values, rerank_top_n_values, rerank_top_n_sweep_values;
    std::size_t batch_size = 10000, top_k = 10, search_width = 1, rerank_top_n = 100, rank_tile_size = 16;
    std::size_t max_expansions = 1024, rvq_entry_count = 64;
    topoanns::RerankExecutionMode rerank_mode = topoanns::RerankExecutionMode::kPersistent;
    bool use_pq2_refine = false, use_pq2_bound_filter = false, use_early_stop = false;
    std::size_t early_stop_min_prefix = 32, early_stop_patience_tiles = 1;
    bool use_learned_stop = false;
    std::filesystem::path learned_stop_model;
    std::string vector_residency = "hbm", topology_residency = "hbm";
    std::uint64_t topology_cached_rows = 0;
    std::size_t repeats = 1;
    bool neighbor_code_layout = false;
};

struct FloatMatrix { std::uint32_t rows = 0, cols = 0; std::vector<float> values; };
struct IntMatrix { std::uint32_t rows = 0, cols = 0; std::vector<std::int32_t> values; };
struct SweepPoint {
    std::size_t top_l, rerank_top_n;
    topoanns::RerankExecutionMode mode;
    std::size_t num_queries;
    double qps, wall_qps, recall;
};

[[noreturn]] void Usage() {
    std::cerr << "Usage: topoanns_eval_sift --index-dir <path> --rvq-model <path> --query-bin <path> [--gt-bin <path>]"
                 " --num-queries <count> [--eval-query-counts <csv>] --top-l-values <csv> [--batch-size <count>]"
                 " [--top-k <count>] [--search-width <count>] [--rerank-top-n <count>] [--rerank-top-n-values <csv>]"
                 " [--rerank-top-n-sweep-values <csv>] [--rerank-mode <linear|tiled|page|persistent>]"
                 " [--rerank-rank-tile-size <count>] [--pq2-pivots <path> --pq2-codes <path> [--pq2-error-bounds <path>]"
                 " --rerank-use-pq2] [--rerank-use-pq2-bound-filter] [--rerank-use-early-stop]"
                 " [--rerank-early-stop-min-prefix <count>] [--rerank-early-stop-patience-tiles <count>] [--max-expansions <count>] [--rvq-entry-count <count>]"
                 " [--vector-residency <hbm|pinned-host>] [--topology-residency <hbm|pinned-host>]"
                 " [--topology-cached-rows <count>] [--repeats <count>] [--neighbor-code-layout]"
                 " [--rerank-use-learned-stop --rerank-learned-stop-model <path>]"
                 " (flags of the NVMe backend, --bam-* and --frontier-pq-modes, are accepted and ignored)"
              << std::endl;
    std::exit(1);
}

std::vector<std::size_t> ParseCsv(const std::string& text) {
    std::vector<std::size_t> out;
    std::stringstream ss(text);
    std::string item;
    while (std::getline(ss, item, ',')) {
        if (!item.empty()) out.push_back(static_cast<std::size_t>(std::stoull(item)));
    }
    return out;
}

const char* ModeName(topoanns::RerankExecutionMode mode) {
    switch (mode) {
        case topoanns::RerankExecutionMode::kLinear: return "linear";
        case topoanns::RerankExecutionMode::kTiled: return "tiled";
        case topoanns::RerankExecutionMode::kPageByPage: return "page";
        default: return "persistent";
    }
}

topoanns::RerankExecutionMode ParseMode(const std::string& text) {
    if (text == "linear") return topoanns::RerankExecutionMode::kLinear;
    if (text == "tiled") return topoanns::RerankExecutionMode::kTiled;
    if (text == "page" || text == "page_by_page") return topoanns::RerankExecutionMode::kPageByPage;
    if (text == "persistent") return topoanns::RerankExecutionMode::kPersistent;
    throw std::runtime_error("Unknown rerank mode: " + text);
}

Args Parse(int argc, char** argv) {
    Args a;
    // flags with one value that this library has no use for
    const char* ignored_with_value[] = {"--frontier-pq-modes", "--bam-config-path", "--bam-controller-path",
                                        "--bam-device-offset-bytes", "--bam-page-cache-bytes", "--bam-queue-depth",
                                        "--bam-num-queues", "--bam-cuda-device", "--rerank-mode-sweep"};
    const char* ignored_flags[] = {"--allow-bam-controller-override"};
    for (int i = 1; i < argc; ++i) {
        const std::string f = argv[i];
        auto value = [&]() -> std::string {
            if (i + 1 >= argc) Usage();
            return argv[++i];
        };
        bool skipped = false;
        for (const char* name : ignored_with_value)
            if (f == name) { value(); std::cerr << "[topoanns_eval] note: " << f << " is ignored" << std::endl; skipped = true; }
        for (const char* name : ignored_flags)
            if (f == name) { std::cerr << "[topoanns_eval] note: " << f << " is ignored" << std::endl; skipped = true; }
        if (skipped) continue;
        if (f == "--index-dir") a.index_dir = value();
        else if (f == "--rvq-model") a.rvq_model = value();
        else if (f == "--query-bin") a.query_bin = value();
        else if (f == "--gt-bin") { a.gt_bin = value(); a.has_gt = true; }
        else if (f == "--num-queries") a.num_queries = std::stoull(value());
        else if (f == "--eval-query-counts") a.eval_query_counts = ParseCsv(value());
        else if (f == "--top-l-values") a.top_l_values = ParseCsv(value());
        else if (f == "--batch-size") a.batch_size = std::stoull(value());
        else if (f == "--top-k") a.top_k = std::stoull(value());
        else if (f == "--search-width") a.search_width = std::stoull(value());
        else if (f == "--rerank-top-n") a.rerank_top_n = std::stoull(value());
        else if (f == "--rerank-top-n-values") a.rerank_top_n_values = ParseCsv(value());
        else if (f == "--rerank-top-n-sweep-values") a.rerank_top_n_sweep_values = ParseCsv(value());
        else if (f == "--rerank-mode") a.rerank_mode = ParseMode(value());
        else if (f == "--rerank-rank-tile-size") a.rank_tile_size = std::stoull(value());
        else if (f == "--pq2-pivots") a.pq2_pivots = value();
        else if (f == "--pq2-codes") a.pq2_codes = value();
        else if (f == "--pq2-error-bounds") a.pq2_error_bounds = value();
        else if (f == "--rerank-use-pq2") a.use_pq2_refine = true;
        else if (f == "--rerank-use-pq2-bound-filter") a.use_pq2_bound_filter = true;
        else if (f == "--rerank-use-early-stop") a.use_early_stop = true;
        else if (f == "--rerank-use-learned-stop") a.use_learned_stop = true;
        else if (f == "--rerank-learned-stop-model") a.learned_stop_model = value();
        else if (f == "--rerank-early-stop-min-prefix") a.early_stop_min_prefix = std::stoull(value());
        else if (f == "--rerank-early-stop-patience-tiles") a.early_stop_patience_tiles = std::stoull(value());
        else if (f == "--max-expansions") a.max_expansions = std::stoull(value());
        else if (f == "--rvq-entry-count") a.rvq_entry_count = std::stoull(value());
        else if (f == "--vector-residency") a.vector_residency = value();
        else if (f == "--topology-residency") a.topology_residency = value();
        else if (f == "--topology-cached-rows") a.topology_cached_rows = std::stoull(value());
        else if (f == "--repeats") a.repeats = std::max<std::size_t>(1, std::stoull(value()));
        else if (f == "--neighbor-code-layout") a.neighbor_code_layout = true;
        else { std::cerr << "Unknown flag: " << f << std::endl; Usage(); }
    }
    if (a.index_dir.empty() || a.rvq_model.empty() || a.query_bin.empty() || a.num_queries == 0 || a.top_l_values.empty())
        Usage();
    if (a.use_learned_stop && a.learned_stop_model.empty())
        throw std::runtime_error("rerank-use-learned-stop requires rerank-learned-stop-model.");
    if (a.use_learned_stop && a.use_early_stop)
        throw std::runtime_error("rerank-use-learned-stop cannot be combined with rerank-use-early-stop.");
    if (a.eval_query_counts.empty()) a.eval_query_counts.push_back(a.num_queries);
    if (!a.rerank_top_n_values.empty() && a.rerank_top_n_values.size() != a.top_l_values.size())
        throw std::runtime_error("--rerank-top-n-values must have one value per --top-l-values entry.");
    return a;
}

template <typename Matrix, typename T>
Matrix LoadMatrix(const std::filesystem::path& path, bool allow_trailing_distances) {
    std::ifstream in(path, std::ios::binary);
    if (!in.is_open()) throw std::runtime_error("Failed to open matrix: " + path.string());
    Matrix m;
    in.read(reinterpret_cast<char*>(&m.rows), 4);
    in.read(reinterpret_cast<char*>(&m.cols), 4);
    if (!in.good() || m.rows == 0 || m.cols == 0) throw std::runtime_error("Invalid matrix header: " + path.string());
    const std::uint64_t body = static_cast<std::uint64_t>(m.rows) * m.cols * sizeof(T);
    const std::uint64_t size = std::filesystem::file_size(path);
    if (size != 8 + body && !(allow_trailing_distances && size == 8 + 2 * body))
        throw std::runtime_error("Unsupported file layout: " + path.string());
    m.values.resize(static_cast<std::size_t>(m.rows) * m.cols);
    in.read(reinterpret_cast<char*>(m.values.data()), static_cast<std::streamsize>(body));
    if (static_cast<std::uint64_t>(in.gcount()) != body) throw std::runtime_error("Short read: " + path.string());
    return m;
}

// tools/topoanns_eval_sift.cpp:570-590
double RecallAtK(const topoanns::TopoAnnsBatchResult& result, const IntMatrix& gt, std::size_t gt_offset, std::size_t top_k) {
    std::size_t matched = 0;
    for (std::size_t q = 0; q < result.queries.size(); ++q) {
        const std::int32_t* row = gt.values.data() + (gt_offset + q) * static_cast<std::size_t>(gt.cols);
        for (const auto& c : result.queries[q].rerank.topk)
            for (std::size_t r = 0; r < top_k; ++r)
                if (static_cast<std::int32_t>(c.node_id) == row[r]) { ++matched; break; }
    }
    return static_cast<double>(matched) / static_cast<double>(result.queries.size() * top_k);
}

// :1068-1086
std::vector<SweepPoint> ParetoFrontier(std::vector<SweepPoint> points) {
    std::sort(points.begin(), points.end(), [](const SweepPoint& l, const SweepPoint& r) {
        if (l.recall != r.recall) return l.recall < r.recall;
        return l.qps > r.qps;
    });
    std::vector<SweepPoint> frontier;
    double best = -1.0;
    for (auto it = points.rbegin(); it != points.rend(); ++it)
        if (it->qps > best) { frontier.push_back(*it); best = it->qps; }
    std::reverse(frontier.begin(), frontier.end());
    return frontier;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        const Args args = Parse(argc, argv);
        const FloatMatrix queries = LoadMatrix<FloatMatrix, float>(args.query_bin, false);
        if (args.num_queries > queries.rows) throw std::runtime_error("Requested num_queries exceeds query file rows.");
        IntMatrix gt;
        if (args.has_gt) {
            gt = LoadMatrix<IntMatrix, std::int32_t>(args.gt_bin, true);
            if (args.num_queries > gt.rows || args.top_k > gt.cols)
                throw std::runtime_error("GT rows/cols are smaller than requested evaluation.");
        }
        topoanns::SearchResources resources = topoanns::SearchResources::FromTopologyFile(args.index_dir / "topology.bin");
        resources.LoadPqIndex(args.index_dir / "_pq_pivots.bin", args.index_dir / "_pq_compressed.bin");
        if (!args.pq2_pivots.empty()) resources.LoadPq2Index(args.pq2_pivots, args.pq2_codes, args.pq2_error_bounds);
        resources.LoadVectorStore(args.index_dir / "vectors.ssd");
        if (args.vector_residency == "pinned-host")
            resources.AttachVectorPageProvider(std::make_shared<topoanns::PinnedHostVectorPageProvider>(args.index_dir / "vectors.ssd"));
        else
            resources.AttachVectorPageProvider(std::make_shared<topoanns::HbmVectorPageProvider>(args.index_dir / "vectors.ssd"));
        if (args.topology_residency == "pinned-host")
            resources.mutable_topology().SetResidency(topoanns::TopologyResidency::kPinnedHost, args.topology_cached_rows);
        if (args.neighbor_code_layout) resources.BuildNeighborCodeLayout();
        if (resources.vector_store_header().dim != queries.cols) throw std::runtime_error("Query dim and vector store dim do not match.");
        topoanns::RvqModel rvq_model = topoanns::RvqModel::Load(args.rvq_model);
        if (rvq_model.dim() != queries.cols) throw std::runtime_error("RVQ model dim and query dim do not match.");
        rvq_model.WarmUp();
        std::cout << "[topoanns_eval] providers vectors=" << args.vector_residency << " topology=" << args.topology_residency
                  << " topology_cached_rows=" << args.topology_cached_rows << std::endl;

        std::vector<SweepPoint> sweep;
        for (std::size_t li = 0; li < args.top_l_values.size(); ++li) {
            const std::size_t top_l = args.top_l_values[li];
            std::vector<std::size_t> top_ns = args.rerank_top_n_sweep_values;
            if (top_ns.empty()) top_ns.push_back(args.rerank_top_n_values.empty() ? args.rerank_top_n : args.rerank_top_n_values[li]);
            for (const std::size_t rerank_top_n : top_ns) {
                for (const std::size_t eval_queries : args.eval_query_counts) {
                    if (eval_queries > args.num_queries) throw std::runtime_error("eval query count exceeds --num-queries.");
                    const std::size_t batch = std::min(args.batch_size, eval_queries);
                    topoanns::TopoAnnsSearchParams params;
                    params.topology.top_k = std::max(args.top_k, rerank_top_n);
                    params.topology.top_l = top_l;
                    params.topology.search_width = args.search_width;
                    params.topology.max_expansions = args.max_expansions;
                    params.rerank.top_k = args.top_k;
                    params.rerank.top_n = rerank_top_n;
                    params.rerank.mode = args.rerank_mode;
                    params.rerank.rank_tile_size = args.rank_tile_size;
                    params.rerank.use_pq2_refine = args.use_pq2_refine;
                    params.rerank.use_pq2_bound_filter = args.use_pq2_bound_filter;
                    params.rerank.pq2_refine_top_l = top_l;
                    params.rerank.use_early_stop = args.use_early_stop;
                    params.rerank.early_stop_min_prefix = args.early_stop_min_prefix;
                    params.rerank.early_stop_patience_tiles = args.early_stop_patience_tiles;
                    params.rerank.use_learned_stop = args.use_learned_stop;
                    params.rerank.learned_stop_model_path = args.learned_stop_model;
                    std::size_t stop_queries = 0, stop_prefix_sum = 0, stop_prefix_min = 0, stop_prefix_max = 0, stop_checkpoints = 0;
                    double best_elapsed = 0.0, recall = -1.0;
                    std::size_t io_pages = 0, exact = 0, filtered = 0, visited = 0, expanded = 0;
                    for (std::size_t rep = 0; rep < args.repeats; ++rep) {   // the first pass is the cold one
                        double recall_sum = 0.0;
                        io_pages = exact = filtered = visited = expanded = 0;
                        stop_queries = stop_prefix_sum = stop_prefix_min = stop_prefix_max = stop_checkpoints = 0;
                        const auto start = std::chrono::steady_clock::now();
                        for (std::size_t off = 0; off < eval_queries; off += batch) {
                            const std::size_t n = std::min(batch, eval_queries - off);
                            const float* begin = queries.values.data() + off * static_cast<std::size_t>(queries.cols);
                            std::vector<float> buffer(begin, begin + n * static_cast<std::size_t>(queries.cols));
                            topoanns::DeviceEntryBatch entries =
                                rvq_model.ComputeFloat32DeviceEntryBatch(buffer, n, args.rvq_entry_count, 0, nullptr);
                            const topoanns::TopoAnnsBatchResult result =
                                topoanns::TopoAnnsSearch::RunBatchFloat32Fused(resources, entries, buffer, n, params);
                            io_pages += result.rerank_stats.io_pages;
                            exact += result.rerank_stats.exact_distance_count;
                            filtered += result.rerank_stats.bound_filtered_count;
                            const topoanns::RerankBatchProfile& rp = result.rerank_profile;
                            if (rp.learned_stop_queries != 0) {
                                stop_prefix_min = stop_queries == 0 ? rp.learned_stop_prefix_min : std::min(stop_prefix_min, rp.learned_stop_prefix_min);
                                stop_prefix_max = std::max(stop_prefix_max, rp.learned_stop_prefix_max);
                                stop_queries += rp.learned_stop_queries;
                                stop_prefix_sum += rp.learned_stop_prefix_sum;
                                stop_checkpoints += rp.learned_stop_checkpoints;
                            }
                            for (const auto& q : result.queries) {
                                visited += q.topology.stats.visited_nodes;
                                expanded += q.topology.stats.expanded_nodes;
                            }
                            if (args.has_gt) recall_sum += RecallAtK(result, gt, off, args.top_k) * static_cast<double>(n);
                            if (rep == 0)
                                std::cout << "[topoanns_eval] frontier_pq_mode=default top_l=" << top_l << " rerank_top_n=" << rerank_top_n
                                          << " finished queries " << (off + n) << " / " << eval_queries << std::endl;
                        }
                        const double elapsed = std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count();
                        if (rep == 0 || elapsed < best_elapsed) best_elapsed = elapsed;
                        if (args.has_gt) recall = recall_sum / static_cast<double>(eval_queries);
                    }
                    const double qps = best_elapsed > 0.0 ? static_cast<double>(eval_queries) / best_elapsed : 0.0;
                    const double nq = static_cast<double>(eval_queries);
                    std::cout << "[topoanns_eval] frontier_pq_mode=default top_l=" << top_l << " rerank_top_n=" << rerank_top_n
                              << " rerank_mode=" << ModeName(args.rerank_mode) << " queries=" << eval_queries
                              << " elapsed_sec=" << best_elapsed << " wall_elapsed_sec=" << best_elapsed << " qps=" << qps
                              << " wall_qps=" << qps;
                    if (recall >= 0.0) std::cout << " recall@10=" << recall;
                    std::cout << " avg_io_pages=" << io_pages / nq << " avg_exact=" << exact / nq << " avg_bound_filtered=" << filtered / nq
                              << " avg_visited=" << visited / nq << " avg_expanded=" << expanded / nq;
                    if (args.use_learned_stop)   // tools/topoanns_eval_sift.cpp:804-857
                        std::cout << " avg_learned_checkpoints=" << stop_checkpoints / nq << " learned_stop_queries=" << stop_queries
                                  << " avg_learned_stop_prefix=" << stop_prefix_sum / nq << " learned_stop_prefix_min=" << stop_prefix_min
                                  << " learned_stop_prefix_max=" << stop_prefix_max;
                    std::cout << std::endl;
                    sweep.push_back(SweepPoint{top_l, rerank_top_n, args.rerank_mode, eval_queries, qps, qps, recall});
                }
            }
        }
        for (const SweepPoint& p : ParetoFrontier(sweep))
            std::cout << "[topoanns_pareto] frontier_pq_mode=default top_l=" << p.top_l << " rerank_top_n=" << p.rerank_top_n
                      << " rerank_mode=" << ModeName(p.mode) << " queries=" << p.num_queries << " qps=" << p.qps
                      << " wall_qps=" << p.wall_qps << " recall@10=" << p.recall << std::endl;
        return 0;
    } catch (const std::exception& e) {
        std::cerr << "topoanns_eval_sift: " << e.what() << std::endl;
        return 2;
    }
}
