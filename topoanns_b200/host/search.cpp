// Search entry points of the API over the C ABI: query tables / oracle, traversal, rerank and the
// whole-path drivers. Control flow, parameter rules, error texts and result shapes follow the
// reference (src/search/pq_query_tables.cu, pq_distance_oracle.cpp, topology_search.cpp,
// topology_search_kernel.cu:3135-3169,3728-3877, rerank_exact.cu:1205-1737,2533-2695,
// topoanns_search.cpp); the device work is one C-ABI call per stage.
#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <unordered_set>

#include "topoanns/api.hpp"

namespace topoanns {
namespace {

using Clock = std::chrono::steady_clock;
double MsSince(const Clock::time_point& t0) { return std::chrono::duration<double, std::milli>(Clock::now() - t0).count(); }

struct DeviceCand {  // the 8-byte candidate record of the C ABI
    float distance;
    std::uint32_t node_id;
};
constexpr std::uint32_t kExpandedBit = 0x80000000u;

std::uint32_t NextPow2(std::size_t v) {
    std::uint32_t p = 1;
    while (p < v) p <<= 1;
    return p;
}

std::string Trim(std::string s) {
    const char* ws = " \t\r\n";
    const std::size_t b = s.find_first_not_of(ws);
    if (b == std::string::npos) return "";
    return s.substr(b, s.find_last_not_of(ws) - b + 1);
}
bool EnvTruthy(const char* name) {
    const char* env = std::getenv(name);
    if (env == nullptr) return false;
    const std::string v = Trim(env);
    return !(v.empty() || v == "0" || v == "false" || v == "FALSE");
}
template <typename T, typename F>
std::vector<T> ParseCsv(const std::string& value, F conv) {
    std::vector<T> out;
    std::stringstream ss(value);
    std::string item;
    while (std::getline(ss, item, ',')) {
        item = Trim(item);
        if (!item.empty()) out.push_back(conv(item));
    }
    return out;
}

// Learned traversal-stop model: text file of key=value lines named by TOPOANNS_LEARNED_STOP_MODEL;
// mean / inverse-std are folded into the weights and the bias
// (src/search/topology_search_kernel.cu:248-380).
TannLearnedStop LoadLearnedStop(const std::string& path, std::uint32_t top_l, std::uint32_t top_k) {
    std::ifstream in(path);
    if (!in.is_open()) throw std::runtime_error(BuildErrorMessage("LoadLearnedStopConfigFromFile", "Failed to open " + path));
    std::vector<std::uint32_t> prefixes, mask;
    std::vector<float> means, inv_stds, weights;
    float bias = 0.0f, threshold = 0.0f;
    std::uint32_t file_top_k = 0;
    std::string churn_mode, next64_mode, line;
    std::map<std::uint32_t, float> per_l;
    auto to_f = [](const std::string& s) { return std::stof(s); };
    auto to_u = [](const std::string& s) { return static_cast<std::uint32_t>(std::stoul(s)); };
    while (std::getline(in, line)) {
        line = Trim(line);
        if (line.empty() || line[0] == '#') continue;
        const std::size_t eq = line.find('=');
        if (eq == std::string::npos)
            throw std::runtime_error(BuildErrorMessage("LoadLearnedStopConfigFromFile", "Invalid learned-stop config line: " + line));
        const std::string key = Trim(line.substr(0, eq)), value = Trim(line.substr(eq + 1));
        const std::string per_l_prefix = "threshold_logit_top_l_";
        if (key == "stage_prefixes") prefixes = ParseCsv<std::uint32_t>(value, to_u);
        else if (key == "feature_means") means = ParseCsv<float>(value, to_f);
        else if (key == "feature_inv_stds") inv_stds = ParseCsv<float>(value, to_f);
        else if (key == "weights") weights = ParseCsv<float>(value, to_f);
        else if (key == "bias") bias = std::stof(value);
        else if (key == "threshold_logit") threshold = std::stof(value);
        else if (key == "top_k") file_top_k = to_u(value);
        else if (key == "topk_churn_mode") churn_mode = value;
        else if (key == "next64_mode") next64_mode = value;
        else if (key == "feature_mask") mask = ParseCsv<std::uint32_t>(value, to_u);
        else if (key.rfind(per_l_prefix, 0) == 0 && key.size() > per_l_prefix.size())
            per_l[to_u(key.substr(per_l_prefix.size()))] = std::stof(value);
    }
    if (means.size() != TANN_STOP_FEATURES || inv_stds.size() != TANN_STOP_FEATURES || weights.size() != TANN_STOP_FEATURES)
        throw std::runtime_error(BuildErrorMessage("LoadLearnedStopConfigFromFile",
                                                   "learned-stop feature vectors must all have length 12."));
    TannLearnedStop c{};
    c.top_k = file_top_k != 0 ? file_top_k : top_k;
    c.inv_top_l = top_l == 0 ? 0.0f : 1.0f / static_cast<float>(top_l);
    c.shadow_mode = EnvTruthy("TOPOANNS_LEARNED_STOP_SHADOW") ? 1u : 0u;
    c.topk_churn_flag_mode = churn_mode == "flag" ? 1u : 0u;
    c.next64_flag_mode = next64_mode == "flag" ? 1u : 0u;
    const auto it = per_l.find(top_l);
    c.threshold_logit = it != per_l.end() ? it->second : threshold;
    float folded_bias = bias;
    for (std::size_t i = 0; i < TANN_STOP_FEATURES; ++i) {
        c.feature_mask[i] = i < mask.size() ? mask[i] : 1u;
        const float w = c.feature_mask[i] != 0 ? weights[i] : 0.0f;
        c.weights[i] = w * inv_stds[i];
        folded_bias -= means[i] * c.weights[i];
    }
    c.bias = folded_bias;
    for (std::uint32_t p : prefixes) {
        if (p == 0 || p >= top_l) continue;
        if (c.num_stages >= TANN_MAX_STOP_STAGES) break;
        c.stage_prefixes[c.num_stages++] = p;
    }
    c.enabled = c.num_stages == 0 ? 0u : 1u;
    if (c.top_k == 0 || c.top_k > 32) c.enabled = 0;
    return c;
}

// TopologySearchParams + the result-affecting environment switches -> kernel parameters
// (src/search/topology_search_kernel.cu:3207-3213,3445-3486).
TannBeamParams MakeBeamParams(const TopologySearchParams& p) {
    TannBeamParams b{};
    b.top_l = static_cast<std::uint32_t>(p.top_l);
    b.search_width = static_cast<std::uint32_t>(p.search_width);
    b.max_expansions = static_cast<std::uint32_t>(std::min<std::size_t>(p.max_expansions, 0xffffffffu));
    const std::size_t limit = std::max(p.top_l, p.candidate_queue_size == 0 ? p.top_l : p.candidate_queue_size);
    b.candidate_capacity = NextPow2(limit);
    std::uint32_t divisor = 1, min_prefix = 32;
    if (const char* e = std::getenv("TOPOANNS_CANDIDATE_STOP_DIVISOR")) {
        const auto v = static_cast<std::uint32_t>(std::strtoul(e, nullptr, 10));
        if (v > 1) divisor = v;
    }
    if (const char* e = std::getenv("TOPOANNS_CANDIDATE_STOP_MIN_PREFIX")) {
        const auto v = static_cast<std::uint32_t>(std::strtoul(e, nullptr, 10));
        if (v != 0) min_prefix = v;
    }
    b.stop_prefix = b.top_l;
    if (divisor > 1) b.stop_prefix = std::min(std::max(min_prefix, b.top_l / divisor), b.top_l);
    if (const char* e = std::getenv("TOPOANNS_CANDIDATE_STOP_PREFIX")) {
        const auto v = static_cast<std::uint32_t>(std::strtoul(e, nullptr, 10));
        if (v != 0) b.stop_prefix = std::min(v, b.top_l);
    }
    b.stop_use_expanded = EnvTruthy("TOPOANNS_CANDIDATE_STOP_USE_EXPANDED") ? 1u : 0u;
    if (const char* e = std::getenv("TOPOANNS_LEARNED_STOP_MODEL"))
        b.learned_stop = LoadLearnedStop(e, b.top_l, static_cast<std::uint32_t>(p.top_k));
    return b;
}

void ValidateTopologyParams(const TopologySearchParams& p, const char* ctx) {
    if (p.top_k == 0) throw std::runtime_error(BuildErrorMessage(ctx, "top_k must be positive."));
    if (p.top_l == 0) throw std::runtime_error(BuildErrorMessage(ctx, "top_l must be positive."));
    if (p.candidate_queue_size != 0 && p.candidate_queue_size < p.top_l)
        throw std::runtime_error(BuildErrorMessage(ctx, "candidate_queue_size must be zero or at least top_l."));
    if (p.search_width == 0) throw std::runtime_error(BuildErrorMessage(ctx, "search_width must be positive."));
}

struct DeviceTraversal {
    std::size_t num_queries = 0;
    std::uint32_t capacity = 0;
    CudaBuffer<DeviceCand> candidates;
    CudaBuffer<std::uint32_t> stats;  // 8 per query
    double kernel_ms = 0.0;
};

// One traversal launch; `lut` may be null (table built inside the kernel from device queries).
DeviceTraversal RunTraversal(const SearchResources& resources, const TopologySearchParams& params, const float* lut,
                             const void* device_queries, std::uint32_t query_kind, std::size_t num_queries,
                             const std::uint32_t* entry_offsets, const std::uint32_t* entry_ids) {
    const char* ctx = "RunTopologySearchKernelBatch";
    DeviceTraversal out;
    out.num_queries = num_queries;
    if (num_queries == 0) return out;
    if (params.search_width > TANN_MAX_SEARCH_WIDTH) throw std::runtime_error(BuildErrorMessage(ctx, "search_width must be at most 32."));
    const TannBeamParams bp = MakeBeamParams(params);
    const TannIndexView view = resources.MakeIndexView(false);
    out.capacity = bp.candidate_capacity;
    out.candidates = CudaBuffer<DeviceCand>::Allocate(num_queries * out.capacity);
    out.stats = CudaBuffer<std::uint32_t>::Allocate(num_queries * 8);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    ThrowIfCudaError(cudaEventCreate(&e0), "cudaEventCreate");
    ThrowIfCudaError(cudaEventCreate(&e1), "cudaEventCreate");
    ThrowIfCudaError(cudaEventRecord(e0), "cudaEventRecord");
    const TannStatus st = tann_beam_search(&view, &bp, lut, device_queries, query_kind, num_queries, entry_offsets,
                                           entry_ids, out.candidates.get(), out.stats.get(), nullptr, nullptr);
    if (st != TANN_OK) {
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        ThrowIfTannError(st, ctx);
    }
    ThrowIfCudaError(cudaEventRecord(e1), "cudaEventRecord");
    ThrowIfCudaError(cudaEventSynchronize(e1), "cudaEventSynchronize");
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    out.kernel_ms = ms;
    return out;
}

std::size_t RankIndex(std::size_t n, std::size_t num, std::size_t den) {
    const std::size_t rank = (num * n + den - 1) / den;
    return std::min(n - 1, std::max<std::size_t>(1, rank) - 1);
}

void FillBatchSummaries(const std::vector<std::uint32_t>& stats, TopologySearchBatchProfile* p) {
    const std::size_t n = stats.size() / 8;
    if (n == 0) return;
    std::vector<std::size_t> expanded(n), iterations(n), full;
    for (std::size_t q = 0; q < n; ++q) {
        expanded[q] = stats[q * 8 + 1];
        iterations[q] = stats[q * 8 + 3];
        if (stats[q * 8 + 5] != 0xffffffffu) full.push_back(stats[q * 8 + 5]);
    }
    auto summarize = [](std::vector<std::size_t> v, double* avg, std::size_t* p50, std::size_t* p95, std::size_t* mx) {
        if (v.empty()) return;
        std::sort(v.begin(), v.end());
        std::size_t total = 0;
        for (std::size_t x : v) total += x;
        *avg = static_cast<double>(total) / static_cast<double>(v.size());
        *p50 = v[RankIndex(v.size(), 50, 100)];
        *p95 = v[RankIndex(v.size(), 95, 100)];
        *mx = v.back();
    };
    std::sort(expanded.begin(), expanded.end());
    p->batch_max_expanded_nodes = expanded.back();
    p->batch_p95_expanded_nodes = expanded[RankIndex(n, 95, 100)];
    summarize(iterations, &p->batch_avg_iterations, &p->batch_p50_iterations, &p->batch_p95_iterations, &p->batch_max_iterations);
    p->batch_full_prefix_reached_queries = full.size();
    summarize(full, &p->batch_avg_full_prefix_iteration, &p->batch_p50_full_prefix_iteration,
              &p->batch_p95_full_prefix_iteration, &p->batch_max_full_prefix_iteration);
}

// Device candidate lists -> per-query results (src/search/topology_search_kernel.cu:3135-3169,3728-3840).
std::vector<TopologySearchResult> Materialize(const DeviceTraversal& t, const TopologySearchParams& params,
                                              TopologySearchBatchProfile* out_profile) {
    std::vector<TopologySearchResult> results(t.num_queries);
    if (t.num_queries == 0) return results;
    const std::size_t limit = std::max(params.top_l, params.candidate_queue_size == 0 ? params.top_l : params.candidate_queue_size);
    auto t0 = Clock::now();
    const std::vector<DeviceCand> cand = t.candidates.CopyToHost();
    const double cand_ms = MsSince(t0);
    t0 = Clock::now();
    const std::vector<std::uint32_t> stats = t.stats.CopyToHost();
    const double stats_ms = MsSince(t0);
    t0 = Clock::now();
    for (std::size_t q = 0; q < t.num_queries; ++q) {
        TopologySearchResult& r = results[q];
        r.sorted_candidates.reserve(limit);
        for (std::uint32_t i = 0; i < t.capacity && r.sorted_candidates.size() < limit; ++i) {
            const DeviceCand& c = cand[q * t.capacity + i];
            if (c.node_id == kInvalidNodeId) continue;
            r.sorted_candidates.push_back(RankedCandidate{c.distance, c.node_id & ~kExpandedBit, (c.node_id & kExpandedBit) != 0});
        }
        for (const RankedCandidate& c : r.sorted_candidates) {
            if (!c.valid()) continue;
            r.topk.push_back(c);
            if (r.topk.size() == params.top_k) break;
        }
        r.stats.visited_nodes = stats[q * 8 + 0];
        r.stats.expanded_nodes = stats[q * 8 + 1];
        r.stats.topology_io_pages = stats[q * 8 + 2];
        r.stats.iterations = stats[q * 8 + 3];
    }
    if (out_profile != nullptr) {
        out_profile->kernel_ms += t.kernel_ms;
        out_profile->candidate_download_ms += cand_ms;
        out_profile->stats_download_ms += stats_ms;
        out_profile->host_postprocess_ms += MsSince(t0);
        FillBatchSummaries(stats, out_profile);
    }
    return results;
}

std::vector<TopologySearchResult> RunHostEntries(const SearchResources& resources, const PqDistanceOracle& oracle,
                                                 const std::vector<std::vector<std::uint32_t>>& entries,
                                                 std::size_t query_offset, std::size_t num_queries,
                                                 const TopologySearchParams& params, TopologySearchBatchProfile* profile) {
    if (entries.size() < num_queries)
        throw std::runtime_error(BuildErrorMessage("RunTopologySearchKernelBatch", "entries_by_query is smaller than num_queries."));
    if (query_offset + num_queries > oracle.num_queries())
        throw std::runtime_error(BuildErrorMessage("RunTopologySearchKernelBatch", "query range is out of bounds."));
    std::vector<std::uint32_t> offsets(num_queries + 1, 0), ids;
    for (std::size_t q = 0; q < num_queries; ++q) {
        offsets[q + 1] = offsets[q] + static_cast<std::uint32_t>(entries[q].size());
        ids.insert(ids.end(), entries[q].begin(), entries[q].end());
    }
    const CudaBuffer<std::uint32_t> d_offsets = CudaBuffer<std::uint32_t>::CopyFromHost(offsets);
    const CudaBuffer<std::uint32_t> d_ids = CudaBuffer<std::uint32_t>::CopyFromHost(ids.empty() ? std::vector<std::uint32_t>{kInvalidNodeId} : ids);
    const std::size_t stride = oracle.pq_index().host().num_chunks * kNumPqCentroids;
    const float* lut = oracle.query_tables().device_tables().get() + query_offset * stride;
    return Materialize(RunTraversal(resources, params, lut, nullptr, TANN_KIND_FLOAT32, num_queries, d_offsets.get(), d_ids.get()),
                       params, profile);
}

// ---- rerank helpers -----------------------------------------------------------------------------------------
struct DeviceRerank {
    std::vector<float> dists;          // [Q][top_n] sorted
    std::vector<std::uint32_t> ids;
    std::size_t n_exact = 0, n_filtered = 0;
    double kernel_ms = 0.0;
};

DeviceRerank RunRerankKernel(const SearchResources& resources, const TannIndexView& view, const TannRerankParams& rp,
                             const DeviceCand* cand, std::uint32_t capacity, std::size_t num_queries, const void* d_queries,
                             std::uint32_t query_kind, const float* error_bounds, const char* ctx) {
    (void)resources;
    DeviceRerank out;
    const std::size_t flat = num_queries * rp.top_n;
    CudaBuffer<float> d_dists = CudaBuffer<float>::Allocate(flat);
    CudaBuffer<std::uint32_t> d_ids = CudaBuffer<std::uint32_t>::Allocate(flat);
    CudaBuffer<unsigned long long> d_counts = CudaBuffer<unsigned long long>::CopyFromHost({0ull, 0ull});
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    ThrowIfCudaError(cudaEventCreate(&e0), "cudaEventCreate");
    ThrowIfCudaError(cudaEventCreate(&e1), "cudaEventCreate");
    ThrowIfCudaError(cudaEventRecord(e0), "cudaEventRecord");
    const TannStatus st = tann_rerank_exact(&view, &rp, cand, capacity, num_queries, d_queries, query_kind, error_bounds,
                                            d_dists.get(), d_ids.get(), d_counts.get(), nullptr, nullptr);
    if (st != TANN_OK) {
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        ThrowIfTannError(st, ctx);
    }
    ThrowIfCudaError(cudaEventRecord(e1), "cudaEventRecord");
    ThrowIfCudaError(cudaEventSynchronize(e1), "cudaEventSynchronize");
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    out.kernel_ms = ms;
    out.dists = d_dists.CopyToHost();
    out.ids = d_ids.CopyToHost();
    const std::vector<unsigned long long> counts = d_counts.CopyToHost();
    out.n_exact = counts[0];
    out.n_filtered = counts[1];
    return out;
}

// ---- learned rerank stop: stop-prefix traces ------------------------------------------------------------------
// File of records {u32 magic "RSP1", u32 budget_top_n, u32 num_queries, u32 prefix[num_queries]}, one per
// batch (src/io/rerank_stop_prefix_trace.hpp:16-88). A process truncates a record file the first time it
// writes to it and appends afterwards; a replay file is read record by record in batch order.
constexpr std::uint32_t kStopPrefixTraceMagic = 0x52535031u;
std::mutex g_trace_mutex;

void AppendStopPrefixTrace(const std::string& path, std::size_t budget_top_n, const std::vector<std::uint32_t>& prefixes) {
    static std::map<std::string, bool> written;
    std::lock_guard<std::mutex> lock(g_trace_mutex);
    bool& seen = written[path];
    std::ofstream out(path, std::ios::binary | (seen ? std::ios::app : std::ios::trunc));
    if (!out.is_open()) throw std::runtime_error("Failed to open rerank stop-prefix trace for writing: " + path);
    const std::uint32_t header[3] = {kStopPrefixTraceMagic, static_cast<std::uint32_t>(budget_top_n),
                                     static_cast<std::uint32_t>(prefixes.size())};
    out.write(reinterpret_cast<const char*>(header), sizeof(header));
    out.write(reinterpret_cast<const char*>(prefixes.data()), static_cast<std::streamsize>(prefixes.size() * sizeof(std::uint32_t)));
    if (!out) throw std::runtime_error("Failed to write rerank stop-prefix trace: " + path);
    seen = true;
}

std::vector<std::uint32_t> ReadStopPrefixTrace(const std::string& path, std::size_t budget_top_n, std::size_t num_queries) {
    static std::map<std::string, std::unique_ptr<std::ifstream>> open_files;
    std::lock_guard<std::mutex> lock(g_trace_mutex);
    std::unique_ptr<std::ifstream>& in = open_files[path];
    if (!in) in = std::make_unique<std::ifstream>(path, std::ios::binary);
    if (!in->is_open()) throw std::runtime_error("Failed to open rerank stop-prefix trace for reading: " + path);
    std::uint32_t header[3] = {0, 0, 0};
    in->read(reinterpret_cast<char*>(header), sizeof(header));
    if (!*in || header[0] != kStopPrefixTraceMagic || header[1] != budget_top_n || header[2] != num_queries)
        throw std::runtime_error("Rerank stop-prefix trace mismatch or premature EOF: " + path);
    std::vector<std::uint32_t> prefixes(num_queries);
    in->read(reinterpret_cast<char*>(prefixes.data()), static_cast<std::streamsize>(prefixes.size() * sizeof(std::uint32_t)));
    if (!*in) throw std::runtime_error("Truncated rerank stop-prefix trace payload: " + path);
    return prefixes;
}

std::string EnvOrEmpty(const char* name) {
    const char* v = std::getenv(name);
    return v == nullptr ? std::string{} : std::string(v);
}

struct DeviceLearnedRerank {
    std::vector<float> dists;          // [Q][top_k] sorted
    std::vector<std::uint32_t> ids;
    std::vector<std::uint32_t> stop_prefixes, checkpoint_counts;
    std::size_t n_exact = 0, n_filtered = 0;
    bool evaluated = false;            // the model ran (no replay, model enabled)
    double kernel_ms = 0.0;
};

// Host side of the persistent rerank with the learned stop (RunPersistentBamRerankFloat32,
// src/io/bam_vector_provider.cu:2471-2774): model file, record / replay environment variables, one kernel.
DeviceLearnedRerank RunLearnedRerankKernel(const TannIndexView& view, const TannRerankParams& rp, const RerankExactParams& params,
                                           const DeviceCand* cand, std::uint32_t capacity, std::size_t num_queries,
                                           const void* d_queries, const float* error_bounds) {
    const char* ctx = "RunPersistentBamRerankFloat32";
    const std::size_t budget = std::min<std::size_t>(rp.top_n, capacity);
    const std::string record_path = EnvOrEmpty("TOPOANNS_RERANK_STOP_PREFIX_RECORD_PATH");
    const std::string replay_path = EnvOrEmpty("TOPOANNS_RERANK_STOP_PREFIX_REPLAY_PATH");
    if (!record_path.empty() && !replay_path.empty())
        throw std::runtime_error(BuildErrorMessage(ctx, "Record and replay modes are mutually exclusive."));
    TannRerankLearnedStop model{};
    ThrowIfTannError(tann_rerank_learned_stop_load(params.learned_stop_model_path.string().c_str(),
                                                   static_cast<std::uint32_t>(budget), rp.top_k, &model), ctx);
    CudaBuffer<std::uint32_t> d_replay;
    if (!replay_path.empty()) {
        const std::vector<std::uint32_t> prefixes = ReadStopPrefixTrace(replay_path, budget, num_queries);
        for (std::uint32_t prefix : prefixes)
            if (prefix < rp.top_k || prefix > budget) throw std::runtime_error(BuildErrorMessage(ctx, "Invalid replay stop prefix."));
        d_replay = CudaBuffer<std::uint32_t>::CopyFromHost(prefixes);
    }
    DeviceLearnedRerank out;
    out.evaluated = model.enabled != 0 && replay_path.empty();
    const std::size_t flat = num_queries * rp.top_k;
    CudaBuffer<float> d_dists = CudaBuffer<float>::Allocate(flat);
    CudaBuffer<std::uint32_t> d_ids = CudaBuffer<std::uint32_t>::Allocate(flat);
    CudaBuffer<unsigned long long> d_counts = CudaBuffer<unsigned long long>::CopyFromHost({0ull, 0ull});
    CudaBuffer<std::uint32_t> d_prefixes = CudaBuffer<std::uint32_t>::Allocate(num_queries);
    CudaBuffer<std::uint32_t> d_checkpoints = CudaBuffer<std::uint32_t>::Allocate(num_queries);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    ThrowIfCudaError(cudaEventCreate(&e0), "cudaEventCreate");
    ThrowIfCudaError(cudaEventCreate(&e1), "cudaEventCreate");
    ThrowIfCudaError(cudaEventRecord(e0), "cudaEventRecord");
    const TannStatus st = tann_rerank_exact_learned_stop(&view, &rp, &model, cand, capacity, num_queries, d_queries,
                                                         TANN_KIND_FLOAT32, error_bounds, replay_path.empty() ? nullptr : d_replay.get(),
                                                         d_dists.get(), d_ids.get(), d_counts.get(), d_prefixes.get(),
                                                         d_checkpoints.get(), nullptr, nullptr, nullptr);
    if (st != TANN_OK) {
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        ThrowIfTannError(st, ctx);
    }
    ThrowIfCudaError(cudaEventRecord(e1), "cudaEventRecord");
    ThrowIfCudaError(cudaEventSynchronize(e1), "cudaEventSynchronize");
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    out.kernel_ms = ms;
    out.dists = d_dists.CopyToHost();
    out.ids = d_ids.CopyToHost();
    out.stop_prefixes = d_prefixes.CopyToHost();
    out.checkpoint_counts = d_checkpoints.CopyToHost();
    const std::vector<unsigned long long> counts = d_counts.CopyToHost();
    out.n_exact = counts[0];
    out.n_filtered = counts[1];
    if (out.evaluated && !record_path.empty()) AppendStopPrefixTrace(record_path, budget, out.stop_prefixes);
    return out;
}

template <typename QueryT>
std::uint32_t KindOf();
template <> std::uint32_t KindOf<float>() { return TANN_KIND_FLOAT32; }
template <> std::uint32_t KindOf<std::uint8_t>() { return TANN_KIND_UINT8; }
template <> std::uint32_t KindOf<std::int8_t>() { return TANN_KIND_INT8; }

// Host-materialised rerank (src/search/rerank_exact.cu:1426-1737): the first top_n valid candidates
// of every query, one exact distance each, (distance, id) sort, first top_k.
template <typename QueryT>
RerankBatchResult RerankFromHostResults(const SearchResources& resources, const std::vector<TopologySearchResult>& topo,
                                        const std::vector<QueryT>& queries, std::size_t num_queries,
                                        const RerankExactParams& params, const char* ctx, RerankBatchProfile* out_profile) {
    const auto total_begin = Clock::now();
    if (!resources.has_vector_store()) throw std::runtime_error(BuildErrorMessage(ctx, "Vector store must be loaded before rerank."));
    const VectorStoreHeader& header = resources.vector_store_header();
    const VectorPageLayout& layout = resources.vector_store_layout();
    if (topo.size() != num_queries) throw std::runtime_error(BuildErrorMessage(ctx, "topology_results.size() must equal num_queries."));
    if (queries.size() != num_queries * header.dim) throw std::runtime_error(BuildErrorMessage(ctx, "query buffer size must equal num_queries * dim."));
    RerankBatchResult result;
    result.queries.resize(num_queries);
    const std::uint32_t top_n = static_cast<std::uint32_t>(params.top_n);
    std::vector<DeviceCand> flat(num_queries * std::max<std::size_t>(top_n, 1), DeviceCand{std::numeric_limits<float>::infinity(), kInvalidNodeId});
    std::unordered_set<std::uint64_t> pages;
    std::size_t count = 0;
    for (std::size_t q = 0; q < num_queries; ++q) {
        const auto& sorted = topo[q].sorted_candidates;
        const std::size_t limit = std::min<std::size_t>(params.top_n, sorted.size());
        std::size_t w = 0;
        for (std::size_t r = 0; r < limit; ++r) {
            if (!sorted[r].valid()) continue;
            flat[q * top_n + w++] = DeviceCand{sorted[r].distance, sorted[r].node_id};
            pages.insert(layout.Resolve(sorted[r].node_id).page_id);
            ++count;
        }
    }
    result.stats.exact_distance_count = count;
    if (count == 0 || top_n == 0) return result;
    result.stats.io_pages = pages.size();
    const double prepare_ms = MsSince(total_begin);
    if (!resources.vector_page_provider().SupportsDeviceReads() || resources.vector_page_provider().DeviceReadHandle() == nullptr)
        throw std::runtime_error(BuildErrorMessage(ctx, "rerank requires a device-resident page provider (HBM, peer or pinned host)."));
    const TannIndexView view = resources.MakeIndexView(true);
    const CudaBuffer<DeviceCand> d_cand = CudaBuffer<DeviceCand>::CopyFromHost(flat);
    auto t0 = Clock::now();
    const CudaBuffer<QueryT> d_queries = CudaBuffer<QueryT>::CopyFromHost(queries);
    const double upload_ms = MsSince(t0);
    TannRerankParams rp{top_n, static_cast<std::uint32_t>(params.top_k), 0, 0, 0, 0, 0, 0};
    const DeviceRerank rr = RunRerankKernel(resources, view, rp, d_cand.get(), top_n, num_queries, d_queries.get(),
                                            KindOf<QueryT>(), nullptr, ctx);
    t0 = Clock::now();
    for (std::size_t q = 0; q < num_queries; ++q) {
        auto& out = result.queries[q];
        for (std::uint32_t r = 0; r < top_n; ++r) {
            const std::uint32_t id = rr.ids[q * top_n + r];
            if (id == kInvalidNodeId) break;  // only the flattened (valid) candidates are listed
            out.sorted_candidates.push_back(RankedCandidate{rr.dists[q * top_n + r], id, true});
        }
        for (const RankedCandidate& c : out.sorted_candidates) {
            out.topk.push_back(c);
            if (out.topk.size() == params.top_k) break;
        }
    }
    RerankBatchProfile& p = result.profile;
    p.prepare_ms = prepare_ms;
    p.query_upload_ms = upload_ms;
    p.exact_distance_kernel_ms = rr.kernel_ms;
    p.exact_distance_total_ms = upload_ms + rr.kernel_ms;
    p.sorted_candidates_materialize_ms = MsSince(t0);
    p.total_ms = MsSince(total_begin);
    if (out_profile != nullptr) {
        out_profile->total_ms += p.total_ms;
        out_profile->prepare_ms += p.prepare_ms;
        out_profile->query_upload_ms += p.query_upload_ms;
        out_profile->exact_distance_kernel_ms += p.exact_distance_kernel_ms;
        out_profile->exact_distance_total_ms += p.exact_distance_total_ms;
        out_profile->sorted_candidates_materialize_ms += p.sorted_candidates_materialize_ms;
    }
    return result;
}

// Device-fused rerank (src/search/rerank_exact.cu:2533-2695 and the drivers it dispatches to).
RerankBatchResult RerankFromDeviceTraversal(const SearchResources& resources, const DeviceTraversal& topo,
                                            const CudaBuffer<float>& d_queries, const std::vector<float>& queries,
                                            std::size_t num_queries, const RerankExactParams& params,
                                            RerankBatchProfile* out_profile) {
    const char* ctx = "RunBatchFloat32FromDeviceTopology";
    const auto total_begin = Clock::now();
    if (!resources.has_vector_store()) throw std::runtime_error(BuildErrorMessage(ctx, "Vector store must be loaded before rerank."));
    const VectorStoreHeader& header = resources.vector_store_header();
    if (queries.size() != num_queries * header.dim) throw std::runtime_error(BuildErrorMessage(ctx, "query buffer size must equal num_queries * dim."));
    if (topo.num_queries != num_queries) throw std::runtime_error(BuildErrorMessage(ctx, "topology_result size mismatch."));
    if (!resources.vector_page_provider().SupportsDeviceReads())
        throw std::runtime_error(BuildErrorMessage(ctx, "Fused rerank requires device-direct reads."));
    if (num_queries == 0 || params.top_n == 0) return RerankBatchResult{};
    if (params.use_pq2_bound_filter) {
        if (!params.use_pq2_refine) throw std::runtime_error(BuildErrorMessage(ctx, "PQ2 bound filter requires PQ2 refine to be enabled."));
        if (params.top_k == 0 || params.top_k > 128) throw std::runtime_error(BuildErrorMessage(ctx, "PQ2 bound filter requires 1 <= top_k <= 128."));
        if (params.mode == RerankExecutionMode::kLinear) throw std::runtime_error(BuildErrorMessage(ctx, "PQ2 bound filter requires a non-linear GPU rerank path."));
        if (!resources.has_pq2_error_bounds()) throw std::runtime_error(BuildErrorMessage(ctx, "PQ2 bound filter requires residual PQ2 error bounds."));
    }
    if (params.use_learned_stop) {   // src/search/rerank_exact.cu:2586-2602
        if (params.mode != RerankExecutionMode::kPersistent)
            throw std::runtime_error(BuildErrorMessage(ctx, "learned rerank stop requires the persistent GPU rerank path."));
        if (!params.use_pq2_bound_filter)
            throw std::runtime_error(BuildErrorMessage(ctx, "learned rerank stop requires PQ34 refine + bound filter."));
        if (params.learned_stop_model_path.empty())
            throw std::runtime_error(BuildErrorMessage(ctx, "learned rerank stop requires learned_stop_model_path."));
        if (params.top_k == 0 || params.top_k > 128)
            throw std::runtime_error(BuildErrorMessage(ctx, "learned rerank stop requires 1 <= top_k <= 128."));
    } else if (!EnvOrEmpty("TOPOANNS_RERANK_STOP_PREFIX_RECORD_PATH").empty() ||
               !EnvOrEmpty("TOPOANNS_RERANK_STOP_PREFIX_REPLAY_PATH").empty()) {
        if (params.mode == RerankExecutionMode::kPersistent)   // src/io/bam_vector_provider.cu:2541-2545
            throw std::runtime_error(BuildErrorMessage("RunPersistentBamRerankFloat32", "Stop-prefix profiling requires learned stop."));
    }
    if (params.use_early_stop) {
        if (params.mode != RerankExecutionMode::kPersistent && params.mode != RerankExecutionMode::kTiled)
            throw std::runtime_error(BuildErrorMessage(ctx, "rerank early stop requires the persistent or tiled mode."));
        if (params.top_k == 0 || params.top_k > 128) throw std::runtime_error(BuildErrorMessage(ctx, "rerank early stop requires 1 <= top_k <= 128."));
        if (params.early_stop_patience_tiles == 0) throw std::runtime_error(BuildErrorMessage(ctx, "rerank early stop requires early_stop_patience_tiles >= 1."));
    }
    if (params.top_k > params.top_n) throw std::runtime_error(BuildErrorMessage(ctx, "top_k must not exceed top_n."));

    RerankBatchResult result;
    RerankBatchProfile& prof = result.profile;
    const DeviceCand* cand = topo.candidates.get();
    std::uint32_t capacity = topo.capacity;
    CudaBuffer<DeviceCand> refined;
    CudaBuffer<float> lut2;
    if (params.use_pq2_refine) {
        const char* rctx = "RunPq2RefineBatchDevice";
        if (!resources.has_pq2_index()) throw std::runtime_error(BuildErrorMessage(rctx, "PQ2 index must be loaded."));
        const PqIndex& pq2 = resources.pq2_index();
        const std::uint32_t lr = static_cast<std::uint32_t>(
            std::min<std::size_t>(params.pq2_refine_top_l == 0 ? capacity : params.pq2_refine_top_l, capacity));
        const bool residual = resources.pq2_is_residual_refine();
        if (residual && !resources.has_pq_index())
            throw std::runtime_error(BuildErrorMessage(rctx, "Base PQ index must be loaded for residual PQ2 refine."));
        const auto t0 = Clock::now();
        const std::uint32_t M = static_cast<std::uint32_t>(pq2.host().num_chunks);
        lut2 = CudaBuffer<float>::Allocate(num_queries * M * kNumPqCentroids);
        ThrowIfTannError(tann_lut_build(pq2.device().tables_col_major.get(), pq2.device().centroid.get(),
                                        pq2.device().chunk_offsets.get(), static_cast<std::uint32_t>(pq2.host().ndims), M,
                                        d_queries.get(), TANN_KIND_FLOAT32, num_queries, lut2.get(), nullptr), rctx);
        refined = CudaBuffer<DeviceCand>::Allocate(num_queries * lr);
        TannShards pq2_codes{};
        pq2_codes.num_shards = 1;
        pq2_codes.base[0] = pq2.device_codes();
        TannShards base_codes{};
        base_codes.num_shards = 1;
        if (residual) base_codes.base[0] = resources.pq_index().device_codes();
        ThrowIfTannError(tann_pq2_refine(cand, topo.stats.get(), num_queries, capacity, lr, residual ? &base_codes : nullptr,
                                         &pq2_codes, M, lut2.get(), residual ? resources.pq2_cross_terms().get() : nullptr,
                                         refined.get(), nullptr, nullptr), rctx);
        ThrowIfCudaError(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        prof.pq2_refine_kernel_ms = MsSince(t0);
        prof.pq2_refine_top_l = lr;
        prof.pq2_refine_batches = 1;
        prof.pq2_residual_refine_batches = residual ? 1 : 0;
        cand = refined.get();
        capacity = lr;
    }
    std::uint32_t tile = 0;
    switch (params.mode) {
        case RerankExecutionMode::kLinear: tile = 0; break;
        case RerankExecutionMode::kPageByPage: tile = 1; break;
        case RerankExecutionMode::kTiled:
        case RerankExecutionMode::kPersistent:
            tile = static_cast<std::uint32_t>(std::max<std::size_t>(1, std::min(params.rank_tile_size, params.top_n)));
            break;
    }
    const TannIndexView view = resources.MakeIndexView(true);
    TannRerankParams rp{static_cast<std::uint32_t>(params.top_n), static_cast<std::uint32_t>(params.top_k), tile,
                        params.use_pq2_bound_filter ? 1u : 0u, params.use_early_stop ? 1u : 0u,
                        static_cast<std::uint32_t>(params.early_stop_min_prefix),
                        static_cast<std::uint32_t>(params.early_stop_patience_tiles), 0u};
    if (params.use_learned_stop) {
        // The persistent rerank keeps only the top_k list per query (result_top_n = top_k,
        // src/io/bam_vector_provider.cu:2546, src/search/rerank_exact.cu:2202-2228).
        const DeviceLearnedRerank lr = RunLearnedRerankKernel(view, rp, params, cand, capacity, num_queries, d_queries.get(),
                                                              resources.pq2_error_bounds_fp32().get());
        result.stats.exact_distance_count = lr.n_exact;
        result.stats.bound_filtered_count = lr.n_filtered;
        result.stats.io_pages = lr.n_exact;
        const auto t1 = Clock::now();
        result.queries.resize(num_queries);
        for (std::size_t q = 0; q < num_queries; ++q) {
            auto& out = result.queries[q];
            for (std::size_t r = 0; r < params.top_k; ++r) {
                const std::uint32_t id = lr.ids[q * params.top_k + r];
                out.sorted_candidates.push_back(RankedCandidate{lr.dists[q * params.top_k + r], id, id != kInvalidNodeId});
                if (id != kInvalidNodeId) out.topk.push_back(out.sorted_candidates.back());
            }
        }
        prof.sorted_candidates_materialize_ms = MsSince(t1);
        prof.exact_distance_kernel_ms = lr.kernel_ms;
        prof.requested_top_n = params.top_n;
        prof.effective_top_n = std::min<std::size_t>(params.top_n, capacity);
        prof.exact_candidates = lr.n_exact;
        prof.bound_filtered_candidates = lr.n_filtered;
        prof.rerank_batches = 1;
        prof.rerank_tile_size = tile;
        if (lr.evaluated) {
            prof.learned_stop_queries = num_queries;
            prof.learned_stop_prefix_min = prof.effective_top_n;
            for (std::size_t q = 0; q < num_queries; ++q) {
                prof.learned_stop_checkpoints += lr.checkpoint_counts[q];
                prof.learned_stop_prefix_sum += lr.stop_prefixes[q];
                prof.learned_stop_prefix_min = std::min<std::size_t>(prof.learned_stop_prefix_min, lr.stop_prefixes[q]);
                prof.learned_stop_prefix_max = std::max<std::size_t>(prof.learned_stop_prefix_max, lr.stop_prefixes[q]);
            }
        }
        prof.total_ms = MsSince(total_begin);
        if (out_profile != nullptr) {
            out_profile->total_ms += prof.total_ms;
            out_profile->pq2_refine_kernel_ms += prof.pq2_refine_kernel_ms;
            out_profile->pq2_refine_batches += prof.pq2_refine_batches;
            out_profile->pq2_residual_refine_batches += prof.pq2_residual_refine_batches;
            out_profile->exact_distance_kernel_ms += prof.exact_distance_kernel_ms;
            out_profile->exact_candidates += prof.exact_candidates;
            out_profile->bound_filtered_candidates += prof.bound_filtered_candidates;
            out_profile->rerank_batches += 1;
            out_profile->requested_top_n += prof.requested_top_n;
            out_profile->effective_top_n += prof.effective_top_n;
            out_profile->sorted_candidates_materialize_ms += prof.sorted_candidates_materialize_ms;
            out_profile->learned_stop_checkpoints += prof.learned_stop_checkpoints;
            out_profile->learned_stop_queries += prof.learned_stop_queries;
            out_profile->learned_stop_prefix_sum += prof.learned_stop_prefix_sum;
            if (prof.learned_stop_prefix_max != 0 || prof.learned_stop_prefix_min != 0) {
                if (out_profile->learned_stop_prefix_max == 0 && out_profile->learned_stop_prefix_min == 0) {
                    out_profile->learned_stop_prefix_min = prof.learned_stop_prefix_min;
                    out_profile->learned_stop_prefix_max = prof.learned_stop_prefix_max;
                } else {
                    out_profile->learned_stop_prefix_min = std::min(out_profile->learned_stop_prefix_min, prof.learned_stop_prefix_min);
                    out_profile->learned_stop_prefix_max = std::max(out_profile->learned_stop_prefix_max, prof.learned_stop_prefix_max);
                }
            }
        }
        return result;
    }
    const DeviceRerank rr = RunRerankKernel(resources, view, rp, cand, capacity, num_queries, d_queries.get(),
                                            TANN_KIND_FLOAT32,
                                            params.use_pq2_bound_filter ? resources.pq2_error_bounds_fp32().get() : nullptr, ctx);
    // statistics as the reference's drivers count them (:1743-1849 linear, :1851-2165 tiled)
    result.stats.exact_distance_count = rr.n_exact;
    result.stats.bound_filtered_count = rr.n_filtered;
    result.stats.io_pages = params.mode == RerankExecutionMode::kLinear ? num_queries * params.top_n : rr.n_exact;
    const auto t0 = Clock::now();
    result.queries.resize(num_queries);
    for (std::size_t q = 0; q < num_queries; ++q) {
        auto& out = result.queries[q];
        out.sorted_candidates.reserve(params.top_n);
        for (std::size_t r = 0; r < params.top_n; ++r) {
            const std::uint32_t id = rr.ids[q * params.top_n + r];
            out.sorted_candidates.push_back(RankedCandidate{rr.dists[q * params.top_n + r], id, id != kInvalidNodeId});
        }
        for (const RankedCandidate& c : out.sorted_candidates) {
            if (!c.valid()) continue;
            out.topk.push_back(c);
            if (out.topk.size() == params.top_k) break;
        }
    }
    prof.sorted_candidates_materialize_ms = MsSince(t0);
    prof.exact_distance_kernel_ms = rr.kernel_ms;
    prof.requested_top_n = params.top_n;
    prof.effective_top_n = std::min<std::size_t>(params.top_n, capacity);
    prof.exact_candidates = rr.n_exact;
    prof.bound_filtered_candidates = rr.n_filtered;
    prof.rerank_batches = 1;
    prof.rerank_gpu_sort_batches = 1;
    prof.rerank_tile_size = tile;
    prof.total_ms = MsSince(total_begin);
    if (out_profile != nullptr) {
        out_profile->total_ms += prof.total_ms;
        out_profile->pq2_refine_kernel_ms += prof.pq2_refine_kernel_ms;
        out_profile->pq2_refine_batches += prof.pq2_refine_batches;
        out_profile->pq2_residual_refine_batches += prof.pq2_residual_refine_batches;
        out_profile->exact_distance_kernel_ms += prof.exact_distance_kernel_ms;
        out_profile->exact_candidates += prof.exact_candidates;
        out_profile->bound_filtered_candidates += prof.bound_filtered_candidates;
        out_profile->rerank_batches += 1;
        out_profile->rerank_gpu_sort_batches += 1;
        out_profile->requested_top_n += prof.requested_top_n;
        out_profile->effective_top_n += prof.effective_top_n;
        out_profile->sorted_candidates_materialize_ms += prof.sorted_candidates_materialize_ms;
    }
    return result;
}

void CheckEndToEnd(const SearchResources& resources, std::size_t query_elems, std::size_t num_queries, const char* ctx) {
    if (!resources.has_pq_index()) throw std::runtime_error(BuildErrorMessage(ctx, "PQ index must be loaded before search."));
    if (!resources.has_vector_store()) throw std::runtime_error(BuildErrorMessage(ctx, "Vector store must be loaded before rerank."));
    if (resources.pq_index().host().ndims != resources.vector_store_header().dim)
        throw std::runtime_error(BuildErrorMessage(ctx, "PQ ndims must match vector store dim for end-to-end search."));
    if (query_elems != num_queries * static_cast<std::size_t>(resources.pq_index().host().ndims))
        throw std::runtime_error(BuildErrorMessage(ctx, "Query buffer size must equal num_queries * pq_ndims."));
}

TopoAnnsSearchParams EffectiveParams(const TopoAnnsSearchParams& params) {
    TopoAnnsSearchParams e = params;
    e.topology.candidate_queue_size = std::max({e.topology.top_l, e.topology.candidate_queue_size, e.rerank.top_n});
    return e;
}

template <typename QueryT, typename OracleFn, typename TopoFn, typename RerankFn>
TopoAnnsBatchResult RunMaterialised(const SearchResources& resources, const std::vector<QueryT>& queries, std::size_t n,
                                    const TopoAnnsSearchParams& params, OracleFn make_oracle, TopoFn run_topology,
                                    RerankFn run_rerank, const char* ctx) {
    CheckEndToEnd(resources, queries.size(), n, ctx);
    const PqDistanceOracle oracle = make_oracle();
    const TopoAnnsSearchParams eff = EffectiveParams(params);
    TopoAnnsBatchResult result;
    result.pq_profile = oracle.query_tables().profile();
    const std::vector<TopologySearchResult> topo = run_topology(oracle, eff, &result.topology_profile);
    const RerankBatchResult rr = run_rerank(topo, eff.rerank, &result.rerank_profile);
    result.queries.resize(n);
    result.rerank_stats = rr.stats;
    for (std::size_t q = 0; q < n; ++q) {
        result.queries[q].topology = topo[q];
        if (q < rr.queries.size()) result.queries[q].rerank = rr.queries[q];
    }
    return result;
}

struct FusedTraversal {
    DeviceTraversal device;
    CudaBuffer<float> d_queries;
    std::vector<std::uint32_t> host_stats;
    PqQueryTablesProfile pq_profile;
    TopologySearchBatchProfile topology_profile;
};

// Table build happens inside the traversal kernel: no Q x M x 256 table in HBM, no D2H of it.
FusedTraversal RunFusedTraversal(const SearchResources& resources, const DeviceEntryBatch& entries,
                                 const std::vector<float>& queries, std::size_t n, const TopologySearchParams& topology,
                                 std::size_t required_queue) {
    const char* ctx = "BuildFusedTopologyArtifacts";
    if (entries.num_queries != n) throw std::runtime_error(BuildErrorMessage(ctx, "entry batch size must equal num_queries."));
    if (!resources.has_pq_index()) throw std::runtime_error(BuildErrorMessage(ctx, "PQ index must be loaded before search."));
    if (!resources.has_vector_store()) throw std::runtime_error(BuildErrorMessage(ctx, "Vector store must be loaded before rerank."));
    if (queries.size() != n * static_cast<std::size_t>(resources.pq_index().host().ndims))
        throw std::runtime_error(BuildErrorMessage("FromFloatQueries", "Query buffer size must equal num_queries * ndims."));
    ValidateTopologyParams(topology, ctx);
    TopologySearchParams eff = topology;
    eff.candidate_queue_size = std::max({eff.top_l, eff.candidate_queue_size, required_queue});
    FusedTraversal f;
    const auto t0 = Clock::now();
    f.d_queries = CudaBuffer<float>::CopyFromHost(queries);
    f.pq_profile.query_upload_ms = MsSince(t0);
    f.device = RunTraversal(resources, eff, nullptr, f.d_queries.get(), TANN_KIND_FLOAT32, n, entries.offsets.get(), entries.ids.get());
    f.topology_profile.kernel_ms = f.device.kernel_ms;
    const auto t1 = Clock::now();
    f.host_stats = f.device.stats.CopyToHost();
    f.topology_profile.stats_download_ms = MsSince(t1);
    FillBatchSummaries(f.host_stats, &f.topology_profile);
    f.pq_profile.total_ms = f.pq_profile.query_upload_ms;
    return f;
}

TopoAnnsBatchResult AssembleFused(std::size_t n, const FusedTraversal& f, RerankBatchResult rr, const RerankBatchProfile& rp) {
    TopoAnnsBatchResult result;
    result.queries.resize(n);
    result.rerank_stats = rr.stats;
    result.pq_profile = f.pq_profile;
    result.topology_profile = f.topology_profile;
    result.rerank_profile = rp;
    for (std::size_t q = 0; q < n; ++q) {
        auto& st = result.queries[q].topology.stats;
        st.visited_nodes = f.host_stats[q * 8 + 0];
        st.expanded_nodes = f.host_stats[q * 8 + 1];
        st.iterations = f.host_stats[q * 8 + 3];
        if (q < rr.queries.size()) result.queries[q].rerank = std::move(rr.queries[q]);
    }
    return result;
}

}  // namespace

// ---- PqQueryDistanceTables ------------------------------------------------------------------------------------
PqQueryDistanceTables PqQueryDistanceTables::Build(const PqIndex& pq, const void* host_queries, std::uint32_t kind,
                                                   std::size_t element_count, std::size_t n, bool materialize,
                                                   const char* ctx) {
    if (pq.host().ndims == 0 || pq.host().num_chunks == 0) throw std::runtime_error(BuildErrorMessage(ctx, "PQ index is empty."));
    const std::size_t dim = pq.host().ndims;
    if (element_count != n * dim) throw std::runtime_error(BuildErrorMessage(ctx, "Query buffer size must equal num_queries * ndims."));
    PqQueryDistanceTables t;
    const auto total0 = Clock::now();
    const std::size_t M = pq.host().num_chunks;
    t.device_tables_ = CudaBuffer<float>::Allocate(n * M * kNumPqCentroids);
    const std::size_t qbytes = element_count * (kind == TANN_KIND_FLOAT32 ? 4 : 1);
    auto t0 = Clock::now();
    CudaBuffer<std::uint8_t> d_q = CudaBuffer<std::uint8_t>::Allocate(qbytes);
    if (qbytes != 0) ThrowIfCudaError(cudaMemcpy(d_q.get(), host_queries, qbytes, cudaMemcpyHostToDevice), "cudaMemcpyHostToDevice");
    t.profile_.query_upload_ms = MsSince(t0);
    t0 = Clock::now();
    ThrowIfTannError(tann_lut_build(pq.device().tables_col_major.get(), pq.device().centroid.get(), pq.device().chunk_offsets.get(),
                                    static_cast<std::uint32_t>(dim), static_cast<std::uint32_t>(M), d_q.get(), kind, n,
                                    t.device_tables_.get(), nullptr), ctx);
    ThrowIfCudaError(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    t.profile_.kernel_ms = MsSince(t0);
    t.num_queries_ = n;
    t.num_chunks_ = M;
    t.host_tables_materialized_ = materialize;
    t0 = Clock::now();
    if (materialize) t.host_tables_ = t.device_tables_.CopyToHost();
    t.profile_.table_download_ms = MsSince(t0);
    t.profile_.total_ms = MsSince(total0);
    return t;
}
PqQueryDistanceTables PqQueryDistanceTables::FromFloatQueries(const PqIndex& pq, const std::vector<float>& q, std::size_t n) {
    return Build(pq, q.data(), TANN_KIND_FLOAT32, q.size(), n, true, "FromFloatQueries");
}
PqQueryDistanceTables PqQueryDistanceTables::FromFloatQueriesDeviceOnly(const PqIndex& pq, const std::vector<float>& q, std::size_t n) {
    return Build(pq, q.data(), TANN_KIND_FLOAT32, q.size(), n, false, "FromFloatQueriesDeviceOnly");
}
PqQueryDistanceTables PqQueryDistanceTables::FromUint8Queries(const PqIndex& pq, const std::vector<std::uint8_t>& q, std::size_t n) {
    return Build(pq, q.data(), TANN_KIND_UINT8, q.size(), n, true, "FromUint8Queries");
}
PqQueryDistanceTables PqQueryDistanceTables::FromInt8Queries(const PqIndex& pq, const std::vector<std::int8_t>& q, std::size_t n) {
    return Build(pq, q.data(), TANN_KIND_INT8, q.size(), n, true, "FromInt8Queries");
}
PqQueryDistanceTables PqQueryDistanceTables::FromFloatQueriesDeviceBufferAsync(const PqIndex& pq, const CudaBuffer<float>& dq,
                                                                               std::size_t n, cudaStream_t stream) {
    const char* ctx = "FromFloatQueriesDeviceBufferAsync";
    if (pq.host().ndims == 0 || pq.host().num_chunks == 0) throw std::runtime_error(BuildErrorMessage(ctx, "PQ index is empty."));
    if (dq.size() != n * pq.host().ndims)
        throw std::runtime_error(BuildErrorMessage(ctx, "Device query buffer size must equal num_queries * ndims."));
    PqQueryDistanceTables t;
    const std::size_t M = pq.host().num_chunks;
    t.device_tables_ = CudaBuffer<float>::Allocate(n * M * kNumPqCentroids);
    ThrowIfTannError(tann_lut_build(pq.device().tables_col_major.get(), pq.device().centroid.get(), pq.device().chunk_offsets.get(),
                                    static_cast<std::uint32_t>(pq.host().ndims), static_cast<std::uint32_t>(M), dq.get(),
                                    TANN_KIND_FLOAT32, n, t.device_tables_.get(), stream), ctx);
    t.num_queries_ = n;
    t.num_chunks_ = M;
    return t;
}
float PqQueryDistanceTables::Lookup(std::size_t q, std::size_t chunk, std::uint32_t centroid) const {
    if (!host_tables_materialized_)
        throw std::runtime_error(BuildErrorMessage("PqQueryDistanceTables::Lookup", "Host query-distance tables are not materialized for this instance."));
    if (q >= num_queries_ || chunk >= num_chunks_ || centroid >= kNumPqCentroids)
        throw std::runtime_error(BuildErrorMessage("PqQueryDistanceTables::Lookup", "index out of range."));
    return host_tables_[(q * num_chunks_ + chunk) * kNumPqCentroids + centroid];
}
float PqQueryDistanceTables::Distance(std::size_t q, std::uint32_t node, const PqIndex& pq) const {
    if (!host_tables_materialized_)
        throw std::runtime_error(BuildErrorMessage("PqQueryDistanceTables::Distance", "Host query-distance tables are not materialized for this instance."));
    if (q >= num_queries_ || node >= pq.host().num_points)
        throw std::runtime_error(BuildErrorMessage("PqQueryDistanceTables::Distance", "index out of range."));
    std::vector<std::uint8_t> tmp;
    const std::uint8_t* codes = nullptr;
    if (pq.host().codes_on_host) {
        codes = pq.host_codes() + static_cast<std::size_t>(node) * num_chunks_;
    } else {
        tmp.resize(num_chunks_);
        ThrowIfCudaError(cudaMemcpy(tmp.data(), pq.device_codes() + static_cast<std::size_t>(node) * num_chunks_, num_chunks_,
                                    cudaMemcpyDeviceToHost), "cudaMemcpyDeviceToHost");
        codes = tmp.data();
    }
    float d = 0.0f;
    for (std::size_t m = 0; m < num_chunks_; ++m) d += Lookup(q, m, codes[m]);
    return d;
}

// ---- PqDistanceOracle --------------------------------------------------------------------------------------------
PqDistanceOracle::PqDistanceOracle(const PqIndex& pq, PqQueryDistanceTables tables) : pq_index_(&pq), query_tables_(std::move(tables)) {}
PqDistanceOracle PqDistanceOracle::FromFloatQueries(const PqIndex& pq, const std::vector<float>& q, std::size_t n) {
    return PqDistanceOracle(pq, PqQueryDistanceTables::FromFloatQueries(pq, q, n));
}
PqDistanceOracle PqDistanceOracle::FromFloatQueriesDeviceOnly(const PqIndex& pq, const std::vector<float>& q, std::size_t n) {
    return PqDistanceOracle(pq, PqQueryDistanceTables::FromFloatQueriesDeviceOnly(pq, q, n));
}
PqDistanceOracle PqDistanceOracle::FromFloatQueries(const SearchResources& r, const std::vector<float>& q, std::size_t n) {
    return FromFloatQueries(r.pq_index(), q, n);
}
PqDistanceOracle PqDistanceOracle::FromFloatQueriesDeviceOnly(const SearchResources& r, const std::vector<float>& q, std::size_t n) {
    return FromFloatQueriesDeviceOnly(r.pq_index(), q, n);
}
PqDistanceOracle PqDistanceOracle::FromUint8Queries(const PqIndex& pq, const std::vector<std::uint8_t>& q, std::size_t n) {
    return PqDistanceOracle(pq, PqQueryDistanceTables::FromUint8Queries(pq, q, n));
}
PqDistanceOracle PqDistanceOracle::FromUint8Queries(const SearchResources& r, const std::vector<std::uint8_t>& q, std::size_t n) {
    return FromUint8Queries(r.pq_index(), q, n);
}
PqDistanceOracle PqDistanceOracle::FromInt8Queries(const PqIndex& pq, const std::vector<std::int8_t>& q, std::size_t n) {
    return PqDistanceOracle(pq, PqQueryDistanceTables::FromInt8Queries(pq, q, n));
}
PqDistanceOracle PqDistanceOracle::FromInt8Queries(const SearchResources& r, const std::vector<std::int8_t>& q, std::size_t n) {
    return FromInt8Queries(r.pq_index(), q, n);
}
float PqDistanceOracle::Distance(std::size_t q, std::uint32_t node) const { return query_tables_.Distance(q, node, pq_index()); }
const PqIndex& PqDistanceOracle::pq_index() const {
    if (pq_index_ == nullptr) throw std::runtime_error(BuildErrorMessage("PqDistanceOracle::pq_index", "PQ index is not set."));
    return *pq_index_;
}

// ---- TopologySearch --------------------------------------------------------------------------------------------------
TopologySearchResult TopologySearch::Run(const SearchResources& resources, const EntryProvider& entries,
                                         const PqDistanceOracle& oracle, std::size_t query_id,
                                         const TopologySearchParams& params, TopologySearchBatchProfile* profile) {
    ValidateTopologyParams(params, "TopologySearch::Run");
    if (query_id >= oracle.num_queries()) throw std::runtime_error(BuildErrorMessage("TopologySearch::Run", "query_id is out of range."));
    return RunHostEntries(resources, oracle, {entries.GetEntryPoints(query_id)}, query_id, 1, params, profile).front();
}
std::vector<TopologySearchResult> TopologySearch::RunBatch(const SearchResources& resources, const EntryProvider& entries,
                                                           const PqDistanceOracle& oracle, const TopologySearchParams& params,
                                                           TopologySearchBatchProfile* profile) {
    ValidateTopologyParams(params, "TopologySearch::RunBatch");
    std::vector<std::vector<std::uint32_t>> by_query(oracle.num_queries());
    for (std::size_t q = 0; q < by_query.size(); ++q) by_query[q] = entries.GetEntryPoints(q);
    return RunHostEntries(resources, oracle, by_query, 0, oracle.num_queries(), params, profile);
}
std::vector<TopologySearchResult> TopologySearch::RunBatch(const SearchResources& resources, const DeviceEntryBatch& batch,
                                                           const PqDistanceOracle& oracle, const TopologySearchParams& params,
                                                           TopologySearchBatchProfile* profile) {
    ValidateTopologyParams(params, "TopologySearch::RunBatch");
    if (batch.num_queries != oracle.num_queries())
        throw std::runtime_error(BuildErrorMessage("TopologySearch::RunBatch", "entry batch size must match oracle query count."));
    return Materialize(RunTraversal(resources, params, oracle.query_tables().device_tables().get(), nullptr, TANN_KIND_FLOAT32,
                                    batch.num_queries, batch.offsets.get(), batch.ids.get()),
                       params, profile);
}

// ---- HpqRefine (src/search/rerank_exact.cu:2457-2531) --------------------------------------------------------------
std::vector<std::vector<RankedCandidate>> HpqRefine::RunBatchFloat32(const SearchResources& resources,
                                                                     const DeviceEntryBatch& batch,
                                                                     const std::vector<float>& queries, std::size_t num_queries,
                                                                     const TopologySearchParams& params, std::size_t refine_top_l) {
    const char* ctx = "RunHpqRefineBatchDevice";
    ValidateTopologyParams(params, ctx);
    if (!resources.has_hpq_index()) throw std::runtime_error(BuildErrorMessage(ctx, "HPQ index must be loaded."));
    if (batch.num_queries != num_queries) throw std::runtime_error(BuildErrorMessage(ctx, "topology_result size mismatch."));
    std::vector<std::vector<RankedCandidate>> out(num_queries);
    if (num_queries == 0 || refine_top_l == 0) return out;
    const HpqIndex& hpq = resources.hpq_index();
    const PqIndex& base = hpq.base_index();
    const PqIndex& outlier = hpq.outlier_index();
    const std::uint32_t M = static_cast<std::uint32_t>(outlier.host().num_chunks);
    const std::uint32_t dim = static_cast<std::uint32_t>(outlier.host().ndims);
    if (queries.size() != num_queries * dim) throw std::runtime_error(BuildErrorMessage(ctx, "queries size must equal num_queries * dim."));
    const CudaBuffer<float> d_queries = CudaBuffer<float>::CopyFromHost(queries);
    const DeviceTraversal topo = RunTraversal(resources, params, nullptr, d_queries.get(), TANN_KIND_FLOAT32, num_queries,
                                              batch.offsets.get(), batch.ids.get());
    if (refine_top_l > topo.capacity || refine_top_l > 2048)
        throw std::runtime_error(BuildErrorMessage(ctx, "HPQ refine size exceeds candidate limits."));
    CudaBuffer<float> base_lut = CudaBuffer<float>::Allocate(num_queries * M * kNumPqCentroids);
    CudaBuffer<float> outlier_lut = CudaBuffer<float>::Allocate(num_queries * M * kNumPqCentroids);
    ThrowIfTannError(tann_lut_build(base.device().tables_col_major.get(), base.device().centroid.get(),
                                    base.device().chunk_offsets.get(), dim, M, d_queries.get(), TANN_KIND_FLOAT32, num_queries,
                                    base_lut.get(), nullptr), ctx);
    ThrowIfTannError(tann_lut_build(outlier.device().tables_col_major.get(), outlier.device().centroid.get(),
                                    outlier.device().chunk_offsets.get(), dim, M, d_queries.get(), TANN_KIND_FLOAT32, num_queries,
                                    outlier_lut.get(), nullptr), ctx);
    CudaBuffer<DeviceCand> refined = CudaBuffer<DeviceCand>::Allocate(num_queries * refine_top_l);
    TannShards codes{};
    codes.num_shards = 1;
    codes.base[0] = outlier.device_codes();
    ThrowIfTannError(tann_hpq_refine(topo.candidates.get(), topo.stats.get(), num_queries, topo.capacity,
                                     static_cast<std::uint32_t>(refine_top_l), &codes, hpq.device_selector_bits(), M,
                                     base_lut.get(), outlier_lut.get(), refined.get(), nullptr, nullptr), ctx);
    ThrowIfCudaError(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    const std::vector<DeviceCand> host = refined.CopyToHost();
    for (std::size_t q = 0; q < num_queries; ++q)
        for (std::size_t i = 0; i < refine_top_l; ++i) {
            const DeviceCand& c = host[q * refine_top_l + i];
            if (c.node_id == kInvalidNodeId) continue;
            out[q].push_back(RankedCandidate{c.distance, c.node_id & ~kExpandedBit, false});
        }
    return out;
}

// ---- RerankExact -----------------------------------------------------------------------------------------------------
RerankBatchResult RerankExact::RunBatchFloat32(const SearchResources& r, const std::vector<TopologySearchResult>& topo,
                                               const std::vector<float>& q, std::size_t n, const RerankExactParams& p,
                                               RerankBatchProfile* prof) {
    return RerankFromHostResults(r, topo, q, n, p, "RerankExact::RunBatchFloat32", prof);
}
RerankBatchResult RerankExact::RunBatchUint8(const SearchResources& r, const std::vector<TopologySearchResult>& topo,
                                             const std::vector<std::uint8_t>& q, std::size_t n, const RerankExactParams& p,
                                             RerankBatchProfile* prof) {
    return RerankFromHostResults(r, topo, q, n, p, "RerankExact::RunBatchUint8", prof);
}
RerankBatchResult RerankExact::RunBatchInt8(const SearchResources& r, const std::vector<TopologySearchResult>& topo,
                                            const std::vector<std::int8_t>& q, std::size_t n, const RerankExactParams& p,
                                            RerankBatchProfile* prof) {
    return RerankFromHostResults(r, topo, q, n, p, "RerankExact::RunBatchInt8", prof);
}

// ---- TopoAnnsSearch --------------------------------------------------------------------------------------------------
TopoAnnsBatchResult TopoAnnsSearch::RunBatchFloat32(const SearchResources& r, const EntryProvider& entries,
                                                    const std::vector<float>& q, std::size_t n, const TopoAnnsSearchParams& p) {
    return RunMaterialised(
        r, q, n, p, [&] { return PqDistanceOracle::FromFloatQueries(r, q, n); },
        [&](const PqDistanceOracle& o, const TopoAnnsSearchParams& e, TopologySearchBatchProfile* tp) {
            return TopologySearch::RunBatch(r, entries, o, e.topology, tp);
        },
        [&](const std::vector<TopologySearchResult>& t, const RerankExactParams& rp, RerankBatchProfile* pr) {
            return RerankExact::RunBatchFloat32(r, t, q, n, rp, pr);
        },
        "TopoAnnsSearch::RunBatchFloat32");
}
TopoAnnsBatchResult TopoAnnsSearch::RunBatchFloat32(const SearchResources& r, const DeviceEntryBatch& batch,
                                                    const std::vector<float>& q, std::size_t n, const TopoAnnsSearchParams& p) {
    if (batch.num_queries != n)
        throw std::runtime_error(BuildErrorMessage("TopoAnnsSearch::RunBatchFloat32", "entry batch size must equal num_queries."));
    return RunMaterialised(
        r, q, n, p, [&] { return PqDistanceOracle::FromFloatQueries(r, q, n); },
        [&](const PqDistanceOracle& o, const TopoAnnsSearchParams& e, TopologySearchBatchProfile* tp) {
            return TopologySearch::RunBatch(r, batch, o, e.topology, tp);
        },
        [&](const std::vector<TopologySearchResult>& t, const RerankExactParams& rp, RerankBatchProfile* pr) {
            return RerankExact::RunBatchFloat32(r, t, q, n, rp, pr);
        },
        "TopoAnnsSearch::RunBatchFloat32");
}
TopoAnnsBatchResult TopoAnnsSearch::RunBatchUint8(const SearchResources& r, const EntryProvider& entries,
                                                  const std::vector<std::uint8_t>& q, std::size_t n, const TopoAnnsSearchParams& p) {
    return RunMaterialised(
        r, q, n, p, [&] { return PqDistanceOracle::FromUint8Queries(r, q, n); },
        [&](const PqDistanceOracle& o, const TopoAnnsSearchParams& e, TopologySearchBatchProfile* tp) {
            return TopologySearch::RunBatch(r, entries, o, e.topology, tp);
        },
        [&](const std::vector<TopologySearchResult>& t, const RerankExactParams& rp, RerankBatchProfile* pr) {
            return RerankExact::RunBatchUint8(r, t, q, n, rp, pr);
        },
        "TopoAnnsSearch::RunBatchUint8");
}
TopoAnnsBatchResult TopoAnnsSearch::RunBatchInt8(const SearchResources& r, const EntryProvider& entries,
                                                 const std::vector<std::int8_t>& q, std::size_t n, const TopoAnnsSearchParams& p) {
    return RunMaterialised(
        r, q, n, p, [&] { return PqDistanceOracle::FromInt8Queries(r, q, n); },
        [&](const PqDistanceOracle& o, const TopoAnnsSearchParams& e, TopologySearchBatchProfile* tp) {
            return TopologySearch::RunBatch(r, entries, o, e.topology, tp);
        },
        [&](const std::vector<TopologySearchResult>& t, const RerankExactParams& rp, RerankBatchProfile* pr) {
            return RerankExact::RunBatchInt8(r, t, q, n, rp, pr);
        },
        "TopoAnnsSearch::RunBatchInt8");
}
TopoAnnsBatchResult TopoAnnsSearch::RunBatchFloat32Fused(const SearchResources& r, const DeviceEntryBatch& batch,
                                                         const std::vector<float>& q, std::size_t n, const TopoAnnsSearchParams& p) {
    const FusedTraversal f = RunFusedTraversal(r, batch, q, n, p.topology, p.rerank.top_n);
    RerankBatchProfile rp;
    RerankBatchResult rr = RerankFromDeviceTraversal(r, f.device, f.d_queries, q, n, p.rerank, &rp);
    return AssembleFused(n, f, std::move(rr), rp);
}
std::vector<TopoAnnsBatchResult> TopoAnnsSearch::RunBatchFloat32FusedRerankSweep(
    const SearchResources& r, const DeviceEntryBatch& batch, const std::vector<float>& q, std::size_t n,
    const TopologySearchParams& topology, const std::vector<RerankExactParams>& rerank_list) {
    std::vector<TopoAnnsBatchResult> out;
    if (rerank_list.empty()) return out;
    std::size_t max_top_n = 0;
    for (const auto& rp : rerank_list) max_top_n = std::max(max_top_n, rp.top_n);
    const FusedTraversal f = RunFusedTraversal(r, batch, q, n, topology, max_top_n);
    for (const auto& params : rerank_list) {
        RerankBatchProfile rp;
        RerankBatchResult rr = RerankFromDeviceTraversal(r, f.device, f.d_queries, q, n, params, &rp);
        out.push_back(AssembleFused(n, f, std::move(rr), rp));
    }
    return out;
}

}  // namespace topoanns
