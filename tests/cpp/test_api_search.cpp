// The search entry points of the C++ API on the reference's toy fixtures (needs a GPU). Mirrors
// tests/test_pq_query_tables.cpp, test_pq_distance_oracle.cpp, test_pinned_topology_uva.cu,
// test_topology_search_gpu.cpp, test_topology_search_batch_gpu.cpp, test_rerank_exact.cpp,
// test_topoanns_search_batch.cpp, test_topoanns_search_device_entries.cpp,
// test_topoanns_search_fused.cpp, test_topoanns_search_fused_sweep.cpp, test_pq2_residual_refine.cpp,
// test_pq2_bound_filter.cpp and test_search_resources.cpp of the reference.
#include "fixtures.hpp"

using namespace topoanns;

namespace {

DeviceEntryBatch MakeEntryBatch(std::size_t n, const std::vector<std::uint32_t>& entries) {
    DeviceEntryBatch b;
    b.num_queries = n;
    b.entries_per_query = entries.size();
    std::vector<std::uint32_t> offsets(n + 1), ids;
    for (std::size_t q = 0; q <= n; ++q) offsets[q] = static_cast<std::uint32_t>(q * entries.size());
    for (std::size_t q = 0; q < n; ++q) ids.insert(ids.end(), entries.begin(), entries.end());
    b.offsets = CudaBuffer<std::uint32_t>::CopyFromHost(offsets);
    b.ids = CudaBuffer<std::uint32_t>::CopyFromHost(ids);
    return b;
}

std::vector<float> Constant(const std::vector<float>& values, std::size_t dim) {
    std::vector<float> q;
    for (float v : values) q.insert(q.end(), dim, v);
    return q;
}

void TestQueryTablesAndOracle() {
    std::vector<float> tables(256 * 2, 0.0f);
    tables[2] = 1.0f; tables[5] = 2.0f; tables[6] = 1.0f; tables[7] = 2.0f;   // centres 1,2,3 = (1,0) (0,2) (1,2)
    fx::WritePq(fx::Tmp("qt_pivots.bin"), fx::Tmp("qt_codes.bin"), 2, tables, {1, 2, 3});
    const PqIndex pq = PqIndex::LoadFromSeparatePaths(fx::Tmp("qt_pivots.bin"), fx::Tmp("qt_codes.bin"));
    CHECK_EQ(pq.host().num_points, std::uint64_t{3});
    CHECK_EQ(pq.host().ndims, std::uint64_t{2});
    CHECK_EQ(pq.host().num_chunks, std::uint64_t{1});
    CHECK_EQ(pq.host().tables_col_major[1 * 256 + 2], 2.0f);
    const std::vector<float> queries = {1.0f, 2.0f, 0.0f, 0.0f};
    const auto qt = PqQueryDistanceTables::FromFloatQueries(pq, queries, 2);
    CHECK_EQ(qt.num_queries(), std::size_t{2});
    CHECK_TRUE(qt.has_host_tables() && qt.device_tables().get() != nullptr);
    CHECK_EQ(qt.Lookup(0, 0, 0), 5.0f); CHECK_EQ(qt.Lookup(0, 0, 1), 4.0f);
    CHECK_EQ(qt.Lookup(0, 0, 2), 1.0f); CHECK_EQ(qt.Lookup(0, 0, 3), 0.0f);
    CHECK_EQ(qt.Lookup(1, 0, 0), 0.0f); CHECK_EQ(qt.Lookup(1, 0, 3), 5.0f);
    CHECK_EQ(qt.Distance(0, 0, pq), 4.0f); CHECK_EQ(qt.Distance(0, 1, pq), 1.0f);
    CHECK_EQ(qt.Distance(0, 2, pq), 0.0f); CHECK_EQ(qt.Distance(1, 2, pq), 5.0f);
    const auto dev_only = PqQueryDistanceTables::FromFloatQueriesDeviceOnly(pq, queries, 2);
    CHECK_TRUE(!dev_only.has_host_tables());
    CHECK_THROWS(dev_only.Lookup(0, 0, 0));
    CHECK_THROWS(dev_only.Distance(0, 0, pq));
    CHECK_THROWS(PqQueryDistanceTables::FromFloatQueries(pq, queries, 3));
    const auto u8 = PqQueryDistanceTables::FromUint8Queries(pq, {1, 2, 0, 0}, 2);
    CHECK_EQ(u8.Lookup(0, 0, 3), 0.0f);
    const PqDistanceOracle oracle = PqDistanceOracle::FromFloatQueries(pq, queries, 2);
    CHECK_EQ(oracle.Distance(0, 2), 0.0f);
    CHECK_EQ(oracle.Distance(1, 0), 1.0f);
}

SearchResources ToyResources(std::size_t dim, const std::string& tag, bool with_vectors) {
    fx::WritePq(fx::Tmp(tag + "_pivots.bin"), fx::Tmp(tag + "_codes.bin"), dim, fx::RampTables(dim), fx::ToyCodes());
    SearchResources r = SearchResources::FromDataset(fx::ToyGraph());
    r.LoadPqIndex(fx::Tmp(tag + "_pivots.bin"), fx::Tmp(tag + "_codes.bin"));
    if (with_vectors) {
        const VectorPageLayout layout = VectorPageLayout::Create(static_cast<std::uint32_t>(dim), ScalarKind::kFloat32);
        std::vector<std::vector<std::uint8_t>> vectors;
        for (float v : {9.0f, 6.0f, 7.0f, 2.0f, 3.0f, 1.0f}) vectors.push_back(fx::FloatBytes(std::vector<float>(dim, v)));
        VectorStoreBuilder::WriteFile(fx::Tmp(tag + "_vectors.ssd"), layout, ScalarKind::kFloat32, static_cast<std::uint32_t>(dim), vectors);
        r.LoadVectorStore(fx::Tmp(tag + "_vectors.ssd"));
        r.AttachVectorPageProvider(std::make_shared<HbmVectorPageProvider>(fx::Tmp(tag + "_vectors.ssd")));
    }
    return r;
}

void TestTopologyAndResources() {
    SearchResources r = ToyResources(1, "topo", false);
    CHECK_EQ(r.num_nodes(), std::uint64_t{6});
    CHECK_EQ(r.degree(), 64u);
    CHECK_TRUE(r.ReadHostNeighbors(0)[1] == 2u && r.ReadHostNeighbors(5)[0] == kInvalidNodeId);
    CHECK_TRUE(r.topology().CopyNodeFromDevice(2)[0] == 4u);       // UVA / HBM copy agrees with the host copy
    CHECK_TRUE(r.has_pq_index() && !r.has_pq2_index() && !r.has_vector_store());
    CHECK_THROWS(r.pq2_index());
    CHECK_THROWS(r.vector_store_header());
    CHECK_THROWS(r.topology().ReadHostNode(6));

    FixedEntryProvider entries({0});
    const std::vector<float> queries = {0.0f, 8.0f};
    const auto oracle = PqDistanceOracle::FromFloatQueries(r, queries, 2);
    TopologySearchParams p;
    p.top_k = 2; p.top_l = 2; p.search_width = 1; p.max_expansions = 16;
    const auto single = TopologySearch::Run(r, entries, oracle, 0, p);
    CHECK_EQ(single.topk.size(), std::size_t{2});
    CHECK_EQ(single.topk[0].node_id, 5u); CHECK_EQ(single.topk[1].node_id, 3u);
    CHECK_EQ(single.topk[0].distance, 1.0f); CHECK_EQ(single.topk[1].distance, 4.0f);
    CHECK_EQ(single.stats.visited_nodes, std::size_t{5});      // the exact-visited-set search of the reference's test
    CHECK_EQ(single.stats.expanded_nodes, std::size_t{4});
    CHECK_EQ(single.stats.iterations, std::size_t{4});
    CHECK_TRUE(SearchStopCondition::BestUnexpandedRank(single.sorted_candidates) >= p.top_l);
    TopologySearchBatchProfile prof;
    const auto batch = TopologySearch::RunBatch(r, entries, oracle, p, &prof);
    CHECK_EQ(batch.size(), std::size_t{2});
    CHECK_EQ(batch[0].topk[0].node_id, 5u); CHECK_EQ(batch[0].topk[1].node_id, 3u);
    CHECK_EQ(batch[1].topk[0].node_id, 0u); CHECK_EQ(batch[1].topk[1].node_id, 2u);
    CHECK_EQ(TopologySearch::Run(r, entries, oracle, 1, p).topk[1].node_id, 2u);
    CHECK_EQ(prof.batch_max_iterations, std::size_t{4});
    // parameter rules
    TopologySearchParams bad = p;
    bad.top_k = 0; CHECK_THROWS(TopologySearch::RunBatch(r, entries, oracle, bad));
    bad = p; bad.top_l = 0; CHECK_THROWS(TopologySearch::RunBatch(r, entries, oracle, bad));
    bad = p; bad.candidate_queue_size = 1; CHECK_THROWS(TopologySearch::RunBatch(r, entries, oracle, bad));
    bad = p; bad.search_width = 0; CHECK_THROWS(TopologySearch::RunBatch(r, entries, oracle, bad));
    bad = p; bad.search_width = 33; CHECK_THROWS(TopologySearch::RunBatch(r, entries, oracle, bad));
    CHECK_THROWS(TopologySearch::Run(r, entries, oracle, 2, p));
    // pinned-host topology tier with and without an HBM cache of the first rows gives the same search
    for (std::uint64_t cached : {std::uint64_t{0}, std::uint64_t{3}}) {
        r.mutable_topology().SetResidency(TopologyResidency::kPinnedHost, cached);
        const auto again = TopologySearch::RunBatch(r, entries, oracle, p);
        CHECK_EQ(again[0].topk[0].node_id, 5u); CHECK_EQ(again[1].topk[1].node_id, 2u);
        CHECK_EQ(again[0].stats.visited_nodes, std::size_t{5});
    }
    r.mutable_topology().SetResidency(TopologyResidency::kHbm);
}

void TestRerankAndEndToEnd() {
    constexpr std::size_t kDim = 300;
    SearchResources r = ToyResources(kDim, "e2e", true);
    FixedEntryProvider entries({0});
    const std::vector<float> queries = Constant({0.0f, 8.0f}, kDim);

    // tests/test_rerank_exact.cpp: both queries zero
    {
        const std::vector<float> zero(2 * kDim, 0.0f);
        const auto oracle = PqDistanceOracle::FromFloatQueries(r, zero, 2);
        TopologySearchParams sp;
        sp.top_k = 5; sp.top_l = 5; sp.search_width = 1; sp.max_expansions = 16;
        const auto topo = TopologySearch::RunBatch(r, entries, oracle, sp);
        RerankExactParams rp;
        rp.top_k = 2; rp.top_n = 5;
        const auto rr = RerankExact::RunBatchFloat32(r, topo, zero, 2, rp);
        CHECK_EQ(rr.queries.size(), std::size_t{2});
        CHECK_EQ(rr.stats.exact_distance_count, std::size_t{10});
        CHECK_EQ(rr.stats.io_pages, std::size_t{2});
        for (int q = 0; q < 2; ++q) {
            CHECK_EQ(rr.queries[q].topk[0].node_id, 5u); CHECK_EQ(rr.queries[q].topk[1].node_id, 3u);
            CHECK_EQ(rr.queries[q].topk[0].distance, 300.0f); CHECK_EQ(rr.queries[q].topk[1].distance, 1200.0f);
        }
    }
    TopoAnnsSearchParams params;
    params.topology.top_k = 5; params.topology.top_l = 4; params.topology.search_width = 1;
    params.topology.max_expansions = 16;
    params.rerank.top_k = 2; params.rerank.top_n = 5;
    // tests/test_topoanns_search_batch.cpp
    const auto base = TopoAnnsSearch::RunBatchFloat32(r, entries, queries, 2, params);
    CHECK_EQ(base.queries.size(), std::size_t{2});
    CHECK_EQ(base.rerank_stats.exact_distance_count, std::size_t{10});
    CHECK_EQ(base.rerank_stats.io_pages, std::size_t{2});
    CHECK_EQ(base.queries[0].topology.sorted_candidates.size(), std::size_t{5});
    CHECK_EQ(base.queries[0].topology.topk[0].node_id, 5u); CHECK_EQ(base.queries[1].topology.topk[1].node_id, 2u);
    CHECK_EQ(base.queries[0].rerank.topk[0].node_id, 5u); CHECK_EQ(base.queries[0].rerank.topk[1].node_id, 3u);
    CHECK_EQ(base.queries[0].rerank.topk[0].distance, 300.0f); CHECK_EQ(base.queries[0].rerank.topk[1].distance, 1200.0f);
    CHECK_EQ(base.queries[1].rerank.topk[0].node_id, 0u); CHECK_EQ(base.queries[1].rerank.topk[1].node_id, 2u);
    CHECK_EQ(base.queries[1].rerank.topk[0].distance, 300.0f); CHECK_EQ(base.queries[1].rerank.topk[1].distance, 300.0f);
    // tests/test_topoanns_search_device_entries.cpp: device entries == host entries
    const DeviceEntryBatch dev_entries = MakeEntryBatch(2, {0});
    const auto dev = TopoAnnsSearch::RunBatchFloat32(r, dev_entries, queries, 2, params);
    for (int q = 0; q < 2; ++q) {
        CHECK_EQ(dev.queries[q].rerank.topk.size(), base.queries[q].rerank.topk.size());
        for (std::size_t i = 0; i < dev.queries[q].rerank.topk.size(); ++i) {
            CHECK_EQ(dev.queries[q].rerank.topk[i].node_id, base.queries[q].rerank.topk[i].node_id);
            CHECK_EQ(dev.queries[q].rerank.topk[i].distance, base.queries[q].rerank.topk[i].distance);
        }
        CHECK_EQ(dev.queries[q].topology.stats.visited_nodes, base.queries[q].topology.stats.visited_nodes);
    }
    CHECK_THROWS(TopoAnnsSearch::RunBatchFloat32(r, MakeEntryBatch(1, {0}), queries, 2, params));
    // tests/test_topoanns_search_fused.cpp: every fused mode == the materialised baseline
    for (RerankExecutionMode mode : {RerankExecutionMode::kLinear, RerankExecutionMode::kTiled,
                                     RerankExecutionMode::kPageByPage, RerankExecutionMode::kPersistent}) {
        TopoAnnsSearchParams fp = params;
        fp.rerank.mode = mode;
        fp.rerank.rank_tile_size = 2;
        const auto fused = TopoAnnsSearch::RunBatchFloat32Fused(r, dev_entries, queries, 2, fp);
        CHECK_EQ(fused.rerank_stats.exact_distance_count, std::size_t{10});
        for (int q = 0; q < 2; ++q) {
            CHECK_EQ(fused.queries[q].rerank.sorted_candidates.size(), std::size_t{5});
            CHECK_EQ(fused.queries[q].rerank.topk.size(), std::size_t{2});
            for (std::size_t i = 0; i < 2; ++i) {
                CHECK_EQ(fused.queries[q].rerank.topk[i].node_id, base.queries[q].rerank.topk[i].node_id);
                CHECK_EQ(fused.queries[q].rerank.topk[i].distance, base.queries[q].rerank.topk[i].distance);
            }
            CHECK_EQ(fused.queries[q].topology.stats.expanded_nodes, base.queries[q].topology.stats.expanded_nodes);
        }
    }
    // tests/test_topoanns_search_fused_sweep.cpp: one traversal, several rerank settings
    std::vector<RerankExactParams> sweep(2, params.rerank);
    sweep[0].mode = RerankExecutionMode::kLinear; sweep[0].top_n = 3;
    sweep[1].mode = RerankExecutionMode::kTiled; sweep[1].top_n = 5; sweep[1].rank_tile_size = 2;
    const auto swept = TopoAnnsSearch::RunBatchFloat32FusedRerankSweep(r, dev_entries, queries, 2, params.topology, sweep);
    CHECK_EQ(swept.size(), std::size_t{2});
    for (std::size_t s = 0; s < 2; ++s) {
        TopoAnnsSearchParams one = params;
        one.rerank = sweep[s];
        one.topology.candidate_queue_size = 5;   // the sweep sizes the queue for the largest top_n
        const auto single = TopoAnnsSearch::RunBatchFloat32Fused(r, dev_entries, queries, 2, one);
        for (int q = 0; q < 2; ++q)
            for (std::size_t i = 0; i < 2; ++i) {
                CHECK_EQ(swept[s].queries[q].rerank.topk[i].node_id, single.queries[q].rerank.topk[i].node_id);
                CHECK_EQ(swept[s].queries[q].rerank.topk[i].distance, single.queries[q].rerank.topk[i].distance);
            }
    }
    // unsupported stops and inconsistent settings are errors
    TopoAnnsSearchParams badp = params;
    badp.rerank.use_pq2_bound_filter = true;
    CHECK_THROWS(TopoAnnsSearch::RunBatchFloat32Fused(r, dev_entries, queries, 2, badp));
    badp = params; badp.rerank.use_learned_stop = true;
    CHECK_THROWS(TopoAnnsSearch::RunBatchFloat32Fused(r, dev_entries, queries, 2, badp));
    // rerank early stop (stable-tile rule): with tiles of one rank, min_prefix 1 and patience 1 the rerank of
    // query 0 ends at the first tile that does not improve the best distance, so fewer than the 10 exact
    // distances of the full run are computed; a rule that can never fire changes nothing; linear mode rejects it
    {
        TopoAnnsSearchParams ep = params;
        ep.rerank.top_k = 1;
        ep.rerank.mode = RerankExecutionMode::kPersistent;
        ep.rerank.rank_tile_size = 1;
        ep.rerank.use_early_stop = true;
        ep.rerank.early_stop_min_prefix = 1;
        ep.rerank.early_stop_patience_tiles = 1;
        const auto early = TopoAnnsSearch::RunBatchFloat32Fused(r, dev_entries, queries, 2, ep);
        CHECK_TRUE(early.rerank_stats.exact_distance_count < std::size_t{10});
        CHECK_TRUE(early.rerank_stats.exact_distance_count >= std::size_t{4});   // at least two tiles per query
        ep.rerank.early_stop_min_prefix = 1000;
        const auto never = TopoAnnsSearch::RunBatchFloat32Fused(r, dev_entries, queries, 2, ep);
        CHECK_EQ(never.rerank_stats.exact_distance_count, std::size_t{10});
        CHECK_EQ(never.queries[0].rerank.topk[0].node_id, base.queries[0].rerank.topk[0].node_id);
        ep.rerank.mode = RerankExecutionMode::kLinear;
        CHECK_THROWS(TopoAnnsSearch::RunBatchFloat32Fused(r, dev_entries, queries, 2, ep));
    }
    // the neighbour-code layout changes where the code rows are read from, not what is found
    {
        r.BuildNeighborCodeLayout();
        CHECK_TRUE(r.has_neighbor_code_layout());
        const auto inl = TopoAnnsSearch::RunBatchFloat32Fused(r, dev_entries, queries, 2, params);
        for (int q = 0; q < 2; ++q) {
            CHECK_EQ(inl.queries[q].topology.stats.visited_nodes, base.queries[q].topology.stats.visited_nodes);
            CHECK_EQ(inl.queries[q].topology.stats.expanded_nodes, base.queries[q].topology.stats.expanded_nodes);
            for (std::size_t i = 0; i < 2; ++i) {
                CHECK_EQ(inl.queries[q].rerank.topk[i].node_id, base.queries[q].rerank.topk[i].node_id);
                CHECK_EQ(inl.queries[q].rerank.topk[i].distance, base.queries[q].rerank.topk[i].distance);
            }
        }
        r.DropNeighborCodeLayout();
    }
    // the pinned-host page provider gives the same fused result
    r.AttachVectorPageProvider(std::make_shared<PinnedHostVectorPageProvider>(fx::Tmp("e2e_vectors.ssd")));
    const auto hosted = TopoAnnsSearch::RunBatchFloat32Fused(r, dev_entries, queries, 2, params);
    CHECK_EQ(hosted.queries[1].rerank.topk[1].node_id, 2u);
    CHECK_EQ(hosted.queries[0].rerank.topk[1].distance, 1200.0f);
}

void TestUint8EntryPoint() {
    // uint8 queries on a uint8 store: the integer rerank path through RunBatchUint8
    constexpr std::size_t kDim = 128;
    fx::WritePq(fx::Tmp("u8_pivots.bin"), fx::Tmp("u8_codes.bin"), kDim, fx::RampTables(kDim), fx::ToyCodes());
    SearchResources r = SearchResources::FromDataset(fx::ToyGraph());
    r.LoadPqIndex(fx::Tmp("u8_pivots.bin"), fx::Tmp("u8_codes.bin"));
    std::vector<std::vector<std::uint8_t>> vectors;
    for (std::uint8_t v : {9, 6, 7, 2, 3, 1}) vectors.push_back(std::vector<std::uint8_t>(kDim, v));
    VectorStoreBuilder::WriteFile(fx::Tmp("u8_vectors.ssd"), VectorPageLayout::Create(kDim, ScalarKind::kUint8), ScalarKind::kUint8, kDim, vectors);
    r.LoadVectorStore(fx::Tmp("u8_vectors.ssd"));
    r.AttachVectorPageProvider(std::make_shared<HbmVectorPageProvider>(fx::Tmp("u8_vectors.ssd")));
    TopoAnnsSearchParams params;
    params.topology.top_k = 5; params.topology.top_l = 4; params.topology.search_width = 1; params.topology.max_expansions = 16;
    params.rerank.top_k = 2; params.rerank.top_n = 5;
    std::vector<std::uint8_t> q(2 * kDim, 0);
    std::fill(q.begin() + kDim, q.end(), std::uint8_t{8});
    const auto res = TopoAnnsSearch::RunBatchUint8(r, FixedEntryProvider({0}), q, 2, params);
    CHECK_EQ(res.queries[0].rerank.topk[0].node_id, 5u); CHECK_EQ(res.queries[0].rerank.topk[0].distance, 128.0f);
    CHECK_EQ(res.queries[0].rerank.topk[1].node_id, 3u); CHECK_EQ(res.queries[0].rerank.topk[1].distance, 512.0f);
    CHECK_EQ(res.queries[1].rerank.topk[0].node_id, 0u); CHECK_EQ(res.queries[1].rerank.topk[1].node_id, 2u);
    CHECK_EQ(res.queries[1].rerank.topk[0].distance, 128.0f);
}

void TestPq2() {
    // tests/test_pq2_residual_refine.cpp and tests/test_pq2_bound_filter.cpp, end to end through the fused path
    std::vector<float> t1(256 * 2, 0.0f), t2(256 * 2, 0.0f);
    t1[2] = 1.0f; t1[5] = 2.0f;                 // base centres 1 = (1,0), 2 = (0,2)
    t2[3] = 1.0f; t2[4] = 1.0f; t2[5] = 1.0f;   // residual centres 1 = (0,1), 2 = (1,1)
    fx::WritePq(fx::Tmp("pq2_base_pivots.bin"), fx::Tmp("pq2_base_codes.bin"), 2, t1, {1, 2});
    fx::WritePq(fx::Tmp("pq2_res_pivots.bin"), fx::Tmp("pq2_res_codes.bin"), 2, t2, {1, 2});
    fx::WriteErrorBounds(fx::Tmp("pq2_eps.bin"), {0.0f, 0.0f});
    SearchResources r = SearchResources::FromDataset(TopologyLayout::MakePadded(2, {{1}, {}}));
    r.LoadPqIndex(fx::Tmp("pq2_base_pivots.bin"), fx::Tmp("pq2_base_codes.bin"));
    r.LoadPq2Index(fx::Tmp("pq2_res_pivots.bin"), fx::Tmp("pq2_res_codes.bin"), fx::Tmp("pq2_eps.bin"));
    CHECK_TRUE(r.has_pq2_index() && r.pq2_is_residual_refine() && r.has_pq2_error_bounds());
    CHECK_EQ(r.pq2_cross_terms().size(), std::size_t{256 * 256});        // one chunk
    CHECK_EQ(r.pq2_error_bounds_fp32().size(), std::size_t{2});
    const std::vector<float> cross = r.pq2_cross_terms().CopyToHost();
    CHECK_EQ(cross[1 * 256 + 1], 0.0f);      // 2 * (1,0).(0,1)
    CHECK_EQ(cross[2 * 256 + 2], 4.0f);      // 2 * (0,2).(1,1)
    fx::WriteErrorBounds(fx::Tmp("pq2_eps_bad.bin"), {0.0f});
    CHECK_THROWS(r.LoadPq2Index(fx::Tmp("pq2_res_pivots.bin"), fx::Tmp("pq2_res_codes.bin"), fx::Tmp("pq2_eps_bad.bin")));
    r.LoadPq2Index(fx::Tmp("pq2_res_pivots.bin"), fx::Tmp("pq2_res_codes.bin"), fx::Tmp("pq2_eps.bin"));
    const VectorPageLayout layout = VectorPageLayout::Create(2, ScalarKind::kFloat32);
    VectorStoreBuilder::WriteFile(fx::Tmp("pq2_vectors.ssd"), layout, ScalarKind::kFloat32, 2,
                                  {fx::FloatBytes({1.0f, 1.0f}), fx::FloatBytes({1.0f, 3.0f})});
    r.LoadVectorStore(fx::Tmp("pq2_vectors.ssd"));
    r.AttachVectorPageProvider(std::make_shared<HbmVectorPageProvider>(fx::Tmp("pq2_vectors.ssd")));
    // Query (1,1): base PQ distances are node 0 -> 1, node 1 -> 2; the refined distances are 2 and 6,
    // node 0's exact distance is 0, and node 1's lower bound (6 - |q|^2 = 4) exceeds it, so it is filtered.
    TopoAnnsSearchParams p;
    p.topology.top_k = 2; p.topology.top_l = 2; p.topology.search_width = 1; p.topology.max_expansions = 8;
    p.rerank.top_k = 1; p.rerank.top_n = 2; p.rerank.mode = RerankExecutionMode::kPageByPage; p.rerank.rank_tile_size = 1;
    p.rerank.use_pq2_refine = true; p.rerank.use_pq2_bound_filter = true; p.rerank.pq2_refine_top_l = 2;
    const auto res = TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {1.0f, 1.0f}, 1, p);
    CHECK_EQ(res.rerank_stats.exact_distance_count, std::size_t{1});
    CHECK_EQ(res.rerank_stats.bound_filtered_count, std::size_t{1});
    CHECK_EQ(res.queries[0].rerank.topk.size(), std::size_t{1});
    CHECK_EQ(res.queries[0].rerank.topk[0].node_id, 0u);
    p.rerank.use_pq2_bound_filter = false;
    const auto plain = TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {1.0f, 1.0f}, 1, p);
    CHECK_EQ(plain.rerank_stats.exact_distance_count, std::size_t{2});
    CHECK_EQ(plain.queries[0].rerank.sorted_candidates[1].node_id, 1u);
    CHECK_EQ(plain.queries[0].rerank.sorted_candidates[1].distance, 4.0f);
    p.rerank.use_pq2_bound_filter = true; p.rerank.mode = RerankExecutionMode::kLinear;
    CHECK_THROWS(TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {1.0f, 1.0f}, 1, p));
}

void TestHpqIndexAndRefine() {
    // Hybrid PQ (include/topoanns/hpq_index.hpp, src/io/hpq_index.cpp, refine src/search/rerank_exact.cu:667-771):
    // one chunk of one dim; base table[c] = c, outlier table[c] = 100 + c; node n's hybrid code is n + 1 and the
    // selector bit of node 1 picks the outlier codebook. Query 0: hybrid distances are node 0 -> 1^2,
    // node 1 -> 102^2, node 2 -> 3^2, so the refined order is 0, 2, 1 although the base codes order them 0, 1, 2.
    std::vector<float> out_tables(256);
    for (std::size_t c = 0; c < 256; ++c) out_tables[c] = 100.0f + static_cast<float>(c);
    fx::WritePq(fx::Tmp("hpq_base_pivots.bin"), fx::Tmp("hpq_base_codes.bin"), 1, fx::RampTables(1), {1, 2, 3});
    fx::WritePq(fx::Tmp("hpq_outlier_pivots.bin"), fx::Tmp("hpq_codes.bin"), 1, out_tables, {1, 2, 3});
    {
        std::ofstream f(fx::Tmp("hpq_selector.bin"), std::ios::binary | std::ios::trunc);
        const std::int32_t rows = 3, cols = 1;
        const std::uint8_t bits[3] = {0, 1, 0};
        f.write(reinterpret_cast<const char*>(&rows), 4);
        f.write(reinterpret_cast<const char*>(&cols), 4);
        f.write(reinterpret_cast<const char*>(bits), 3);
    }
    SearchResources r = SearchResources::FromDataset(TopologyLayout::MakePadded(3, {{1, 2}, {}, {}}));
    CHECK_THROWS(r.LoadHpqIndex(fx::Tmp("hpq_base_pivots.bin"), fx::Tmp("hpq_outlier_pivots.bin"), fx::Tmp("hpq_codes.bin"),
                                fx::Tmp("hpq_selector.bin")));   // base PQ index first
    r.LoadPqIndex(fx::Tmp("hpq_base_pivots.bin"), fx::Tmp("hpq_base_codes.bin"));
    CHECK_TRUE(!r.has_hpq_index());
    CHECK_THROWS(r.hpq_index());
    r.LoadHpqIndex(fx::Tmp("hpq_base_pivots.bin"), fx::Tmp("hpq_outlier_pivots.bin"), fx::Tmp("hpq_codes.bin"),
                   fx::Tmp("hpq_selector.bin"));
    CHECK_TRUE(r.has_hpq_index());
    CHECK_EQ(r.hpq_index().selector_stride_bytes(), std::size_t{1});
    CHECK_TRUE(r.hpq_index().outlier_index().codes_are_mapped());
    CHECK_TRUE(r.hpq_index().device_selector_bits() != nullptr);
    TopologySearchParams tp;
    tp.top_k = 3; tp.top_l = 4; tp.search_width = 1; tp.max_expansions = 8;
    const auto lists = HpqRefine::RunBatchFloat32(r, MakeEntryBatch(1, {0}), {0.0f}, 1, tp, 4);
    CHECK_EQ(lists.size(), std::size_t{1});
    CHECK_EQ(lists[0].size(), std::size_t{3});
    CHECK_EQ(lists[0][0].node_id, 0u);
    CHECK_EQ(lists[0][0].distance, 1.0f);
    CHECK_EQ(lists[0][1].node_id, 2u);
    CHECK_EQ(lists[0][1].distance, 9.0f);
    CHECK_EQ(lists[0][2].node_id, 1u);
    CHECK_EQ(lists[0][2].distance, 102.0f * 102.0f);
    // a selector file of the wrong shape is refused
    {
        std::ofstream f(fx::Tmp("hpq_selector_bad.bin"), std::ios::binary | std::ios::trunc);
        const std::int32_t rows = 2, cols = 1;
        const std::uint8_t bits[2] = {0, 1};
        f.write(reinterpret_cast<const char*>(&rows), 4);
        f.write(reinterpret_cast<const char*>(&cols), 4);
        f.write(reinterpret_cast<const char*>(bits), 2);
    }
    CHECK_THROWS(HpqIndex::Load(fx::Tmp("hpq_base_pivots.bin"), fx::Tmp("hpq_outlier_pivots.bin"), fx::Tmp("hpq_codes.bin"),
                                fx::Tmp("hpq_selector_bad.bin")));
}

void TestLearnedRerankStop() {
    // Persistent rerank with the learned stop (src/io/bam_vector_provider.cu:721-1323, :2471-2774) through the
    // fused entry point. 24 nodes on a line, query at 0: node i is at i + 1 (exact distance (i + 1)^2) but its
    // PQ code says 24 - i, so the candidate list is ranked 23, 22, ..., 0 and every window of four ranks
    // improves the best-2 list. Error bounds of 100 make every lower bound 0: nothing is filtered.
    const std::size_t n = 24;
    std::vector<std::uint8_t> base_codes(n), zero_codes(n, 0);
    std::vector<float> eps(n, 100.0f);
    std::vector<std::vector<std::uint8_t>> rows;
    std::vector<std::vector<std::uint32_t>> lists(n);
    for (std::size_t i = 0; i < n; ++i) {
        base_codes[i] = static_cast<std::uint8_t>(n - i);
        rows.push_back(fx::FloatBytes({static_cast<float>(i + 1)}));
        if (i > 0) lists[0].push_back(static_cast<std::uint32_t>(i));
    }
    fx::WritePq(fx::Tmp("ls_base_pivots.bin"), fx::Tmp("ls_base_codes.bin"), 1, fx::RampTables(1), base_codes);
    fx::WritePq(fx::Tmp("ls_res_pivots.bin"), fx::Tmp("ls_res_codes.bin"), 1, std::vector<float>(256, 0.0f), zero_codes);
    fx::WriteErrorBounds(fx::Tmp("ls_eps.bin"), eps);
    SearchResources r = SearchResources::FromDataset(TopologyLayout::MakePadded(n, lists));
    r.LoadPqIndex(fx::Tmp("ls_base_pivots.bin"), fx::Tmp("ls_base_codes.bin"));
    r.LoadPq2Index(fx::Tmp("ls_res_pivots.bin"), fx::Tmp("ls_res_codes.bin"), fx::Tmp("ls_eps.bin"));
    const VectorPageLayout layout = VectorPageLayout::Create(1, ScalarKind::kFloat32);
    VectorStoreBuilder::WriteFile(fx::Tmp("ls_vectors.ssd"), layout, ScalarKind::kFloat32, 1, rows);
    r.LoadVectorStore(fx::Tmp("ls_vectors.ssd"));
    r.AttachVectorPageProvider(std::make_shared<HbmVectorPageProvider>(fx::Tmp("ls_vectors.ssd")));
    // logit = 1 - 4 * (ranks scored / 24): 1/3 after the bootstrap window (no stage there), -1/3 at the
    // stage at 8, -1 at the stage at 12, which is below the threshold -0.5.
    {
        std::ofstream model(fx::Tmp("ls_model.txt"));
        model << "# synthetic model\nstage_prefixes = 8, 12, 16\nbootstrap_prefix = 4\n"
              << "feature_means = 0,0,0,0,0,0,0,0,0,0,0,0,0\nfeature_inv_stds = 1,1,1,1,1,1,1,1,1,1,1,1,1\n"
              << "weights = 0,-4,0,0,0,0,0,0,0,0,0,0,0\nbias = 1\nthreshold_logit = -0.5\n";
    }
    TopoAnnsSearchParams p;
    p.topology.top_k = 24; p.topology.top_l = 24; p.topology.search_width = 1; p.topology.max_expansions = 64;
    p.rerank.top_k = 2; p.rerank.top_n = 24; p.rerank.mode = RerankExecutionMode::kPersistent; p.rerank.rank_tile_size = 4;
    p.rerank.use_pq2_refine = true; p.rerank.use_pq2_bound_filter = true; p.rerank.pq2_refine_top_l = 24;
    p.rerank.use_learned_stop = true; p.rerank.learned_stop_model_path = fx::Tmp("ls_model.txt");
    unsetenv("TOPOANNS_RERANK_STOP_PREFIX_RECORD_PATH");
    unsetenv("TOPOANNS_RERANK_STOP_PREFIX_REPLAY_PATH");
    const auto check_stopped_at_12 = [&](const TopoAnnsBatchResult& res) {
        CHECK_EQ(res.rerank_stats.exact_distance_count, std::size_t{12});
        CHECK_EQ(res.rerank_stats.bound_filtered_count, std::size_t{0});
        CHECK_EQ(res.queries[0].rerank.sorted_candidates.size(), std::size_t{2});   // the top_k list only
        CHECK_EQ(res.queries[0].rerank.topk.size(), std::size_t{2});
        CHECK_EQ(res.queries[0].rerank.topk[0].node_id, 12u);
        CHECK_EQ(res.queries[0].rerank.topk[0].distance, 169.0f);
        CHECK_EQ(res.queries[0].rerank.topk[1].node_id, 13u);
        CHECK_EQ(res.queries[0].rerank.topk[1].distance, 196.0f);
    };
    const auto res = TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {0.0f}, 1, p);
    check_stopped_at_12(res);
    CHECK_EQ(res.rerank_profile.learned_stop_queries, std::size_t{1});
    CHECK_EQ(res.rerank_profile.learned_stop_checkpoints, std::size_t{2});
    CHECK_EQ(res.rerank_profile.learned_stop_prefix_sum, std::size_t{12});
    CHECK_EQ(res.rerank_profile.learned_stop_prefix_min, std::size_t{12});
    CHECK_EQ(res.rerank_profile.learned_stop_prefix_max, std::size_t{12});
    // record the stop prefixes of two batches, then replay them: same lists, the model is not evaluated
    const std::string trace = fx::Tmp("ls_trace.bin").string();
    setenv("TOPOANNS_RERANK_STOP_PREFIX_RECORD_PATH", trace.c_str(), 1);
    check_stopped_at_12(TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {0.0f}, 1, p));
    check_stopped_at_12(TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {0.0f}, 1, p));
    CHECK_EQ(std::filesystem::file_size(trace), std::uintmax_t{2 * (12 + 4)});
    setenv("TOPOANNS_RERANK_STOP_PREFIX_REPLAY_PATH", trace.c_str(), 1);
    CHECK_THROWS(TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {0.0f}, 1, p));   // both set
    unsetenv("TOPOANNS_RERANK_STOP_PREFIX_RECORD_PATH");
    for (int batch = 0; batch < 2; ++batch) {
        const auto again = TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {0.0f}, 1, p);
        check_stopped_at_12(again);
        CHECK_EQ(again.rerank_profile.learned_stop_queries, std::size_t{0});
        CHECK_EQ(again.rerank_profile.learned_stop_checkpoints, std::size_t{0});
    }
    CHECK_THROWS(TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {0.0f}, 1, p));   // the trace has two records
    unsetenv("TOPOANNS_RERANK_STOP_PREFIX_REPLAY_PATH");
    // a threshold that nothing reaches: every rank is scored, the list is the true best two
    {
        std::ofstream model(fx::Tmp("ls_model_never.txt"));
        model << "stage_prefixes = 8, 12, 16\nbootstrap_prefix = 4\nfeature_means = 0,0,0,0,0,0,0,0,0,0,0,0,0\n"
              << "feature_inv_stds = 1,1,1,1,1,1,1,1,1,1,1,1,1\nweights = 0,-4,0,0,0,0,0,0,0,0,0,0,0\nbias = 1\n"
              << "threshold_logit = -100\n";
    }
    TopoAnnsSearchParams never = p;
    never.rerank.learned_stop_model_path = fx::Tmp("ls_model_never.txt");
    const auto full = TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {0.0f}, 1, never);
    CHECK_EQ(full.rerank_stats.exact_distance_count, std::size_t{24});
    CHECK_EQ(full.queries[0].rerank.topk[0].node_id, 0u);
    CHECK_EQ(full.queries[0].rerank.topk[1].node_id, 1u);
    CHECK_EQ(full.rerank_profile.learned_stop_checkpoints, std::size_t{3});
    CHECK_EQ(full.rerank_profile.learned_stop_prefix_sum, std::size_t{24});
    // the reference's parameter checks (src/search/rerank_exact.cu:2586-2602)
    TopoAnnsSearchParams bad = p;
    bad.rerank.mode = RerankExecutionMode::kTiled;
    CHECK_THROWS(TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {0.0f}, 1, bad));
    bad = p;
    bad.rerank.use_pq2_bound_filter = false;
    CHECK_THROWS(TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {0.0f}, 1, bad));
    bad = p;
    bad.rerank.learned_stop_model_path.clear();
    CHECK_THROWS(TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {0.0f}, 1, bad));
    bad = p;
    bad.rerank.learned_stop_model_path = fx::Tmp("ls_no_such_model.txt");
    CHECK_THROWS(TopoAnnsSearch::RunBatchFloat32Fused(r, MakeEntryBatch(1, {0}), {0.0f}, 1, bad));
}

void TestRvqModel() {
    // two coarse x two fine centroids in 2-d; model file in the reference's layout
    const auto path = fx::Tmp("rvq_model.bin");
    {
        std::ofstream out(path, std::ios::binary | std::ios::trunc);
        const std::int32_t hdr[3] = {2, 2, 2};
        out.write(reinterpret_cast<const char*>(hdr), sizeof(hdr));
        const float coarse[4] = {0, 0, 10, 10}, fine[4] = {-1, 0, 1, 0};
        out.write(reinterpret_cast<const char*>(coarse), sizeof(coarse));
        out.write(reinterpret_cast<const char*>(fine), sizeof(fine));
        const std::uint64_t two = 2;
        out.write(reinterpret_cast<const char*>(&two), 8);
        const std::vector<std::vector<std::int32_t>> buckets = {{4, 5, 6}, {}, {7}, {8, 9}};
        for (int c = 0; c < 2; ++c) {
            out.write(reinterpret_cast<const char*>(&two), 8);
            for (int f = 0; f < 2; ++f) {
                const auto& b = buckets[c * 2 + f];
                const std::uint64_t n = b.size();
                out.write(reinterpret_cast<const char*>(&n), 8);
                out.write(reinterpret_cast<const char*>(b.data()), static_cast<std::streamsize>(n * 4));
            }
        }
    }
    const RvqModel model = RvqModel::Load(path);
    CHECK_EQ(model.dim(), 2u); CHECK_EQ(model.coarse_centroids(), 2u); CHECK_EQ(model.fine_centroids(), 2u);
    model.WarmUp();
    // q0 near coarse 0, residual (+0.9, 0) -> fine 1 is empty -> falls to fine 0 = bucket {4,5,6}
    // q1 near coarse 1, residual (+1, 0) -> fine 1 -> bucket {8,9}
    const std::vector<float> q = {0.9f, 0.0f, 11.0f, 10.0f};
    const auto host_entries = model.ComputeFloat32EntryPoints(q, 2, 2);
    CHECK_TRUE(host_entries[0] == (std::vector<std::uint32_t>{4, 5}));
    CHECK_TRUE(host_entries[1] == (std::vector<std::uint32_t>{8, 9}));
    const DeviceEntryBatch batch = model.ComputeFloat32DeviceEntryBatch(q, 2, 4, 77);
    CHECK_EQ(batch.entries_per_query, std::size_t{4});
    CHECK_TRUE(batch.offsets.CopyToHost() == (std::vector<std::uint32_t>{0, 4, 8}));
    CHECK_TRUE(batch.ids.CopyToHost() == (std::vector<std::uint32_t>{4, 5, 6, kInvalidNodeId, 8, 9, kInvalidNodeId, kInvalidNodeId}));
    CHECK_THROWS(model.ComputeFloat32DeviceEntryBatch(q, 2, 0));
    CHECK_THROWS(model.ComputeFloat32DeviceEntryBatch(q, 3, 2));
    const RvqEntryProvider provider = RvqEntryProvider::FromFloatQueries(model, q, 2, 3);
    CHECK_EQ(provider.num_queries(), std::size_t{2});
    CHECK_TRUE(provider.GetEntryPoints(0) == (std::vector<std::uint32_t>{4, 5, 6}));
    CHECK_THROWS(provider.GetEntryPoints(2));
    CHECK_THROWS(RvqModel().dim());
}

}  // namespace

int main() {
    TestQueryTablesAndOracle();
    TestTopologyAndResources();
    TestRerankAndEndToEnd();
    TestUint8EntryPoint();
    TestPq2();
    TestHpqIndexAndRefine();
    TestLearnedRerankStop();
    TestRvqModel();
    std::cout << "test_api_search passed" << std::endl;
    return 0;
}
