// Host-only parts of the API: layouts, file round trips, entry providers, the stop rule.
// Mirrors tests/test_topology_layout.cpp, test_vector_page_layout.cpp, test_vector_store_builder.cpp,
// test_entry_provider.cpp and test_search_stop_condition.cpp of the reference.
#include "fixtures.hpp"

using namespace topoanns;

int main() {
    // topology layout: padding to 64 slots with 0xffffffff, offsets, file round trip
    const TopologyDataset ds = TopologyLayout::MakePadded(3, {{1, 2}, {}, {0}});
    CHECK_EQ(ds.degree, 64u);
    CHECK_EQ(ds.adjacency.size(), std::size_t{3 * 64});
    CHECK_EQ(ds.NodeNeighbors(0)[1], 2u);
    CHECK_EQ(ds.NodeNeighbors(0)[2], kInvalidNodeId);
    CHECK_EQ(TopologyLayout::NodeBytes(), std::size_t{256});
    CHECK_EQ(TopologyLayout::NodeOffsetBytes(2), std::uint64_t{4096 + 512});
    CHECK_THROWS(ds.NodeNeighbors(3));
    CHECK_THROWS(TopologyLayout::MakePadded(2, {{1}}));
    CHECK_THROWS(TopologyLayout::MakePadded(1, {std::vector<std::uint32_t>(65, 0u)}));
    const auto path = fx::Tmp("tann_api_topology.bin");
    TopologyLayout::WriteFile(path, ds);
    CHECK_EQ(std::filesystem::file_size(path), std::uintmax_t{4096 + 3 * 64 * 4});
    const TopologyHeader h = TopologyLayout::ReadHeader(path);
    CHECK_EQ(h.num_nodes, std::uint64_t{3});
    CHECK_EQ(h.payload_bytes, std::uint64_t{3 * 64 * 4});
    const TopologyDataset back = TopologyLayout::ReadFile(path);
    CHECK_TRUE(back.adjacency == ds.adjacency);
    // compact degree-32 records load too
    const TopologyDataset d32 = TopologyLayout::MakePaddedDegree(2, 32, {{1}, {0}});
    TopologyLayout::WriteFile(path, d32);
    CHECK_EQ(TopologyLayout::ReadFile(path).degree, 32u);
    { std::ofstream f(path, std::ios::binary | std::ios::trunc); f << "short"; }
    CHECK_THROWS(TopologyLayout::ReadFile(path));

    // vector page layout: 512-byte vectors -> 8 per page, 100-byte -> 40, > 4 KB throws
    CHECK_EQ(VectorPageLayout::Create(128, ScalarKind::kFloat32).vectors_per_page(), std::size_t{8});
    CHECK_EQ(VectorPageLayout::CreateFromVectorBytes(100).vectors_per_page(), std::size_t{40});
    CHECK_THROWS(VectorPageLayout::Create(2000, ScalarKind::kFloat32));
    const VectorPageLayout lay = VectorPageLayout::Create(96, ScalarKind::kFloat32);
    CHECK_EQ(lay.vectors_per_page(), std::size_t{10});
    const VectorPageAddress a = lay.Resolve(23);
    CHECK_EQ(a.page_id, std::uint64_t{2});
    CHECK_EQ(a.slot_id, 3u);
    CHECK_EQ(a.byte_offset, std::uint64_t{4096 + 2 * 4096 + 3 * 384});
    CHECK_EQ(lay.PageCountForVectors(21), std::uint64_t{3});

    // vector store round trip
    const auto vpath = fx::Tmp("tann_api_vectors.ssd");
    const VectorPageLayout l8 = VectorPageLayout::Create(128, ScalarKind::kUint8);
    std::vector<std::vector<std::uint8_t>> vecs(70, std::vector<std::uint8_t>(128));
    for (std::size_t i = 0; i < vecs.size(); ++i)
        for (std::size_t k = 0; k < 128; ++k) vecs[i][k] = static_cast<std::uint8_t>((i * 7 + k) & 255);
    VectorStoreBuilder::WriteFile(vpath, l8, ScalarKind::kUint8, 128, vecs);
    const VectorStoreHeader vh = VectorStoreBuilder::ReadHeader(vpath);
    CHECK_EQ(vh.num_vectors, std::uint64_t{70});
    CHECK_EQ(vh.vectors_per_page, std::uint64_t{32});
    CHECK_EQ(std::filesystem::file_size(vpath), std::uintmax_t{4096 + 3 * 4096});
    CHECK_TRUE(VectorStoreBuilder::ReadVectorById(vpath, l8, 45) == vecs[45]);

    // entry providers
    FixedEntryProvider fixed({3, 4});
    CHECK_TRUE(fixed.GetEntryPoints(17) == (std::vector<std::uint32_t>{3, 4}));
    PerQueryEntryProvider per({{1}, {2, 3}});
    CHECK_TRUE(per.GetEntryPoints(1) == (std::vector<std::uint32_t>{2, 3}));
    CHECK_THROWS(per.GetEntryPoints(2));

    // stop rule
    std::vector<RankedCandidate> c = {{1.0f, 5, true}, {2.0f, 3, false}, {3.0f, 1, false}};
    CHECK_EQ(SearchStopCondition::CountValid(c), std::size_t{3});
    CHECK_EQ(SearchStopCondition::BestUnexpandedRank(c), std::size_t{1});
    CHECK_TRUE(!SearchStopCondition::TopLHasNoBetterUnexpanded(c, 2));
    CHECK_TRUE(SearchStopCondition::TopLHasNoBetterUnexpanded(c, 1));
    CHECK_TRUE(!SearchStopCondition::TopLHasNoBetterUnexpanded(c, 4));
    CHECK_TRUE(SearchStopCondition::TopLHasNoBetterUnexpanded(c, 0));
    std::cout << "test_api_host passed" << std::endl;
    return 0;
}
