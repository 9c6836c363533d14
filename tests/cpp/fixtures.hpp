// Shared fixtures of the C++ API tests: tiny PQ files, vector stores and a check macro. The numeric
// fixtures are the ones the reference's tests use (tests/test_*.cpp of szrr/TopoANNS), so the
// expected values below are that project's own known answers.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <iostream>
#include <sstream>
#include <vector>

#include "topoanns/api.hpp"

#define CHECK_TRUE(expr)                                                                   \
    do {                                                                                   \
        if (!(expr)) {                                                                     \
            std::cerr << __FILE__ << ":" << __LINE__ << ": check failed: " #expr << "\n";  \
            std::exit(1);                                                                  \
        }                                                                                  \
    } while (0)
#define CHECK_EQ(a, b)                                                                                     \
    do {                                                                                                   \
        const auto va__ = (a);                                                                             \
        const auto vb__ = (b);                                                                             \
        if (!(va__ == vb__)) {                                                                             \
            std::cerr << __FILE__ << ":" << __LINE__ << ": " #a " == " #b " failed (" << va__ << " vs " << vb__ << ")\n"; \
            std::exit(1);                                                                                  \
        }                                                                                                  \
    } while (0)
#define CHECK_THROWS(stmt)                                                                 \
    do {                                                                                   \
        bool threw__ = false;                                                              \
        try { stmt; } catch (const std::runtime_error&) { threw__ = true; }                \
        if (!threw__) {                                                                    \
            std::cerr << __FILE__ << ":" << __LINE__ << ": expected a throw: " #stmt << "\n"; \
            std::exit(1);                                                                  \
        }                                                                                  \
    } while (0)

namespace fx {

inline std::filesystem::path Tmp(const std::string& name) {
    const char* dir = std::getenv("TANN_TEST_TMP");
    return std::filesystem::path(dir != nullptr ? dir : "/tmp") / name;
}

template <typename T>
void PutBlock(std::vector<char>& buf, std::size_t offset, std::int32_t rows, std::int32_t cols, const std::vector<T>& data) {
    if (buf.size() < offset + 8 + data.size() * sizeof(T)) buf.resize(offset + 8 + data.size() * sizeof(T), 0);
    std::memcpy(buf.data() + offset, &rows, 4);
    std::memcpy(buf.data() + offset + 4, &cols, 4);
    if (!data.empty()) std::memcpy(buf.data() + offset + 8, data.data(), data.size() * sizeof(T));
}

// DiskANN-style pivots + compressed files with one chunk covering all `dim` dims.
inline void WritePq(const std::filesystem::path& pivots, const std::filesystem::path& codes_path, std::size_t dim,
                    const std::vector<float>& tables /*256 x dim*/, const std::vector<std::uint8_t>& codes /*N x 1*/) {
    const std::size_t t_off = 4096, c_off = t_off + 8 + 256 * dim * 4, o_off = c_off + 8 + dim * 4;
    std::vector<char> buf(4096, 0);
    PutBlock<std::size_t>(buf, 0, 4, 1, {t_off, c_off, o_off, 0});
    PutBlock<float>(buf, t_off, 256, static_cast<std::int32_t>(dim), tables);
    PutBlock<float>(buf, c_off, static_cast<std::int32_t>(dim), 1, std::vector<float>(dim, 0.0f));
    PutBlock<std::uint32_t>(buf, o_off, 2, 1, {0u, static_cast<std::uint32_t>(dim)});
    std::ofstream(pivots, std::ios::binary | std::ios::trunc).write(buf.data(), static_cast<std::streamsize>(buf.size()));
    std::ofstream out(codes_path, std::ios::binary | std::ios::trunc);
    const std::int32_t rows = static_cast<std::int32_t>(codes.size()), cols = 1;
    out.write(reinterpret_cast<const char*>(&rows), 4);
    out.write(reinterpret_cast<const char*>(&cols), 4);
    out.write(reinterpret_cast<const char*>(codes.data()), static_cast<std::streamsize>(codes.size()));
}

inline std::vector<float> RampTables(std::size_t dim) {  // tables[c][*] = c
    std::vector<float> t(256 * dim);
    for (std::size_t c = 0; c < 256; ++c)
        for (std::size_t k = 0; k < dim; ++k) t[c * dim + k] = static_cast<float>(c);
    return t;
}

inline std::vector<std::uint8_t> FloatBytes(const std::vector<float>& v) {
    std::vector<std::uint8_t> b(v.size() * 4);
    std::memcpy(b.data(), v.data(), b.size());
    return b;
}

inline void WriteErrorBounds(const std::filesystem::path& path, const std::vector<float>& eps) {
    std::vector<char> buf;
    PutBlock<float>(buf, 0, static_cast<std::int32_t>(eps.size()), 1, eps);
    std::ofstream(path, std::ios::binary | std::ios::trunc).write(buf.data(), static_cast<std::streamsize>(buf.size()));
}

// The 6-node graph and codes used throughout the reference's search tests.
inline topoanns::TopologyDataset ToyGraph() { return topoanns::TopologyLayout::MakePadded(6, {{1, 2}, {3}, {4}, {5}, {5}, {}}); }
inline std::vector<std::uint8_t> ToyCodes() { return {9, 6, 7, 2, 3, 1}; }

}  // namespace fx
