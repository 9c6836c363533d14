// CPU restatement of the TopoANNS batched graph-search path.
//
// TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA path: it is called by the
// tests, by the smoke check and by the benchmark's CPU-baseline leg. Nothing that ships may call
// it, and the product library never falls back to it.
//
// Every function restates, in plain scalar C++, what the reference computes for one step of the
// path; citations are file:line inside the reference project (szrr/TopoANNS).
//
// Pinning: the functions below are checked against the known-answer values asserted by the
// reference's own tests (tests/test_pq_query_tables.cpp:102-116,
// tests/test_topology_search_gpu.cpp:182-221, tests/test_topology_search_batch_gpu.cpp:182-199,
// tests/test_rerank_exact.cpp:133-145, tests/test_pq2_residual_refine.cpp:134-138,
// tests/test_pq2_bound_filter.cpp:167-171), and against outputs of the reference's own kernels: the
// reference's sources for this path compile in place (oracle/ref_build.sh) and, run on a B200, give
// tables, candidate lists, per-query statistics, refined lists and rerank output that this file
// reproduces bit for bit (tests/test_reference_pin.py; a small recorded case is committed as
// tests/golden/reference_small.npz and checked on the CPU). That covers the Bloom filter's
// false-positive behaviour and the visited-set protocol as well. Still "parity unpinned": RVQ entry
// selection (the reference scores with a cuBLAS GEMM whose summation order is not published) and
// the learned traversal stop (no model file or known-answer test in the reference).
//
// Floating point: where the reference's device code is `acc += a * b` nvcc contracts it to one
// fused multiply-add, so the restatement calls fmaf() explicitly; this file is compiled with
// -ffp-contract=off so that nothing else is fused.

#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr uint32_t kInvalid = 0xffffffffu;        // include/topoanns/common.hpp:15
constexpr uint32_t kExpandedBit = 0x80000000u;    // src/search/topology_search_kernel.hpp:16
constexpr uint32_t kRawMask = 0x7fffffffu;        // src/search/topology_search_kernel.hpp:17
constexpr uint32_t kBloomWords = 1024;            // src/search/topology_search_kernel.cu:55
constexpr uint32_t kCentroids = 256;              // include/topoanns/pq_index.hpp:15

struct Cand {
    float dist;
    uint32_t id;  // bit 31 = expanded; 0xffffffff = invalid
};

inline uint32_t RawId(uint32_t packed) { return packed == kInvalid ? kInvalid : (packed & kRawMask); }
inline bool IsExpanded(uint32_t packed) { return packed != kInvalid && (packed & kExpandedBit); }

// src/search/topology_search_kernel.cu:414-420
inline bool CandLess(const Cand& a, const Cand& b) {
    if (a.dist != b.dist) return a.dist < b.dist;
    return RawId(a.id) < RawId(b.id);
}

// src/search/topology_search_kernel.cu:382-385
const uint32_t kSeeds[10] = {0x924ed183u, 0xd854fc0au, 0xecf5e3b7u, 0x1bead407u, 0x28a30449u,
                             0xbfc4d99fu, 0x715030e2u, 0xffcfb45bu, 0x6e4ce166u, 0xeb53c362u};

// src/search/topology_search_kernel.cu:611-619
inline uint32_t BloomHash(int h, uint32_t v) {
    v ^= v >> 16;
    v *= kSeeds[h << 1];
    v ^= v >> 13;
    v *= kSeeds[(h << 1) + 1];
    v ^= v >> 16;
    return v % (kBloomWords << 5);
}

// src/search/topology_search_kernel.cu:637-653
inline void BloomAdd(uint32_t v, uint32_t* words) {
    for (int h = 0; h < 3; ++h) {
        const uint32_t bit = BloomHash(h, v);
        words[bit % kBloomWords] |= 1u << (bit / kBloomWords);
    }
}
inline bool BloomTest(uint32_t v, const uint32_t* words) {
    bool ok = true;
    for (int h = 0; h < 3; ++h) {
        const uint32_t bit = BloomHash(h, v);
        ok &= ((words[bit % kBloomWords] >> (bit / kBloomWords)) & 1u) != 0u;
    }
    return ok;
}

// The 16/8/4/2/1 shuffle-down tree of src/search/topology_search_kernel.cu:444-451 (same tree in
// src/search/rerank_exact.cu:267-271,609-613): lane 0 ends up with the value computed here.
inline float WarpTree(float* lane) {
    for (int off = 16; off >= 1; off >>= 1) {
        for (int i = 0; i < off; ++i) lane[i] = lane[i] + lane[i + off];
    }
    return lane[0];
}

// src/search/topology_search_kernel.cu:656-692 (generic branch): per group of 32 chunks one tree,
// group results added in order.
inline float AdcTree(const float* lut, const uint8_t* codes, uint32_t M) {
    float partial = 0.0f;
    for (uint32_t base = 0; base < M; base += 32) {
        float lane[32];
        for (uint32_t l = 0; l < 32; ++l) {
            const uint32_t c = base + l;
            float v = 0.0f;
            if (c < M) v += lut[c * kCentroids + codes[c]];
            lane[l] = v;
        }
        partial += WarpTree(lane);
    }
    return partial;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------------------------
// a1. PQ query tables. src/search/pq_query_tables.cu:13-53: shared_query = float(q) - centroid;
// out[c] accumulates (table[c][dim] - shared_query[dim])^2 over the chunk's dims in ascending
// order, starting from the zero-filled buffer (:78-80); `+= diff * diff` is one FMA on device.
// tables_row_major is [256][d] as stored in the pivots file (src/io/pq_index.cpp:147-155).
// query_kind: 0 = int8, 1 = uint8, 2 = float32 (include/topoanns/common.hpp:17-21).
void orc_lut_build(const void* queries, int query_kind, uint64_t Q, uint32_t d, uint32_t M,
                   const float* tables_row_major, const float* centroid,
                   const uint32_t* chunk_offsets, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < (int64_t)Q; ++q) {
        std::vector<float> sq(d);
        for (uint32_t i = 0; i < d; ++i) {
            float v;
            if (query_kind == 2) v = static_cast<const float*>(queries)[q * d + i];
            else if (query_kind == 1) v = static_cast<float>(static_cast<const uint8_t*>(queries)[q * d + i]);
            else v = static_cast<float>(static_cast<const int8_t*>(queries)[q * d + i]);
            sq[i] = v - centroid[i];
        }
        float* o = out + (uint64_t)q * M * kCentroids;
        for (uint32_t m = 0; m < M; ++m) {
            for (uint32_t c = 0; c < kCentroids; ++c) {
                float acc = 0.0f;
                for (uint32_t dim = chunk_offsets[m]; dim < chunk_offsets[m + 1]; ++dim) {
                    const float diff = tables_row_major[(uint64_t)c * d + dim] - sq[dim];
                    acc = fmaf(diff, diff, acc);
                }
                o[m * kCentroids + c] = acc;
            }
        }
    }
}

// Host-side distance of the reference: serial sum over chunks,
// src/search/pq_query_tables.cu:206-237.
float orc_adc_serial(const float* lut, const uint8_t* codes, uint32_t M) {
    float dist = 0.0f;
    for (uint32_t m = 0; m < M; ++m) dist += lut[m * kCentroids + codes[m]];
    return dist;
}

// Device-side distance of the reference traversal kernel (tree order), see AdcTree above.
float orc_adc_tree(const float* lut, const uint8_t* codes, uint32_t M) { return AdcTree(lut, codes, M); }

// ---------------------------------------------------------------------------------------------
// a4. Learned traversal stop, folded form. src/search/topology_search_kernel.cu:98-112 (device
// struct), :327-380 (folding of mean / inverse std into weights and bias, done by the caller).
struct OrcLearnedStop {
    uint32_t enabled;
    uint32_t num_stages;
    uint32_t top_k;
    uint32_t shadow_mode;
    uint32_t topk_churn_flag_mode;  // 1 = "flag", 0 = ratio
    uint32_t next64_flag_mode;      // 1 = "flag", 0 = fraction
    uint32_t stage_prefixes[32];
    uint32_t feature_mask[12];
    float weights[12];
    float bias;
    float threshold_logit;
    float inv_top_l;
};

struct OrcBeamParams {
    uint64_t num_nodes;
    uint32_t degree;
    uint32_t num_chunks;
    uint32_t top_l;
    uint32_t search_width;
    uint32_t max_expansions;
    uint32_t candidate_capacity;   // power of two, >= top_l
    uint32_t stop_prefix;          // = top_l unless TOPOANNS_CANDIDATE_STOP_* narrows it
    uint32_t stop_use_expanded;
    uint32_t two_phase;            // 1: per round of 128 slots all Bloom tests, then all adds; 0: slot by slot
    uint32_t reserved;
};

}  // extern "C"

namespace {

struct BeamState {
    std::vector<Cand> cand;
    std::vector<Cand> frontier;
    std::vector<uint32_t> bloom;
    std::vector<uint32_t> unexpanded;
    uint32_t valid = 0, visited = 0, expanded = 0, iterations = 0;
    uint32_t first_full = 0xffffffffu;
    uint32_t hash_iter = 0;
    // learned stop
    uint32_t ls_stage = 0, ls_has_prev = 0, ls_topk_changed = 0;
    float ls_prev_dk = std::numeric_limits<float>::infinity();
    float ls_prev_boundary = std::numeric_limits<float>::infinity();
    uint32_t ls_prev_ids[32];
};

// src/search/topology_search_kernel.cu:856-893
uint32_t CountBitsInRange(const uint32_t* bits, uint32_t b, uint32_t e) {
    uint32_t n = 0;
    for (uint32_t i = b; i < e; ++i) n += (bits[i >> 5] >> (i & 31)) & 1u;
    return n;
}
uint32_t FindFirstSetBit(const uint32_t* bits, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i)
        if ((bits[i >> 5] >> (i & 31)) & 1u) return i;
    return limit;
}

// src/search/topology_search_kernel.cu:953-1137. The "core7" fast variant (:999-1038) evaluates
// the same FMA chain with the masked terms left out; a masked term contributes fmaf(0, 0, x) = x,
// so the generic chain below gives the same bits.
bool LearnedStopSaysStop(const OrcLearnedStop& ls, BeamState& s, uint32_t top_l) {
    if (!ls.enabled) return false;
    while (s.ls_stage < ls.num_stages) {
        const uint32_t p = ls.stage_prefixes[s.ls_stage];
        if (p == 0 || p >= top_l || p < ls.top_k) { ++s.ls_stage; continue; }
        if (s.valid < top_l || s.valid < p || s.valid < ls.top_k || s.expanded < p) break;
        const float dk = s.cand[ls.top_k - 1].dist;
        const float boundary = s.cand[p - 1].dist;
        const uint32_t next64_end = std::min(p + 64u, top_l);
        const uint32_t next256_end = std::min(p + 256u, top_l);
        const uint32_t next64_span = next64_end > p ? next64_end - p : 1u;
        const uint32_t next256_span = next256_end > p ? next256_end - p : 1u;
        const uint32_t gap32_index = std::min(std::max(ls.top_k - 1u, 31u), p - 1u);
        const bool has_prev = s.ls_has_prev != 0;
        float f[12];
        f[0] = ls.feature_mask[0] ? (float)p * ls.inv_top_l : 0.0f;
        f[1] = ls.feature_mask[1] ? (float)s.expanded * ls.inv_top_l : 0.0f;
        f[2] = ls.feature_mask[2] ? (float)s.visited * ls.inv_top_l : 0.0f;
        const bool need_best = ls.feature_mask[3] || (ls.feature_mask[4] && ls.next64_flag_mode);
        uint32_t best = top_l;
        if (need_best) {
            best = FindFirstSetBit(s.unexpanded.data(), top_l);
            f[3] = ls.feature_mask[3] ? (float)best * ls.inv_top_l : 0.0f;
        } else {
            f[3] = 0.0f;
        }
        if (ls.feature_mask[4]) {
            if (ls.next64_flag_mode) f[4] = best < next64_end ? 1.0f : 0.0f;
            else f[4] = (float)CountBitsInRange(s.unexpanded.data(), p, next64_end) / (float)next64_span;
        } else {
            f[4] = 0.0f;
        }
        f[5] = ls.feature_mask[5]
                   ? (float)CountBitsInRange(s.unexpanded.data(), p, next256_end) / (float)next256_span
                   : 0.0f;
        f[6] = ls.feature_mask[6] ? dk : 0.0f;
        f[7] = ls.feature_mask[7] ? (boundary - dk) : 0.0f;
        f[8] = ls.feature_mask[8] ? (s.cand[gap32_index].dist - dk) : 0.0f;
        f[9] = (ls.feature_mask[9] && has_prev) ? (s.ls_prev_dk - dk) : 0.0f;
        f[10] = (ls.feature_mask[10] && has_prev) ? (s.ls_prev_boundary - boundary) : 0.0f;
        if (!ls.feature_mask[11]) {
            f[11] = 0.0f;
        } else if (ls.topk_churn_flag_mode) {
            f[11] = s.ls_topk_changed ? 1.0f : 0.0f;
        } else if (!has_prev) {  // :895-915
            f[11] = 1.0f;
        } else {
            uint32_t changed = 0;
            for (uint32_t i = 0; i < ls.top_k; ++i) {
                const uint32_t cur = RawId(s.cand[i].id);
                bool found = false;
                for (uint32_t j = 0; j < ls.top_k; ++j)
                    if (s.ls_prev_ids[j] == cur) { found = true; break; }
                changed += found ? 0u : 1u;
            }
            f[11] = (float)changed / (float)ls.top_k;
        }
        float logit = ls.bias;  // :917-932
        for (int i = 0; i < 12; ++i) logit = fmaf(f[i], ls.weights[i], logit);
        s.ls_prev_dk = dk;
        s.ls_prev_boundary = boundary;
        s.ls_has_prev = 1;
        s.ls_topk_changed = 0;
        if (ls.feature_mask[11] && !ls.topk_churn_flag_mode)
            for (uint32_t i = 0; i < ls.top_k; ++i) s.ls_prev_ids[i] = RawId(s.cand[i].id);
        if (logit < ls.threshold_logit) {
            if (ls.shadow_mode) { s.ls_stage = ls.num_stages; break; }
            return true;
        }
        ++s.ls_stage;
    }
    return false;
}

// One "push": Bloom-filter the slot ids, score survivors, sort the frontier, merge, rebuild
// prefix state. src/search/topology_search_kernel.cu:2307-2412 (entries), :2543-2654 (expansion),
// :1338-1424 (merge), :822-845 (prefix state).
void PushBatch(const OrcBeamParams& P, const OrcLearnedStop& ls, BeamState& s,
               const uint32_t* ids, uint32_t nslots, const float* lut, const uint8_t* codes,
               bool is_entry_batch) {
    const uint32_t F = (uint32_t)s.frontier.size();
    const Cand inval{std::numeric_limits<float>::infinity(), kInvalid};
    std::fill(s.frontier.begin(), s.frontier.end(), inval);
    if (P.two_phase) {
        // The reference block has 128 threads (:59); thread t handles slots t, t+128, ... and does
        // test-then-add on each, so within a round of 128 slots every test precedes every add, and
        // a later round sees the adds of the earlier ones.
        constexpr uint32_t kRound = 128;
        std::vector<uint8_t> pass(kRound, 0);
        for (uint32_t base = 0; base < nslots; base += kRound) {
            const uint32_t n = std::min(kRound, nslots - base);
            for (uint32_t i = 0; i < n; ++i) {
                const uint32_t id = ids[base + i];
                pass[i] = !(id == kInvalid || id >= P.num_nodes || BloomTest(id, s.bloom.data()));
            }
            for (uint32_t i = 0; i < n; ++i) {
                if (!pass[i]) continue;
                s.frontier[base + i].id = ids[base + i];
                BloomAdd(ids[base + i], s.bloom.data());
                ++s.visited;
            }
        }
    } else {
        for (uint32_t i = 0; i < nslots; ++i) {
            const uint32_t id = ids[i];
            if (id == kInvalid || id >= P.num_nodes || BloomTest(id, s.bloom.data())) continue;
            s.frontier[i].id = id;
            BloomAdd(id, s.bloom.data());
            ++s.visited;
        }
    }
    for (uint32_t i = 0; i < nslots && i < F; ++i) {
        if (s.frontier[i].id == kInvalid) continue;
        s.frontier[i].dist = AdcTree(lut, codes + (uint64_t)s.frontier[i].id * P.num_chunks, P.num_chunks);
    }
    std::sort(s.frontier.begin(), s.frontier.end(), CandLess);
    uint32_t fv = 0;
    for (const Cand& c : s.frontier) fv += c.id != kInvalid;
    const uint32_t C = P.candidate_capacity;
    const uint32_t nv = std::min<uint64_t>(C, (uint64_t)s.valid + fv);
    uint32_t accepted = 0;
    while (accepted < fv && accepted < nv) {
        if (!CandLess(s.frontier[accepted], s.cand[nv - 1 - accepted])) break;
        ++accepted;
    }
    bool topk_changed = false;
    if (accepted != 0) {
        int64_t ci = (int64_t)(nv - accepted) - 1, fi = (int64_t)accepted - 1, oi = (int64_t)nv - 1;
        while (fi >= 0) {
            if (ci >= 0 && !CandLess(s.cand[ci], s.frontier[fi])) {
                s.cand[oi] = s.cand[ci];
                --ci;
            } else {
                s.cand[oi] = s.frontier[fi];
                if (oi >= 0 && (uint32_t)oi < ls.top_k) topk_changed = true;
                --fi;
            }
            --oi;
        }
    }
    if (topk_changed) s.ls_topk_changed = 1;
    s.valid = nv;
    if (s.first_full == 0xffffffffu && nv >= P.top_l) s.first_full = is_entry_batch ? 0u : s.iterations;
    ++s.hash_iter;
    const bool rebuild = s.hash_iter >= 3;
    std::fill(s.unexpanded.begin(), s.unexpanded.end(), 0u);
    if (rebuild) std::fill(s.bloom.begin(), s.bloom.end(), 0u);
    const uint32_t prefix = std::min(s.valid, P.top_l);
    for (uint32_t i = 0; i < prefix; ++i) {
        const Cand c = s.cand[i];
        if (c.id == kInvalid) continue;
        if (!IsExpanded(c.id)) s.unexpanded[i >> 5] |= 1u << (i & 31);
        if (rebuild) BloomAdd(RawId(c.id), s.bloom.data());
    }
    if (rebuild) s.hash_iter = 0;
}

void BeamSearchOne(const OrcBeamParams& P, const OrcLearnedStop& ls, const uint32_t* adjacency,
                   const uint8_t* codes, const float* lut, const uint32_t* entries,
                   uint32_t num_entries, Cand* out_cand, uint32_t* out_stats) {
    const uint32_t slots = P.search_width * P.degree;
    uint32_t F = 1;
    while (F < std::max(slots, 1u)) F <<= 1;  // :3212-3213
    BeamState s;
    const Cand inval{std::numeric_limits<float>::infinity(), kInvalid};
    s.cand.assign(P.candidate_capacity, inval);
    s.frontier.assign(F, inval);
    s.bloom.assign(kBloomWords, 0u);
    const uint32_t uw = (P.top_l + 31) / 32;
    s.unexpanded.assign(std::max(uw, 1u), 0u);
    for (auto& x : s.ls_prev_ids) x = kInvalid;

    std::vector<uint32_t> ids(std::max(slots, 1u));
    const uint32_t batches = slots == 0 ? 0 : (num_entries + slots - 1) / slots;  // :2307-2308
    for (uint32_t b = 0; b < batches; ++b) {
        for (uint32_t i = 0; i < slots; ++i) {
            const uint64_t e = (uint64_t)b * slots + i;
            ids[i] = e < num_entries ? entries[e] : kInvalid;
        }
        PushBatch(P, ls, s, ids.data(), slots, lut, codes, true);
    }
    while (s.expanded < P.max_expansions) {  // :2414
        if (s.valid == 0) break;
        if (LearnedStopSaysStop(ls, s, P.top_l)) break;
        // :2439-2464
        bool stop;
        const bool prefix_stop = P.stop_prefix != 0 && P.stop_prefix < P.top_l;
        if (prefix_stop) {
            if (P.stop_use_expanded) {
                stop = s.valid >= P.top_l && s.expanded >= P.stop_prefix;
            } else {
                const uint32_t words = s.valid >= P.stop_prefix ? (P.stop_prefix + 31) / 32 : uw;
                stop = true;
                for (uint32_t w = 0; w < words; ++w) stop &= s.unexpanded[w] == 0;
            }
        } else {
            stop = true;
            for (uint32_t w = 0; w < uw; ++w) stop &= s.unexpanded[w] == 0;
        }
        if (stop) break;
        ++s.iterations;
        // :2479-2513 selection: first W set bits in rank order; no max_expansions re-check inside.
        uint32_t selected[32];
        uint32_t nsel = 0;
        for (uint32_t w = 0; w < uw && nsel < P.search_width; ++w) {
            uint32_t word = s.unexpanded[w];
            while (word != 0 && nsel < P.search_width) {
                const uint32_t bit = (uint32_t)__builtin_ctz(word);
                const uint32_t idx = w * 32 + bit;
                word &= word - 1;
                s.unexpanded[w] &= ~(1u << bit);
                if (idx >= P.candidate_capacity || idx >= P.top_l || idx >= s.valid ||
                    s.cand[idx].id == kInvalid || IsExpanded(s.cand[idx].id))
                    continue;
                s.cand[idx].id |= kExpandedBit;
                selected[nsel++] = RawId(s.cand[idx].id);
                ++s.expanded;
            }
        }
        if (nsel == 0) break;
        for (uint32_t k = 0; k < nsel; ++k)
            for (uint32_t j = 0; j < P.degree; ++j)
                ids[k * P.degree + j] = adjacency[(uint64_t)selected[k] * P.degree + j];
        PushBatch(P, ls, s, ids.data(), nsel * P.degree, lut, codes, false);
    }
    for (uint32_t i = 0; i < P.candidate_capacity; ++i) out_cand[i] = s.cand[i];
    // src/search/topology_search_kernel.hpp:56-65
    out_stats[0] = s.visited;
    out_stats[1] = s.expanded;
    out_stats[2] = 0;
    out_stats[3] = s.iterations;
    out_stats[4] = s.valid;
    out_stats[5] = s.first_full;
    out_stats[6] = 0;
    out_stats[7] = 0;
}

}  // namespace

extern "C" {

// a3. Batched beam search. lut: Q x M x 256 (or, when lut_stride == 0, one table shared by all
// queries). entry_offsets: Q+1 (CSR). out_cand: Q x C x {f32 dist, u32 packed id};
// out_stats: Q x 8 u32.
void orc_beam_search(const OrcBeamParams* P, const OrcLearnedStop* ls, const uint32_t* adjacency,
                     const uint8_t* codes, const float* lut, uint64_t lut_stride, uint64_t Q,
                     const uint32_t* entry_offsets, const uint32_t* entry_ids, void* out_cand,
                     uint32_t* out_stats) {
    OrcLearnedStop off;
    std::memset(&off, 0, sizeof(off));
    const OrcLearnedStop& L = ls ? *ls : off;
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t q = 0; q < (int64_t)Q; ++q) {
        BeamSearchOne(*P, L, adjacency, codes, lut + (uint64_t)q * lut_stride,
                      entry_ids + entry_offsets[q], entry_offsets[q + 1] - entry_offsets[q],
                      static_cast<Cand*>(out_cand) + (uint64_t)q * P->candidate_capacity,
                      out_stats + (uint64_t)q * 8);
    }
}

// ---------------------------------------------------------------------------------------------
// a2. RVQ entry selection.
//   norms: legacy_rvq .../functions/distance_kernel.cu:25-111 (block of 128 threads: thread t sums
//          columns t, t+128, ...; warp tree; then one tree over the four warp sums),
//   scores: D = ((-2 * q.c) + |q|^2) + |c|^2, distance_kernel.cu:114-124,187-199,229-323. The dot
//          product is a cuBLAS SGEMM in the reference, whose summation order is not published;
//          this restatement accumulates k in ascending order with FMA ("parity unpinned" there),
//   argmin: first strict minimum, functions/selectMin1.cu:9-23; fine level starts from FLT_MAX
//          and skips empty buckets, :66-81,
//   residual: RVQ/RVQ.cu:180-188; cluster id = coarse * fine_count + fine, selectMin1.cu:80,
//   entries: src/search/rvq_device_entries.cu:15-52 over the CSR of posting lists capped at 256
//          ids per bucket (src/search/rvq_entry_provider.cpp:21,115-144).
static float RvqNorm(const float* x, uint32_t d) {
    float warp_sum[4];
    for (int w = 0; w < 4; ++w) {
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (uint32_t col = w * 32 + l; col < d; col += 128) acc = fmaf(x[col], x[col], acc);
            lane[l] = acc;
        }
        warp_sum[w] = WarpTree(lane);
    }
    float lane[32] = {0};
    for (int w = 0; w < 4; ++w) lane[w] = warp_sum[w];
    return WarpTree(lane);
}

static float RvqDot(const float* a, const float* b, uint32_t d) {
    float acc = 0.0f;
    for (uint32_t k = 0; k < d; ++k) acc = fmaf(a[k], b[k], acc);
    return acc;
}

void orc_rvq_clusters(const float* queries, uint64_t Q, uint32_t d, const float* coarse,
                      uint32_t num_coarse, const float* fine, uint32_t num_fine,
                      const int32_t* bucket_sizes, int32_t* out_cluster, float* out_coarse_score,
                      float* out_fine_score) {
    std::vector<float> cn(num_coarse), fn(num_fine);
    for (uint32_t c = 0; c < num_coarse; ++c) cn[c] = RvqNorm(coarse + (uint64_t)c * d, d);
    for (uint32_t c = 0; c < num_fine; ++c) fn[c] = RvqNorm(fine + (uint64_t)c * d, d);
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < (int64_t)Q; ++q) {
        const float* x = queries + (uint64_t)q * d;
        const float qn = RvqNorm(x, d);
        float best = 0.0f;
        int best_c = 0;
        for (uint32_t c = 0; c < num_coarse; ++c) {
            const float D = (-2.0f * RvqDot(x, coarse + (uint64_t)c * d, d) + qn) + cn[c];
            if (c == 0 || D < best) { best = D; best_c = (int)c; }
        }
        std::vector<float> r(d);
        for (uint32_t i = 0; i < d; ++i) r[i] = x[i] - coarse[(uint64_t)best_c * d + i];
        const float rn = RvqNorm(r.data(), d);
        float fbest = FLT_MAX;
        int best_f = 0;
        for (uint32_t c = 0; c < num_fine; ++c) {
            const float D = (-2.0f * RvqDot(r.data(), fine + (uint64_t)c * d, d) + rn) + fn[c];
            if (D < fbest && bucket_sizes[(uint64_t)best_c * num_fine + c] > 0) { fbest = D; best_f = (int)c; }
        }
        out_cluster[q] = best_c * (int)num_fine + best_f;
        if (out_coarse_score) out_coarse_score[q] = best;
        if (out_fine_score) out_fine_score[q] = fbest;
    }
}

void orc_rvq_gather(const int32_t* clusters, uint64_t Q, const uint32_t* cluster_offsets,
                    const uint32_t* cluster_ids, uint32_t entry_count, uint32_t fallback_entry,
                    uint32_t* out_entry_ids) {
    for (uint64_t q = 0; q < Q; ++q) {
        uint32_t* o = out_entry_ids + q * entry_count;
        for (uint32_t i = 0; i < entry_count; ++i) o[i] = kInvalid;
        const int32_t c = clusters[q];
        if (c < 0) { if (entry_count) o[0] = fallback_entry; continue; }
        const uint32_t b = cluster_offsets[c], e = cluster_offsets[c + 1];
        const uint32_t n = std::min(e - b, entry_count);
        if (n == 0) { if (entry_count) o[0] = fallback_entry; continue; }
        for (uint32_t i = 0; i < n; ++i) o[i] = cluster_ids[b + i];
    }
}

// ---------------------------------------------------------------------------------------------
// a5. pq2 cross terms, src/search/search_resources.cpp:52-91 (host code, no FMA): X[m][b][r] =
// 2 * sum_dim (T1[b][dim] + mu1[dim]) * (T2[r][dim] + mu2[dim]).
void orc_pq2_cross_terms(uint32_t d, uint32_t M, const uint32_t* chunk_offsets, const float* t1,
                         const float* mu1, const float* t2, const float* mu2, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < (int64_t)M; ++m) {
        for (uint32_t b = 0; b < kCentroids; ++b)
            for (uint32_t r = 0; r < kCentroids; ++r) {
                float dot = 0.0f;
                for (uint32_t dim = chunk_offsets[m]; dim < chunk_offsets[m + 1]; ++dim) {
                    const float bv = t1[(uint64_t)b * d + dim] + mu1[dim];
                    const float rv = t2[(uint64_t)r * d + dim] + mu2[dim];
                    const float prod = bv * rv;
                    dot = dot + prod;
                }
                out[((uint64_t)m * kCentroids + b) * kCentroids + r] = 2.0f * dot;
            }
    }
}

// a5. pq2 refine + re-sort, src/search/rerank_exact.cu:573-665 (plain: base_codes == nullptr,
// distance = tree of LUT2 lookups) and :773-879 (residual: candidate distance + tree of
// (LUT2 + cross term)); lanes take chunks lane, lane+32, ...; output is refine_top_l entries
// sorted by (distance, id), invalid = (+inf, 0xffffffff), expanded flag cleared.
void orc_pq2_refine(const void* cand_in, const uint32_t* stats, uint64_t Q, uint32_t capacity,
                    uint32_t refine_top_l, const uint8_t* base_codes, const uint8_t* pq2_codes,
                    uint32_t M, const float* lut2, const float* cross_terms, void* cand_out) {
    const Cand* in = static_cast<const Cand*>(cand_in);
    Cand* out = static_cast<Cand*>(cand_out);
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < (int64_t)Q; ++q) {
        const uint32_t valid = std::min(stats[q * 8 + 4], refine_top_l);
        const float* lut = lut2 + (uint64_t)q * M * kCentroids;
        std::vector<Cand> v(refine_top_l);
        for (uint32_t rank = 0; rank < refine_top_l; ++rank) {
            Cand o{std::numeric_limits<float>::infinity(), kInvalid};
            if (rank < valid) {
                const Cand c = in[(uint64_t)q * capacity + rank];
                const uint32_t id = RawId(c.id);
                o.id = id;
                if (id != kInvalid) {
                    float lane[32];
                    for (uint32_t l = 0; l < 32; ++l) {
                        float partial = 0.0f;
                        for (uint32_t m = l; m < M; m += 32) {
                            const uint32_t rc = pq2_codes[(uint64_t)id * M + m];
                            if (base_codes) {
                                const uint32_t bc = base_codes[(uint64_t)id * M + m];
                                partial += lut[m * kCentroids + rc] +
                                           cross_terms[((uint64_t)m * kCentroids + bc) * kCentroids + rc];
                            } else {
                                partial += lut[m * kCentroids + rc];
                            }
                        }
                        lane[l] = partial;
                    }
                    const float t = WarpTree(lane);
                    o.dist = base_codes ? c.dist + t : t;
                }
            }
            v[rank] = o;
        }
        std::sort(v.begin(), v.end(), [](const Cand& a, const Cand& b) {
            if (a.dist != b.dist) return a.dist < b.dist;
            return a.id < b.id;  // src/search/rerank_exact.cu:92-100 (unpacked ids)
        });
        for (uint32_t i = 0; i < refine_top_l; ++i) out[(uint64_t)q * refine_top_l + i] = v[i];
    }
}

// ---------------------------------------------------------------------------------------------
// a7. Exact distance, src/search/rerank_exact.cu:242-276: lane-strided FMA partials of
// (float(v) - float(q))^2, then the shuffle tree. kinds as in orc_lut_build.
static inline float LoadScalar(const void* p, int kind, uint64_t i) {
    if (kind == 2) return static_cast<const float*>(p)[i];
    if (kind == 1) return (float)static_cast<const uint8_t*>(p)[i];
    return (float)static_cast<const int8_t*>(p)[i];
}
float orc_exact_distance(const void* query, int query_kind, const void* vec, int vec_kind, uint32_t d) {
    float lane[32];
    for (uint32_t l = 0; l < 32; ++l) {
        float acc = 0.0f;
        for (uint32_t i = l; i < d; i += 32) {
            const float diff = LoadScalar(vec, vec_kind, i) - LoadScalar(query, query_kind, i);
            acc = fmaf(diff, diff, acc);
        }
        lane[l] = acc;
    }
    return WarpTree(lane);
}

// src/search/rerank_exact.cu:137-142
static inline float LowerBound(float approx_sq, float err) {
    const float a = sqrtf(fmaxf(approx_sq, 0.0f));
    const float lo = fmaxf(0.0f, a - err);
    return lo * lo;
}

// a6 + a7. Rerank of ranks [0, top_n) of a device candidate list (valid or not), in tiles of
// `tile` ranks, src/search/rerank_exact.cu:1851-2165: with the bound filter on, a valid candidate
// is skipped when the per-query threshold (k-th smallest exact distance over the ranks handled so
// far, :541-571) is finite and LowerBound(d' - |q|^2, eps[id]) exceeds it (:434-497); |q|^2 is
// summed in double and rounded once (:1892-1899). Then sort by (distance, id) (:153-204) with
// skipped / invalid ranks as (+inf, 0xffffffff). vectors are addressed through the page layout:
// byte offset = (id / vpp) * page_bytes + (id % vpp) * vector_bytes
// (src/io/vector_page_layout.cpp:50-57), without the file header.
// out_ids/out_dists: Q x top_n. counts[0] += exact distances, counts[1] += filtered.
void orc_rerank(const void* cand_in, uint64_t Q, uint32_t capacity, uint32_t top_n, uint32_t top_k,
                uint32_t tile, const void* queries, int query_kind, uint32_t d,
                const uint8_t* vector_pages, int vec_kind, uint64_t vectors_per_page,
                uint64_t page_bytes, uint64_t vector_bytes, int use_bound_filter,
                const float* error_bounds, float* out_dists, uint32_t* out_ids, uint64_t* counts,
                uint32_t early_stop_min_prefix, uint32_t early_stop_patience_tiles) {
    // early_stop_patience_tiles == 0: no early stop. Otherwise the rule of the reference's persistent
    // rerank, src/io/bam_vector_provider.cu:852-975 (tile loop, k-th distance before / after the tile)
    // and :1124-1135 (stable-tile count).
    const bool early = early_stop_patience_tiles != 0;
    const Cand* in = static_cast<const Cand*>(cand_in);
    const uint64_t qbytes = (uint64_t)d * (query_kind == 2 ? 4 : 1);
    uint64_t n_exact = 0, n_filtered = 0;
    if (tile == 0) tile = top_n;
#pragma omp parallel for schedule(static) reduction(+ : n_exact, n_filtered)
    for (int64_t q = 0; q < (int64_t)Q; ++q) {
        const uint8_t* qp = static_cast<const uint8_t*>(queries) + (uint64_t)q * qbytes;
        float qnorm = 0.0f;
        if (use_bound_filter) {
            double s = 0.0;
            for (uint32_t i = 0; i < d; ++i) {
                const double v = (double)LoadScalar(qp, query_kind, i);
                s += v * v;
            }
            qnorm = (float)s;
        }
        std::vector<float> fd(top_n, std::numeric_limits<float>::infinity());
        std::vector<uint32_t> fi(top_n, kInvalid);
        float threshold = std::numeric_limits<float>::infinity();
        float previous_kth = std::numeric_limits<float>::infinity();
        uint32_t stable_tiles = 0;
        for (uint32_t rb = 0; rb < top_n; rb += tile) {
            const uint32_t rc = std::min(tile, top_n - rb);
            for (uint32_t r = rb; r < rb + rc; ++r) {
                if (r >= capacity) continue;
                const Cand c = in[(uint64_t)q * capacity + r];
                if (c.id == kInvalid) continue;
                const uint32_t id = RawId(c.id);
                if (use_bound_filter && std::isfinite(threshold)) {
                    if (LowerBound(c.dist - qnorm, error_bounds[id]) > threshold) { ++n_filtered; continue; }
                }
                const uint8_t* vp = vector_pages + (id / vectors_per_page) * page_bytes +
                                    (id % vectors_per_page) * vector_bytes;
                fd[r] = orc_exact_distance(qp, query_kind, vp, vec_kind, d);
                fi[r] = id;
                ++n_exact;
            }
            if (use_bound_filter || early) {  // :541-571
                std::vector<float> best(top_k, std::numeric_limits<float>::infinity());
                const uint32_t prefix = std::min(top_n, rb + rc);
                for (uint32_t r = 0; r < prefix; ++r) {
                    const float x = fd[r];
                    if (!(x < best[top_k - 1])) continue;
                    uint32_t ins = top_k - 1;
                    while (ins > 0 && x < best[ins - 1]) { best[ins] = best[ins - 1]; --ins; }
                    best[ins] = x;
                }
                const float kth = best[top_k - 1];
                if (use_bound_filter) threshold = kth;
                if (early) {
                    bool stop = false;
                    if (rb + rc >= early_stop_min_prefix && std::isfinite(kth)) {
                        if (kth < previous_kth) stable_tiles = 0; else ++stable_tiles;
                        stop = stable_tiles >= early_stop_patience_tiles;
                    }
                    previous_kth = kth;
                    if (stop) break;
                }
            }
        }
        std::vector<uint32_t> order(top_n);
        for (uint32_t i = 0; i < top_n; ++i) order[i] = i;
        std::sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
            if (fd[a] != fd[b]) return fd[a] < fd[b];
            return fi[a] < fi[b];
        });
        for (uint32_t i = 0; i < top_n; ++i) {
            out_dists[(uint64_t)q * top_n + i] = fd[order[i]];
            out_ids[(uint64_t)q * top_n + i] = fi[order[i]];
        }
    }
    if (counts) { counts[0] += n_exact; counts[1] += n_filtered; }
}

// Hybrid-PQ refine + re-sort, src/search/rerank_exact.cu:667-771: one code per chunk, one selector bit per
// chunk (bit m & 7 of byte m >> 3 of the node's row) choosing the base or the outlier query table;
// lanes take chunks lane, lane + 32, ...; tree sum; sort by (distance, id).
void orc_hpq_refine(const void* cand_in, const uint32_t* stats, uint64_t Q, uint32_t capacity,
                    uint32_t refine_top_l, const uint8_t* hybrid_codes, const uint8_t* selector_bits, uint32_t M,
                    const float* base_lut, const float* outlier_lut, void* cand_out) {
    const Cand* in = static_cast<const Cand*>(cand_in);
    Cand* out = static_cast<Cand*>(cand_out);
    const uint32_t stride = (M + 7) / 8;
    for (uint64_t q = 0; q < Q; ++q) {
        const uint32_t valid = std::min(stats[q * 8 + 4], refine_top_l);
        const float* tables[2] = {base_lut + q * M * kCentroids, outlier_lut + q * M * kCentroids};
        std::vector<Cand> v(refine_top_l);
        for (uint32_t rank = 0; rank < refine_top_l; ++rank) {
            Cand o{std::numeric_limits<float>::infinity(), kInvalid};
            if (rank < valid) {
                const uint32_t id = RawId(in[q * capacity + rank].id);
                o.id = id;
                if (id != kInvalid) {
                    float lane[32];
                    for (uint32_t l = 0; l < 32; ++l) {
                        float partial = 0.0f;
                        for (uint32_t m = l; m < M; m += 32) {
                            const uint32_t bit = (selector_bits[(uint64_t)id * stride + (m >> 3)] >> (m & 7)) & 1u;
                            partial += tables[bit][m * kCentroids + hybrid_codes[(uint64_t)id * M + m]];
                        }
                        lane[l] = partial;
                    }
                    o.dist = WarpTree(lane);
                }
            }
            v[rank] = o;
        }
        std::sort(v.begin(), v.end(), [](const Cand& a, const Cand& b) {
            if (a.dist != b.dist) return a.dist < b.dist;
            return a.id < b.id;
        });
        for (uint32_t i = 0; i < refine_top_l; ++i) out[q * refine_top_l + i] = v[i];
    }
}

// Folded learned rerank-stop model, field for field the reference's DeviceRerankLearnedStopConfig
// (src/io/bam_vector_provider.cu:65-79).
struct OrcRerankStop {
    uint32_t enabled, feature_variant, num_stages, top_k, bootstrap_prefix, initial_stage_index;
    uint32_t stage_prefixes[64];
    float linear_weights[13];
    float bias, threshold_logit, budget_log2, inv_budget_top_n, inv_top_k;
};

// src/io/bam_vector_provider.cu:542-596
static float OrcStopLogit13(const OrcRerankStop& c, uint32_t processed_prefix, float current_kth, float delta_kth_last,
                            float delta_kth_prev, float topk_changed_flag, uint32_t entered_topk_count, float topk_spread,
                            uint32_t next_window_live_count, uint32_t next_window_count, float best_live_lb,
                            uint32_t window_exact_count, uint32_t window_candidate_count, uint32_t cumulative_exact_count) {
    const float f1 = (float)processed_prefix * c.inv_budget_top_n;
    const float f6 = (float)entered_topk_count * c.inv_top_k;
    const float f8 = next_window_count == 0 ? 0.0f : (float)next_window_live_count / (float)next_window_count;
    const float f9 = std::isfinite(best_live_lb) ? (best_live_lb - current_kth) : 0.0f;
    const float inv_window = window_candidate_count == 0 ? 0.0f : 1.0f / (float)window_candidate_count;
    const float f10 = (float)window_exact_count * inv_window;
    const float f11 = (float)(window_candidate_count - window_exact_count) * inv_window;
    const float f12 = processed_prefix == 0 ? 0.0f : (float)cumulative_exact_count / (float)processed_prefix;
    const float f[13] = {c.budget_log2, f1, current_kth, delta_kth_last, delta_kth_prev, topk_changed_flag, f6,
                         topk_spread, f8, f9, f10, f11, f12};
    float logit = c.bias;
    for (int i = 0; i < 13; ++i) logit = fmaf(f[i], c.linear_weights[i], logit);
    return logit;
}

// src/io/bam_vector_provider.cu:598-617: features 0, 1, 2, 5, 7, 9 only
static float OrcStopLogit6(const OrcRerankStop& c, uint32_t processed_prefix, float current_kth,
                           float topk_changed_flag, float topk_spread, float best_live_lb) {
    const float f1 = (float)processed_prefix * c.inv_budget_top_n;
    const float f9 = std::isfinite(best_live_lb) ? (best_live_lb - current_kth) : 0.0f;
    float logit = c.bias;
    logit = fmaf(c.budget_log2, c.linear_weights[0], logit);
    logit = fmaf(f1, c.linear_weights[1], logit);
    logit = fmaf(current_kth, c.linear_weights[2], logit);
    logit = fmaf(topk_changed_flag, c.linear_weights[5], logit);
    logit = fmaf(topk_spread, c.linear_weights[7], logit);
    return fmaf(f9, c.linear_weights[9], logit);
}

static bool PairLess(float ad, uint32_t ai, float bd, uint32_t bi) {   // :525-533
    if (ad != bd) return ad < bd;
    return ai < bi;
}

// Persistent rerank with the learned stop, the stage schedule and stop-prefix replay:
// src/io/bam_vector_provider.cu:721-1323, one query at a time, in the kernel's own order (window
// scored, window sorted, ascending insertion into the top_k list with one "entered" count, then
// the checkpoint / replay / early-stop rule of thread 0). model may be null (plain tiles).
// replay may be null. use_bound_filter needs error_bounds; the lower bounds of :655-681 are
// computed where they are read. Outputs: out_dists / out_ids [Q][top_k]; stop_prefixes,
// checkpoint_counts, stop_flags [Q]; counts[0] += exact, counts[1] += filtered.
void orc_rerank_learned(const void* cand_in, uint64_t Q, uint32_t capacity, uint32_t top_n, uint32_t top_k,
                        uint32_t tile, const void* queries, int query_kind, uint32_t d,
                        const uint8_t* vector_pages, int vec_kind, uint64_t vectors_per_page,
                        uint64_t page_bytes, uint64_t vector_bytes, int use_bound_filter,
                        const float* error_bounds, const OrcRerankStop* model, const uint32_t* replay,
                        int use_early_stop, uint32_t early_stop_min_prefix, uint32_t early_stop_patience_tiles,
                        float* out_dists, uint32_t* out_ids, uint64_t* counts, uint32_t* stop_prefixes,
                        uint32_t* checkpoint_counts, uint32_t* stop_flags) {
    const Cand* in = static_cast<const Cand*>(cand_in);
    const float inf = std::numeric_limits<float>::infinity();
    const uint64_t qbytes = (uint64_t)d * (query_kind == 2 ? 4 : 1);
    const uint32_t budget = std::min(top_n, capacity);
    if (tile == 0) tile = budget;
    OrcRerankStop ls;
    std::memset(&ls, 0, sizeof(ls));
    if (model) ls = *model;
    const bool use_schedule = ls.enabled != 0;                 // :2561-2567
    const bool evaluate = use_schedule && replay == nullptr;   // :2568-2569
    uint64_t n_exact = 0, n_filtered = 0;
    for (uint64_t q = 0; q < Q; ++q) {
        const uint8_t* qp = static_cast<const uint8_t*>(queries) + q * qbytes;
        float qnorm = 0.0f;
        if (use_bound_filter) {
            double s = 0.0;
            for (uint32_t i = 0; i < d; ++i) {
                const double v = (double)LoadScalar(qp, query_kind, i);
                s += v * v;
            }
            qnorm = (float)s;
        }
        const auto lower_bound_of_rank = [&](uint32_t r) {
            const Cand c = in[q * capacity + r];
            if (c.id == kInvalid) return inf;
            return LowerBound(c.dist - qnorm, error_bounds[RawId(c.id)]);
        };
        std::vector<float> top_d(top_k, inf);
        std::vector<uint32_t> top_i(top_k, kInvalid);
        float current_kth = inf, previous_checkpoint_kth = inf, previous_delta = 0.0f;
        uint32_t exact_count = 0, stable_tiles = 0, stage = ls.initial_stage_index, checkpoints = 0;
        uint32_t next_prefix = use_schedule ? std::min(budget, ls.bootstrap_prefix) : std::min(budget, tile);
        uint32_t stop_prefix = budget;
        bool has_previous = false, stop = false;
        for (uint32_t rank_begin = 0; rank_begin < budget && !stop;) {
            const uint32_t rank_end = use_schedule ? next_prefix : std::min(budget, rank_begin + tile);
            const uint32_t rank_count = rank_end - rank_begin;
            std::vector<std::pair<float, uint32_t>> window;
            for (uint32_t r = rank_begin; r < rank_end; ++r) {
                const Cand c = in[q * capacity + r];
                if (c.id == kInvalid) continue;
                const uint32_t id = RawId(c.id);
                if (use_bound_filter && std::isfinite(current_kth) && lower_bound_of_rank(r) > current_kth) {
                    ++n_filtered;
                    continue;
                }
                const uint8_t* vp = vector_pages + (id / vectors_per_page) * page_bytes + (id % vectors_per_page) * vector_bytes;
                window.emplace_back(orc_exact_distance(qp, query_kind, vp, vec_kind, d), id);
                ++exact_count;
                ++n_exact;
            }
            std::stable_sort(window.begin(), window.end(), [](const auto& a, const auto& b) {
                return PairLess(a.first, a.second, b.first, b.second);
            });
            const float previous_window_kth = top_d[top_k - 1];
            uint32_t entered = 0;
            for (const auto& e : window) {   // :619-642
                if (!PairLess(e.first, e.second, top_d[top_k - 1], top_i[top_k - 1])) continue;
                uint32_t ins = top_k - 1;
                while (ins > 0 && PairLess(e.first, e.second, top_d[ins - 1], top_i[ins - 1])) {
                    top_d[ins] = top_d[ins - 1];
                    top_i[ins] = top_i[ins - 1];
                    --ins;
                }
                top_d[ins] = e.first;
                top_i[ins] = e.second;
                ++entered;
            }
            const uint32_t processed = rank_end;
            current_kth = top_d[top_k - 1];
            if (evaluate && ls.enabled && std::isfinite(current_kth) && stage < ls.num_stages &&
                processed >= ls.stage_prefixes[stage]) {
                const float delta_last = has_previous ? (previous_checkpoint_kth - current_kth) : 0.0f;
                const float spread = current_kth - top_d[0];
                const float changed = entered == 0 ? 0.0f : 1.0f;
                uint32_t next_end = (stage + 1 < ls.num_stages) ? std::min(budget, ls.stage_prefixes[stage + 1])
                                                                : std::min(budget, rank_end + tile);
                if (next_end < rank_end) next_end = rank_end;
                next_end = std::min(next_end, rank_end + 8u);   // head probe, :56,1008-1009
                uint32_t live = 0;
                float best_lb = inf;
                if (ls.linear_weights[8] != 0.0f || ls.linear_weights[9] != 0.0f) {
                    for (uint32_t r = rank_end; r < next_end; ++r) {
                        const float lb = lower_bound_of_rank(r);
                        if (lb <= current_kth) {
                            ++live;
                            best_lb = fminf(best_lb, lb);
                        }
                    }
                }
                const float logit =
                    ls.feature_variant == 1
                        ? OrcStopLogit6(ls, processed, current_kth, changed, spread, best_lb)
                        : OrcStopLogit13(ls, processed, current_kth, delta_last, previous_delta, changed, entered, spread,
                                         live, next_end - rank_end, best_lb, (uint32_t)window.size(), rank_count,
                                         exact_count);
                ++checkpoints;
                if (logit < ls.threshold_logit) {
                    stop = true;
                    stop_prefix = processed;
                }
                previous_checkpoint_kth = current_kth;
                previous_delta = delta_last;
                has_previous = true;
                ++stage;
            } else if (replay != nullptr) {
                while (stage < ls.num_stages && ls.stage_prefixes[stage] <= processed) ++stage;
                if (processed >= replay[q]) {
                    stop = true;
                    stop_prefix = processed;
                }
            } else if (use_early_stop && processed >= early_stop_min_prefix && std::isfinite(current_kth)) {
                if (current_kth < previous_window_kth) stable_tiles = 0; else ++stable_tiles;
                if (stable_tiles >= early_stop_patience_tiles) {
                    stop = true;
                    stop_prefix = processed;
                }
            }
            if (use_schedule && !stop)
                next_prefix = stage < ls.num_stages ? std::min(budget, ls.stage_prefixes[stage])
                                                    : std::min(budget, processed + tile);
            rank_begin = rank_end;
        }
        for (uint32_t i = 0; i < top_k; ++i) {
            out_dists[q * top_k + i] = top_d[i];
            out_ids[q * top_k + i] = top_i[i];
        }
        if (stop_prefixes) stop_prefixes[q] = stop_prefix;
        if (checkpoint_counts) checkpoint_counts[q] = checkpoints;
        if (stop_flags) stop_flags[q] = stop ? 1u : 0u;
    }
    if (counts) { counts[0] += n_exact; counts[1] += n_filtered; }
}

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}

}  // extern "C"
