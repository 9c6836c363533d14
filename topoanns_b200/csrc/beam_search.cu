// Fused Bloom-filtered beam search, one query per 128-thread block (the grid is the batch; the loop over
// queries only matters when a caller launches fewer blocks than queries).
//
// What it computes is the traversal of the reference kernel
// (src/search/topology_search_kernel.cu:2190-2664): same Bloom filter (hashes :382-385,611-653,
// cleared and rebuilt from the top-L prefix on every third merge :2394-2411,2636-2654), same
// candidate order (distance, raw id) (:414-420), same merge tie rule (:1338-1424), same selection
// of the first W unexpanded ranks without a max_expansions re-check (:2479-2513), same ADC
// summation tree (:656-692), same learned stop (:953-1137). Visited tests and adds of one batch
// of slots run as two phases per round of 128 slots (all tests, barrier, all adds). That is what the
// reference's 128-thread block does in practice (each thread tests then adds its slot, round by
// round, :2543-2564) and it is the explicit protocol of its micro-batch kernels (:2078-2106); run
// on a B200 the compiled reference kernel agrees with this order on every query tested.
//
// How it differs in construction: the query's look-up table lives in shared memory (built in
// place from the query and the PQ pivots, or staged from HBM), the Bloom filter lives in shared
// memory, every thread owns one frontier slot (its own 4-byte adjacency load, its own 16-byte
// code loads, a register-resident tree sum), candidates and frontier entries are 64-bit keys,
// frontier entries that cannot enter a full list are dropped before sorting, the rest are
// rank-sorted, and the merge is a parallel merge-path into a second buffer instead of a
// single-thread backward merge.

#include "beam_args.h"
#include "tann_launch.h"

// Optional per-phase cycle counters (development builds only: -DTANN_BEAM_PROFILE). Thread 0 adds
// clock64() deltas per phase into a [Q][12] uint64 array passed through BeamArgs::status.
#ifdef TANN_BEAM_PROFILE
#define TANN_PHASE(i)                                            \
    do {                                                         \
        if (tid == 0) {                                          \
            const long long now__ = clock64();                   \
            prof_acc[i] += (unsigned long long)(now__ - prof_t); \
            prof_t = now__;                                      \
        }                                                        \
    } while (0)
#else
#define TANN_PHASE(i) do {} while (0)
#endif

namespace tann {

constexpr int kBeamThreads = 128;

// State written by thread 0 (or benignly by any thread) and read by the block after a barrier.
// Counters every thread can derive identically (valid, visited, merges since the last Bloom
// rebuild) are kept in registers instead.
struct BeamCtl {
    uint32_t first_full;
    uint32_t nsel, stop, stop_scan;
    // learned stop state (:2252-2258)
    uint32_t ls_stage, ls_has_prev, ls_topk_changed;
    float ls_prev_dk, ls_prev_boundary;
    uint32_t ls_prev_ids[32];
};

// Candidates and frontier entries are 64-bit keys in shared memory: high word = order-preserving
// bits of the distance, low word = packed node id (bit 31 = expanded). Comparing two keys with
// bit 31 masked off is the reference's CandidateLess (distance, then raw id).
constexpr unsigned long long kInvalidKey = 0xff800000ffffffffull;  // (+inf, 0xffffffff)
constexpr unsigned long long kCmpMask = 0xffffffff7fffffffull;
__device__ __forceinline__ float KeyDist(unsigned long long k) { return FromOrderedBits((uint32_t)(k >> 32)); }
__device__ __forceinline__ uint32_t KeyPackedId(unsigned long long k) { return (uint32_t)k; }
__device__ __forceinline__ uint32_t KeyRawId(unsigned long long k) { return RawId((uint32_t)k); }

__device__ __forceinline__ uint32_t CountBitsInRange(const uint32_t* bits, uint32_t b, uint32_t e) {
    uint32_t n = 0;
    for (uint32_t i = b; i < e; ++i) n += (bits[i >> 5] >> (i & 31)) & 1u;
    return n;
}
__device__ __forceinline__ uint32_t FindFirstSetBit(const uint32_t* bits, uint32_t limit) {
    const uint32_t words = (limit + 31) / 32;
    for (uint32_t w = 0; w < words; ++w) {
        uint32_t word = bits[w];
        if (w + 1 == words && (limit & 31)) word &= (1u << (limit & 31)) - 1u;
        if (word) return w * 32 + __ffs(word) - 1;
    }
    return limit;
}

// Position of set bit number n (0-based) in a bitmap of up to four words; n must be below its popcount.
__device__ __forceinline__ uint32_t NthSetBit(const uint32_t (&wd)[4], uint32_t n) {
    uint32_t word = wd[0], base = 0;
    const uint32_t c0 = __popc(wd[0]), c1 = __popc(wd[1]), c2 = __popc(wd[2]);
    if (n >= c0) {
        n -= c0; word = wd[1]; base = 32;
        if (n >= c1) {
            n -= c1; word = wd[2]; base = 64;
            if (n >= c2) { n -= c2; word = wd[3]; base = 96; }
        }
    }
    for (uint32_t i = 0; i < n; ++i) word &= word - 1u;
    return base + __ffs(word) - 1;
}

// Sets the expanded flag of the list elements this lane picked (the picks sel_begin..sel_end-1 are
// the lowest set bits of its bitmap word). Runs on warp 0 once every warp has read the ids.
__device__ __forceinline__ void MarkExpanded(unsigned long long* cur, uint32_t word, uint32_t sel_begin,
                                             uint32_t sel_end, uint32_t lane, uint32_t mark_pos) {
    if (mark_pos != kInvalid) cur[mark_pos] |= kExpandedBit;
    for (uint32_t sidx = sel_begin; sidx < sel_end; ++sidx) {
        const uint32_t bit = __ffs(word) - 1;
        word &= word - 1u;
        cur[lane * 32 + bit] |= kExpandedBit;
    }
}

// Learned stop on one thread; returns true when the traversal has to stop.
__device__ bool LearnedStop(const TannLearnedStop& ls, BeamCtl& s, uint32_t valid, uint32_t visited,
                            uint32_t expanded, const unsigned long long* cand, const uint32_t* unexp,
                            uint32_t top_l) {
    while (s.ls_stage < ls.num_stages) {
        const uint32_t p = ls.stage_prefixes[s.ls_stage];
        if (p == 0 || p >= top_l || p < ls.top_k) { ++s.ls_stage; continue; }
        if (valid < top_l || valid < p || valid < ls.top_k || expanded < p) break;
        const float dk = KeyDist(cand[ls.top_k - 1]);
        const float boundary = KeyDist(cand[p - 1]);
        const uint32_t next64_end = min(p + 64u, top_l);
        const uint32_t next256_end = min(p + 256u, top_l);
        const uint32_t next64_span = next64_end > p ? next64_end - p : 1u;
        const uint32_t next256_span = next256_end > p ? next256_end - p : 1u;
        const uint32_t gap32_index = min(max(ls.top_k - 1u, 31u), p - 1u);
        const bool has_prev = s.ls_has_prev != 0;
        float f[TANN_STOP_FEATURES];
        f[0] = ls.feature_mask[0] ? (float)p * ls.inv_top_l : 0.0f;
        f[1] = ls.feature_mask[1] ? (float)expanded * ls.inv_top_l : 0.0f;
        f[2] = ls.feature_mask[2] ? (float)visited * ls.inv_top_l : 0.0f;
        const bool need_best = ls.feature_mask[3] || (ls.feature_mask[4] && ls.next64_flag_mode);
        uint32_t best = top_l;
        if (need_best) {
            best = FindFirstSetBit(unexp, top_l);
            f[3] = ls.feature_mask[3] ? (float)best * ls.inv_top_l : 0.0f;
        } else {
            f[3] = 0.0f;
        }
        if (ls.feature_mask[4]) {
            if (ls.next64_flag_mode) f[4] = best < next64_end ? 1.0f : 0.0f;
            else f[4] = (float)CountBitsInRange(unexp, p, next64_end) / (float)next64_span;
        } else {
            f[4] = 0.0f;
        }
        f[5] = ls.feature_mask[5] ? (float)CountBitsInRange(unexp, p, next256_end) / (float)next256_span
                                  : 0.0f;
        f[6] = ls.feature_mask[6] ? dk : 0.0f;
        f[7] = ls.feature_mask[7] ? (boundary - dk) : 0.0f;
        f[8] = ls.feature_mask[8] ? (KeyDist(cand[gap32_index]) - dk) : 0.0f;
        f[9] = (ls.feature_mask[9] && has_prev) ? (s.ls_prev_dk - dk) : 0.0f;
        f[10] = (ls.feature_mask[10] && has_prev) ? (s.ls_prev_boundary - boundary) : 0.0f;
        if (!ls.feature_mask[11]) {
            f[11] = 0.0f;
        } else if (ls.topk_churn_flag_mode) {
            f[11] = s.ls_topk_changed ? 1.0f : 0.0f;
        } else if (!has_prev) {
            f[11] = 1.0f;
        } else {
            uint32_t changed = 0;
            for (uint32_t i = 0; i < ls.top_k; ++i) {
                const uint32_t cur = KeyRawId(cand[i]);
                bool found = false;
                for (uint32_t j = 0; j < ls.top_k; ++j)
                    if (s.ls_prev_ids[j] == cur) { found = true; break; }
                changed += found ? 0u : 1u;
            }
            f[11] = (float)changed / (float)ls.top_k;
        }
        float logit = ls.bias;
#pragma unroll
        for (int i = 0; i < TANN_STOP_FEATURES; ++i) logit = fmaf(f[i], ls.weights[i], logit);
        s.ls_prev_dk = dk;
        s.ls_prev_boundary = boundary;
        s.ls_has_prev = 1;
        s.ls_topk_changed = 0;
        if (ls.feature_mask[11] && !ls.topk_churn_flag_mode)
            for (uint32_t i = 0; i < ls.top_k; ++i) s.ls_prev_ids[i] = KeyRawId(cand[i]);
        if (logit < ls.threshold_logit) {
            if (ls.shadow_mode) { s.ls_stage = ls.num_stages; break; }
            return true;
        }
        ++s.ls_stage;
    }
    return false;
}

// The code row of a node as 32-bit words (specialised chunk counts only): loading is split from
// summing so that the loads can be issued before a barrier and consumed after it.
template <int kM>
__device__ __forceinline__ void LoadCodeWords(const uint8_t* row, uint32_t (&w)[kM > 0 ? kM / 4 : 1]) {
    const uint4* r4 = reinterpret_cast<const uint4*>(row);
#pragma unroll
    for (int i = 0; i < kM / 16; ++i) {
        const uint4 v = __ldg(r4 + i);
        w[4 * i + 0] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
    }
}

// ADC distance of one node by one thread, in the reference's order: per group of 32 chunks the
// 16/8/4/2/1 tree over "lanes", groups added in order. Terms beyond M are exact zeros in the
// reference and are simply left out here.
template <int kM>
__device__ __forceinline__ float AdcFromWords(const float* lut, const uint32_t (&w)[kM > 0 ? kM / 4 : 1]) {
    static_assert(kM > 0 && kM % 16 == 0, "specialised chunk counts are multiples of 16");
    float total = 0.0f;
#pragma unroll
    for (int base = 0; base < kM; base += 32) {
        const int n = (kM - base) < 32 ? (kM - base) : 32;
        float x[32];
#pragma unroll
        for (int l = 0; l < 32; ++l) {
            if (l < n) {
                const int c = base + l;
                const uint32_t code = (w[c >> 2] >> ((c & 3) * 8)) & 0xffu;
                x[l] = lut[c * kCentroids + code];
            }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
            for (int i = 0; i < off; ++i)
                if (i + off < n) x[i] = x[i] + x[i + off];
        }
        total = (base == 0) ? x[0] : total + x[0];
    }
    return total;
}

template <int kM>
__device__ __forceinline__ float AdcTreeThread(const float* lut, const uint8_t* row, uint32_t M) {
    float total = 0.0f;
    if constexpr (kM > 0) {
        uint32_t w[kM / 4];
        LoadCodeWords<kM>(row, w);
        total = AdcFromWords<kM>(lut, w);
    } else {
        for (uint32_t base = 0; base < M; base += 32) {
            const uint32_t n = min(32u, M - base);
            float x[32];
#pragma unroll
            for (uint32_t l = 0; l < 32; ++l) {
                x[l] = 0.0f;
                if (l < n) x[l] = lut[(base + l) * kCentroids + __ldg(row + base + l)];
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
                for (int i = 0; i < off; ++i) x[i] = x[i] + x[i + off];
            }
            total = total + x[0];
        }
    }
    return total;
}

// Bitonic sort of F keys held in shared memory (any power of two F).
__device__ void SortKeysShared(unsigned long long* keys, uint32_t F) {
    for (uint32_t k = 2; k <= F; k <<= 1) {
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
            for (uint32_t t = threadIdx.x; t < F / 2; t += kBeamThreads) {
                const uint32_t lo = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                const uint32_t hi = lo | j;
                const bool asc = (lo & k) == 0;
                const unsigned long long a = keys[lo], b = keys[hi];
                if ((a > b) == asc) { keys[lo] = b; keys[hi] = a; }
            }
            __syncthreads();
        }
    }
}

// Row n of an array: the plain form knows there is one shard.
template <bool kOneShard>
__device__ __forceinline__ const uint8_t* Row(const TannShards& s, uint64_t n, uint64_t row_bytes) {
    if constexpr (kOneShard) return static_cast<const uint8_t*>(s.base[0]) + n * row_bytes;
    else return ShardRow(s, n, row_bytes);
}

// kSingle: W * degree <= 128, so every thread owns at most one frontier slot per batch: its key
// stays in a register until the survivors are compacted and rank-sorted.
// kSub > 0 selects the plain form: no caller-provided table, no learned stop, the default stop prefix, at most 128 list
// ranks that matter (top_l <= 128), no adjacency cache and (unless kSharded) every array in one shard - the launcher checks these - with
// chunks kSub dims wide (checked here; other widths take the generic table builder). Compiling those paths out shrinks
// the loop that five blocks in different phases run at once.
// The plain form is also compiled per layout (kNbr: 1 = neighbour-code layout present, 0 = absent, -1 = look at the
// index view) and for lists whose traversal prefix fits one bitmap word (kOneWord: top_l <= 32).
template <int kM, bool kSingle, int kSub, int kNbr = -1, bool kOneWord = false, bool kSharded = false>
__global__ void __launch_bounds__(kBeamThreads)
beam_search_kernel(const __grid_constant__ BeamArgs a) {
    constexpr bool kPlain = kSub > 0;
    constexpr bool kOneShard = kPlain && !kSharded;   // rows of node-id-range shards are resolved per gather
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const uint32_t M = kM > 0 ? (uint32_t)kM : a.ix.num_chunks;
    const uint32_t C = a.p.candidate_capacity;
    const uint32_t F = a.frontier_capacity;
    const uint32_t L = a.p.top_l;
    const uint32_t W = a.p.search_width;
    const uint32_t deg = a.ix.degree;
    const uint32_t slots = W * deg;
    const uint32_t UW = (L + 31) / 32;
    const uint32_t d = a.ix.dim;
    const uint64_t N = a.ix.num_nodes;
    const uint32_t FK = kSingle ? (uint32_t)kBeamThreads : F;  // keys held in shared memory

    float* lut = reinterpret_cast<float*>(smem_raw);
    unsigned long long* cand_a = reinterpret_cast<unsigned long long*>(lut + (size_t)M * kCentroids);
    unsigned long long* cand_b = cand_a + C;
    unsigned long long* fkey = cand_b + C;        // frontier keys (compacted survivors when kSingle)
    unsigned long long* skey = fkey + FK;         // sorted frontier (kSingle only)
    uint32_t* bloom = reinterpret_cast<uint32_t*>(skey + (kSingle ? FK : 0));
    uint32_t* unexp = bloom + kBloomWords;
    uint32_t* offs = unexp + UW;
    float* sq = reinterpret_cast<float*>(offs + M + 1);

    __shared__ BeamCtl ctl;
    __shared__ uint32_t s_surv, s_pass;
    __shared__ uint32_t s_half_rank[64];   // partial ranks of the split rank count (33..64 survivors)
    __shared__ uint32_t s_sel[kBeamThreads / 32][TANN_MAX_SEARCH_WIDTH];  // selected nodes, one copy per warp
    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31;
    const uint32_t my_k = deg ? tid / deg : 0u, my_j = tid - my_k * deg;  // slot of this thread (kSingle)

    __shared__ __align__(8) unsigned long long lut_barrier;   // completion of the bulk copy of a caller's table
    uint32_t lut_phase = 0;
    if (!kPlain && a.lut != nullptr) {
        if (tid == 0) BarrierInit(&lut_barrier, 1);
        __syncthreads();
    }
    // Chunks of equal width (the usual case) take the unrolled table build.
    uint32_t uniform_sub = 0;
    if (kPlain || a.lut == nullptr) {
        const uint32_t sub0 = __ldg(a.ix.pq_chunk_offsets + 1) - __ldg(a.ix.pq_chunk_offsets);
        bool same = __ldg(a.ix.pq_chunk_offsets) == 0u;
        for (uint32_t i = tid; i < M; i += kBeamThreads)
            same = same && (__ldg(a.ix.pq_chunk_offsets + i + 1) - __ldg(a.ix.pq_chunk_offsets + i)) == sub0;
        uniform_sub = __syncthreads_and(same) ? sub0 : 0u;
    }

    for (uint64_t q = blockIdx.x; q < a.num_queries; q += gridDim.x) {
#ifdef TANN_BEAM_PROFILE
        unsigned long long prof_acc[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
        long long prof_t = clock64();
#endif
        // ---- per-query set-up --------------------------------------------------------------
        bool lut_copy_pending = false;
        if (!kPlain && a.lut != nullptr) {
            // A table given by the caller is staged with one bulk asynchronous copy while the block clears
            // its lists.
            const float* src_lut = a.lut + q * (uint64_t)M * kCentroids;
            // (the host side rejects tables that are not 16-byte aligned; rows are 1 KB)
            if (tid == 0) BulkLoadToShared(lut, src_lut, M * kCentroids * 4, &lut_barrier);
            lut_copy_pending = true;
        } else {
            // src/search/pq_query_tables.cu:33-52
            for (uint32_t i = tid; i < d; i += kBeamThreads)
                sq[i] = LoadAsFloat<float>(a.queries, a.query_kind, q * d + i) - __ldg(a.ix.pq_centroid + i);
            for (uint32_t i = tid; i <= M; i += kBeamThreads) offs[i] = __ldg(a.ix.pq_chunk_offsets + i);
            __syncthreads();
            if constexpr (kPlain) {
                if (uniform_sub == (uint32_t)kSub) BuildLutUniform<kSub, kBeamThreads>(lut, sq, a.ix.pq_tables_col_major, M, tid);
                else BuildLutGeneric<kBeamThreads>(lut, sq, offs, a.ix.pq_tables_col_major, M, tid);
            } else
            switch (uniform_sub) {
                case 1: BuildLutUniform<1, kBeamThreads>(lut, sq, a.ix.pq_tables_col_major, M, tid); break;
                case 2: BuildLutUniform<2, kBeamThreads>(lut, sq, a.ix.pq_tables_col_major, M, tid); break;
                case 3: BuildLutUniform<3, kBeamThreads>(lut, sq, a.ix.pq_tables_col_major, M, tid); break;
                case 4: BuildLutUniform<4, kBeamThreads>(lut, sq, a.ix.pq_tables_col_major, M, tid); break;
                case 6: BuildLutUniform<6, kBeamThreads>(lut, sq, a.ix.pq_tables_col_major, M, tid); break;
                case 8: BuildLutUniform<8, kBeamThreads>(lut, sq, a.ix.pq_tables_col_major, M, tid); break;
                default: BuildLutGeneric<kBeamThreads>(lut, sq, offs, a.ix.pq_tables_col_major, M, tid); break;
            }
        }
        // cand_b needs no clear: a merge writes all C elements of the buffer it fills.
        for (uint32_t i = tid; i < C; i += kBeamThreads) cand_a[i] = kInvalidKey;
        for (uint32_t i = tid; i < kBloomWords; i += kBeamThreads) bloom[i] = 0u;
        for (uint32_t i = tid; i < UW; i += kBeamThreads) unexp[i] = 0u;
        if (tid == 0) {
            ctl.first_full = 0xffffffffu;
            ctl.nsel = 0; ctl.stop = 0;
            ctl.ls_stage = 0; ctl.ls_has_prev = 0; ctl.ls_topk_changed = 0;
            ctl.ls_prev_dk = __int_as_float(0x7f800000);
            ctl.ls_prev_boundary = __int_as_float(0x7f800000);
            s_surv = 0; s_pass = 0;
        }
        if (tid < 32) ctl.ls_prev_ids[tid] = kInvalid;
        if (lut_copy_pending) {
            const bool arrived = BarrierWaitBounded(&lut_barrier, lut_phase & 1u);
            ++lut_phase;
            if (!__syncthreads_and(arrived)) {
                // Never seen. The copy may still land in `lut` later, so the block must not use that memory
                // again: it reports the timeout, gives the copy one more bounded wait and ends without results
                // for its remaining queries.
                if (tid == 0 && a.status != nullptr) atomicOr(a.status, TANN_STATUS_COPY_TIMEOUT);
                BarrierWaitBounded(&lut_barrier, (lut_phase - 1u) & 1u);
                return;
            }
        }
        __syncthreads();

        TANN_PHASE(0);  // 0: set-up (table build, clears)
        // block-uniform state, identical in every thread
        uint32_t valid = 0, visited = 0, hash_iter = 0, expanded = 0, iterations = 0;
        unsigned long long* cur = cand_a;
        unsigned long long* nxt = cand_b;
        const uint32_t entry_begin = a.entry_offsets[q];
        const uint32_t num_entries = a.entry_offsets[q + 1] - entry_begin;
        const uint32_t entry_batches = slots == 0 ? 0 : (num_entries + slots - 1) / slots;
        uint32_t batch = 0;
        bool in_entries = entry_batches > 0;

        // ---- one pass per batch of slot ids: entry batches first, then expansions ----------
        while (true) {
            uint32_t nslots;
            uint32_t sel_word = 0, sel_begin = 0, sel_end = 0;  // this lane's share of the selection
            uint32_t mark_pos = kInvalid;   // list rank this lane marks as expanded (bitmaps of <= 4 words)
            uint32_t my_node = kInvalid;    // kSingle, bitmaps of <= 4 words: the node of this thread's slot
            if (in_entries) {
                nslots = slots;
            } else {
                // Stop tests and selection (:2414-2513). The unexpanded bitmap was rebuilt from the
                // list after the last merge, so every set bit is a valid, unexpanded rank below
                // min(valid, L): the first W set bits are exactly what the reference's serial scan
                // picks. Every warp finds them by itself with one popcount scan over the words (all
                // inputs are block-uniform), so no barrier separates the bitmap from the adjacency
                // loads; warp 0 marks the picked elements as expanded after the next barrier.
                uint32_t stop = 0, nsel = 0;
                if (expanded >= a.p.max_expansions || valid == 0) {
                    stop = 2;
                } else if (!kPlain && a.p.learned_stop.enabled) {
                    if (tid == 0)
                        ctl.stop = LearnedStop(a.p.learned_stop, ctl, valid, visited, expanded, cur, unexp, L) ? 2u : 0u;
                    __syncthreads();
                    stop = ctl.stop;
                }
                if (!stop) {
                    const bool prefix_stop = !kPlain && a.p.stop_prefix != 0 && a.p.stop_prefix < L;
                    if (kPlain || UW <= 4) {
                        // up to 128 list ranks: every thread reads the whole bitmap and finds the
                        // pick of its own slot directly (no scan, no exchange)
                        uint32_t wd[4];
#pragma unroll
                        for (uint32_t u = 0; u < 4; ++u) wd[u] = (u < UW && (!kOneWord || u == 0)) ? unexp[u] : 0u;
                        bool any;
                        if (prefix_stop && a.p.stop_use_expanded) {
                            any = !(valid >= L && expanded >= a.p.stop_prefix);
                        } else {
                            const uint32_t words = (prefix_stop && valid >= a.p.stop_prefix)
                                                       ? (a.p.stop_prefix + 31) / 32 : UW;
                            uint32_t acc = 0;
#pragma unroll
                            for (uint32_t u = 0; u < 4; ++u) acc |= u < words ? wd[u] : 0u;
                            any = acc != 0u;
                        }
                        if (!any) {
                            stop = 2;
                        } else {
                            nsel = min((uint32_t)(__popc(wd[0]) + __popc(wd[1]) + __popc(wd[2]) + __popc(wd[3])), W);
                            if (nsel == 0) {
                                stop = 1;
                            } else if (kSingle) {
                                if (my_k < nsel) my_node = KeyPackedId(cur[NthSetBit(wd, my_k)]) & kRawMask;
                                if (tid < nsel) mark_pos = NthSetBit(wd, tid);   // warp 0 marks them later
                            } else {
                                if (lane < nsel) {
                                    const uint32_t pos = NthSetBit(wd, lane);
                                    s_sel[tid >> 5][lane] = KeyPackedId(cur[pos]) & kRawMask;
                                    if (tid < 32) mark_pos = pos;
                                }
                                __syncwarp();
                            }
                        }
                    } else if (UW <= 32) {
                        sel_word = lane < UW ? unexp[lane] : 0u;
                        bool any;
                        if (prefix_stop && a.p.stop_use_expanded) {
                            any = !(valid >= L && expanded >= a.p.stop_prefix);
                        } else {
                            const uint32_t words = (prefix_stop && valid >= a.p.stop_prefix)
                                                       ? (a.p.stop_prefix + 31) / 32 : UW;
                            any = __ballot_sync(kFull, lane < words && sel_word != 0u) != 0u;
                        }
                        if (!any) {
                            stop = 2;
                        } else {
                            const uint32_t cnt = __popc(sel_word);
                            uint32_t incl = cnt;
#pragma unroll
                            for (int off = 1; off < 32; off <<= 1) {
                                const uint32_t t = __shfl_up_sync(kFull, incl, off);
                                if (lane >= (uint32_t)off) incl += t;
                            }
                            nsel = min(__shfl_sync(kFull, incl, 31), W);
                            sel_begin = incl - cnt;
                            sel_end = min(incl, nsel);
                            uint32_t w = sel_word;
                            for (uint32_t sidx = sel_begin; sidx < sel_end; ++sidx) {
                                const uint32_t bit = __ffs(w) - 1;
                                w &= w - 1u;
                                s_sel[tid >> 5][sidx] = KeyPackedId(cur[lane * 32 + bit]) & kRawMask;
                            }
                            __syncwarp();
                            if (nsel == 0) stop = 1;
                        }
                    } else {
                        // more than 1024 list ranks: serial scan by one thread, shared through a barrier
                        if (tid == 0) {
                            bool any = false;
                            if (prefix_stop && a.p.stop_use_expanded) {
                                any = !(valid >= L && expanded >= a.p.stop_prefix);
                            } else {
                                const uint32_t words = (prefix_stop && valid >= a.p.stop_prefix)
                                                           ? (a.p.stop_prefix + 31) / 32 : UW;
                                for (uint32_t w = 0; w < words; ++w) any |= unexp[w] != 0u;
                            }
                            uint32_t found = 0;
                            for (uint32_t w = 0; any && w < UW && found < W; ++w) {
                                uint32_t word = unexp[w];
                                while (word != 0u && found < W) {
                                    const uint32_t idx = w * 32 + __ffs(word) - 1;
                                    word &= word - 1u;
                                    const unsigned long long k = cur[idx];
                                    cur[idx] = k | kExpandedBit;
                                    for (int wp = 0; wp < kBeamThreads / 32; ++wp)
                                        s_sel[wp][found] = KeyPackedId(k) & kRawMask;
                                    ++found;
                                }
                            }
                            ctl.nsel = found;
                            ctl.stop_scan = !any ? 2u : (found == 0 ? 1u : 0u);
                        }
                        __syncthreads();
                        stop = ctl.stop_scan;
                        nsel = ctl.nsel;
                    }
                }
                if (stop) {
                    // the reference counts an iteration whenever the scan for nodes ran, also when
                    // it found none (:2479-2513); stop == 2 marks the stops taken before the scan
                    if (stop == 1) ++iterations;
                    break;
                }
                ++iterations;
                expanded += nsel;
                nslots = nsel * deg;
            }
            TANN_PHASE(1);  // 1: stop tests + selection

            // ---- phase 1: gather slot ids, Bloom tests ----------------------------------------
            unsigned long long my_key = kInvalidKey;  // kSingle: this thread's slot
            uint32_t my_words[kM > 0 ? kM / 4 : 1];     // kSingle: its code row
            BloomBits my_bits;                          // kSingle: its visited-set positions
            if (!kSingle)
                for (uint32_t i = tid; i < F; i += kBeamThreads) fkey[i] = kInvalidKey;
            const uint32_t rounds = kSingle ? 1u : (nslots + kBeamThreads - 1) / kBeamThreads;
            if (!kSingle) {
                __syncthreads();
                if (tid < 32) MarkExpanded(cur, sel_word, sel_begin, sel_end, lane, mark_pos);
            }
            for (uint32_t r = 0; r < rounds; ++r) {
                const uint32_t s = r * kBeamThreads + tid;
                uint32_t id = kInvalid;
                bool codes_requested = false;   // kSingle: my_words already on their way (neighbour-code layout)
                if (s < nslots) {
                    if (in_entries) {
                        const uint64_t e = (uint64_t)batch * slots + s;
                        if (e < num_entries) id = __ldg(a.entry_ids + entry_begin + e);
                    } else {
                        uint32_t k, j, node;
                        if (kSingle) { k = my_k; j = my_j; } else { k = s / deg; j = s - k * deg; }
                        if (kSingle && UW <= 4) node = my_node; else node = s_sel[tid >> 5][k];
                        const uint32_t* row =
                            (!kPlain && node < a.ix.adjacency_cached_rows)
                                ? a.ix.adjacency_cache + (uint64_t)node * deg
                                : reinterpret_cast<const uint32_t*>(
                                      Row<kOneShard>(a.ix.adjacency, node, (uint64_t)deg * 4));
                        id = __ldg(row + j);
                        // With the neighbour-code layout the slot's code row sits at (node, j): its address
                        // does not depend on the id just requested, so both loads share one round trip.
                        if constexpr (kSingle && kM > 0) {
                            if (kNbr < 0 ? a.ix.neighbor_codes.base[0] != nullptr : kNbr == 1) {
                                LoadCodeWords<kM>(Row<kOneShard>(a.ix.neighbor_codes, node, (uint64_t)deg * kM) + (size_t)j * kM, my_words);
                                codes_requested = true;
                            }
                        }
                    }
                }
                const BloomBits bits = BloomPositions(id);
                const bool in_range = id < N;
#ifndef TANN_BEAM_PROFILE
                // an id that is neither the padding value nor a node of the index is skipped (as the
                // reference does) and reported through the caller's status word
                if (id != kInvalid && !in_range && a.status != nullptr) atomicOr(a.status, TANN_STATUS_BEAM_ID_RANGE);
#endif
                const bool pass = id != kInvalid && in_range && !BloomTest(bits, bloom);
                if (kSingle) my_bits = bits;
                // The code row does not depend on the barrier below: request it now.
                if constexpr (kSingle && kM > 0)
                    if (pass && !codes_requested) LoadCodeWords<kM>(Row<kOneShard>(a.ix.codes, id, M), my_words);
                // Park the surviving id in the key slot; phase 2 turns it into a key.
                const unsigned long long parked = pass ? (unsigned long long)id : kInvalidKey;
                if (kSingle) {
                    my_key = parked;
                } else {
                    // More slots than threads: the reference's 128 threads walk the slots in rounds
                    // of 128, so the tests of a round see the adds of the rounds before it
                    // (src/search/topology_search_kernel.cu:2543-2564). Same here, made explicit.
                    if (s < F) fkey[s] = parked;
                    __syncthreads();
                    if (pass) BloomAdd(bits, bloom);
                    __syncthreads();
                }
            }
            // kSingle: the adds of this round and the expanded marks wait for the compaction barrier below, which
            // every test of the round precedes as well
            TANN_PHASE(2);  // 2: slot ids (adjacency / entries) + Bloom tests
            // ---- phase 2: Bloom adds, code gathers, ADC sums ------------------------------------
            uint32_t fv = 0;
            for (uint32_t r = 0; r < rounds; ++r) {
                const uint32_t s = r * kBeamThreads + tid;
                const unsigned long long parked = kSingle ? my_key : (s < F ? fkey[s] : kInvalidKey);
                const bool pass = parked != kInvalidKey;
                if (pass) {
                    const uint32_t id = (uint32_t)parked;
                    float dist;
                    if constexpr (kSingle && kM > 0) {
                        dist = AdcFromWords<kM>(lut, my_words);
                    } else {
                        dist = AdcTreeThread<kM>(lut, Row<kOneShard>(a.ix.codes, id, M), M);
                    }
                    const unsigned long long key = ((unsigned long long)OrderedBits(dist) << 32) | id;
                    if (kSingle) my_key = key; else fkey[s] = key;
                }
                if (!kSingle) fv += __syncthreads_count(pass);
            }
            TANN_PHASE(3);  // 3: Bloom adds + code rows + table sums

            // ---- order the frontier and merge it into the list (:1338-1424) ---------------------
            // sorted[0 .. n) = the frontier entries that can still enter the list, ascending;
            // entry x is accepted while sorted[x] < list[nv-1-x] (a prefix, the test is monotone).
            const unsigned long long* sorted;
            uint32_t nv, accepted = 0;
            if (kSingle) {
                // When the list is full an entry not below its last element can never be accepted,
                // so only the others are kept; they are compacted and rank-sorted (each survivor
                // counts the survivors in front of it), which costs ~4 instructions per pair
                // instead of a 28-step bitonic network over all 128 slots. The same thread then
                // tests its entry for acceptance and finds its place in the list: an accepted entry
                // is below list[nv - accepted], so its lower bound in the whole list is also its
                // lower bound among the elements that stay.
                const bool pass = my_key != kInvalidKey;
                const unsigned long long thr = valid == C ? (cur[C - 1] & kCmpMask) : ~0ull;
                const bool surv = pass && my_key < thr;
                const uint32_t ballot_pass = __ballot_sync(kFull, pass);
                const uint32_t ballot = __ballot_sync(kFull, surv);
                uint32_t base = 0;
                if (lane == 0) {
                    if (ballot != 0u) base = atomicAdd(&s_surv, (uint32_t)__popc(ballot));
                    if (ballot_pass != 0u) atomicAdd(&s_pass, (uint32_t)__popc(ballot_pass));
                }
                base = __shfl_sync(kFull, base, 0);
                if (surv) fkey[base + __popc(ballot & ((1u << lane) - 1u))] = my_key;
                __syncthreads();
                if (pass) BloomAdd(my_bits, bloom);
                if (tid < 32) MarkExpanded(cur, sel_word, sel_begin, sel_end, lane, mark_pos);
                TANN_PHASE(8);  // 8: filter + compaction (waits for every code row)
                const uint32_t n = s_surv;
                fv = s_pass;
                nv = (uint32_t)min((uint64_t)C, (uint64_t)valid + fv);
                bool pred = false;
                unsigned long long k = kInvalidKey;
                uint32_t rank = 0;
                if (n > 32 && n <= 64) {
                    // 33..64 survivors: the n x n comparisons are split over all 128 threads. Thread t
                    // compares key t & 63 with one half of the keys (a warp reads the same key at a time,
                    // i.e. broadcasts); the half counts meet in shared memory.
                    const uint32_t i = tid & 63u, part = tid >> 6;
                    const uint32_t half = (n + 1) / 2;
                    const uint32_t jb = part * half, je = min(n, jb + half);
                    uint32_t cnt = 0;
                    if (i < n) {
                        k = fkey[i];
#pragma unroll 8
                        for (uint32_t j = jb; j < je; ++j) {
                            const unsigned long long kj = fkey[j];
                            cnt += (kj < k || (kj == k && j < i)) ? 1u : 0u;
                        }
                        if (part == 1) s_half_rank[i] = cnt;
                    }
                    __syncthreads();
                    if (part == 0 && i < n) rank = cnt + s_half_rank[i];
                    else k = kInvalidKey;   // the upper half only helped counting
                } else if (n > 64) {
                    // Long survivor lists (the list is not full yet): every warp sorts its 32 keys
                    // with shuffles, then a key's rank is its place in its own run plus its lower /
                    // upper bounds in the other runs (runs in front win ties, so ranks are distinct).
                    k = tid < n ? fkey[tid] : kInvalidKey;
                    k = WarpSortKey(k, lane);
                    fkey[tid] = k;
                    __syncthreads();
                    rank = lane;
                    const uint32_t w = tid >> 5;
                    uint32_t cnt[kBeamThreads / 32];
#pragma unroll
                    for (uint32_t o = 0; o < kBeamThreads / 32; ++o) cnt[o] = 0;
#pragma unroll
                    for (uint32_t b = 32; b > 0; b >>= 1) {       // the searches of the other runs, side by side
#pragma unroll
                        for (uint32_t o = 0; o < kBeamThreads / 32; ++o) {
                            const uint32_t t = cnt[o] + b;
                            if (o != w && t <= 32) {
                                const unsigned long long x = fkey[o * 32 + t - 1];
                                if (o < w ? x <= k : x < k) cnt[o] = t;
                            }
                        }
                    }
#pragma unroll
                    for (uint32_t o = 0; o < kBeamThreads / 32; ++o) rank += cnt[o];
                } else if (tid < n) {
                    k = fkey[tid];
#pragma unroll 8
                    for (uint32_t j = 0; j < n; ++j) {
                        const unsigned long long kj = fkey[j];
                        rank += (kj < k || (kj == k && j < tid)) ? 1u : 0u;
                    }
                }
                TANN_PHASE(9);  // 9: ranks of the survivors
                if (k != kInvalidKey) {
                    skey[rank] = k;
                    if (rank < nv) pred = k < (cur[nv - 1 - rank] & kCmpMask);
                    if (pred) {
                        uint32_t lo = 0;  // list elements < k stay in front of it (fixed-trip count)
                        if (valid != 0) {
                            for (uint32_t b = 1u << (31 - __clz(valid)); b > 0; b >>= 1) {
                                const uint32_t t = lo + b;
                                if (t <= valid && (cur[t - 1] & kCmpMask) < k) lo = t;
                            }
                        }
                        nxt[rank + lo] = k;
                        if (!kPlain && rank + lo < a.p.learned_stop.top_k) ctl.ls_topk_changed = 1;
                    }
                }
                accepted = __syncthreads_count(pred);
                if (tid == 0) { s_surv = 0; s_pass = 0; }
                sorted = skey;
                TANN_PHASE(4);  // 4: filter + compaction + rank sort + acceptance
            } else {
                nv = (uint32_t)min((uint64_t)C, (uint64_t)valid + fv);
                SortKeysShared(fkey, F);
                sorted = fkey;
                TANN_PHASE(4);
                const uint32_t lim = min(fv, nv);
                uint32_t base = 0;
                do {
                    const uint32_t x = base + tid;
                    bool pred = false;
                    if (x < lim) pred = sorted[x] < (cur[nv - 1 - x] & kCmpMask);
                    const uint32_t cnt = __syncthreads_count(pred);
                    accepted += cnt;
                    if (cnt < (uint32_t)kBeamThreads) break;
                    base += kBeamThreads;
                } while (base < lim);
                const uint32_t kept = nv - accepted;
                bool changed = false;
                for (uint32_t j = tid; j < accepted; j += kBeamThreads) {
                    const unsigned long long fk = sorted[j];
                    uint32_t lo = 0, hi = kept;  // kept candidates < fk stay in front of it
                    while (lo < hi) {
                        const uint32_t mid = (lo + hi) >> 1;
                        if ((cur[mid] & kCmpMask) < fk) lo = mid + 1; else hi = mid;
                    }
                    nxt[j + lo] = fk;
                    changed |= (j + lo) < a.p.learned_stop.top_k;
                }
                if (changed) ctl.ls_topk_changed = 1;
            }
            if (accepted != 0) {
                const uint32_t kept = nv - accepted;
                // Every kept element moves back by the number of accepted keys <= it (those go in front
                // of it). The count is a fixed-trip binary search, two elements per thread at a time so
                // that their shared-memory reads overlap.
                const uint32_t top_bit = 1u << (31 - __clz(accepted));
                for (uint32_t i0 = tid; i0 < kept; i0 += 2 * kBeamThreads) {
                    const uint32_t i1 = i0 + kBeamThreads;
                    const bool two = i1 < kept;
                    const unsigned long long c0 = cur[i0];
                    const unsigned long long c1 = two ? cur[i1] : 0ull;
                    const unsigned long long ck0 = c0 & kCmpMask, ck1 = c1 & kCmpMask;
                    uint32_t p0 = 0, p1 = 0;
                    for (uint32_t b = top_bit; b > 0; b >>= 1) {
                        const uint32_t t0 = p0 + b, t1 = p1 + b;
                        const bool in0 = t0 <= accepted, in1 = two && t1 <= accepted;
                        const unsigned long long s0 = in0 ? sorted[t0 - 1] : ~0ull;
                        const unsigned long long s1 = in1 ? sorted[t1 - 1] : ~0ull;
                        if (s0 <= ck0) p0 = t0;
                        if (s1 <= ck1) p1 = t1;
                    }
                    nxt[i0 + p0] = c0;
                    if (two) nxt[i1 + p1] = c1;
                }
                for (uint32_t i = nv + tid; i < C; i += kBeamThreads) nxt[i] = kInvalidKey;
                unsigned long long* t = cur; cur = nxt; nxt = t;
            }
            valid = nv;
            visited += fv;
            ++hash_iter;
            const bool rebuild = hash_iter >= 3;
            if (rebuild) {
                hash_iter = 0;
                for (uint32_t i = tid; i < kBloomWords; i += kBeamThreads) bloom[i] = 0u;
            }
            if (tid == 0 && ctl.first_full == 0xffffffffu && nv >= L)
                ctl.first_full = in_entries ? 0u : iterations;
            __syncthreads();
            TANN_PHASE(5);  // 5: acceptance + merge
            // ---- prefix state (:822-845): unexpanded bitmap, Bloom rebuild every third merge ----
            const uint32_t prefix = min(nv, L);
            for (uint32_t base = 0; base < UW * 32; base += kBeamThreads) {
                const uint32_t i = base + tid;
                bool un = false;
                if (i < prefix) {
                    const uint32_t pid = KeyPackedId(cur[i]);
                    if (pid != kInvalid) {
                        un = (pid & kExpandedBit) == 0;
                        if (rebuild) BloomAdd(pid & kRawMask, bloom);
                    }
                }
                const uint32_t word = __ballot_sync(kFull, un);
                if (lane == 0 && (i >> 5) < UW) unexp[i >> 5] = word;
            }
            __syncthreads();
            TANN_PHASE(6);  // 6: bitmap + Bloom rebuild

            if (in_entries) {
                ++batch;
                if (batch >= entry_batches) in_entries = false;
            }
        }

        // ---- results -----------------------------------------------------------------------------
        Cand* out = a.out_cand + q * (uint64_t)C;
        for (uint32_t i = tid; i < C; i += kBeamThreads) {
            const unsigned long long k = cur[i];
            Cand c;
            c.dist = KeyDist(k);
            c.id = KeyPackedId(k);
            out[i] = c;
        }
        if (tid == 0) {
            uint32_t* st = a.out_stats + q * 8;
            st[0] = visited; st[1] = expanded; st[2] = 0; st[3] = iterations;
            st[4] = valid; st[5] = ctl.first_full; st[6] = 0; st[7] = 0;
        }
        __syncthreads();
        TANN_PHASE(7);  // 7: output
#ifdef TANN_BEAM_PROFILE
        if (tid == 0 && a.status != nullptr) {
            unsigned long long* o = reinterpret_cast<unsigned long long*>(a.status) + q * 12;
            for (int i = 0; i < 12; ++i) o[i] = prof_acc[i];
        }
#endif
    }
}

size_t BeamSmemBytes(uint32_t M, uint32_t C, uint32_t F, uint32_t L, uint32_t d) {
    const size_t uw = (L + 31) / 32;
    // single-round kernels keep two 128-key buffers (compacted and sorted frontier)
    const size_t fk = F <= (uint32_t)kBeamThreads ? (size_t)2 * kBeamThreads : F;
    size_t bytes = (size_t)M * kCentroids * 4 + (size_t)2 * C * 8 + fk * 8 + kBloomWords * 4 +
                   uw * 4 + ((size_t)M + 1) * 4 + (size_t)d * 4;
    return (bytes + 15) & ~(size_t)15;
}

typedef void (*BeamKernel)(const BeamArgs);

template <bool kSingle>
static BeamKernel PickByChunks(uint32_t M) {
    switch (M) {
        case 16: return beam_search_kernel<16, kSingle, 0>;
        case 32: return beam_search_kernel<32, kSingle, 0>;
        case 48: return beam_search_kernel<48, kSingle, 0>;
        case 64: return beam_search_kernel<64, kSingle, 0>;
        case 96: return beam_search_kernel<96, kSingle, 0>;
        default: return beam_search_kernel<0, kSingle, 0>;
    }
}

// The plain form exists for the chunk counts and widths of the benchmark configurations (128 dims in 32 chunks,
// 96 in 48, 768 in 96) with at most 128 slots per batch.
static bool PlainCase(const BeamArgs& a) {
    const TannIndexView& ix = a.ix;
    const TannBeamParams& p = a.p;
    return a.lut == nullptr && !p.learned_stop.enabled && (p.stop_prefix == 0 || p.stop_prefix >= p.top_l) &&
           !p.stop_use_expanded && p.top_l <= 128 && ix.adjacency_cached_rows == 0 &&
           p.search_width * ix.degree <= (uint32_t)kBeamThreads;
}

template <int kM, int kSub>
static BeamKernel PickPlain(bool nbr, bool one_word, bool sharded) {
    if (sharded)   // node-id-range shards: the layout is looked up in the index view
        return one_word ? beam_search_kernel<kM, true, kSub, -1, true, true> : beam_search_kernel<kM, true, kSub, -1, false, true>;
    if (nbr) return one_word ? beam_search_kernel<kM, true, kSub, 1, true> : beam_search_kernel<kM, true, kSub, 1, false>;
    return one_word ? beam_search_kernel<kM, true, kSub, 0, true> : beam_search_kernel<kM, true, kSub, 0, false>;
}

BeamKernel PickBeamKernel(uint32_t M, uint32_t slots, uint32_t plain_sub, bool nbr, bool one_word, bool sharded) {
    if (plain_sub != 0 && slots <= (uint32_t)kBeamThreads) {
        if (M == 32 && plain_sub == 4) return PickPlain<32, 4>(nbr, one_word, sharded);
        if (M == 48 && plain_sub == 2) return PickPlain<48, 2>(nbr, one_word, sharded);
        if (M == 96 && plain_sub == 8) return PickPlain<96, 8>(nbr, one_word, sharded);
    }
    return slots <= (uint32_t)kBeamThreads ? PickByChunks<true>(M) : PickByChunks<false>(M);
}

static uint32_t PlainSub(const BeamArgs& a) {
    if (!PlainCase(a) || a.ix.num_chunks == 0 || a.ix.dim % a.ix.num_chunks != 0) return 0;
    return a.ix.dim / a.ix.num_chunks;
}

cudaError_t LaunchBeam(const BeamArgs& a, size_t smem, uint32_t grid, cudaStream_t stream) {
    BeamKernel k = PickBeamKernel(a.ix.num_chunks, a.p.search_width * a.ix.degree, PlainSub(a),
                                  a.ix.neighbor_codes.base[0] != nullptr, a.p.top_l <= 32,
                                  a.ix.adjacency.num_shards > 1 || a.ix.codes.num_shards > 1 || a.ix.neighbor_codes.num_shards > 1);
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    k<<<grid, kBeamThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t BeamOccupancy(uint32_t M, uint32_t slots, size_t smem, int* blocks_per_sm) {
    BeamKernel k = PickBeamKernel(M, slots, 0, false, false, false);   // the plain forms use the same shared memory and no more registers
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocks_per_sm, k, kBeamThreads, smem);
}

}  // namespace tann
