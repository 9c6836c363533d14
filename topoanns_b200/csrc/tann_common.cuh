// Shared device helpers of the B200 graph-search kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "topoanns_b200.h"

namespace tann {

constexpr uint32_t kInvalid = 0xffffffffu;
constexpr uint32_t kExpandedBit = 0x80000000u;
constexpr uint32_t kRawMask = 0x7fffffffu;
constexpr uint32_t kBloomWords = 1024;  // 32 768-bit filter, src/search/topology_search_kernel.cu:55
constexpr uint32_t kCentroids = 256;
constexpr unsigned kFull = 0xffffffffu;

struct __align__(8) Cand {
    float dist;
    uint32_t id;
};

__host__ __device__ inline uint32_t RawId(uint32_t packed) {
    return packed == kInvalid ? kInvalid : (packed & kRawMask);
}

// Order-preserving map float -> uint32 (total order of the reals; -0 sorts just below +0, which
// never meets here because every distance on this path is a sum of squares or +inf).
__device__ __forceinline__ uint32_t OrderedBits(float f) {
    const uint32_t b = __float_as_uint(f);
    return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}
__device__ __forceinline__ float FromOrderedBits(uint32_t o) {
    const uint32_t b = o ^ ((o >> 31) ? 0x80000000u : 0xffffffffu);
    return __uint_as_float(b);
}

// 64-bit sort key of a candidate: (distance, raw id) ascending, the order of CandidateLess
// (src/search/topology_search_kernel.cu:414-420). Invalid = (+inf, 0xffffffff) sorts last.
__device__ __forceinline__ unsigned long long KeyOf(float dist, uint32_t packed_id) {
    return (static_cast<unsigned long long>(OrderedBits(dist)) << 32) | RawId(packed_id);
}
__device__ __forceinline__ unsigned long long KeyOf(const Cand& c) { return KeyOf(c.dist, c.id); }

__device__ __forceinline__ uint32_t BloomHash(int h, uint32_t v) {
    // src/search/topology_search_kernel.cu:382-385,611-619
    constexpr uint32_t s[6] = {0x924ed183u, 0xd854fc0au, 0xecf5e3b7u,
                               0x1bead407u, 0x28a30449u, 0xbfc4d99fu};
    v ^= v >> 16;
    v *= s[h << 1];
    v ^= v >> 13;
    v *= s[(h << 1) + 1];
    v ^= v >> 16;
    return v & (kBloomWords * 32 - 1);
}
// The three bit positions of a value; computed once and used for the test and, later, the add.
struct BloomBits {
    uint32_t b[3];
};
__device__ __forceinline__ BloomBits BloomPositions(uint32_t v) {
    BloomBits r;
#pragma unroll
    for (int h = 0; h < 3; ++h) r.b[h] = BloomHash(h, v);
    return r;
}
__device__ __forceinline__ bool BloomTest(const BloomBits& p, const uint32_t* words) {
    bool ok = true;
#pragma unroll
    for (int h = 0; h < 3; ++h) ok &= ((words[p.b[h] & (kBloomWords - 1)] >> (p.b[h] >> 10)) & 1u) != 0u;
    return ok;
}
__device__ __forceinline__ void BloomAdd(const BloomBits& p, uint32_t* words) {
#pragma unroll
    for (int h = 0; h < 3; ++h) atomicOr(&words[p.b[h] & (kBloomWords - 1)], 1u << (p.b[h] >> 10));
}
__device__ __forceinline__ bool BloomTest(uint32_t v, const uint32_t* words) { return BloomTest(BloomPositions(v), words); }
__device__ __forceinline__ void BloomAdd(uint32_t v, uint32_t* words) { BloomAdd(BloomPositions(v), words); }

// Resolve row `n` of a sharded array; rows are `row_bytes` apart inside a shard.
__device__ __forceinline__ const uint8_t* ShardRow(const TannShards& s, uint64_t n, uint64_t row_bytes) {
    if (s.num_shards <= 1) return static_cast<const uint8_t*>(s.base[0]) + n * row_bytes;
    const uint64_t shard = n / s.rows_per_shard;
    const uint64_t local = n - shard * s.rows_per_shard;
    return static_cast<const uint8_t*>(s.base[shard]) + local * row_bytes;
}

// The shuffle-down tree of the reference (16, 8, 4, 2, 1); lane 0 holds the result.
__device__ __forceinline__ float WarpTreeSum(float v) {
    v += __shfl_down_sync(kFull, v, 16);
    v += __shfl_down_sync(kFull, v, 8);
    v += __shfl_down_sync(kFull, v, 4);
    v += __shfl_down_sync(kFull, v, 2);
    v += __shfl_down_sync(kFull, v, 1);
    return v;
}

// Bitonic sort of one key per lane across a warp, ascending by lane.
__device__ __forceinline__ unsigned long long WarpSortKey(unsigned long long k, uint32_t lane) {
#pragma unroll
    for (uint32_t size = 2; size <= 32; size <<= 1) {
#pragma unroll
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            const unsigned long long o = __shfl_xor_sync(kFull, k, stride);
            const bool upper = (lane & stride) != 0;          // this lane holds the pair's upper slot
            const bool asc = (lane & size) == 0 || size == 32;
            const bool take_min = upper != asc;
            k = take_min ? (o < k ? o : k) : (o > k ? o : k);
        }
    }
    return k;
}

// Query look-up table (src/search/pq_query_tables.cu:33-52), four consecutive centroids per thread
// and step: one 16-byte load per dim and the same per-entry FMA chain (ascending dim) as the
// one-entry form. kSub = dims per chunk when every chunk has that many: the loads of a step
// (sixteen per thread) are then all issued before the first is used, which is what keeps the
// 128 KB table stream from L2 from being latency-bound.
template <int kSub, int kThreads>
__device__ __forceinline__ void BuildLutUniform(float* lut /*shared or global, 16-byte aligned*/, const float* sq, const float* tables,
                                                uint32_t M, uint32_t tid) {
    constexpr int kItems = kSub <= 2 ? 8 : (kSub <= 4 ? 4 : 2);   // 16 loads in flight per thread
    const uint32_t total = M * (kCentroids / 4);
    for (uint32_t item0 = tid; item0 < total; item0 += kThreads * kItems) {
        float4 t[kItems][kSub];
#pragma unroll
        for (int u = 0; u < kItems; ++u) {
            const uint32_t item = item0 + u * kThreads;
            if (item < total) {
                const uint32_t m = item >> 6, c4 = (item & 63u) * 4u;
#pragma unroll
                for (int sd = 0; sd < kSub; ++sd)
                    t[u][sd] = __ldg(reinterpret_cast<const float4*>(
                        tables + (size_t)(m * kSub + sd) * kCentroids + c4));
            }
        }
#pragma unroll
        for (int u = 0; u < kItems; ++u) {
            const uint32_t item = item0 + u * kThreads;
            if (item < total) {
                const uint32_t m = item >> 6, c4 = (item & 63u) * 4u;
                float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int sd = 0; sd < kSub; ++sd) {
                    const float sv = sq[m * kSub + sd];
                    float df = t[u][sd].x - sv; acc.x = fmaf(df, df, acc.x);
                    df = t[u][sd].y - sv; acc.y = fmaf(df, df, acc.y);
                    df = t[u][sd].z - sv; acc.z = fmaf(df, df, acc.z);
                    df = t[u][sd].w - sv; acc.w = fmaf(df, df, acc.w);
                }
                *reinterpret_cast<float4*>(lut + m * kCentroids + c4) = acc;
            }
        }
    }
}

template <int kThreads>
__device__ __noinline__ void BuildLutGeneric(float* lut, const float* sq, const uint32_t* offs,
                                             const float* tables, uint32_t M, uint32_t tid) {
    for (uint32_t item = tid; item < M * (kCentroids / 4); item += kThreads) {
        const uint32_t m = item >> 6, c4 = (item & 63u) * 4u;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (uint32_t dim = offs[m]; dim < offs[m + 1]; ++dim) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(tables + (size_t)dim * kCentroids + c4));
            const float sv = sq[dim];
            float df = t.x - sv; acc.x = fmaf(df, df, acc.x);
            df = t.y - sv; acc.y = fmaf(df, df, acc.y);
            df = t.z - sv; acc.z = fmaf(df, df, acc.z);
            df = t.w - sv; acc.w = fmaf(df, df, acc.w);
        }
        *reinterpret_cast<float4*>(lut + m * kCentroids + c4) = acc;
    }
}

// ---- bulk asynchronous copy (TMA, untiled form) of a contiguous global range into shared memory ----
// One thread arms an mbarrier with the byte count and issues the copies; every thread then polls the
// barrier's phase. Source, destination and size are multiples of 16 bytes. The poll is bounded: if the
// phase does not complete within the limit the caller loads the range with ordinary loads instead.
__device__ __forceinline__ uint32_t SmemAddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void BarrierInit(unsigned long long* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(arrivals) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void BulkLoadToShared(void* dst, const void* src, uint32_t bytes, unsigned long long* bar) {
    constexpr uint32_t kChunk = 32768;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier generic accesses to dst come first
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
    for (uint32_t off = 0; off < bytes; off += kChunk) {
        const uint32_t n = min(kChunk, bytes - off);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(SmemAddr(static_cast<char*>(dst) + off)), "l"(static_cast<const char*>(src) + off), "r"(n),
                       "r"(SmemAddr(bar))
                     : "memory");
    }
}
__device__ __forceinline__ bool BarrierWaitBounded(unsigned long long* bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(SmemAddr(bar)), "r"(parity) : "memory");
        if (done) return true;
        __nanosleep(32);
    }
    return false;
}

template <typename T>
__device__ __forceinline__ float LoadAsFloat(const void* p, uint32_t kind, uint64_t i) {
    if (kind == TANN_KIND_FLOAT32) return static_cast<const float*>(p)[i];
    if (kind == TANN_KIND_UINT8) return static_cast<float>(static_cast<const uint8_t*>(p)[i]);
    return static_cast<float>(static_cast<const int8_t*>(p)[i]);
}

}  // namespace tann
