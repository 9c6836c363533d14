// Exact rerank by the owner of the rows, for indexes sharded by node-id range over several GPUs.
// NO COUNTERPART IN THE REFERENCE (it is single-GPU).
//
// Reading a candidate's vector from the shard of another GPU costs one random access into that GPU's memory.
// With shards of tens of GB the peers' memory is hundreds of GB of address space touched at random, and the
// rate of such accesses falls far below what NVLink carries. The candidates can travel instead: the GPU
// that ran a query's traversal splits its candidate list by owner (partition_candidates_kernel: one list per
// owner, ids rewritten to the owner's local row numbers), the lists are exchanged, every owner scores what it
// received against its own shard with the ordinary rerank kernel, the k best of every (query, owner) pair
// travel back, and merge_topk_lists_kernel merges them by (distance, global id). Exact distances and the
// order do not depend on where a row is scored, so the result is the unsharded one bit for bit.
#include "tann_common.cuh"
#include "tann_launch.h"
#include "topoanns_b200.h"

namespace tann {

void SetLastError(const char* message);  // capi.cu

constexpr uint32_t kPartitionMaxOwners = 64;

// One warp per query. Ranks [0, top_n) of the query's candidate list in rank order; the record of owner o's
// c-th candidate goes to out[o][q][c] with its local row number; a list that would exceed `slot` records
// raises *overflow (the caller then falls back to wider lists) and drops the excess.
__global__ void __launch_bounds__(128)
partition_candidates_kernel(const Cand* __restrict__ cand, uint32_t capacity, uint32_t top_n, uint64_t Q,
                            uint32_t rows_per_shard, uint32_t owners, uint32_t slot, Cand* __restrict__ out,
                            uint32_t* __restrict__ overflow) {
    __shared__ uint32_t s_count[4][kPartitionMaxOwners];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t q = (uint64_t)blockIdx.x * 4 + warp;
    if (q >= Q) return;
    uint32_t* count = s_count[warp];
    for (uint32_t o = lane; o < owners; o += 32) count[o] = 0;
    __syncwarp();
    const uint32_t n = top_n < capacity ? top_n : capacity;
    bool over = false;
    for (uint32_t r0 = 0; r0 < n; r0 += 32) {
        const uint32_t r = r0 + lane;
        Cand c;
        c.id = kInvalid;
        c.dist = 0.0f;
        if (r < n) c = cand[q * capacity + r];
        const uint32_t raw = RawId(c.id);
        uint32_t owner = kInvalid;
        if (raw != kInvalid) {
            owner = raw / rows_per_shard;
            if (owner >= owners) owner = kInvalid;   // an id beyond the last shard: dropped
        }
        // position among the lanes of this round that have the same owner, in rank order
        const uint32_t same = __match_any_sync(kFull, owner);
        const uint32_t before = __popc(same & ((1u << lane) - 1u));
        if (owner != kInvalid) {
            const uint32_t pos = count[owner] + before;
            if (pos < slot) {
                Cand w;
                w.id = raw - owner * rows_per_shard;
                w.dist = c.dist;
                out[((uint64_t)owner * Q + q) * slot + pos] = w;
            } else {
                over = true;
            }
        }
        __syncwarp();
        if (owner != kInvalid && before == 0) count[owner] += __popc(same);   // one lane per owner
        __syncwarp();
    }
    // the unused tail of every list
    for (uint32_t o = 0; o < owners; ++o) {
        const uint32_t used = count[o] < slot ? count[o] : slot;
        for (uint32_t p = used + lane; p < slot; p += 32) {
            Cand w;
            w.id = kInvalid;
            w.dist = 0.0f;
            out[((uint64_t)o * Q + q) * slot + p] = w;
        }
    }
    if (__any_sync(kFull, over) && lane == 0) atomicOr(overflow, 1u);
}

// One warp per query: `lists` sorted lists of k <= 32 (distance, local id) pairs, list l holding rows of shard
// l (global id = local id + l * rows_per_shard); the k smallest by (distance, global id) come out sorted.
__global__ void __launch_bounds__(128)
merge_topk_lists_kernel(const float* __restrict__ dists, const uint32_t* __restrict__ ids, uint32_t lists, uint64_t Q,
                        uint32_t k, uint32_t rows_per_shard, float* __restrict__ out_dists,
                        uint32_t* __restrict__ out_ids) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t q = (uint64_t)blockIdx.x * 4 + warp;
    if (q >= Q) return;
    constexpr unsigned long long kNone = 0xff800000ffffffffull;   // (+inf, invalid id)
    unsigned long long best = kNone;
    for (uint32_t l = 0; l < lists; ++l) {
        unsigned long long key = kNone;
        if (lane < k) {
            const uint64_t at = ((uint64_t)l * Q + q) * k + lane;
            const uint32_t id = ids[at];
            if (id != kInvalid) key = KeyOf(dists[at], id + l * rows_per_shard);
        }
        key = WarpSortKey(key, lane);
        if (l == 0) {
            best = key;
            continue;
        }
        // the 32 smallest of two sorted runs: element-wise minimum of one and the other reversed is a bitonic
        // sequence of exactly those; five compare-exchange stages sort it
        const unsigned long long other = __shfl_sync(kFull, key, 31 - lane);
        unsigned long long m = best < other ? best : other;
#pragma unroll
        for (uint32_t sft = 16; sft > 0; sft >>= 1) {
            const unsigned long long o = __shfl_xor_sync(kFull, m, sft);
            const bool upper = (lane & sft) != 0;
            m = upper ? (o > m ? o : m) : (o < m ? o : m);
        }
        best = m;
    }
    if (lane < k) {
        out_dists[q * k + lane] = FromOrderedBits((uint32_t)(best >> 32));
        out_ids[q * k + lane] = (uint32_t)best;
    }
}

cudaError_t LaunchPartitionCandidates(const void* cand, uint32_t capacity, uint32_t top_n, uint64_t Q,
                                      uint32_t rows_per_shard, uint32_t owners, uint32_t slot, void* out,
                                      uint32_t* overflow, cudaStream_t stream) {
    if (Q == 0) return cudaSuccess;
    partition_candidates_kernel<<<(unsigned)((Q + 3) / 4), 128, 0, stream>>>(
        static_cast<const Cand*>(cand), capacity, top_n, Q, rows_per_shard, owners, slot, static_cast<Cand*>(out),
        overflow);
    return cudaGetLastError();
}

cudaError_t LaunchMergeTopkLists(const float* dists, const uint32_t* ids, uint32_t lists, uint64_t Q, uint32_t k,
                                 uint32_t rows_per_shard, float* out_dists, uint32_t* out_ids, cudaStream_t stream) {
    if (Q == 0) return cudaSuccess;
    merge_topk_lists_kernel<<<(unsigned)((Q + 3) / 4), 128, 0, stream>>>(dists, ids, lists, Q, k, rows_per_shard,
                                                                          out_dists, out_ids);
    return cudaGetLastError();
}

TannStatus OwnerFail(TannStatus st, const char* message) {
    SetLastError(message);
    return st;
}

}  // namespace tann

extern "C" {

TannStatus tann_partition_candidates(const void* candidates, uint32_t capacity, uint32_t top_n, uint64_t num_queries,
                                     uint64_t rows_per_shard, uint32_t num_owners, uint32_t slot, void* out,
                                     uint32_t* overflow, tann_stream_t stream) {
    if (num_queries == 0 || top_n == 0) return TANN_OK;
    if (!candidates || !out || !overflow)
        return tann::OwnerFail(TANN_ERR_INVALID_ARGUMENT, "tann_partition_candidates: null pointer.");
    if (num_owners == 0 || num_owners > tann::kPartitionMaxOwners || slot == 0 || rows_per_shard == 0 ||
        rows_per_shard > 0x7fffffffull)
        return tann::OwnerFail(TANN_ERR_INVALID_ARGUMENT,
                               "tann_partition_candidates: 1 to 64 owners, a non-empty slot and rows_per_shard below 2^31.");
    cudaError_t e = tann::LaunchPartitionCandidates(candidates, capacity, top_n, num_queries, (uint32_t)rows_per_shard,
                                                    num_owners, slot, out, overflow, (cudaStream_t)stream);
    if (e != cudaSuccess) return tann::OwnerFail(TANN_ERR_CUDA, cudaGetErrorString(e));
    return TANN_OK;
}

TannStatus tann_merge_topk_lists(const float* dists, const uint32_t* ids, uint32_t num_lists, uint64_t num_queries,
                                 uint32_t top_k, uint64_t rows_per_shard, float* out_dists, uint32_t* out_ids,
                                 tann_stream_t stream) {
    if (num_queries == 0 || top_k == 0) return TANN_OK;
    if (!dists || !ids || !out_dists || !out_ids)
        return tann::OwnerFail(TANN_ERR_INVALID_ARGUMENT, "tann_merge_topk_lists: null pointer.");
    if (num_lists == 0 || top_k > 32 || rows_per_shard > 0x7fffffffull ||
        (uint64_t)num_lists * rows_per_shard > 0x80000000ull)
        return tann::OwnerFail(TANN_ERR_INVALID_ARGUMENT,
                               "tann_merge_topk_lists: at least one list, top_k at most 32, num_lists * rows_per_shard "
                               "at most 2^31 (node ids have 31 bits).");
    cudaError_t e = tann::LaunchMergeTopkLists(dists, ids, num_lists, num_queries, top_k, (uint32_t)rows_per_shard,
                                               out_dists, out_ids, (cudaStream_t)stream);
    if (e != cudaSuccess) return tann::OwnerFail(TANN_ERR_CUDA, cudaGetErrorString(e));
    return TANN_OK;
}

}  // extern "C"
