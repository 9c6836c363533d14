// tann_rerank_topk_static: exact rerank + top-k of one batch with every intermediate buffer in a
// fixed device array of this file, so the call allocates nothing (no cudaMalloc / cudaFree, no
// allocating library routine). It exists for callers that may not allocate at the point where they
// rerank: cudaMalloc and cudaFree synchronise the whole device, so a process that reranks while other
// streams are in the middle of a batch, or that hands its entire HBM budget to another allocator at
// start-up, has no work space to give tann_rerank_exact + tann_topk_pack. The reference has no such
// entry point.
//
// Scratch use (TANN_STATIC_SCRATCH_BYTES in total, 256-byte aligned pieces): a 4-byte "queries are not
// uint8-valued" flag, the uint8 copy of float queries [Q][dim], and the sorted rerank lists
// [Q][top_n] distances + ids. Batches that need more are rejected.
//
// The first call on a device looks up the array's address (cudaGetSymbolAddress) with that device
// current; make that call before any stream capture. Two calls that overlap on the GPU (different
// streams, or different host threads) use the same array and race: serialise them.
#include <cuda_runtime.h>
#include <stdio.h>

#include <mutex>

#include "tann_common.cuh"
#include "tann_launch.h"
#include "topoanns_b200.h"

namespace tann {
void SetLastError(const char* message);  // capi.cu
}

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[TANN_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_scratch_addr[kMaxDevices] = {};

TannStatus StaticFail(TannStatus st, const char* message) {
    tann::SetLastError(message);
    return st;
}

// Address of the array on the current device; looked up once per device.
TannStatus ScratchForCurrentDevice(unsigned char** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return StaticFail(TANN_ERR_CUDA, cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices)
        return StaticFail(TANN_ERR_UNSUPPORTED, "tann_rerank_topk_static: device ordinal out of range.");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            char msg[256];
            snprintf(msg, sizeof(msg), "tann_rerank_topk_static: cudaGetSymbolAddress: %s",
                     cudaGetErrorString(e));
            return StaticFail(TANN_ERR_CUDA, msg);
        }
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return TANN_OK;
}

size_t Align256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

extern "C" TannStatus tann_rerank_topk_static(const TannIndexView* index, const TannRerankParams* params,
                                              const void* candidates, uint32_t candidate_capacity,
                                              uint64_t num_queries, const void* queries, uint32_t query_kind,
                                              const float* error_bounds, float* out_dists, uint32_t* out_ids,
                                              tann_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!index || !params) return StaticFail(TANN_ERR_INVALID_ARGUMENT, "tann_rerank_topk_static: null index or params.");
    if (num_queries == 0 || params->top_k == 0) return TANN_OK;
    if (!candidates || !queries || !out_dists || !out_ids || query_kind > TANN_KIND_FLOAT32)
        return StaticFail(TANN_ERR_INVALID_ARGUMENT, "tann_rerank_topk_static: null pointer or unknown query kind.");
    if (params->top_n == 0) return StaticFail(TANN_ERR_UNSUPPORTED, "tann_rerank_topk_static: top_n must be 1..2048.");
    // the rules of tann_rerank_exact (vector store, top_n, bound filter, early stop, shard coverage)
    TannStatus st = tann::CheckRerank("tann_rerank_topk_static", index, params, error_bounds);
    if (st != TANN_OK) return st;
    if (params->top_k > params->top_n)
        return StaticFail(TANN_ERR_INVALID_ARGUMENT, "tann_rerank_topk_static: need top_k <= top_n.");
    // bounds the products below well inside size_t before they are formed
    if (num_queries > (uint64_t)TANN_STATIC_SCRATCH_BYTES || index->dim > (uint32_t)TANN_STATIC_SCRATCH_BYTES)
        return StaticFail(TANN_ERR_UNSUPPORTED,
                          "tann_rerank_topk_static: batch is larger than the static work space; split the batch or use "
                          "tann_rerank_exact.");
    const bool u8_copy = query_kind == TANN_KIND_FLOAT32 && index->vector_kind == TANN_KIND_UINT8 &&
                         !params->use_bound_filter;
    const size_t flag_bytes = 256;
    const size_t q8_bytes = u8_copy ? Align256((size_t)num_queries * index->dim) : 0;
    const size_t list_bytes = Align256((size_t)num_queries * params->top_n * 4);
    const size_t need = flag_bytes + q8_bytes + 2 * list_bytes;
    if (need > (size_t)TANN_STATIC_SCRATCH_BYTES) {
        char msg[256];
        snprintf(msg, sizeof(msg),
                 "tann_rerank_topk_static: batch needs %zu bytes of work space, the static area holds %zu; "
                 "split the batch or use tann_rerank_exact.", need, (size_t)TANN_STATIC_SCRATCH_BYTES);
        return StaticFail(TANN_ERR_UNSUPPORTED, msg);
    }
    unsigned char* scratch = nullptr;
    st = ScratchForCurrentDevice(&scratch);
    if (st != TANN_OK) return st;
    uint32_t* flag = reinterpret_cast<uint32_t*>(scratch);
    uint8_t* q8 = scratch + flag_bytes;
    float* list_dists = reinterpret_cast<float*>(scratch + flag_bytes + q8_bytes);
    uint32_t* list_ids = reinterpret_cast<uint32_t*>(scratch + flag_bytes + q8_bytes + list_bytes);
    cudaError_t e;
    if (u8_copy) {
        // clears the flag (it must start at zero), then converts and checks the queries
        e = tann::LaunchF32ToU8Checked(static_cast<const float*>(queries), num_queries * index->dim, q8, flag, stream);
        if (e != cudaSuccess) return StaticFail(TANN_ERR_CUDA, cudaGetErrorString(e));
    }
    e = tann::LaunchRerank(*index, *params, candidates, candidate_capacity, num_queries, queries, query_kind,
                           error_bounds, list_dists, list_ids, nullptr, stream, u8_copy ? q8 : nullptr,
                           u8_copy ? flag : nullptr);
    if (e != cudaSuccess) return StaticFail(TANN_ERR_CUDA, cudaGetErrorString(e));
    e = tann::LaunchTopkPack(list_dists, list_ids, num_queries, params->top_n, params->top_k, out_dists, out_ids, stream);
    if (e != cudaSuccess) return StaticFail(TANN_ERR_CUDA, cudaGetErrorString(e));
    return TANN_OK;
}
