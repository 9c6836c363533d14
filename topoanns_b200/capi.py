"""ctypes binding of ``libtopoanns_b200.so`` (declared in ``include/topoanns_b200.h``).

The library is the product; this module only loads it and mirrors its structs. There is no
fallback: if the shared library is missing or a call returns a non-zero status, an exception is
raised.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtopoanns_b200.so")

MAX_SHARDS = 8
KIND_INT8, KIND_UINT8, KIND_FLOAT32 = 0, 1, 2
INVALID_NODE = 0xFFFFFFFF
IPC_HANDLE_BYTES = 64


class TannError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[status {status}] {message}")
        self.status = status
        self.message = message


class Shards(C.Structure):
    _fields_ = [("num_shards", C.c_uint32), ("reserved", C.c_uint32), ("rows_per_shard", C.c_uint64),
                ("base", C.c_void_p * MAX_SHARDS)]


class IndexView(C.Structure):
    _fields_ = [
        ("num_nodes", C.c_uint64), ("degree", C.c_uint32), ("num_chunks", C.c_uint32),
        ("dim", C.c_uint32), ("vector_kind", C.c_uint32), ("vector_bytes", C.c_uint64),
        ("vectors_per_page", C.c_uint64), ("page_bytes", C.c_uint64), ("adjacency", Shards),
        ("codes", Shards), ("vectors", Shards), ("adjacency_cache", C.c_void_p),
        ("adjacency_cached_rows", C.c_uint64), ("pq_tables_col_major", C.c_void_p),
        ("pq_centroid", C.c_void_p), ("pq_chunk_offsets", C.c_void_p), ("neighbor_codes", Shards),
    ]


class LearnedStop(C.Structure):
    _fields_ = [
        ("enabled", C.c_uint32), ("num_stages", C.c_uint32), ("top_k", C.c_uint32),
        ("shadow_mode", C.c_uint32), ("topk_churn_flag_mode", C.c_uint32),
        ("next64_flag_mode", C.c_uint32), ("stage_prefixes", C.c_uint32 * 32),
        ("feature_mask", C.c_uint32 * 12), ("weights", C.c_float * 12), ("bias", C.c_float),
        ("threshold_logit", C.c_float), ("inv_top_l", C.c_float),
    ]


class BeamParams(C.Structure):
    _fields_ = [
        ("top_l", C.c_uint32), ("search_width", C.c_uint32), ("max_expansions", C.c_uint32),
        ("candidate_capacity", C.c_uint32), ("stop_prefix", C.c_uint32),
        ("stop_use_expanded", C.c_uint32), ("reserved0", C.c_uint32), ("reserved1", C.c_uint32),
        ("learned_stop", LearnedStop),
    ]


class RerankParams(C.Structure):
    _fields_ = [("top_n", C.c_uint32), ("top_k", C.c_uint32), ("tile", C.c_uint32),
                ("use_bound_filter", C.c_uint32), ("use_early_stop", C.c_uint32),
                ("early_stop_min_prefix", C.c_uint32), ("early_stop_patience_tiles", C.c_uint32),
                ("reserved", C.c_uint32)]


class RerankLearnedStop(C.Structure):
    """TannRerankLearnedStop: the folded learned rerank-stop model and its stage schedule."""
    _fields_ = [("enabled", C.c_uint32), ("feature_variant", C.c_uint32), ("num_stages", C.c_uint32),
                ("top_k", C.c_uint32), ("bootstrap_prefix", C.c_uint32), ("initial_stage_index", C.c_uint32),
                ("stage_prefixes", C.c_uint32 * 64), ("linear_weights", C.c_float * 13), ("bias", C.c_float),
                ("threshold_logit", C.c_float), ("budget_log2", C.c_float), ("inv_budget_top_n", C.c_float),
                ("inv_top_k", C.c_float)]


class RvqModelView(C.Structure):
    _fields_ = [
        ("dim", C.c_uint32), ("num_coarse", C.c_uint32), ("num_fine", C.c_uint32),
        ("entry_count", C.c_uint32), ("fallback_entry", C.c_uint32), ("reserved", C.c_uint32),
        ("coarse", C.c_void_p), ("coarse_t", C.c_void_p), ("coarse_norms", C.c_void_p),
        ("fine_t", C.c_void_p), ("fine_norms", C.c_void_p), ("bucket_sizes", C.c_void_p),
        ("cluster_offsets", C.c_void_p), ("cluster_ids", C.c_void_p),
    ]


class Pq2View(C.Structure):
    _fields_ = [
        ("enabled", C.c_uint32), ("residual", C.c_uint32), ("refine_top_l", C.c_uint32),
        ("reserved", C.c_uint32), ("codes", Shards), ("tables_col_major", C.c_void_p),
        ("centroid", C.c_void_p), ("chunk_offsets", C.c_void_p), ("cross_terms", C.c_void_p),
        ("error_bounds", C.c_void_p),
    ]


# Every symbol include/topoanns_b200.h declares, with its argument types.
_VP, _U32, _U64, _I = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int
SIGNATURES = {
    "tann_version": (C.c_char_p, []),
    "tann_last_error": (C.c_char_p, []),
    "tann_lut_build": (_I, [_VP, _VP, _VP, _U32, _U32, _VP, _U32, _U64, _VP, _VP]),
    "tann_beam_search": (_I, [C.POINTER(IndexView), C.POINTER(BeamParams), _VP, _VP, _U32, _U64, _VP,
                              _VP, _VP, _VP, _VP, _VP]),
    "tann_beam_search_occupancy": (_I, [C.POINTER(IndexView), C.POINTER(BeamParams), _I,
                                        C.POINTER(_U32), C.POINTER(_U32), C.POINTER(_U32)]),
    "tann_rvq_norms": (_I, [_VP, _U32, _U32, _VP, _VP]),
    "tann_rvq_entries": (_I, [_VP, _U64, _U32, _VP, _VP, _VP, _U32, _VP, _VP, _U32, _VP, _VP, _VP, _U32,
                              _U32, _VP, _VP, _VP, _VP]),
    "tann_pq2_refine": (_I, [_VP, _VP, _U64, _U32, _U32, C.POINTER(Shards), C.POINTER(Shards), _U32, _VP,
                             _VP, _VP, _VP, _VP]),
    "tann_hpq_refine": (_I, [_VP, _VP, _U64, _U32, _U32, C.POINTER(Shards), _VP, _U32, _VP, _VP, _VP, _VP, _VP]),
    "tann_pq2_cross_terms": (_I, [_U32, _U32, _VP, _VP, _VP, _VP, _VP, _VP, _VP]),
    "tann_rerank_exact": (_I, [C.POINTER(IndexView), C.POINTER(RerankParams), _VP, _U32, _U64, _VP, _U32,
                               _VP, _VP, _VP, _VP, _VP, _VP]),
    "tann_rerank_learned_stop_load": (_I, [C.c_char_p, _U32, _U32, C.POINTER(RerankLearnedStop)]),
    "tann_rerank_exact_learned_stop": (_I, [C.POINTER(IndexView), C.POINTER(RerankParams),
                                            C.POINTER(RerankLearnedStop), _VP, _U32, _U64, _VP, _U32, _VP, _VP,
                                            _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP]),
    "tann_topk_pack": (_I, [_VP, _VP, _U64, _U32, _U32, _VP, _VP, _VP]),
    "tann_partition_candidates": (_I, [_VP, _U32, _U32, _U64, _U64, _U32, _U32, _VP, _VP, _VP]),
    "tann_merge_topk_lists": (_I, [_VP, _VP, _U32, _U64, _U32, _U64, _VP, _VP, _VP]),
    "tann_rerank_topk_static": (_I, [C.POINTER(IndexView), C.POINTER(RerankParams), _VP, _U32, _U64, _VP, _U32,
                                     _VP, _VP, _VP, _VP]),
    "tann_neighbor_codes_build": (_I, [C.POINTER(IndexView), _U64, _U64, _VP, _VP]),
    "tann_device_alloc": (_I, [_U64, C.POINTER(_VP)]),
    "tann_device_free": (_I, [_VP]),
    "tann_host_alloc_mapped": (_I, [_U64, C.POINTER(_VP), C.POINTER(_VP)]),
    "tann_host_free": (_I, [_VP]),
    "tann_ipc_export": (_I, [_VP, C.c_char_p]),
    "tann_ipc_open": (_I, [C.c_char_p, C.POINTER(_VP)]),
    "tann_ipc_close": (_I, [_VP]),
    "tann_enable_peer_access": (_I, [_I]),
    "tann_searcher_create": (_I, [C.POINTER(IndexView), _U64, _U32, _U32, _U32, C.POINTER(_VP)]),
    "tann_searcher_set_rvq": (_I, [_VP, C.POINTER(RvqModelView)]),
    "tann_searcher_set_pq2": (_I, [_VP, C.POINTER(Pq2View)]),
    "tann_searcher_run": (_I, [_VP, C.POINTER(BeamParams), C.POINTER(RerankParams), _VP, _U32, _U64, _VP,
                               _U32, _VP, _VP, _VP, _VP]),
    "tann_searcher_set_rerank_learned_stop": (_I, [_VP, C.POINTER(RerankLearnedStop)]),
    "tann_searcher_submit": (_I, [_VP, C.POINTER(BeamParams), C.POINTER(RerankParams), _VP, _U32, _U64, _VP,
                                  _U32, _VP, _VP, _VP, _VP]),
    "tann_searcher_wait": (_I, [_VP]),
    "tann_searcher_run_device": (_I, [_VP, C.POINTER(BeamParams), C.POINTER(RerankParams), _VP, _U32, _U64,
                                      _VP, _VP, C.POINTER(_VP), C.POINTER(_VP), C.POINTER(_VP), _VP]),
    "tann_searcher_destroy": (_I, [_VP]),
    "tann_searcher_status_device": (_I, [_VP, C.POINTER(_VP)]),
    "tann_dependent_load_ns": (_I, [_VP, _U64, _U32, C.POINTER(C.c_float), _VP]),
}

_lib = None


def load():
    """Load the shared library and bind every declared symbol (raises if anything is missing)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `make -C topoanns_b200/csrc` "
                "(or __graft_entry__.build()); there is no CPU fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise TannError(status, load().tann_last_error().decode("utf-8", "replace"))


def next_pow2(v: int) -> int:
    p = 1
    while p < v:
        p <<= 1
    return p


def candidate_capacity(top_l: int, candidate_queue_size: int = 0, rerank_top_n: int = 0) -> int:
    """C = nextpow2(max(top_l, candidate_queue_size, rerank top_n)); reference
    src/search/topoanns_search.cpp:77-81 and src/search/topology_search_kernel.cu:3207-3210."""
    return next_pow2(max(top_l, candidate_queue_size, rerank_top_n))
