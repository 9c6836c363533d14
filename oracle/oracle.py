"""ctypes front end of the CPU checker (``libtann_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the benchmark's
CPU-baseline leg. The product package never imports this module.

All arrays are numpy, C-contiguous. Candidate lists are ``uint32`` arrays of shape
``[Q, C, 2]``: word 0 holds the float32 distance bits, word 1 the packed node id (bit 31 =
expanded, ``0xffffffff`` = invalid), which is the 8-byte record of the reference
(src/search/topology_search_kernel.hpp:37-54).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtann_oracle.so")
INVALID = 0xFFFFFFFF
KIND = {"int8": 0, "uint8": 1, "float32": 2}


def build(force: bool = False) -> str:
    """Compile the restatement with the Makefile beside it (g++ only)."""
    src = os.path.join(_HERE, "tann_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libtann_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


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
        ("num_nodes", C.c_uint64), ("degree", C.c_uint32), ("num_chunks", C.c_uint32),
        ("top_l", C.c_uint32), ("search_width", C.c_uint32), ("max_expansions", C.c_uint32),
        ("candidate_capacity", C.c_uint32), ("stop_prefix", C.c_uint32),
        ("stop_use_expanded", C.c_uint32), ("two_phase", C.c_uint32), ("reserved", C.c_uint32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_adc_serial.restype = C.c_float
        _lib.orc_adc_tree.restype = C.c_float
        _lib.orc_exact_distance.restype = C.c_float
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def next_pow2(v: int) -> int:
    p = 1
    while p < v:
        p <<= 1
    return p


def kind_of(a: np.ndarray) -> int:
    return KIND[str(a.dtype)]


def lut_build(queries, tables_row_major, centroid, chunk_offsets):
    q = np.ascontiguousarray(queries)
    Q, d = q.shape
    M = len(chunk_offsets) - 1
    out = np.empty((Q, M, 256), np.float32)
    lib().orc_lut_build(_p(q), kind_of(q), C.c_uint64(Q), C.c_uint32(d), C.c_uint32(M),
                        _p(_c(tables_row_major, np.float32)), _p(_c(centroid, np.float32)),
                        _p(_c(chunk_offsets, np.uint32)), _p(out))
    return out


def adc_serial(lut_q, codes_row):
    lut_q = _c(lut_q, np.float32)
    codes_row = _c(codes_row, np.uint8)
    return float(lib().orc_adc_serial(_p(lut_q), _p(codes_row), C.c_uint32(len(codes_row))))


def adc_tree(lut_q, codes_row):
    lut_q = _c(lut_q, np.float32)
    codes_row = _c(codes_row, np.uint8)
    return float(lib().orc_adc_tree(_p(lut_q), _p(codes_row), C.c_uint32(len(codes_row))))


def candidate_capacity(top_l: int, candidate_queue_size: int = 0, rerank_top_n: int = 0) -> int:
    """src/search/topoanns_search.cpp:77-81 and topology_search_kernel.cu:3207-3210."""
    cqs = max(top_l, candidate_queue_size, rerank_top_n)
    return next_pow2(max(top_l, cqs))


def beam_search(adjacency, codes, lut, entry_offsets, entry_ids, *, top_l, search_width,
                max_expansions, capacity=None, learned_stop=None, two_phase=True,
                stop_prefix=None, stop_use_expanded=False):
    adjacency = _c(adjacency, np.uint32)
    codes = _c(codes, np.uint8)
    lut = _c(lut, np.float32)
    N, deg = adjacency.shape
    Q = len(entry_offsets) - 1
    M = codes.shape[1]
    if capacity is None:
        capacity = candidate_capacity(top_l)
    P = BeamParams(N, deg, M, top_l, search_width, max_expansions, capacity,
                   top_l if stop_prefix is None else stop_prefix, int(stop_use_expanded),
                   int(two_phase), 0)
    cand = np.empty((Q, capacity, 2), np.uint32)
    stats = np.empty((Q, 8), np.uint32)
    stride = 0 if lut.ndim == 2 else M * 256
    lib().orc_beam_search(C.byref(P), C.byref(learned_stop) if learned_stop is not None else None,
                          _p(adjacency), _p(codes), _p(lut), C.c_uint64(stride), C.c_uint64(Q),
                          _p(_c(entry_offsets, np.uint32)), _p(_c(entry_ids, np.uint32)),
                          _p(cand), _p(stats))
    return cand, stats


def rvq_clusters(queries, coarse, fine, bucket_sizes):
    q = _c(queries, np.float32)
    Q, d = q.shape
    out = np.empty(Q, np.int32)
    cs = np.empty(Q, np.float32)
    fs = np.empty(Q, np.float32)
    lib().orc_rvq_clusters(_p(q), C.c_uint64(Q), C.c_uint32(d), _p(_c(coarse, np.float32)),
                           C.c_uint32(len(coarse)), _p(_c(fine, np.float32)), C.c_uint32(len(fine)),
                           _p(_c(bucket_sizes, np.int32)), _p(out), _p(cs), _p(fs))
    return out, cs, fs


def rvq_gather(clusters, cluster_offsets, cluster_ids, entry_count, fallback_entry=0):
    clusters = _c(clusters, np.int32)
    out = np.empty((len(clusters), entry_count), np.uint32)
    lib().orc_rvq_gather(_p(clusters), C.c_uint64(len(clusters)), _p(_c(cluster_offsets, np.uint32)),
                         _p(_c(cluster_ids, np.uint32)), C.c_uint32(entry_count),
                         C.c_uint32(fallback_entry), _p(out))
    return out


def pq2_cross_terms(chunk_offsets, t1, mu1, t2, mu2):
    t1 = _c(t1, np.float32)
    d = t1.shape[1]
    M = len(chunk_offsets) - 1
    out = np.empty((M, 256, 256), np.float32)
    lib().orc_pq2_cross_terms(C.c_uint32(d), C.c_uint32(M), _p(_c(chunk_offsets, np.uint32)), _p(t1),
                              _p(_c(mu1, np.float32)), _p(_c(t2, np.float32)),
                              _p(_c(mu2, np.float32)), _p(out))
    return out


def pq2_refine(cand, stats, refine_top_l, pq2_codes, lut2, base_codes=None, cross_terms=None):
    cand = _c(cand, np.uint32)
    Q, capacity, _ = cand.shape
    pq2_codes = _c(pq2_codes, np.uint8)
    M = pq2_codes.shape[1]
    out = np.empty((Q, refine_top_l, 2), np.uint32)
    lib().orc_pq2_refine(_p(cand), _p(_c(stats, np.uint32)), C.c_uint64(Q), C.c_uint32(capacity),
                         C.c_uint32(refine_top_l),
                         _p(_c(base_codes, np.uint8)) if base_codes is not None else None,
                         _p(pq2_codes), C.c_uint32(M), _p(_c(lut2, np.float32)),
                         _p(_c(cross_terms, np.float32)) if cross_terms is not None else None, _p(out))
    return out


def hpq_refine(cand, stats, refine_top_l, hybrid_codes, selector_bits, base_lut, outlier_lut):
    """Hybrid-PQ refine (src/search/rerank_exact.cu:667-771). Returns [Q, refine_top_l, 2] uint32 records."""
    cand = _c(cand, np.uint32)
    stats = _c(stats, np.uint32)
    Q, capacity, _ = cand.shape
    codes = _c(hybrid_codes, np.uint8)
    M = codes.shape[1]
    sel = _c(selector_bits, np.uint8)
    assert sel.shape == (codes.shape[0], (M + 7) // 8)
    out = np.empty((Q, refine_top_l, 2), np.uint32)
    lib().orc_hpq_refine(_p(cand), _p(stats), C.c_uint64(Q), C.c_uint32(capacity), C.c_uint32(refine_top_l), _p(codes),
                         _p(sel), C.c_uint32(M), _p(_c(base_lut, np.float32)), _p(_c(outlier_lut, np.float32)), _p(out))
    return out


def exact_distance(query, vec):
    query = np.ascontiguousarray(query)
    vec = np.ascontiguousarray(vec)
    return float(lib().orc_exact_distance(_p(query), kind_of(query), _p(vec), kind_of(vec),
                                          C.c_uint32(len(query))))


def rerank(cand, queries, vector_pages, vec_dtype, *, top_n, top_k, tile=0, vectors_per_page,
           page_bytes, vector_bytes, error_bounds=None, early_stop_min_prefix=0, early_stop_patience_tiles=0):
    """Returns (dists [Q, top_n] f32, ids [Q, top_n] u32, n_exact, n_filtered).
    early_stop_patience_tiles > 0 switches the persistent rerank's early stop on."""
    cand = _c(cand, np.uint32)
    Q, capacity, _ = cand.shape
    queries = np.ascontiguousarray(queries)
    d = queries.shape[1]
    pages = _c(vector_pages, np.uint8)
    dists = np.empty((Q, top_n), np.float32)
    ids = np.empty((Q, top_n), np.uint32)
    counts = np.zeros(2, np.uint64)
    lib().orc_rerank(_p(cand), C.c_uint64(Q), C.c_uint32(capacity), C.c_uint32(top_n),
                     C.c_uint32(top_k), C.c_uint32(tile), _p(queries), kind_of(queries),
                     C.c_uint32(d), _p(pages), KIND[np.dtype(vec_dtype).name],
                     C.c_uint64(vectors_per_page), C.c_uint64(page_bytes), C.c_uint64(vector_bytes),
                     1 if error_bounds is not None else 0,
                     _p(_c(error_bounds, np.float32)) if error_bounds is not None else None,
                     _p(dists), _p(ids), _p(counts), C.c_uint32(early_stop_min_prefix),
                     C.c_uint32(early_stop_patience_tiles))
    return dists, ids, int(counts[0]), int(counts[1])


# ----- learned rerank stop (src/io/bam_vector_provider.cu) -----------------------------------

class RerankStop(C.Structure):
    """DeviceRerankLearnedStopConfig, src/io/bam_vector_provider.cu:65-79."""
    _fields_ = [("enabled", C.c_uint32), ("feature_variant", C.c_uint32), ("num_stages", C.c_uint32),
                ("top_k", C.c_uint32), ("bootstrap_prefix", C.c_uint32), ("initial_stage_index", C.c_uint32),
                ("stage_prefixes", C.c_uint32 * 64), ("linear_weights", C.c_float * 13), ("bias", C.c_float),
                ("threshold_logit", C.c_float), ("budget_log2", C.c_float), ("inv_budget_top_n", C.c_float),
                ("inv_top_k", C.c_float)]


def load_rerank_stop_model(path, budget_top_n, top_k):
    """LoadRerankLearnedStopConfigFromFile, src/io/bam_vector_provider.cu:125-279, in float32 steps."""
    f32 = np.float32
    lists, scalars, per_budget = {}, {}, {}
    with open(path) as fh:
        for raw in fh:
            line = raw.strip()
            if not line or line.startswith("#"):
                continue
            if "=" not in line:
                raise ValueError("Invalid learned-stop config line: " + line)
            key, value = (t.strip() for t in line.split("=", 1))
            if key in ("stage_prefixes", "feature_mask"):
                lists[key] = [int(t) for t in (u.strip() for u in value.split(",")) if t]
            elif key in ("feature_means", "feature_inv_stds", "weights"):
                lists[key] = [f32(t) for t in (u.strip() for u in value.split(",")) if t]
            elif key in ("bias", "threshold_logit"):
                scalars[key] = f32(value)
            elif key in ("top_k", "bootstrap_prefix"):
                scalars[key] = int(value)
            elif key.startswith("threshold_logit_top_l_") and key[len("threshold_logit_top_l_"):]:
                per_budget.setdefault(int(key[len("threshold_logit_top_l_"):]), f32(value))
    means, stds, weights = (lists.get(k, []) for k in ("feature_means", "feature_inv_stds", "weights"))
    mask = lists.get("feature_mask", [])
    n = len(weights)
    if n not in (12, 13) or len(means) != n or len(stds) != n:
        raise ValueError("learned-stop feature vectors must all have length 13 or 12.")
    if mask and len(mask) != n:
        raise ValueError("feature_mask must have length %d." % n)
    c = RerankStop()
    if n == 13 and mask == [1, 1, 1, 0, 0, 1, 0, 1, 0, 1, 0, 0, 0]:
        c.feature_variant = 1
    c.top_k = scalars.get("top_k", 0) or top_k
    c.bootstrap_prefix = scalars.get("bootstrap_prefix", 0)
    c.threshold_logit = per_budget.get(budget_top_n, scalars.get("threshold_logit", f32(0)))
    c.budget_log2 = f32(np.log2(max(f32(1), f32(budget_top_n)), dtype=f32))
    c.inv_budget_top_n = f32(0) if budget_top_n == 0 else f32(1) / f32(budget_top_n)
    c.inv_top_k = f32(0) if c.top_k == 0 else f32(1) / f32(c.top_k)
    bias = f32(scalars.get("bias", f32(0)))
    for src in range(n):
        dst = src + 1 if (n == 12 and src >= 5) else src   # the older single churn ratio is feature 6 now
        w = weights[src] if (not mask or mask[src] != 0) else f32(0)
        folded = f32(w * stds[src])
        c.linear_weights[dst] = folded
        bias = f32(bias - f32(means[src] * folded))
    c.bias = bias
    for prefix in lists.get("stage_prefixes", []):
        if prefix == 0 or prefix > budget_top_n:
            continue
        if c.num_stages >= 64:
            break
        c.stage_prefixes[c.num_stages] = prefix
        c.num_stages += 1
    while c.initial_stage_index < c.num_stages and c.stage_prefixes[c.initial_stage_index] <= c.bootstrap_prefix:
        c.initial_stage_index += 1
    c.enabled = 0 if (c.num_stages == 0 or c.bootstrap_prefix == 0) else 1
    if c.top_k == 0 or c.top_k > 128:
        c.enabled = 0
    return c


def rerank_learned(cand, queries, vector_pages, vec_dtype, *, top_n, top_k, tile, vectors_per_page, page_bytes,
                   vector_bytes, model=None, replay=None, error_bounds=None, use_early_stop=False,
                   early_stop_min_prefix=0, early_stop_patience_tiles=0):
    """Persistent rerank with the learned stop. Returns a dict: dists / ids [Q, top_k], stop_prefixes,
    checkpoint_counts, stop_flags [Q], n_exact, n_filtered."""
    cand = _c(cand, np.uint32)
    Q, capacity, _ = cand.shape
    queries = np.ascontiguousarray(queries)
    pages = _c(vector_pages, np.uint8)
    dists = np.empty((Q, top_k), np.float32)
    ids = np.empty((Q, top_k), np.uint32)
    counts = np.zeros(2, np.uint64)
    stop_prefixes = np.zeros(Q, np.uint32)
    checkpoints = np.zeros(Q, np.uint32)
    flags = np.zeros(Q, np.uint32)
    replay_arr = _c(replay, np.uint32) if replay is not None else None
    lib().orc_rerank_learned(
        _p(cand), C.c_uint64(Q), C.c_uint32(capacity), C.c_uint32(top_n), C.c_uint32(top_k), C.c_uint32(tile),
        _p(queries), kind_of(queries), C.c_uint32(queries.shape[1]), _p(pages), KIND[np.dtype(vec_dtype).name],
        C.c_uint64(vectors_per_page), C.c_uint64(page_bytes), C.c_uint64(vector_bytes),
        1 if error_bounds is not None else 0,
        _p(_c(error_bounds, np.float32)) if error_bounds is not None else None,
        C.byref(model) if model is not None else None, _p(replay_arr) if replay_arr is not None else None,
        1 if use_early_stop else 0, C.c_uint32(early_stop_min_prefix), C.c_uint32(early_stop_patience_tiles),
        _p(dists), _p(ids), _p(counts), _p(stop_prefixes), _p(checkpoints), _p(flags))
    return dict(dists=dists, ids=ids, stop_prefixes=stop_prefixes, checkpoint_counts=checkpoints, stop_flags=flags,
                n_exact=int(counts[0]), n_filtered=int(counts[1]))


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


# ----- small helpers shared by the tests -----------------------------------------------------

def cand_dist(cand):
    return cand[..., 0].view(np.float32)


def cand_raw_id(cand):
    ids = cand[..., 1]
    return np.where(ids == INVALID, INVALID, ids & 0x7FFFFFFF).astype(np.uint32)


def cand_expanded(cand):
    ids = cand[..., 1]
    return (ids != INVALID) & ((ids & 0x80000000) != 0)
