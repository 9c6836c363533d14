"""Whole path on the CPU checker, for parity tests and the timed CPU baseline.

TEST INFRASTRUCTURE ONLY (see oracle.py). Inputs are numpy arrays in the same layouts the device
path uses; stages are the checker's restatements chained the way the reference chains them
(src/search/topoanns_search.cpp:54-270).
"""
from __future__ import annotations

import time

import numpy as np

from . import oracle as orc


def vectors_to_pages(vectors: np.ndarray, page_bytes: int = 4096):
    v = np.ascontiguousarray(vectors)
    n = v.shape[0]
    vb = v.shape[1] * v.dtype.itemsize
    vpp = page_bytes // vb
    pages = np.zeros(((n + vpp - 1) // vpp, page_bytes), np.uint8)
    raw = v.view(np.uint8).reshape(n, vb)
    full = (n // vpp) * vpp
    if full:
        pages[: n // vpp, : vpp * vb] = raw[:full].reshape(n // vpp, vpp * vb)
    if n > full:
        pages[n // vpp, : (n - full) * vb] = raw[full:].reshape(-1)
    return pages.reshape(-1), vpp, vb


def run(index: dict, queries: np.ndarray, *, top_l, search_width, max_expansions, top_n, top_k,
        entry_count=0, fixed_entries=None, use_pq2=False, refine_top_l=0, bound_filter=False, tile=0,
        learned_stop=None, two_phase=True, timings=None, early_stop=None):
    """index: dict with adjacency [N,deg] u32, codes [N,M] u8, pq_tables [256,d], pq_centroid,
    pq_chunk_offsets, vectors [N,d], and optionally rvq_* / pq2_* arrays. Returns a dict."""
    t0 = time.perf_counter()
    Q = queries.shape[0]
    qf = np.ascontiguousarray(queries, np.float32) if queries.dtype != np.float32 else queries
    if fixed_entries is not None:
        fe = np.asarray(fixed_entries, np.uint32)
        entry_ids = np.tile(fe, Q)
        entry_offsets = np.arange(Q + 1, dtype=np.uint32) * fe.size
        clusters = None
    else:
        clusters, _, _ = orc.rvq_clusters(qf, index["rvq_coarse"], index["rvq_fine"], index["rvq_sizes"])
        entry_ids = orc.rvq_gather(clusters, index["rvq_offsets"], index["rvq_ids"], entry_count).reshape(-1)
        entry_offsets = np.arange(Q + 1, dtype=np.uint32) * entry_count
    t1 = time.perf_counter()
    lut = orc.lut_build(queries, index["pq_tables"], index["pq_centroid"], index["pq_chunk_offsets"])
    t2 = time.perf_counter()
    cap = orc.candidate_capacity(top_l, 0, top_n)
    cand, stats = orc.beam_search(index["adjacency"], index["codes"], lut, entry_offsets, entry_ids,
                                  top_l=top_l, search_width=search_width, max_expansions=max_expansions,
                                  capacity=cap, learned_stop=learned_stop, two_phase=two_phase)
    t3 = time.perf_counter()
    src = cand
    err = None
    if use_pq2:
        lr = min(refine_top_l or cap, cap)
        lut2 = orc.lut_build(qf, index["pq2_tables"], index["pq2_centroid"], index["pq_chunk_offsets"])
        residual = index.get("pq2_cross") is not None
        src = orc.pq2_refine(cand, stats, lr, index["pq2_codes"], lut2,
                             index["codes"] if residual else None, index.get("pq2_cross"))
        if bound_filter:
            err = index["pq2_error_bounds"]
    pages = index.get("pages")
    if pages is None:
        pages, vpp, vb = vectors_to_pages(index["vectors"])
        index["pages"], index["vpp"], index["vb"] = pages, vpp, vb
    dists, ids, n_exact, n_filt = orc.rerank(src, queries, pages, index["vectors"].dtype, top_n=top_n,
                                             top_k=top_k, tile=tile, vectors_per_page=index["vpp"],
                                             page_bytes=4096, vector_bytes=index["vb"], error_bounds=err,
                                             early_stop_min_prefix=early_stop[0] if early_stop else 0,
                                             early_stop_patience_tiles=early_stop[1] if early_stop else 0)
    t4 = time.perf_counter()
    if timings is not None:
        timings.update(entries=t1 - t0, lut=t2 - t1, beam=t3 - t2, rerank=t4 - t3, total=t4 - t0)
    return dict(clusters=clusters, entry_ids=entry_ids, entry_offsets=entry_offsets, lut=lut, cand=cand,
                stats=stats, refined=src if use_pq2 else None, dists=dists, ids=ids, n_exact=n_exact,
                n_filtered=n_filt, topk_ids=ids[:, :top_k], topk_dists=dists[:, :top_k])


def index_from_synth(s) -> dict:
    """numpy view of a topoanns_b200.synth.SynthIndex."""
    def n(t):
        return None if t is None else t.detach().cpu().numpy()
    d = dict(adjacency=n(s.adjacency).view(np.uint32), codes=n(s.pq_codes), pq_tables=n(s.pq_tables),
             pq_centroid=n(s.pq_centroid), pq_chunk_offsets=n(s.pq_chunk_offsets).astype(np.uint32),
             vectors=n(s.vectors))
    if s.rvq_coarse is not None:
        d.update(rvq_coarse=n(s.rvq_coarse), rvq_fine=n(s.rvq_fine), rvq_sizes=n(s.rvq_buckets[0]),
                 rvq_offsets=n(s.rvq_buckets[1]).astype(np.uint32), rvq_ids=n(s.rvq_buckets[2]).astype(np.uint32))
    if s.pq2_tables is not None:
        d.update(pq2_tables=n(s.pq2_tables), pq2_centroid=n(s.pq2_centroid), pq2_codes=n(s.pq2_codes),
                 pq2_error_bounds=n(s.pq2_error_bounds))
        d["pq2_cross"] = orc.pq2_cross_terms(d["pq_chunk_offsets"], d["pq_tables"], d["pq_centroid"],
                                             d["pq2_tables"], d["pq2_centroid"])
    return d
