"""Frequency-ordered relabelling for the tiered topology: node ids are renumbered so that the most often expanded
nodes get the smallest ids. The beam kernel serves adjacency rows with id < `adjacency_cached_rows` from HBM and the
rest from the slower tier (pinned host memory or a peer GPU); the reference's id-prefix cache
(`topology_cached_node_count`, include/topoanns/topology_search.hpp:17-32, src/search/topology_search_kernel.cu:551-609)
has the same prefix semantics, so "cache the hot nodes" becomes "cache a prefix" once the ids are ordered by heat.

All functions work on host arrays in the file layouts (adjacency [N, degree] uint32 with 0xffffffff padding, per-node
rows of codes / vectors / error bounds, RVQ posting ids)."""
from __future__ import annotations

import numpy as np

INVALID = 0xFFFFFFFF
EXPANDED_BIT = 0x80000000


def expansion_counts(candidates: np.ndarray, num_nodes: int, counts: np.ndarray | None = None) -> np.ndarray:
    """Adds, per node, how many of the candidate records [Q, capacity, 2] (uint32: distance bits, packed id) carry
    the expanded flag. Nodes expanded and later pushed out of a list are not seen; with list sizes >= top_l they are few."""
    ids = np.ascontiguousarray(candidates)[..., 1].reshape(-1)
    hot = ids[(ids != INVALID) & ((ids & EXPANDED_BIT) != 0)] & ~np.uint32(EXPANDED_BIT)
    out = np.zeros(num_nodes, np.int64) if counts is None else counts
    np.add.at(out, hot[hot < num_nodes], 1)
    return out


def frequency_permutation(counts: np.ndarray, pinned_first=()):
    """Returns (new_id_of_old [N], old_id_of_new [N]): ids by descending count, ties by old id (stable);
    `pinned_first` (e.g. the medoid and fixed entry nodes) come before everything else."""
    n = counts.shape[0]
    key = counts.astype(np.int64).copy()
    if len(pinned_first):
        key[np.asarray(pinned_first, np.int64)] = np.iinfo(np.int64).max
    old_of_new = np.argsort(-key, kind="stable").astype(np.uint32)
    new_of_old = np.empty(n, np.uint32)
    new_of_old[old_of_new] = np.arange(n, dtype=np.uint32)
    return new_of_old, old_of_new


def map_ids(ids: np.ndarray, new_of_old: np.ndarray) -> np.ndarray:
    """Old ids -> new ids; the invalid id stays."""
    ids = np.asarray(ids)
    flat = ids.astype(np.uint32, copy=False).reshape(-1)
    out = np.full(flat.shape, INVALID, np.uint32)
    ok = flat != INVALID
    out[ok] = new_of_old[flat[ok]]
    return out.reshape(ids.shape)


def relabel_index(index: dict, new_of_old: np.ndarray, old_of_new: np.ndarray) -> dict:
    """A copy of a host index dict (keys as oracle.pipeline.index_from_synth: adjacency, codes, vectors and the
    optional pq2_codes, pq2_error_bounds, rvq_ids) under the new ids. Per-node rows move to their new position;
    stored ids (adjacency entries, RVQ postings) are mapped; slot order inside an adjacency row is kept."""
    out = dict(index)
    out["adjacency"] = map_ids(index["adjacency"][old_of_new], new_of_old)
    for key in ("codes", "vectors", "pq2_codes", "pq2_error_bounds"):
        if index.get(key) is not None:
            out[key] = np.ascontiguousarray(index[key][old_of_new])
    if index.get("rvq_ids") is not None:
        out["rvq_ids"] = map_ids(index["rvq_ids"], new_of_old)
    out.pop("pages", None)
    return out


def prefix_hit_rate(candidates: np.ndarray, cached_rows: int) -> float:
    """Share of the expanded records whose id lies in the cached prefix [0, cached_rows)."""
    ids = np.ascontiguousarray(candidates)[..., 1].reshape(-1)
    hot = ids[(ids != INVALID) & ((ids & EXPANDED_BIT) != 0)] & ~np.uint32(EXPANDED_BIT)
    return float(np.count_nonzero(hot < cached_rows)) / max(1, hot.size)
