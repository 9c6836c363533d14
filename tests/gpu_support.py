"""Shared helpers of the GPU parity tests: build a small synthetic index once, put it on the
device, and compare candidate lists record by record."""
import dataclasses
import functools

import numpy as np
import torch

from oracle import pipeline
from topoanns_b200 import search, synth


@functools.lru_cache(maxsize=8)
def small_index(name="cfg1", num_nodes=20000, components=200, num_queries=256, seed=1234, pq_chunks=None,
                knn_edges=None, random_edges=None, dim=None, rvq_coarse=None, rvq_fine=None):
    base = synth.CONFIGS[name]
    kw = dict(num_nodes=num_nodes, components=components, num_queries=num_queries, seed=seed,
              train_sample=32768, kmeans_iters=8)
    if pq_chunks is not None:
        kw["pq_chunks"] = pq_chunks
    if knn_edges is not None:
        kw["knn_edges"] = knn_edges
    if random_edges is not None:
        kw["random_edges"] = random_edges
    if dim is not None:
        kw["dim"] = dim
    if rvq_coarse is not None:
        kw["rvq_coarse"] = rvq_coarse
    if rvq_fine is not None:
        kw["rvq_fine"] = rvq_fine
    cfg = dataclasses.replace(base, **kw)
    s = synth.build(cfg, "cuda" if torch.cuda.is_available() else "cpu")
    host = pipeline.index_from_synth(s)
    return s, host


def device_index(s):
    return search.device_index_from_synth(s, "cuda")


def fixed_entries(Q, entries, device="cuda"):
    e = torch.tensor(list(entries), dtype=torch.int32, device=device)
    ids = e.repeat(Q)
    offsets = torch.arange(Q + 1, dtype=torch.int32, device=device) * e.numel()
    return offsets, ids


def np_u32(t):
    return t.detach().cpu().numpy().view(np.uint32)


def assert_candidates_equal(dev_cand, dev_stats, ref_cand, ref_stats):
    got = np_u32(dev_cand)
    gstats = np_u32(dev_stats)
    bad = np.nonzero((got != ref_cand).reshape(got.shape[0], -1).any(1))[0]
    assert bad.size == 0, f"{bad.size} queries differ, first {bad[:5]}: got {got[bad[0], :4]} want {ref_cand[bad[0], :4]}"
    assert np.array_equal(gstats, ref_stats), "per-query statistics differ"
