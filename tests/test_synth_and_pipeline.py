"""The synthetic generator and the checker's whole-path runner on a small index (CPU)."""
import dataclasses

import numpy as np
import torch

from oracle import pipeline
from topoanns_b200 import synth

INVALID = 0xFFFFFFFF


def _small(name="cfg2", **kw):
    base = dict(num_nodes=6000, components=30, num_queries=64, train_sample=6000, kmeans_iters=4)
    base.update(kw)
    return synth.build(dataclasses.replace(synth.CONFIGS[name], **base), "cpu")


def test_generator_shapes_and_graph_quality():
    s = _small()
    N = s.vectors.shape[0]
    assert s.vectors.dtype == torch.uint8 and s.adjacency.shape == (N, 64) and s.pq_codes.shape == (N, 32)
    assert s.pq_tables.shape == (256, 128) and s.pq_chunk_offsets.tolist() == list(range(0, 129, 4))
    assert int(s.adjacency.min()) >= 0 and int(s.adjacency.max()) < N
    # kNN edges found inside the mixture component equal the brute-force kNN
    x = s.vectors.float()
    probe = torch.arange(0, N, 97)
    d = torch.cdist(x[probe], x) ** 2
    d[torch.arange(probe.numel()), probe] = float("inf")
    kth = d.topk(48, largest=False).values[:, -1]
    nbr = s.adjacency[probe, :48].long()
    nd = ((x[nbr] - x[probe].unsqueeze(1)) ** 2).sum(2)
    assert float((nd <= kth.unsqueeze(1) + 0.5).float().mean()) > 0.999
    # ground truth is the exact top-k
    q = s.queries
    dq = torch.cdist(q, x) ** 2
    want = dq.topk(10, largest=False).values
    got = ((x[s.gt_ids] - q.unsqueeze(1)) ** 2).sum(2)
    assert torch.allclose(got, want)
    sizes, offsets, ids = s.rvq_buckets
    assert int(sizes.sum()) == N and int(offsets[-1]) == ids.numel() and int((offsets[1:] - offsets[:-1]).max()) <= 256


def test_same_seed_same_index():
    a, b = _small(num_nodes=2000, components=10), _small(num_nodes=2000, components=10)
    assert torch.equal(a.vectors, b.vectors) and torch.equal(a.adjacency, b.adjacency)
    assert torch.equal(a.pq_codes, b.pq_codes) and torch.equal(a.gt_ids, b.gt_ids)


def test_whole_path_on_checker_finds_neighbours():
    s = _small()
    host = pipeline.index_from_synth(s)
    q = s.queries.numpy()
    r = pipeline.run(host, q, top_l=64, search_width=2, max_expansions=4096, top_n=64, top_k=10, entry_count=128)
    assert synth.recall_at_k(r["topk_ids"], s.gt_ids.numpy(), 10) > 0.6
    assert (np.diff(r["dists"], axis=1) >= 0).all()
    # both visited-set protocols give valid searches; they may differ only through duplicates
    r2 = pipeline.run(host, q, top_l=64, search_width=2, max_expansions=4096, top_n=64, top_k=10, entry_count=128,
                      two_phase=False)
    assert synth.recall_at_k(r2["topk_ids"], s.gt_ids.numpy(), 10) > 0.6
    # uint8 queries give the same answer as their float copies
    r8 = pipeline.run(host, q.astype(np.uint8), top_l=64, search_width=2, max_expansions=4096, top_n=64, top_k=10,
                      entry_count=128)
    assert np.array_equal(r8["topk_ids"], r["topk_ids"]) and np.array_equal(r8["topk_dists"], r["topk_dists"])


def test_pq2_generation_and_bound_filter_never_lose_the_best():
    s = _small("cfg3", num_nodes=3000, components=15, num_queries=32)
    assert s.vectors.dtype == torch.float32 and s.pq2_codes.shape == s.pq_codes.shape
    host = pipeline.index_from_synth(s)
    q = s.queries.numpy()
    kw = dict(top_l=64, search_width=2, max_expansions=1024, top_n=64, top_k=10, fixed_entries=[s.medoid], use_pq2=True,
              refine_top_l=64)
    plain = pipeline.run(host, q, **kw)
    filt = pipeline.run(host, q, bound_filter=True, tile=16, **kw)
    assert filt["n_exact"] + filt["n_filtered"] == plain["n_exact"]
    # the error bound is a true bound on the reconstruction error, so the filter cannot drop a top-k member
    assert np.array_equal(filt["topk_ids"], plain["topk_ids"])
