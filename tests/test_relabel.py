"""Frequency-ordered relabelling (tiered topology): the relabelled graph is the same graph, and the cached id
prefix then holds the nodes that are expanded most."""
import numpy as np
import pytest

from topoanns_b200 import relabel

INVALID = 0xFFFFFFFF


def _random_index(n=500, degree=64, seed=3):
    rng = np.random.default_rng(seed)
    adj = np.full((n, degree), INVALID, np.uint32)
    for i in range(n):
        k = int(rng.integers(1, 20))
        adj[i, :k] = rng.choice(n, size=k, replace=False)
    return dict(adjacency=adj, codes=rng.integers(0, 256, (n, 8), dtype=np.uint8),
                vectors=rng.integers(0, 256, (n, 16), dtype=np.uint8),
                rvq_ids=rng.integers(0, n, 300).astype(np.uint32)), rng


def test_relabelled_graph_is_the_same_graph():
    index, rng = _random_index()
    n = index["adjacency"].shape[0]
    cand = np.zeros((40, 32, 2), np.uint32)
    ids = rng.integers(0, 60, (40, 32)).astype(np.uint32)             # a hot set of 60 nodes
    flags = rng.integers(0, 2, (40, 32)).astype(np.uint32) << np.uint32(31)
    cand[..., 1] = ids | flags
    cand[0, 0, 1] = INVALID
    counts = relabel.expansion_counts(cand, n)
    assert counts.sum() == np.count_nonzero((cand[..., 1] != INVALID) & (cand[..., 1] >> 31 == 1))
    assert counts[60:].sum() == 0
    new_of_old, old_of_new = relabel.frequency_permutation(counts, pinned_first=[123])
    assert new_of_old[123] == 0 and sorted(new_of_old.tolist()) == list(range(n))
    assert np.array_equal(old_of_new[new_of_old], np.arange(n))
    order_counts = counts[old_of_new[1:]]
    assert np.all(order_counts[:-1] >= order_counts[1:])                  # descending heat after the pinned node
    out = relabel.relabel_index(index, new_of_old, old_of_new)
    for u in rng.integers(0, n, 50):
        old_row = index["adjacency"][u]
        new_row = out["adjacency"][new_of_old[u]]
        assert np.array_equal(new_row == INVALID, old_row == INVALID)     # slots keep their place
        assert np.array_equal(new_row[new_row != INVALID], new_of_old[old_row[old_row != INVALID]])
        assert np.array_equal(out["codes"][new_of_old[u]], index["codes"][u])
        assert np.array_equal(out["vectors"][new_of_old[u]], index["vectors"][u])
    assert np.array_equal(out["rvq_ids"], new_of_old[index["rvq_ids"]])
    # the 60 hot nodes (and the pinned one) now fill the id prefix
    mapped = cand.copy()
    raw = np.where(cand[..., 1] == INVALID, INVALID, cand[..., 1] & 0x7FFFFFFF).astype(np.uint32)
    mapped[..., 1] = np.where(raw == INVALID, INVALID, relabel.map_ids(raw, new_of_old) | (cand[..., 1] & 0x80000000))
    assert relabel.prefix_hit_rate(mapped, 61) == 1.0
    assert relabel.prefix_hit_rate(cand, 30) < 0.7


@pytest.mark.gpu
def test_relabelled_index_searches_the_same_and_heats_the_prefix():
    import torch

    import gpu_support as gs
    from topoanns_b200 import search, synth

    s, host = gs.small_index(name="cfg1", num_nodes=20000, components=200, num_queries=256)
    ix = gs.device_index(s)
    Q = s.queries.shape[0]
    train, test = slice(0, 192), slice(192, Q)
    q = s.queries.cuda().to(torch.uint8).contiguous()
    p = search.TopologySearchParams(top_l=32, search_width=2, max_expansions=4096)
    rp = search.RerankExactParams(top_k=10, top_n=32)
    eo, ei = gs.fixed_entries(192, [s.medoid])
    cand, _ = search.beam_search(ix, p, eo, ei, queries=q[train].contiguous())
    counts = relabel.expansion_counts(gs.np_u32(cand), ix.num_nodes)
    new_of_old, old_of_new = relabel.frequency_permutation(counts, pinned_first=[s.medoid])
    out = relabel.relabel_index(host, new_of_old, old_of_new)
    ix2 = search.device_index_from_arrays(adjacency=out["adjacency"], codes=out["codes"], vectors=out["vectors"],
                                          pq_tables_row_major=host["pq_tables"], pq_centroid=host["pq_centroid"],
                                          pq_chunk_offsets=host["pq_chunk_offsets"])
    nt = Q - 192
    eo_t, ei_t = gs.fixed_entries(nt, [s.medoid])
    eo_t2, ei_t2 = gs.fixed_entries(nt, [int(new_of_old[s.medoid])])
    qt = q[test].contiguous()
    c1, _ = search.beam_search(ix, p, eo_t, ei_t, queries=qt)
    c2, _ = search.beam_search(ix2, p, eo_t2, ei_t2, queries=qt)
    _, i1, _, _ = search.rerank_exact(ix, rp, c1, qt)
    d2, i2, _, _ = search.rerank_exact(ix2, rp, c2, qt)
    gt = s.gt_ids.cpu().numpy()[test]
    r1 = synth.recall_at_k(gs.np_u32(i1[:, :10]), gt, 10)
    back = old_of_new[np.minimum(gs.np_u32(i2[:, :10]), ix.num_nodes - 1)]
    r2 = synth.recall_at_k(back, gt, 10)
    assert abs(r1 - r2) < 0.03            # same graph; only id-dependent tie breaks and filter collisions differ
    # the queries the counts came from: (nearly) all their expansions now fall into the prefix of hot nodes
    hot = int(np.count_nonzero(counts)) + 1
    eo2, ei2 = gs.fixed_entries(192, [int(new_of_old[s.medoid])])
    c_train2, _ = search.beam_search(ix2, p, eo2, ei2, queries=q[train].contiguous())
    assert relabel.prefix_hit_rate(gs.np_u32(c_train2), hot) > 0.95
    assert relabel.prefix_hit_rate(gs.np_u32(cand), hot) < 0.6
    # held-out queries share the first hops from the entry node: the same prefix serves more of their expansions
    before = relabel.prefix_hit_rate(gs.np_u32(c1), hot)
    after = relabel.prefix_hit_rate(gs.np_u32(c2), hot)
    assert after > before, (before, after)
