"""The checker (CPU) and the CUDA path (GPU) against outputs of the reference itself, stored in
tests/golden/reference_small.npz by tests/golden/make_reference_fixtures.py (a tiny index plus what the
reference's own kernels produced for it on a B200). Everything is compared bit for bit."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from oracle import pipeline

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_small.npz")
INVALID = 0xFFFFFFFF
CASES = [(32, 2), (16, 1)]


@pytest.fixture(scope="module")
def gold():
    g = dict(np.load(GOLDEN))
    g["index"] = dict(adjacency=g["adjacency"], codes=g["codes"], pq_tables=g["pq_tables"],
                      pq_centroid=g["pq_centroid"], pq_chunk_offsets=g["pq_chunk_offsets"], vectors=g["vectors"])
    return g


def _packed(dist_bits, ids, limit):
    out = np.stack([dist_bits[:, :limit], ids[:, :limit]], axis=2).copy()
    out[..., 0][out[..., 1] == INVALID] = 0
    return out


def test_checker_tables_equal_reference(gold):
    want = gold["ref_lut"]
    got = orc.lut_build(gold["queries"][:want.shape[0]], gold["pq_tables"], gold["pq_centroid"], gold["pq_chunk_offsets"])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("top_l,width", CASES)
def test_checker_traversal_equals_reference(gold, top_l, width):
    Q = gold["queries"].shape[0]
    top_n = int(gold["top_n"])
    limit = max(top_l, top_n)
    lut = orc.lut_build(gold["queries"], gold["pq_tables"], gold["pq_centroid"], gold["pq_chunk_offsets"])
    entries = gold["entries"]
    eo = np.arange(Q + 1, dtype=np.uint32) * entries.shape[1]
    cand, st = orc.beam_search(gold["adjacency"], gold["codes"], lut, eo, entries.reshape(-1), top_l=top_l,
                               search_width=width, max_expansions=int(gold["max_expansions"]),
                               capacity=orc.candidate_capacity(top_l, 0, top_n))
    tag = f"s{top_l}_{width}"
    want = _packed(gold[f"ref_{tag}_dist"].view(np.uint32), gold[f"ref_{tag}_ids"], limit)
    assert np.array_equal(_packed(cand[..., 0], cand[..., 1], limit), want)
    assert np.array_equal(st[:, [0, 1, 3]], gold[f"ref_{tag}_stats"])   # visited, expanded, iterations


def test_checker_rerank_equals_reference(gold):
    r = pipeline.run(gold["index"], gold["queries"].astype(np.uint8), top_l=32, search_width=2,
                     max_expansions=int(gold["max_expansions"]), top_n=int(gold["top_n"]), top_k=int(gold["top_k"]),
                     fixed_entries=gold["entries"][0])
    assert np.array_equal(r["ids"], gold["ref_rerank_ids"])
    assert np.array_equal(r["dists"].view(np.uint32), gold["ref_rerank_dist"].view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("top_l,width", CASES)
def test_cuda_traversal_and_rerank_equal_reference(gold, top_l, width):
    import torch

    from topoanns_b200 import search
    Q = gold["queries"].shape[0]
    top_n, top_k = int(gold["top_n"]), int(gold["top_k"])
    limit = max(top_l, top_n)
    ix = search.device_index_from_arrays(adjacency=gold["adjacency"], codes=gold["codes"], vectors=gold["vectors"],
                                         pq_tables_row_major=gold["pq_tables"], pq_centroid=gold["pq_centroid"],
                                         pq_chunk_offsets=gold["pq_chunk_offsets"])
    q = torch.from_numpy(gold["queries"]).cuda().contiguous()
    entries = gold["entries"]
    eo = torch.from_numpy((np.arange(Q + 1, dtype=np.uint32) * entries.shape[1]).view(np.int32)).cuda()
    ei = torch.from_numpy(entries.reshape(-1).view(np.int32)).cuda()
    p = search.TopologySearchParams(top_l=top_l, search_width=width, max_expansions=int(gold["max_expansions"]))
    cand, stats = search.beam_search(ix, p, eo, ei, queries=q, capacity=p.capacity(top_n))
    got = cand.cpu().numpy().view(np.uint32)
    tag = f"s{top_l}_{width}"
    want = _packed(gold[f"ref_{tag}_dist"].view(np.uint32), gold[f"ref_{tag}_ids"], limit)
    assert np.array_equal(_packed(got[..., 0], got[..., 1], limit), want)
    assert np.array_equal(stats.cpu().numpy().view(np.uint32)[:, [0, 1, 3]], gold[f"ref_{tag}_stats"])
    if (top_l, width) == (32, 2):
        d, i, _, _ = search.rerank_exact(ix, search.RerankExactParams(top_k=top_k, top_n=top_n), cand, q)
        assert np.array_equal(i.cpu().numpy().view(np.uint32), gold["ref_rerank_ids"])
        assert np.array_equal(d.cpu().numpy().view(np.uint32), gold["ref_rerank_dist"].view(np.uint32))
