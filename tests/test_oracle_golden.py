"""The CPU checker against the known answers asserted by the reference's own tests.

Inputs and expected values are the tiny numeric fixtures of the reference test files named in
each test; they pin the restatement in oracle/tann_oracle.cpp.
"""
import numpy as np

INVALID = 0xFFFFFFFF


def _toy_graph():
    # tests/test_topology_search_gpu.cpp:182-183: MakePadded(6, {{1,2},{3},{4},{5},{5},{}})
    lists = [[1, 2], [3], [4], [5], [5], []]
    adj = np.full((6, 64), INVALID, np.uint32)
    for i, l in enumerate(lists):
        adj[i, :len(l)] = l
    return adj


def _toy_pq_1d():
    # tests/test_topology_search_gpu.cpp:46-54: tables[i] = i (256 x 1), centroid 0, one chunk,
    # codes {9,6,7,2,3,1}
    tables = np.arange(256, dtype=np.float32).reshape(256, 1)
    return tables, np.zeros(1, np.float32), np.array([0, 1], np.uint32), \
        np.array([[9], [6], [7], [2], [3], [1]], np.uint8)


def test_lut_values_and_distances(orc):
    # tests/test_pq_query_tables.cpp:44-57,95-116
    tables = np.zeros((256, 2), np.float32)
    tables[1] = (1, 0)
    tables[2] = (0, 2)
    tables[3] = (1, 2)
    lut = orc.lut_build(np.array([[1, 2], [0, 0]], np.float32), tables, np.zeros(2, np.float32),
                        np.array([0, 2], np.uint32))
    assert lut.shape == (2, 1, 256)
    assert lut[0, 0, :4].tolist() == [5.0, 4.0, 1.0, 0.0]
    assert lut[1, 0, :4].tolist() == [0.0, 1.0, 4.0, 5.0]
    codes = np.array([[1], [2], [3]], np.uint8)
    assert [orc.adc_serial(lut[0], codes[n]) for n in range(3)] == [4.0, 1.0, 0.0]
    assert orc.adc_serial(lut[1], codes[0]) == 1.0
    assert orc.adc_serial(lut[1], codes[2]) == 5.0
    assert orc.adc_tree(lut[1], codes[2]) == 5.0


def test_lut_uint8_and_int8_queries_match_float(orc):
    # src/search/pq_query_tables.cu:33-35: the query is cast to float before anything else.
    rng = np.random.default_rng(0)
    tables = rng.normal(size=(256, 8)).astype(np.float32)
    cen = rng.normal(size=8).astype(np.float32)
    off = np.array([0, 3, 8], np.uint32)
    qu = rng.integers(0, 256, size=(5, 8)).astype(np.uint8)
    qi = rng.integers(-128, 128, size=(5, 8)).astype(np.int8)
    assert np.array_equal(orc.lut_build(qu, tables, cen, off),
                          orc.lut_build(qu.astype(np.float32), tables, cen, off))
    assert np.array_equal(orc.lut_build(qi, tables, cen, off),
                          orc.lut_build(qi.astype(np.float32), tables, cen, off))


def test_toy_graph_single_query(orc):
    # tests/test_topology_search_gpu.cpp:189-212: top_k = top_l = 2, W = 1, max_expansions 16;
    # top-2 = ids (5, 3), distances (1, 4). The reference asserts that visited / expanded /
    # iterations equal its exact-visited-set CPU search (tests/test_topology_search_gpu.cpp:94-171),
    # which gives 5 / 4 / 4 on this graph (0 -> 1 -> 3 -> 5, node 4 is never reached).
    tables, cen, off, codes = _toy_pq_1d()
    lut = orc.lut_build(np.array([[0.0]], np.float32), tables, cen, off)
    for two_phase in (True, False):
        cand, stats = orc.beam_search(_toy_graph(), codes, lut, [0, 1], [0], top_l=2,
                                      search_width=1, max_expansions=16, two_phase=two_phase)
        assert orc.cand_raw_id(cand)[0, :2].tolist() == [5, 3]
        assert orc.cand_dist(cand)[0, :2].tolist() == [1.0, 4.0]
        assert stats[0].tolist()[:5] == [5, 4, 0, 4, 2]


def test_toy_graph_two_queries(orc):
    # tests/test_topology_search_batch_gpu.cpp:174-199: queries {0, 8} -> (5,3) and (0,2)
    tables, cen, off, codes = _toy_pq_1d()
    lut = orc.lut_build(np.array([[0.0], [8.0]], np.float32), tables, cen, off)
    cand, stats = orc.beam_search(_toy_graph(), codes, lut, [0, 1, 2], [0, 0], top_l=2,
                                  search_width=1, max_expansions=16)
    ids = orc.cand_raw_id(cand)
    assert ids[0, :2].tolist() == [5, 3]
    assert ids[1, :2].tolist() == [0, 2]


def test_end_to_end_batch(orc):
    # tests/test_topoanns_search_batch.cpp:107-161: dim 300, tables[c][*] = c, one chunk over all
    # dims, vectors constant {9,6,7,2,3,1}, queries constant {0, 8}; top_l 4, top_k 5, rerank
    # top_n 5 / top_k 2 -> candidate capacity nextpow2(max(4, 5)) = 8, 5 valid candidates each.
    dim = 300
    tables = np.repeat(np.arange(256, dtype=np.float32)[:, None], dim, axis=1)
    codes = np.array([[9], [6], [7], [2], [3], [1]], np.uint8)
    queries = np.repeat(np.array([[0.0], [8.0]], np.float32), dim, axis=1)
    lut = orc.lut_build(queries, tables, np.zeros(dim, np.float32), np.array([0, dim], np.uint32))
    cap = orc.candidate_capacity(4, 0, 5)
    assert cap == 8
    cand, stats = orc.beam_search(_toy_graph(), codes, lut, [0, 1, 2], [0, 0], top_l=4,
                                  search_width=1, max_expansions=16, capacity=cap)
    ids = orc.cand_raw_id(cand)
    assert ids[0, :2].tolist() == [5, 3] and ids[1, :2].tolist() == [0, 2]
    # first max(top_l, cqs) = 5 valid candidates are materialised
    assert int((ids[0] != INVALID).sum()) >= 5 and int((ids[1] != INVALID).sum()) >= 5
    vals = np.array([9, 6, 7, 2, 3, 1], np.float32)
    vpp = 4096 // (dim * 4)
    pages = np.zeros((6 + vpp - 1) // vpp * 4096, np.uint8)
    for n in range(6):
        o = (n // vpp) * 4096 + (n % vpp) * dim * 4
        pages[o:o + dim * 4] = np.full(dim, vals[n], np.float32).view(np.uint8)
    d, i, n_exact, n_filt = orc.rerank(cand, queries, pages, np.float32, top_n=5, top_k=2,
                                       vectors_per_page=vpp, page_bytes=4096, vector_bytes=dim * 4)
    assert n_exact == 10 and n_filt == 0
    assert i[0, :2].tolist() == [5, 3] and d[0, :2].tolist() == [300.0, 1200.0]
    assert i[1, :2].tolist() == [0, 2] and d[1, :2].tolist() == [300.0, 300.0]


def _pq2_fixture(orc):
    # tests/test_pq2_residual_refine.cpp:92-129 and tests/test_pq2_bound_filter.cpp:109-160
    t1 = np.zeros((256, 2), np.float32)
    t1[1] = (1, 0)
    t1[2] = (0, 2)
    t2 = np.zeros((256, 2), np.float32)
    t2[1] = (0, 1)
    t2[2] = (1, 1)
    off = np.array([0, 2], np.uint32)
    zero = np.zeros(2, np.float32)
    base_codes = np.array([[1], [2]], np.uint8)
    res_codes = np.array([[1], [2]], np.uint8)
    cand = np.zeros((1, 2, 2), np.uint32)
    cand[0, 0] = (np.float32(2.0).view(np.uint32), 1)
    cand[0, 1] = (np.float32(1.0).view(np.uint32), 0)
    stats = np.zeros((1, 8), np.uint32)
    stats[0, 4] = 2
    q = np.array([[1.0, 1.0]], np.float32)
    lut2 = orc.lut_build(q, t2, zero, off)
    cross = orc.pq2_cross_terms(off, t1, zero, t2, zero)
    refined = orc.pq2_refine(cand, stats, 2, res_codes, lut2, base_codes, cross)
    return q, refined


def test_pq2_residual_refine(orc):
    # tests/test_pq2_residual_refine.cpp:134-138: ids (0, 1), distances (2, 6)
    _, refined = _pq2_fixture(orc)
    assert orc.cand_raw_id(refined)[0].tolist() == [0, 1]
    assert orc.cand_dist(refined)[0].tolist() == [2.0, 6.0]


def test_pq2_bound_filter(orc):
    # tests/test_pq2_bound_filter.cpp:143-171: vectors (1,1) and (1,3), page-by-page tiles, top_k 1,
    # top_n 2, zero error bounds -> 1 exact distance, 1 filtered, top-1 = node 0.
    q, refined = _pq2_fixture(orc)
    pages = np.zeros(4096, np.uint8)
    pages[0:8] = np.array([1, 1], np.float32).view(np.uint8)
    pages[8:16] = np.array([1, 3], np.float32).view(np.uint8)
    d, i, n_exact, n_filt = orc.rerank(refined, q, pages, np.float32, top_n=2, top_k=1, tile=1,
                                       vectors_per_page=512, page_bytes=4096, vector_bytes=8,
                                       error_bounds=np.zeros(2, np.float32))
    assert n_exact == 1 and n_filt == 1
    assert i[0, 0] == 0 and d[0, 0] == 0.0
    assert i[0, 1] == INVALID and np.isinf(d[0, 1])


def test_uint8_exact_distance_is_integer_exact(orc):
    # src/search/rerank_exact.cu:261-265 accumulates in float; for uint8 d = 128 every partial sum
    # is an integer below 2^24, so the float result equals the integer sum.
    rng = np.random.default_rng(1)
    for _ in range(50):
        a = rng.integers(0, 256, 128).astype(np.uint8)
        b = rng.integers(0, 256, 128).astype(np.uint8)
        want = int(((a.astype(np.int64) - b.astype(np.int64)) ** 2).sum())
        assert orc.exact_distance(a, b) == float(want)
        assert orc.exact_distance(a.astype(np.float32), b) == float(want)
    a = np.zeros(128, np.uint8)
    b = np.full(128, 255, np.uint8)
    assert orc.exact_distance(a, b) == 128 * 255.0 ** 2


def test_rerank_early_stop_rule(orc):
    """The persistent rerank's early stop (src/io/bam_vector_provider.cu:1124-1135) on a hand-made case:
    tiles of 2 ranks, k = 1; the best distance stops improving after the second tile, so with
    min_prefix = 2 and patience 1 the third tile ends the rerank and ranks 6.. are never scored."""
    import numpy as np
    d = 4
    # vector i = (dist_i, 0, 0, 0) against the zero query: squared distances below, in candidate rank order
    sq = np.array([9, 16, 4, 25, 36, 49, 1, 64], np.float32)
    vectors = np.zeros((8, d), np.float32)
    vectors[:, 0] = np.sqrt(sq)
    from oracle import pipeline
    pages, vpp, vb = pipeline.vectors_to_pages(vectors)
    cand = np.zeros((1, 8, 2), np.uint32)
    cand[0, :, 0] = np.arange(8, dtype=np.float32).view(np.uint32)   # PQ distances only order the ranks
    cand[0, :, 1] = np.arange(8)
    q = np.zeros((1, d), np.float32)
    kw = dict(top_n=8, top_k=1, tile=2, vectors_per_page=vpp, page_bytes=4096, vector_bytes=vb)
    dists, ids, n_exact, _ = orc.rerank(cand, q, pages, np.float32, **kw)
    assert n_exact == 8 and ids[0, 0] == 6 and dists[0, 0] == 1.0
    dists, ids, n_exact, _ = orc.rerank(cand, q, pages, np.float32, early_stop_min_prefix=2, early_stop_patience_tiles=1, **kw)
    # tile 1 (ranks 0-1): k-th 9, improved from inf -> stable 0; tile 2: 4 < 9 -> 0; tile 3: 4 == 4 -> stable 1 -> stop
    assert n_exact == 6 and ids[0, 0] == 2 and dists[0, 0] == 4.0
    assert ids[0, 6] == 0xFFFFFFFF and np.isinf(dists[0, 6])
    dists, ids, n_exact, _ = orc.rerank(cand, q, pages, np.float32, early_stop_min_prefix=2, early_stop_patience_tiles=2, **kw)
    assert n_exact == 8 and ids[0, 0] == 6   # tile 4 improves the best again before two stable tiles are seen
