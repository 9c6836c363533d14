"""Parity of the CUDA path (through the C ABI) with the CPU checker. Integer / index work is
compared bit for bit; float tables within the 1e-5 relative tolerance the path states (they come
out bit-identical in practice because both sides use the same FMA order)."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from oracle import pipeline
from topoanns_b200 import capi, formats, search

from gpu_support import (assert_candidates_equal, device_index, fixed_entries, np_u32, small_index)

pytestmark = pytest.mark.gpu
INVALID = 0xFFFFFFFF


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a.view(np.int32) if a.dtype == np.uint32 else a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def _toy_index(dim=1, vectors=None, tables=None, codes=None, lists=None):
    lists = lists if lists is not None else [[1, 2], [3], [4], [5], [5], []]
    n = len(lists)
    adj = np.full((n, 64), INVALID, np.uint32)
    for i, l in enumerate(lists):
        adj[i, :len(l)] = l
    if tables is None:
        tables = np.repeat(np.arange(256, dtype=np.float32)[:, None], dim, axis=1)
    if codes is None:
        codes = np.array([[9], [6], [7], [2], [3], [1]], np.uint8)
    if vectors is None:
        vectors = np.repeat(np.array([9, 6, 7, 2, 3, 1], np.float32)[:, None], dim, axis=1)
    return search.device_index_from_arrays(
        adjacency=adj, codes=codes, vectors=vectors, pq_tables_row_major=tables,
        pq_centroid=np.zeros(dim, np.float32), pq_chunk_offsets=np.array([0, dim], np.uint32))


# ---- the reference's own known answers, through the CUDA path ----------------------------------

def test_golden_lut_values():
    # tests/test_pq_query_tables.cpp:44-57,95-116
    tables = np.zeros((256, 2), np.float32)
    tables[1], tables[2], tables[3] = (1, 0), (0, 2), (1, 2)
    ix = _toy_index(dim=2, tables=tables, codes=np.array([[1], [2], [3]], np.uint8),
                    vectors=np.zeros((3, 2), np.float32), lists=[[], [], []])
    lut = search.lut_build(ix, _dev(np.array([[1, 2], [0, 0]], np.float32))).cpu().numpy()
    assert lut[0, 0, :4].tolist() == [5.0, 4.0, 1.0, 0.0]
    assert lut[1, 0, :4].tolist() == [0.0, 1.0, 4.0, 5.0]


@pytest.mark.parametrize("lut_in_kernel", [False, True])
def test_golden_toy_graph(lut_in_kernel):
    # tests/test_topology_search_gpu.cpp:182-221 and tests/test_topology_search_batch_gpu.cpp:174-199
    ix = _toy_index()
    q = _dev(np.array([[0.0], [8.0]], np.float32))
    eo, ei = fixed_entries(2, [0])
    p = search.TopologySearchParams(top_k=2, top_l=2, search_width=1, max_expansions=16)
    if lut_in_kernel:
        cand, stats = search.beam_search(ix, p, eo, ei, queries=q)
    else:
        cand, stats = search.beam_search(ix, p, eo, ei, lut=search.lut_build(ix, q))
    c = np_u32(cand)
    assert orc.cand_raw_id(c)[0, :2].tolist() == [5, 3]
    assert orc.cand_dist(c)[0, :2].tolist() == [1.0, 4.0]
    assert orc.cand_raw_id(c)[1, :2].tolist() == [0, 2]
    assert np_u32(stats)[0, :5].tolist() == [5, 4, 0, 4, 2]


def test_golden_end_to_end_batch():
    # tests/test_topoanns_search_batch.cpp:107-161
    dim = 300
    ix = _toy_index(dim=dim)
    queries = np.repeat(np.array([[0.0], [8.0]], np.float32), dim, axis=1)
    s = search.Searcher(ix, 2, 8, 5, 4)
    tp = search.TopologySearchParams(top_k=5, top_l=4, search_width=1, max_expansions=16)
    rp = search.RerankExactParams(top_k=2, top_n=5)
    ids, dists, stats = s.run_host(queries, tp, rp, fixed_entries=np.array([0], np.uint32), want_stats=True)
    assert ids[0].tolist() == [5, 3] and dists[0].tolist() == [300.0, 1200.0]
    assert ids[1].tolist() == [0, 2] and dists[1].tolist() == [300.0, 300.0]
    s.close()


def _pq2_fixture():
    # tests/test_pq2_residual_refine.cpp:92-129, tests/test_pq2_bound_filter.cpp:109-160
    t1 = np.zeros((256, 2), np.float32)
    t1[1], t1[2] = (1, 0), (0, 2)
    t2 = np.zeros((256, 2), np.float32)
    t2[1], t2[2] = (0, 1), (1, 1)
    ix = _toy_index(dim=2, tables=t1, codes=np.array([[1], [2]], np.uint8),
                    vectors=np.array([[1, 1], [1, 3]], np.float32), lists=[[1], []])
    cand = np.zeros((1, 2, 2), np.uint32)
    cand[0, 0] = (np.float32(2.0).view(np.uint32), 1)
    cand[0, 1] = (np.float32(1.0).view(np.uint32), 0)
    stats = np.zeros((1, 8), np.uint32)
    stats[0, 4] = 2
    q = _dev(np.array([[1.0, 1.0]], np.float32))
    off = _dev(np.array([0, 2], np.uint32))
    zero = _dev(np.zeros(2, np.float32))
    t2d = _dev(t2)
    lut2 = search.lut_build(ix, q, tables_col_major=t2d.t().contiguous(), centroid=zero, chunk_offsets=off)
    cross = search.pq2_cross_terms(off, _dev(t1), zero, t2d, zero)
    refined = search.pq2_refine(_dev(cand), _dev(stats), 2, _dev(np.array([[1], [2]], np.uint8)), lut2,
                                base_codes=ix.codes, cross_terms=cross)
    return ix, q, refined


def test_golden_pq2_residual_refine():
    # tests/test_pq2_residual_refine.cpp:134-138
    _, _, refined = _pq2_fixture()
    r = np_u32(refined)
    assert orc.cand_raw_id(r)[0].tolist() == [0, 1]
    assert orc.cand_dist(r)[0].tolist() == [2.0, 6.0]


def test_golden_pq2_bound_filter():
    # tests/test_pq2_bound_filter.cpp:143-171
    ix, q, refined = _pq2_fixture()
    rp = search.RerankExactParams(top_k=1, top_n=2, rank_tile_size=1, use_pq2_bound_filter=True)
    d, i, n_exact, n_filt = search.rerank_exact(ix, rp, refined, q, error_bounds=_dev(np.zeros(2, np.float32)))
    assert (n_exact, n_filt) == (1, 1)
    assert np_u32(i)[0].tolist() == [0, INVALID]
    assert d.cpu().numpy()[0, 0] == 0.0


# ---- seeded synthetic indices against the checker ------------------------------------------------

def test_lut_matches_checker_all_query_kinds():
    s, host = small_index()
    ix = device_index(s)
    q = s.queries[:64]
    for qt in (q, q.to(torch.uint8), (q - 128).to(torch.int8)):
        got = search.lut_build(ix, qt.cuda().contiguous()).cpu().numpy()
        want = orc.lut_build(qt.cpu().numpy(), host["pq_tables"], host["pq_centroid"], host["pq_chunk_offsets"])
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=0)
        assert np.array_equal(got, want)  # same FMA order on both sides


@pytest.mark.parametrize("top_l,width", [(16, 1), (64, 2), (100, 2), (256, 4), (1100, 2)])
def test_beam_search_matches_checker(top_l, width):
    s, host = small_index()
    ix = device_index(s)
    q = s.queries.cuda().contiguous()
    Q = q.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid])
    p = search.TopologySearchParams(top_l=top_l, search_width=width, max_expansions=4096)
    cap = p.capacity(32)
    lut_ref = orc.lut_build(s.queries.cpu().numpy(), host["pq_tables"], host["pq_centroid"], host["pq_chunk_offsets"])
    ref_cand, ref_stats = orc.beam_search(host["adjacency"], host["codes"], lut_ref, np_u32(eo), np_u32(ei),
                                          top_l=top_l, search_width=width, max_expansions=4096, capacity=cap)
    for use_lut in (False, True):
        if use_lut:
            cand, stats = search.beam_search(ix, p, eo, ei, lut=search.lut_build(ix, q), capacity=cap)
        else:
            cand, stats = search.beam_search(ix, p, eo, ei, queries=q, capacity=cap)
        assert_candidates_equal(cand, stats, ref_cand, ref_stats)


def test_beam_search_wide_frontier_and_max_expansions():
    # W * degree > 128 takes the multi-round path; max_expansions cuts the search short and may be
    # overshot by up to W - 1 (src/search/topology_search_kernel.cu:2479-2513).
    s, host = small_index()
    ix = device_index(s)
    q = s.queries[:64].cuda().contiguous()
    eo, ei = fixed_entries(64, [s.medoid, 5, 7])
    lut_ref = orc.lut_build(s.queries[:64].cpu().numpy(), host["pq_tables"], host["pq_centroid"], host["pq_chunk_offsets"])
    for width, max_exp in ((8, 4096), (32, 50), (3, 10)):
        p = search.TopologySearchParams(top_l=128, search_width=width, max_expansions=max_exp)
        cand, stats = search.beam_search(ix, p, eo, ei, queries=q)
        ref_cand, ref_stats = orc.beam_search(host["adjacency"], host["codes"], lut_ref, np_u32(eo), np_u32(ei),
                                              top_l=128, search_width=width, max_expansions=max_exp)
        assert_candidates_equal(cand, stats, ref_cand, ref_stats)
        assert np_u32(stats)[:, 1].max() <= max_exp + width - 1


def test_ragged_invalid_and_empty_entries():
    s, host = small_index()
    ix = device_index(s)
    Q = 6
    q = s.queries[:Q].cuda().contiguous()
    lists = [[s.medoid], [], [INVALID, 3, 3, 3],
             list(range(0, 300)), [ix.num_nodes + 5, INVALID], [7]]
    offsets = np.zeros(Q + 1, np.uint32)
    offsets[1:] = np.cumsum([len(l) for l in lists])
    ids = np.array([x for l in lists for x in l], np.uint32)
    eo, ei = _dev(offsets), _dev(ids)
    p = search.TopologySearchParams(top_l=32, search_width=2, max_expansions=512)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cand, stats = search.beam_search(ix, p, eo, ei, queries=q, status=status)
    assert int(status.item()) == 1      # TANN_STATUS_BEAM_ID_RANGE: the id beyond the index was skipped and reported
    clean = torch.zeros(1, dtype=torch.int32, device="cuda")
    search.beam_search(ix, p, eo[:2].contiguous(), ei[:1].contiguous(), queries=q[:1].contiguous(), status=clean)
    assert int(clean.item()) == 0
    lut_ref = orc.lut_build(s.queries[:Q].cpu().numpy(), host["pq_tables"], host["pq_centroid"], host["pq_chunk_offsets"])
    ref_cand, ref_stats = orc.beam_search(host["adjacency"], host["codes"], lut_ref, offsets, ids, top_l=32,
                                          search_width=2, max_expansions=512)
    assert_candidates_equal(cand, stats, ref_cand, ref_stats)
    st = np_u32(stats)
    assert st[1, 4] == 0 and st[4, 4] == 0          # no valid entry -> nothing found
    assert (np_u32(cand)[1, :, 1] == INVALID).all()


def test_empty_batch_is_a_no_op():
    s, _ = small_index()
    ix = device_index(s)
    eo = torch.zeros(1, dtype=torch.int32, device="cuda")
    ei = torch.zeros(0, dtype=torch.int32, device="cuda")
    p = search.TopologySearchParams(top_l=16, search_width=1)
    cand, stats = search.beam_search(ix, p, eo, ei, queries=torch.zeros((0, ix.dim), device="cuda"))
    assert cand.shape[0] == 0 and stats.shape[0] == 0


@pytest.mark.parametrize("chunks,knn,rnd", [(48, 24, 8), (20, 56, 8), (16, 12, 4)])
def test_beam_search_other_chunk_counts_and_degrees(chunks, knn, rnd):
    # M = 48 (two tree groups), M = 20 (generic byte path), degree 64 / 16
    s, host = small_index(num_nodes=8000, components=80, num_queries=64, pq_chunks=chunks, knn_edges=knn,
                          random_edges=rnd, dim=96 if chunks == 48 else 80 if chunks == 20 else 64)
    ix = device_index(s)
    q = s.queries.cuda().contiguous()
    eo, ei = fixed_entries(q.shape[0], [s.medoid])
    p = search.TopologySearchParams(top_l=48, search_width=2, max_expansions=1024)
    cand, stats = search.beam_search(ix, p, eo, ei, queries=q)
    lut_ref = orc.lut_build(s.queries.cpu().numpy(), host["pq_tables"], host["pq_centroid"], host["pq_chunk_offsets"])
    ref_cand, ref_stats = orc.beam_search(host["adjacency"], host["codes"], lut_ref, np_u32(eo), np_u32(ei),
                                          top_l=48, search_width=2, max_expansions=1024)
    assert_candidates_equal(cand, stats, ref_cand, ref_stats)


def test_learned_stop_matches_checker():
    s, host = small_index()
    ix = device_index(s)
    q = s.queries.cuda().contiguous()
    Q = q.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid])
    for churn_flag, next64_flag, mask in ((1, 0, [0, 0, 1, 1, 0, 0, 1, 1, 1, 0, 1, 1]), (0, 1, [1] * 12), (0, 0, [1] * 12)):
        def make(cls):
            ls = cls()
            ls.enabled, ls.num_stages, ls.top_k, ls.shadow_mode = 1, 3, 10, 0
            ls.topk_churn_flag_mode, ls.next64_flag_mode = churn_flag, next64_flag
            for i, pfx in enumerate((16, 32, 48)):
                ls.stage_prefixes[i] = pfx
            w = np.random.default_rng(11).normal(size=12).astype(np.float32) * 1e-4
            for i in range(12):
                ls.feature_mask[i] = mask[i]
                ls.weights[i] = float(w[i]) if mask[i] else 0.0
            ls.bias, ls.threshold_logit, ls.inv_top_l = 0.05, 0.0, 1.0 / 64
            return ls
        p = search.TopologySearchParams(top_l=64, search_width=2, max_expansions=4096, learned_stop=make(capi.LearnedStop))
        cand, stats = search.beam_search(ix, p, eo, ei, queries=q)
        lut_ref = orc.lut_build(s.queries.cpu().numpy(), host["pq_tables"], host["pq_centroid"], host["pq_chunk_offsets"])
        ref_cand, ref_stats = orc.beam_search(host["adjacency"], host["codes"], lut_ref, np_u32(eo), np_u32(ei),
                                              top_l=64, search_width=2, max_expansions=4096,
                                              learned_stop=make(orc.LearnedStop))
        assert_candidates_equal(cand, stats, ref_cand, ref_stats)


def test_rerank_uint8_bit_exact_and_sorted():
    s, host = small_index()
    ix = device_index(s)
    Q = s.queries.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid])
    p = search.TopologySearchParams(top_l=64, search_width=2, max_expansions=4096)
    q_f32 = s.queries.cuda().contiguous()
    cand, stats = search.beam_search(ix, p, eo, ei, queries=q_f32, capacity=p.capacity(32))
    rp = search.RerankExactParams(top_k=10, top_n=32)
    for qt in (q_f32.to(torch.uint8), q_f32):   # integer (dp4a) path and float path
        d, i, n_exact, _ = search.rerank_exact(ix, rp, cand, qt.contiguous())
        rd, ri, rn, _ = orc.rerank(np_u32(cand), qt.cpu().numpy(), host_pages(host), np.uint8, top_n=32, top_k=10,
                                   vectors_per_page=host["vpp"], page_bytes=4096, vector_bytes=host["vb"])
        assert n_exact == rn
        assert np.array_equal(np_u32(i), ri)
        assert np.array_equal(d.cpu().numpy().view(np.uint32), rd.view(np.uint32))   # bit-exact
        dd = d.cpu().numpy()
        assert (np.diff(dd, axis=1) >= 0).all()
        # independent integer check of every returned distance
        ids_np = np_u32(i).astype(np.int64)
        vec = host["vectors"].astype(np.int64)
        qq = s.queries.cpu().numpy().astype(np.int64)
        want = ((vec[ids_np] - qq[:, None, :]) ** 2).sum(2)
        assert np.array_equal(dd.astype(np.int64), want)


@pytest.mark.parametrize("top_n", [1, 7, 40, 100, 300, 600])
def test_rerank_sizes_and_query_kinds(top_n):
    """Every rerank path (8 lanes per candidate with integer, uint8-row/float-query and float rows, the
    warp-per-candidate fallback for int8 queries) at list lengths around the sort's and tiling's
    boundaries, bit for bit against the checker."""
    s, host = small_index()
    ix = device_index(s)
    Q = s.queries.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid])
    L = max(64, min(top_n, 512))
    p = search.TopologySearchParams(top_l=L, search_width=2, max_expansions=4096)
    q_f32 = s.queries.cuda().contiguous()
    cand, _ = search.beam_search(ix, p, eo, ei, queries=q_f32, capacity=p.capacity(top_n))
    rp = search.RerankExactParams(top_k=min(10, top_n), top_n=top_n)
    g = torch.Generator(device="cuda").manual_seed(3)
    q_frac = (q_f32 + torch.rand(q_f32.shape, generator=g, device="cuda") * 0.75).contiguous()   # not uint8-valued
    q_i8 = (q_f32 / 2).to(torch.int8).contiguous()
    for qt in (q_f32.to(torch.uint8).contiguous(), q_f32, q_frac, q_i8):
        d, i, n_exact, _ = search.rerank_exact(ix, rp, cand, qt)
        rd, ri, rn, _ = orc.rerank(np_u32(cand), qt.cpu().numpy(), host_pages(host), np.uint8, top_n=top_n,
                                   top_k=rp.top_k, vectors_per_page=host["vpp"], page_bytes=4096, vector_bytes=host["vb"])
        assert n_exact == rn
        assert np.array_equal(np_u32(i), ri), str(qt.dtype)
        assert np.array_equal(d.cpu().numpy().view(np.uint32), rd.view(np.uint32)), str(qt.dtype)


@pytest.mark.parametrize("top_n", [5, 64, 200])
def test_rerank_float_rows(top_n):
    s, host = small_index(name="cfg3", num_nodes=12000, components=60, num_queries=128)
    ix = device_index(s)
    Q = s.queries.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid])
    p = search.TopologySearchParams(top_l=max(64, top_n), search_width=2, max_expansions=4096)
    q = s.queries.cuda().contiguous()
    cand, _ = search.beam_search(ix, p, eo, ei, queries=q, capacity=p.capacity(top_n))
    rp = search.RerankExactParams(top_k=min(10, top_n), top_n=top_n)
    d, i, n_exact, _ = search.rerank_exact(ix, rp, cand, q)
    rd, ri, rn, _ = orc.rerank(np_u32(cand), q.cpu().numpy(), host_pages(host), np.float32, top_n=top_n, top_k=rp.top_k,
                               vectors_per_page=host["vpp"], page_bytes=4096, vector_bytes=host["vb"])
    assert n_exact == rn
    assert np.array_equal(np_u32(i), ri)
    assert np.array_equal(d.cpu().numpy().view(np.uint32), rd.view(np.uint32))


@pytest.mark.parametrize("min_prefix,patience", [(32, 1), (16, 2), (64, 3)])
def test_rerank_early_stop_matches_checker(min_prefix, patience):
    """Early stop of the persistent rerank: same scored prefix, same lists and the same count of exact
    distances as the checker; fewer distances than without the stop."""
    s, host = small_index()
    ix = device_index(s)
    Q = s.queries.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid])
    top_n = 160
    p = search.TopologySearchParams(top_l=top_n, search_width=2, max_expansions=4096)
    q = s.queries.cuda().to(torch.uint8).contiguous()
    cand, _ = search.beam_search(ix, p, eo, ei, queries=q, capacity=p.capacity(top_n))
    rp = search.RerankExactParams(top_k=10, top_n=top_n, rank_tile_size=16, use_early_stop=True,
                                  early_stop_min_prefix=min_prefix, early_stop_patience_tiles=patience)
    d, i, n_exact, _ = search.rerank_exact(ix, rp, cand, q)
    rd, ri, rn, _ = orc.rerank(np_u32(cand), q.cpu().numpy(), host_pages(host), np.uint8, top_n=top_n, top_k=10, tile=16,
                               vectors_per_page=host["vpp"], page_bytes=4096, vector_bytes=host["vb"],
                               early_stop_min_prefix=min_prefix, early_stop_patience_tiles=patience)
    assert n_exact == rn
    assert np.array_equal(np_u32(i), ri)
    assert np.array_equal(d.cpu().numpy().view(np.uint32), rd.view(np.uint32))
    full = search.RerankExactParams(top_k=10, top_n=top_n, rank_tile_size=16)
    _, _, n_full, _ = search.rerank_exact(ix, full, cand, q)
    assert n_exact < n_full
    # a stop that can never trigger changes nothing
    never = search.RerankExactParams(top_k=10, top_n=top_n, rank_tile_size=16, use_early_stop=True,
                                     early_stop_min_prefix=10 ** 6, early_stop_patience_tiles=1)
    d2, i2, n2, _ = search.rerank_exact(ix, never, cand, q)
    d3, i3, _, _ = search.rerank_exact(ix, full, cand, q)
    assert n2 == n_full and torch.equal(d2, d3) and torch.equal(i2, i3)


@pytest.mark.parametrize("tile,top_k,top_n,float_queries", [(1, 1, 40, False), (16, 32, 160, False), (33, 10, 100, True),
                                                             (64, 5, 300, False), (48, 10, 24, True), (64, 32, 512, True),
                                                             (65, 10, 160, False)])
def test_rerank_short_tiles_match_checker(tile, top_k, top_n, float_queries):
    """Tiles of up to 64 ranks with top_k <= 32 are scored by one warp per query (tile 65: a block per query):
    same lists, same count of exact distances as the checker, for one- and two-round tiles, lists that are not
    powers of two and both query kinds."""
    s, host = small_index()
    ix = device_index(s)
    Q = s.queries.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid])
    L = max(top_n, 16)
    p = search.TopologySearchParams(top_l=L, search_width=2, max_expansions=4096)
    q8 = s.queries.cuda().to(torch.uint8).contiguous()
    cand, _ = search.beam_search(ix, p, eo, ei, queries=q8, capacity=p.capacity(top_n))
    if float_queries:
        q = s.queries.cuda().float().contiguous() + 0.25     # not uint8-valued: float arithmetic on uint8 rows
        q_np = q.cpu().numpy()
    else:
        q, q_np = q8, q8.cpu().numpy()
    rp = search.RerankExactParams(top_k=top_k, top_n=top_n, rank_tile_size=tile, use_early_stop=True,
                                  early_stop_min_prefix=2 * tile, early_stop_patience_tiles=2)
    d, i, n_exact, _ = search.rerank_exact(ix, rp, cand, q)
    rd, ri, rn, _ = orc.rerank(np_u32(cand), q_np, host_pages(host), np.uint8, top_n=top_n, top_k=top_k, tile=tile,
                               vectors_per_page=host["vpp"], page_bytes=4096, vector_bytes=host["vb"],
                               early_stop_min_prefix=2 * tile, early_stop_patience_tiles=2)
    assert n_exact == rn
    assert np.array_equal(np_u32(i), ri)
    assert np.array_equal(d.cpu().numpy().view(np.uint32), rd.view(np.uint32))


@pytest.mark.parametrize("owners,float_queries", [(4, False), (3, True), (7, False)])
def test_rerank_by_owner_matches_plain_rerank(owners, float_queries):
    """Candidate lists split by the owner of the rows, every owner's list scored against its slice of the vector
    pages alone, the per-owner top-k lists merged: ids and distance bits of the plain rerank of the whole list."""
    import ctypes as C
    import dataclasses
    s, host = small_index()
    ix = device_index(s)
    lib = capi.load()
    Q, N = s.queries.shape[0], ix.num_nodes
    top_n, k = 200, 10
    eo, ei = fixed_entries(Q, [s.medoid])
    p = search.TopologySearchParams(top_l=top_n, search_width=2, max_expansions=4096)
    q8 = s.queries.cuda().to(torch.uint8).contiguous()
    cand, _ = search.beam_search(ix, p, eo, ei, queries=q8, capacity=p.capacity(top_n))
    q = (s.queries.cuda().float().contiguous() + 0.5) if float_queries else q8
    rp = search.RerankExactParams(top_k=k, top_n=top_n)
    d, i, _, _ = search.rerank_exact(ix, rp, cand, q)
    want_d, want_i = search.topk_pack(d, i, k)
    vpp = ix.vectors_per_page
    rows = ((N + owners - 1) // owners + vpp - 1) // vpp * vpp
    ptr = lambda t: C.c_void_p(t.data_ptr())
    for slot in (top_n, 8):
        parts = torch.empty((owners, Q, slot, 2), dtype=torch.int32, device="cuda")
        overflow = torch.zeros(1, dtype=torch.int32, device="cuda")
        capi.check(lib.tann_partition_candidates(ptr(cand), cand.shape[1], top_n, Q, rows, owners, slot, ptr(parts),
                                                 ptr(overflow), None))
        if slot < top_n:
            assert int(overflow.item()) == 1      # the mixture's candidates crowd into few owners
            continue
        assert int(overflow.item()) == 0
        raw = parts.cpu().numpy().view(np.uint32)          # records are (distance bits, id)
        all_ids = np_u32(cand)[:, :top_n, 1]
        for o in range(owners):                   # every candidate sits in its owner's list, in rank order
            for qi in (0, Q // 2, Q - 1):
                valid = all_ids[qi] != 0xffffffff
                rid = all_ids[qi] & 0x7fffffff
                pick = valid & (rid // rows == o)
                assert np.array_equal(raw[o, qi, :pick.sum(), 1], rid[pick] - o * rows)
                assert np.array_equal(raw[o, qi, :pick.sum(), 0], np_u32(cand)[qi, :top_n, 0][pick])
                assert (raw[o, qi, pick.sum():, 1] == 0xffffffff).all()
        lists_d = torch.empty((owners, Q, k), dtype=torch.float32, device="cuda")
        lists_i = torch.empty((owners, Q, k), dtype=torch.int32, device="cuda")
        for o in range(owners):
            n_o = min(rows, N - o * rows)
            first_page = o * rows // vpp
            local = dataclasses.replace(ix, num_nodes=n_o,
                                        vector_pages=ix.vector_pages[first_page * ix.page_bytes:])
            od, oi, _, _ = search.rerank_exact(local, search.RerankExactParams(top_k=k, top_n=slot), parts[o], q)
            pd, pi = search.topk_pack(od, oi, k)
            lists_d[o], lists_i[o] = pd, pi
        out_d = torch.empty((Q, k), dtype=torch.float32, device="cuda")
        out_i = torch.empty((Q, k), dtype=torch.int32, device="cuda")
        capi.check(lib.tann_merge_topk_lists(ptr(lists_d), ptr(lists_i), owners, Q, k, rows, ptr(out_d), ptr(out_i), None))
        assert torch.equal(out_i, want_i)
        assert np.array_equal(out_d.cpu().numpy().view(np.uint32), want_d.cpu().numpy().view(np.uint32))


def test_rerank_int8_vectors():
    """Stored int8 vectors (the third scalar kind of the vector store) with int8 and float queries."""
    s, host = small_index()
    Q = s.queries.shape[0]
    v8 = (s.vectors.to(torch.int16) - 128).to(torch.int8).cuda().contiguous()          # signed copy of the uint8 data
    base = device_index(s)
    ix = search.device_index_from_arrays(adjacency=host["adjacency"], codes=host["codes"], vectors=v8.cpu().numpy(),
                                         pq_tables_row_major=host["pq_tables"], pq_centroid=host["pq_centroid"],
                                         pq_chunk_offsets=host["pq_chunk_offsets"])
    assert ix.vector_kind == capi.KIND_INT8
    eo, ei = fixed_entries(Q, [s.medoid])
    p = search.TopologySearchParams(top_l=64, search_width=2, max_expansions=4096)
    cand, _ = search.beam_search(base, p, eo, ei, queries=s.queries.cuda().contiguous(), capacity=p.capacity(48))
    pages, vpp, vb = pipeline.vectors_to_pages(v8.cpu().numpy())
    rp = search.RerankExactParams(top_k=10, top_n=48)
    q_i8 = (s.queries - 128).clamp(-128, 127).to(torch.int8).cuda().contiguous()
    for qt in (q_i8, q_i8.float().contiguous()):
        d, i, n_exact, _ = search.rerank_exact(ix, rp, cand, qt)
        rd, ri, rn, _ = orc.rerank(np_u32(cand), qt.cpu().numpy(), pages, np.int8, top_n=48, top_k=10,
                                   vectors_per_page=vpp, page_bytes=4096, vector_bytes=vb)
        assert n_exact == rn
        assert np.array_equal(np_u32(i), ri)
        assert np.array_equal(d.cpu().numpy().view(np.uint32), rd.view(np.uint32))


def host_pages(host):
    if host.get("pages") is None:
        pages, vpp, vb = pipeline.vectors_to_pages(host["vectors"])
        host["pages"], host["vpp"], host["vb"] = pages, vpp, vb
    return host["pages"]


def test_rvq_entries_match_checker():
    s, host = small_index(name="cfg2", num_nodes=40000, components=40, num_queries=300)
    model = search.rvq_model_from_synth(s)
    q = s.queries.cuda().contiguous()
    for entry_count in (128, 3):
        offs, ids, clusters = model.device_entry_batch(q, entry_count)
        rc, _, _ = orc.rvq_clusters(s.queries.cpu().numpy(), host["rvq_coarse"], host["rvq_fine"], host["rvq_sizes"])
        assert np.array_equal(clusters.cpu().numpy(), rc)
        want = orc.rvq_gather(rc, host["rvq_offsets"], host["rvq_ids"], entry_count)
        assert np.array_equal(np_u32(ids), want)
        assert np.array_equal(np_u32(offs), np.arange(q.shape[0] + 1, dtype=np.uint32) * entry_count)
    # empty buckets are skipped and a model with no usable bucket falls back
    empty = search.RvqModel(dim=model.dim, coarse=model.coarse, fine=model.fine,
                            bucket_sizes=torch.zeros_like(model.bucket_sizes),
                            cluster_offsets=torch.zeros_like(model.cluster_offsets), cluster_ids=model.cluster_ids)
    _, ids, _ = empty.device_entry_batch(q[:4], 4, fallback_entry=77)
    assert np_u32(ids).tolist() == [[77, INVALID, INVALID, INVALID]] * 4


@pytest.mark.parametrize("coarse,fine", [(512, 384), (258, 130)])
def test_rvq_entries_with_codebooks_larger_than_shared_memory(coarse, fine):
    # a 512-centroid level of 128 floats does not fit beside a query tile: the levels are streamed in tiles;
    # sizes that are not multiples of 4 take the row-at-a-time kernel
    s, host = small_index(name="cfg2", num_nodes=60000, components=60, num_queries=700, rvq_coarse=coarse, rvq_fine=fine)
    assert host["rvq_coarse"].shape[0] == coarse and host["rvq_fine"].shape[0] == fine
    model = search.rvq_model_from_synth(s)
    q = s.queries.cuda().contiguous()
    offs, ids, clusters = model.device_entry_batch(q, 128)
    rc, _, _ = orc.rvq_clusters(s.queries.cpu().numpy(), host["rvq_coarse"], host["rvq_fine"], host["rvq_sizes"])
    assert np.array_equal(clusters.cpu().numpy(), rc)
    assert np.array_equal(np_u32(ids), orc.rvq_gather(rc, host["rvq_offsets"], host["rvq_ids"], 128))


def test_rvq_clusters_agree_with_gemm_scores():
    """The reference scores RVQ levels with a cuBLAS FP32 GEMM (distance_kernel.cu:114-124), whose summation
    order is not published, so bit parity cannot be pinned there. This test measures the next best thing:
    the clusters chosen by this library's ascending-k FMA scores against clusters chosen from GEMM scores
    (torch.matmul = cuBLAS SGEMM, TF32 off) with the same formula and selection rules. They must agree
    except where the two best scores are numerically tied."""
    s, host = small_index(name="cfg2", num_nodes=40000, components=40, num_queries=300)
    model = search.rvq_model_from_synth(s)
    g = torch.Generator(device="cuda").manual_seed(11)
    pick = torch.randint(0, s.vectors.shape[0], (20000,), generator=g, device="cuda")
    q = (s.vectors.cuda()[pick].float() + torch.randn((20000, model.dim), generator=g, device="cuda") * 10.0).contiguous()
    _, _, clusters = model.device_entry_batch(q, 8)
    torch.backends.cuda.matmul.allow_tf32 = False
    coarse, fine = model.coarse.float(), model.fine.float()
    nf = fine.shape[0]

    def scores(x, book):
        return (-2.0 * (x @ book.t()) + (x * x).sum(1, keepdim=True)) + (book * book).sum(1)[None, :]

    d0 = scores(q, coarse)
    c_star = d0.argmin(1)
    resid = q - coarse[c_star]
    d1 = scores(resid, fine)
    sizes = model.bucket_sizes.view(coarse.shape[0], nf)[c_star]
    d1 = torch.where(sizes > 0, d1, torch.full_like(d1, float("inf")))
    f_star = d1.argmin(1)
    want = (c_star * nf + f_star).to(torch.int32)
    same = clusters == want
    agreement = float(same.float().mean())
    assert agreement >= 0.999, agreement
    # every disagreement is a numerical tie of the two best scores at one of the levels
    bad = (~same).nonzero().flatten()
    for i in bad.tolist():
        t0 = torch.topk(d0[i], 2, largest=False).values
        t1 = torch.topk(d1[i], 2, largest=False).values
        gap0 = float((t0[1] - t0[0]) / t0[1].abs().clamp_min(1e-12))
        gap1 = float((t1[1] - t1[0]) / t1[1].abs().clamp_min(1e-12))
        assert min(gap0, gap1) < 1e-4, (i, gap0, gap1)


def test_pipelined_searchers_give_the_results_of_single_calls():
    """tann_searcher_submit / tann_searcher_wait: two searchers on two streams, batches submitted alternately,
    page-locked and pageable buffers; every batch equals the blocking call's answer."""
    s, host = small_index(name="cfg2", num_nodes=40000, components=40, num_queries=300)
    ix = device_index(s)
    model = search.rvq_model_from_synth(s)
    lanes = []
    for _ in range(2):
        sr = search.Searcher(ix, 512, 128, 64, 128)
        sr.set_rvq(model, 128)
        lanes.append((sr, torch.cuda.Stream()))
    tp = search.TopologySearchParams(top_l=32, search_width=2, max_expansions=4096)
    rp = search.RerankExactParams(top_k=10, top_n=32)
    q = s.queries.cpu().numpy()
    batches = [np.ascontiguousarray(q[i * 50:(i + 1) * 50 + 17]) for i in range(5)]
    want = [lanes[0][0].run_host(b, tp, rp)[:2] for b in batches]
    pinned = [torch.from_numpy(b).pin_memory().numpy() for b in batches]
    outs = []
    for i, b in enumerate(batches):
        n = b.shape[0]
        if i % 2 == 0:   # page-locked in and out
            oi = torch.empty((n, 10), dtype=torch.int32).pin_memory().numpy().view(np.uint32)
            od = torch.empty((n, 10), dtype=torch.float32).pin_memory().numpy()
            src = pinned[i]
        else:            # pageable: staged inside the searcher
            oi, od, src = np.empty((n, 10), np.uint32), np.empty((n, 10), np.float32), b
        outs.append((oi, od))
        sr, st = lanes[i % 2]
        sr.wait()
        sr.submit_host(src, tp, rp, oi, od, stream=st)
    with pytest.raises(capi.TannError, match="has not been waited for"):
        lanes[0][0].submit_host(batches[0], tp, rp, *outs[0], stream=lanes[0][1])
    for sr, _ in lanes:
        sr.wait()
        sr.wait()   # nothing pending: no-op
    for (oi, od), (wi, wd) in zip(outs, want):
        assert np.array_equal(oi, wi) and np.array_equal(od.view(np.uint32), wd.view(np.uint32))
    for sr, _ in lanes:
        sr.close()


def test_full_pipeline_matches_checker_with_rvq():
    s, host = small_index(name="cfg2", num_nodes=40000, components=40, num_queries=300)
    ix = device_index(s)
    model = search.rvq_model_from_synth(s)
    sr = search.Searcher(ix, 512, 128, 64, 128)
    sr.set_rvq(model, 128)
    for L, top_n in ((16, 32), (64, 32), (128, 64)):
        tp = search.TopologySearchParams(top_l=L, search_width=2, max_expansions=4096)
        rp = search.RerankExactParams(top_k=10, top_n=top_n)
        ids, dists, stats = sr.run_host(s.queries.cpu().numpy(), tp, rp, want_stats=True)
        ref = pipeline.run(host, s.queries.cpu().numpy(), top_l=L, search_width=2, max_expansions=4096,
                           top_n=top_n, top_k=10, entry_count=128)
        assert np.array_equal(ids, ref["topk_ids"])
        assert np.array_equal(dists.view(np.uint32), ref["topk_dists"].view(np.uint32))
        assert np.array_equal(stats, ref["stats"])
        # uint8 queries through the same call give the same answer (integer rerank path)
        ids8, dists8, _ = sr.run_host(s.queries.cpu().numpy().astype(np.uint8), tp, rp)
        assert np.array_equal(ids8, ids) and np.array_equal(dists8, dists)
    sr.close()


def test_searcher_reports_an_entry_id_outside_the_index():
    """A fixed entry list with an id beyond the index: the id is skipped as the reference skips it (the results are
    those of the valid entries) and the call answers TANN_ERR_DEVICE_CHECK from the device status word."""
    s, _ = small_index()
    ix = device_index(s)
    sr = search.Searcher(ix, 64, 64, 32, 8)
    tp = search.TopologySearchParams(top_l=32, search_width=2, max_expansions=512)
    rp = search.RerankExactParams(top_k=10, top_n=32)
    q = s.queries[:32].cpu().numpy()
    good_ids, good_d, _ = sr.run_host(q, tp, rp, fixed_entries=np.array([s.medoid, 7], np.uint32))
    ids = np.zeros((32, 10), np.uint32)
    dists = np.zeros((32, 10), np.float32)
    with pytest.raises(capi.TannError) as err:
        sr.run_host(q, tp, rp, fixed_entries=np.array([s.medoid, ix.num_nodes + 3, 7], np.uint32), out_ids=ids, out_dists=dists)
    assert err.value.status == 4 and "status bits 0x1" in err.value.message
    assert np.array_equal(ids, good_ids) and np.array_equal(dists, good_d)
    again, _, _ = sr.run_host(q, tp, rp, fixed_entries=np.array([s.medoid, 7], np.uint32))   # the word is cleared per run
    assert np.array_equal(again, good_ids)
    sr.close()


def test_pq2_refine_and_bound_filter_float32():
    s, host = small_index(name="cfg3", num_nodes=12000, components=60, num_queries=128)
    ix = device_index(s)
    q = s.queries.cuda().contiguous()
    Q = q.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid])
    p = search.TopologySearchParams(top_l=64, search_width=2, max_expansions=2048)
    cand, stats = search.beam_search(ix, p, eo, ei, queries=q)
    off = ix.pq_chunk_offsets
    t2 = s.pq2_tables.cuda().contiguous()
    c2 = s.pq2_centroid.cuda().contiguous()
    lut2 = search.lut_build(ix, q, tables_col_major=t2.t().contiguous(), centroid=c2, chunk_offsets=off)
    cross = search.pq2_cross_terms(off, s.pq_tables.cuda().contiguous(), ix.pq_centroid, t2, c2)
    assert np.array_equal(cross.cpu().numpy(), host["pq2_cross"])
    codes2 = s.pq2_codes.cuda().contiguous()
    ref_lut2 = orc.lut_build(s.queries.cpu().numpy(), host["pq2_tables"], host["pq2_centroid"], host["pq_chunk_offsets"])
    np.testing.assert_allclose(lut2.cpu().numpy(), ref_lut2, rtol=1e-5)
    for residual in (True, False):
        refined = search.pq2_refine(cand, stats, 64, codes2, lut2, base_codes=ix.codes if residual else None,
                                    cross_terms=cross if residual else None)
        want = orc.pq2_refine(np_u32(cand), np_u32(stats), 64, host["pq2_codes"], ref_lut2,
                              host["codes"] if residual else None, host["pq2_cross"] if residual else None)
        assert np.array_equal(np_u32(refined), want)
    refined = search.pq2_refine(cand, stats, 64, codes2, lut2, base_codes=ix.codes, cross_terms=cross)
    err = s.pq2_error_bounds.cuda().contiguous()
    for tile, bound in ((16, True), (1, True), (0, False), (16, False)):
        rp = search.RerankExactParams(top_k=10, top_n=64, rank_tile_size=tile, use_pq2_bound_filter=bound)
        d, i, n_exact, n_filt = search.rerank_exact(ix, rp, refined, q, error_bounds=err if bound else None)
        rd, ri, rn, rf = orc.rerank(np_u32(refined), s.queries.cpu().numpy(), host_pages(host), np.float32,
                                    top_n=64, top_k=10, tile=tile, vectors_per_page=host["vpp"], page_bytes=4096,
                                    vector_bytes=host["vb"], error_bounds=host["pq2_error_bounds"] if bound else None)
        assert (n_exact, n_filt) == (rn, rf)
        assert np.array_equal(np_u32(i), ri)
        np.testing.assert_allclose(d.cpu().numpy(), rd, rtol=1e-5)
        assert np.array_equal(d.cpu().numpy().view(np.uint32), rd.view(np.uint32))


def test_hpq_refine_matches_checker():
    """Hybrid-PQ refine (src/search/rerank_exact.cu:667-771): per chunk a selector bit picks the base or the
    outlier codebook's query table. The second codebook of the float configuration stands in for the outlier
    codebook; selector bits are random. With all bits clear it is the plain refine with the base table."""
    s, host = small_index(name="cfg3", num_nodes=12000, components=60, num_queries=128)
    ix = device_index(s)
    q = s.queries.cuda().contiguous()
    Q = q.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid])
    p = search.TopologySearchParams(top_l=64, search_width=2, max_expansions=2048)
    cand, stats = search.beam_search(ix, p, eo, ei, queries=q)
    off = ix.pq_chunk_offsets
    base_lut = search.lut_build(ix, q)
    outlier_lut = search.lut_build(ix, q, tables_col_major=s.pq2_tables.cuda().t().contiguous(),
                                   centroid=s.pq2_centroid.cuda().contiguous(), chunk_offsets=off)
    N, M = host["codes"].shape
    rng = np.random.default_rng(11)
    bits = rng.integers(0, 2, size=(N, M), dtype=np.uint8)
    hybrid = np.where(bits == 1, host["pq2_codes"], host["codes"]).astype(np.uint8)
    selectors = np.packbits(bits, axis=1, bitorder="little")
    assert selectors.shape == (N, (M + 7) // 8)
    for lr in (64, 48):
        got = search.hpq_refine(cand, stats, lr, _dev(hybrid), _dev(selectors), base_lut, outlier_lut)
        want = orc.hpq_refine(np_u32(cand), np_u32(stats), lr, hybrid, selectors, base_lut.cpu().numpy(),
                              outlier_lut.cpu().numpy())
        assert np.array_equal(np_u32(got), want)
    zero = np.zeros_like(selectors)
    got = search.hpq_refine(cand, stats, 64, ix.codes, _dev(zero), base_lut, outlier_lut)
    plain = search.pq2_refine(cand, stats, 64, ix.codes, base_lut)
    assert torch.equal(got, plain)


def test_sharded_and_cached_providers_give_the_same_result():
    s, host = small_index()
    ix = device_index(s)
    q = s.queries.cuda().contiguous()
    Q = q.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid])
    p = search.TopologySearchParams(top_l=64, search_width=2, max_expansions=4096)
    cap = p.capacity(32)
    base_cand, base_stats = search.beam_search(ix, p, eo, ei, queries=q, capacity=cap)
    rp = search.RerankExactParams(top_k=10, top_n=32)
    base_d, base_i, _, _ = search.rerank_exact(ix, rp, base_cand, q)
    # node-id-range shards (here all on one device): rows_per_shard is a multiple of vectors/page
    G = 4
    vpp = ix.vectors_per_page
    rps = ((ix.num_nodes + G - 1) // G + vpp - 1) // vpp * vpp
    adj_parts, code_parts, vec_parts = [], [], []
    for g in range(G):
        lo, hi = g * rps, min(ix.num_nodes, (g + 1) * rps)
        adj_parts.append(ix.adjacency[lo:hi].clone())
        code_parts.append(ix.codes[lo:hi].clone())
        vec_parts.append(ix.vector_pages[(lo // vpp) * 4096:((hi + vpp - 1) // vpp) * 4096].clone())
    sharded = search.DeviceIndex(
        num_nodes=ix.num_nodes, degree=ix.degree, dim=ix.dim, vector_kind=ix.vector_kind,
        pq_tables_col_major=ix.pq_tables_col_major, pq_centroid=ix.pq_centroid, pq_chunk_offsets=ix.pq_chunk_offsets,
        vector_bytes=ix.vector_bytes, vectors_per_page=vpp, page_bytes=4096,
        adjacency_bases=[t.data_ptr() for t in adj_parts], codes_bases=[t.data_ptr() for t in code_parts],
        vector_bases=[t.data_ptr() for t in vec_parts], rows_per_shard=rps, keepalive=[adj_parts, code_parts, vec_parts])
    cand, stats = search.beam_search(sharded, p, eo, ei, queries=q, capacity=cap)
    assert torch.equal(cand, base_cand) and torch.equal(stats, base_stats)
    d, i, _, _ = search.rerank_exact(sharded, rp, cand, q)
    assert torch.equal(d, base_d) and torch.equal(i, base_i)
    # pinned-host (UVA) topology behind an HBM cache of the first rows
    lib = capi.load()
    nbytes = ix.adjacency.numel() * 4
    hp, dp = C.c_void_p(), C.c_void_p()
    capi.check(lib.tann_host_alloc_mapped(nbytes, C.byref(hp), C.byref(dp)))
    try:
        adj_host = ix.adjacency.cpu().numpy()   # keep the array alive across the copy
        C.memmove(hp.value, adj_host.ctypes.data, nbytes)
        for cached_rows in (0, ix.num_nodes // 3):
            hosted = search.DeviceIndex(
                num_nodes=ix.num_nodes, degree=ix.degree, dim=ix.dim, vector_kind=ix.vector_kind, codes=ix.codes,
                vector_pages=ix.vector_pages, pq_tables_col_major=ix.pq_tables_col_major, pq_centroid=ix.pq_centroid,
                pq_chunk_offsets=ix.pq_chunk_offsets, vector_bytes=ix.vector_bytes, vectors_per_page=vpp,
                adjacency_bases=[dp.value], adjacency_cache=ix.adjacency[:max(cached_rows, 1)].clone() if cached_rows else None,
                adjacency_cached_rows=cached_rows)
            cand, stats = search.beam_search(hosted, p, eo, ei, queries=q, capacity=cap)
            torch.cuda.synchronize()
            assert torch.equal(cand, base_cand) and torch.equal(stats, base_stats)
    finally:
        torch.cuda.synchronize()
        capi.check(lib.tann_host_free(hp))


def test_wide_float_configuration_with_pinned_host_vectors():
    """The 768-dimensional float configuration in miniature: M = 96 chunks of 8 dims (the widest specialised
    table), 3 KB vectors at one per page, vector pages in mapped pinned host memory read over UVA, RVQ entries."""
    s, host = small_index(name="cfg5", num_nodes=6000, components=12, num_queries=64)
    assert s.vectors.shape[1] == 768 and s.pq_codes.shape[1] == 96
    ix = device_index(s)
    q = s.queries.cuda().contiguous()
    Q = q.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid, 17])
    p = search.TopologySearchParams(top_l=128, search_width=2, max_expansions=4096)
    cap = p.capacity(64)
    cand, stats = search.beam_search(ix, p, eo, ei, queries=q, capacity=cap)
    lut_ref = orc.lut_build(s.queries.cpu().numpy(), host["pq_tables"], host["pq_centroid"], host["pq_chunk_offsets"])
    ref_cand, ref_stats = orc.beam_search(host["adjacency"], host["codes"], lut_ref, np_u32(eo), np_u32(ei), top_l=128,
                                          search_width=2, max_expansions=4096, capacity=cap)
    assert_candidates_equal(cand, stats, ref_cand, ref_stats)
    rp = search.RerankExactParams(top_k=10, top_n=64)
    rd, ri, rn, _ = orc.rerank(ref_cand, s.queries.cpu().numpy(), host_pages(host), np.float32, top_n=64, top_k=10,
                               vectors_per_page=host["vpp"], page_bytes=4096, vector_bytes=host["vb"])
    lib = capi.load()
    nbytes = ix.vector_pages.numel()
    hp, dp = C.c_void_p(), C.c_void_p()
    capi.check(lib.tann_host_alloc_mapped(nbytes, C.byref(hp), C.byref(dp)))
    try:
        pages_host = ix.vector_pages.cpu().numpy()          # keep the array alive across the copy
        C.memmove(hp.value, pages_host.ctypes.data, nbytes)
        hosted = search.DeviceIndex(
            num_nodes=ix.num_nodes, degree=ix.degree, dim=ix.dim, vector_kind=ix.vector_kind, adjacency=ix.adjacency,
            codes=ix.codes, pq_tables_col_major=ix.pq_tables_col_major, pq_centroid=ix.pq_centroid,
            pq_chunk_offsets=ix.pq_chunk_offsets, vector_bytes=ix.vector_bytes, vectors_per_page=ix.vectors_per_page,
            vector_bases=[dp.value])
        for index in (ix, hosted):
            d, i, n_exact, _ = search.rerank_exact(index, rp, cand, q)
            torch.cuda.synchronize()
            assert n_exact == rn
            assert np.array_equal(np_u32(i), ri)
            assert np.array_equal(d.cpu().numpy().view(np.uint32), rd.view(np.uint32))
    finally:
        torch.cuda.synchronize()
        capi.check(lib.tann_host_free(hp))


def test_neighbor_code_layout_gives_identical_results():
    """The optional layout that stores every node's neighbours' PQ codes next to each other only changes
    where the code rows are read from: candidates and statistics stay bit-identical, also with padded
    adjacency rows and through the searcher."""
    s, host = small_index()
    ix = device_index(s)
    q = s.queries.cuda().contiguous()
    Q = q.shape[0]
    eo, ei = fixed_entries(Q, [s.medoid, 3])
    inl = search.inline_neighbor_codes(device_index(s))
    assert inl.neighbor_codes.shape == (ix.num_nodes, ix.degree, ix.num_chunks)
    for top_l, width in ((64, 2), (16, 1), (256, 4)):
        p = search.TopologySearchParams(top_l=top_l, search_width=width, max_expansions=4096)
        cand, stats = search.beam_search(ix, p, eo, ei, queries=q)
        cand2, stats2 = search.beam_search(inl, p, eo, ei, queries=q)
        assert torch.equal(cand, cand2) and torch.equal(stats, stats2)
    # padded rows (0xffffffff slots) and the whole path
    pad = search.device_index_from_arrays(adjacency=formats.pad_degree(host["adjacency"], 64), codes=host["codes"],
                                          vectors=host["vectors"], pq_tables_row_major=host["pq_tables"],
                                          pq_centroid=host["pq_centroid"], pq_chunk_offsets=host["pq_chunk_offsets"])
    p = search.TopologySearchParams(top_l=64, search_width=2, max_expansions=4096)
    base_cand, base_stats = search.beam_search(pad, p, eo, ei, queries=q)
    search.inline_neighbor_codes(pad)
    cand3, stats3 = search.beam_search(pad, p, eo, ei, queries=q)
    assert torch.equal(base_cand, cand3) and torch.equal(base_stats, stats3)
    sr = search.Searcher(inl, Q, 128, 64, 128)
    sr2 = search.Searcher(ix, Q, 128, 64, 128)
    rp = search.RerankExactParams(top_k=10, top_n=32)
    fe = np.array([s.medoid, 3], np.uint32)
    ids_a, d_a, st_a = sr.run_host(s.queries.cpu().numpy(), p, rp, fixed_entries=fe, want_stats=True)
    ids_b, d_b, st_b = sr2.run_host(s.queries.cpu().numpy(), p, rp, fixed_entries=fe, want_stats=True)
    assert np.array_equal(ids_a, ids_b) and np.array_equal(d_a, d_b) and np.array_equal(st_a, st_b)
    sr.close()
    sr2.close()


def test_parameter_errors_are_reported():
    s, _ = small_index()
    ix = device_index(s)
    eo, ei = fixed_entries(1, [0])
    q = s.queries[:1].cuda().contiguous()
    for kw, msg in ((dict(top_l=0), "top_l must be positive"), (dict(top_l=8, search_width=33), "at most 32"),
                    (dict(top_l=8, search_width=0), "search_width must be positive"),
                    (dict(top_l=8, max_expansions=0), "max_expansions must be positive")):
        with pytest.raises(capi.TannError, match=msg):
            search.beam_search(ix, search.TopologySearchParams(**{**dict(search_width=1), **kw}), eo, ei, queries=q,
                               capacity=8)
    with pytest.raises(capi.TannError, match="shared memory requirement"):
        search.beam_search(ix, search.TopologySearchParams(top_l=16384, search_width=1), eo, ei, queries=q)


def test_full_size_index_properties():
    """The 10 M-vector configuration at full size (10 k queries): properties that hold at any size (the
    checker is not run here) - determinism, sorted output, exact integer distances recomputed on the host,
    statistics within their bounds, recall against brute-force ground truth."""
    import dataclasses

    from topoanns_b200 import synth
    cfg = dataclasses.replace(synth.CONFIGS["cfg2"], kmeans_iters=5)
    s = synth.build(cfg, "cuda")
    assert s.vectors.shape[0] == 10_000_000 and s.queries.shape[0] == 10_000
    ix = device_index(s)
    model = search.rvq_model_from_synth(s)
    sr = search.Searcher(ix, 10_000, 256, 256, 128)
    sr.set_rvq(model, 128)
    tp = search.TopologySearchParams(top_l=128, search_width=2, max_expansions=4096)
    rp = search.RerankExactParams(top_k=10, top_n=64)
    qn = s.queries.cpu().numpy()
    ids, dists, stats = sr.run_host(qn, tp, rp, want_stats=True)
    ids2, dists2, _ = sr.run_host(qn, tp, rp)
    assert np.array_equal(ids, ids2) and np.array_equal(dists, dists2)          # deterministic
    assert (np.diff(dists, axis=1) >= 0).all()                                   # sorted
    valid = ids != INVALID
    assert valid.all()
    picked = s.vectors[torch.from_numpy(ids.astype(np.int64)).cuda()].cpu().numpy().astype(np.int64)   # [Q, k, d]
    want = ((picked - qn.astype(np.int64)[:, None, :]) ** 2).sum(2)
    assert np.array_equal(dists.astype(np.int64), want)                          # exact integer distances
    assert (stats[:, 0] >= stats[:, 1]).all() and (stats[:, 1] <= 4096 + 1).all()
    assert (stats[:, 4] <= 256).all()
    # wider rerank: the operating region of the benchmark reaches its recall bar
    ids3, _, _ = sr.run_host(qn, search.TopologySearchParams(top_l=16, search_width=2, max_expansions=4096),
                             search.RerankExactParams(top_k=10, top_n=256))
    from topoanns_b200.synth import recall_at_k
    assert recall_at_k(ids3, s.gt_ids.cpu().numpy(), 10) >= 0.95
    sr.close()
