"""Learned rerank stop of the reference's persistent rerank (src/io/bam_vector_provider.cu:125-279 model
file, :542-617 logit, :721-1323 kernel): model-file folding, the checker's rule on a hand-made case, and
the CUDA kernel against the checker on seeded indexes (bit for bit: lists, stop prefixes, checkpoint
counts, exact / filtered counts)."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import oracle as orc
from oracle import pipeline

INVALID = 0xFFFFFFFF

MODEL_13 = """# 13-feature model
stage_prefixes = 16, 32, 64, 96, 128, 300
feature_means = 5,0.5,100,1,1,0.5,0.2,50,0.5,3,0.7,0.3,0.8
feature_inv_stds = 0.5,2,0.01,0.3,0.3,2,4,0.02,2,0.1,3,3,2.5
weights = 0.1,-0.7,0.003,0.5,0.25,0.8,0.4,-0.01,0.6,0.05,0.2,-0.2,0.3
bias = 0.25
threshold_logit = {threshold}
bootstrap_prefix = 16
"""

MODEL_NO_NEXT_WINDOW = MODEL_13 + "feature_mask = 1,1,1,1,1,1,1,1,0,0,1,1,1\n"
MODEL_SIX = MODEL_13 + "feature_mask = 1,1,1,0,0,1,0,1,0,1,0,0,0\n"
MODEL_12 = """stage_prefixes = 8, 24, 40, 72, 104
feature_means = 5,0.5,100,1,1,0.2,50,0.5,3,0.7,0.3,0.8
feature_inv_stds = 0.5,2,0.01,0.3,0.3,4,0.02,2,0.1,3,3,2.5
weights = 0.1,-0.7,0.003,0.5,0.25,0.4,-0.01,0.0,0.0,0.2,-0.2,0.3
bias = 0.25
threshold_logit = {threshold}
threshold_logit_top_l_128 = {threshold}
bootstrap_prefix = 8
top_k = 10
"""


def _write(tmp_path, name, text):
    path = os.path.join(str(tmp_path), name)
    with open(path, "w") as fh:
        fh.write(text)
    return path


# ---- CPU: model file and the rule ------------------------------------------------------------------

def test_model_file_folding_matches_between_library_and_checker(tmp_path):
    from topoanns_b200 import capi
    lib = capi.load()
    for name, text in (("m13", MODEL_13), ("mask", MODEL_NO_NEXT_WINDOW), ("six", MODEL_SIX), ("m12", MODEL_12)):
        path = _write(tmp_path, name, text.format(threshold=-0.375))
        for budget in (128, 100, 64, 16, 8):
            want = orc.load_rerank_stop_model(path, budget, 10)
            got = capi.RerankLearnedStop()
            capi.check(lib.tann_rerank_learned_stop_load(path.encode(), budget, 10, C.byref(got)))
            assert bytes(got) == bytes(want), (name, budget)
    six = orc.load_rerank_stop_model(_write(tmp_path, "six2", MODEL_SIX.format(threshold=0)), 128, 10)
    assert six.feature_variant == 1 and six.linear_weights[3] == 0.0 and six.linear_weights[9] != 0.0
    m = orc.load_rerank_stop_model(_write(tmp_path, "m", MODEL_13.format(threshold=0)), 100, 10)
    # prefixes beyond the budget are dropped, those <= bootstrap_prefix are skipped at the start
    assert (m.enabled, m.num_stages, m.initial_stage_index) == (1, 4, 1)
    assert list(m.stage_prefixes[:4]) == [16, 32, 64, 96]
    old = orc.load_rerank_stop_model(_write(tmp_path, "o", MODEL_12.format(threshold=0)), 128, 0)
    # the older layout's churn ratio (index 5) is feature 6 now; feature 5 (changed flag) has no weight
    assert old.linear_weights[5] == 0.0 and old.linear_weights[6] == np.float32(0.4) * np.float32(4)
    assert old.top_k == 10
    # no bootstrap prefix or no stage inside the budget: model off
    off = orc.load_rerank_stop_model(_write(tmp_path, "off", MODEL_13.format(threshold=0)), 12, 10)
    assert off.enabled == 0


def test_model_file_errors(tmp_path):
    from topoanns_b200 import capi
    lib = capi.load()
    out = capi.RerankLearnedStop()
    assert lib.tann_rerank_learned_stop_load(b"/nonexistent/model", 64, 10, C.byref(out)) == 1
    assert b"Failed to open" in lib.tann_last_error()
    bad = _write(tmp_path, "bad", "stage_prefixes 1,2\n")
    assert lib.tann_rerank_learned_stop_load(bad.encode(), 64, 10, C.byref(out)) == 1
    assert b"Invalid learned-stop config line" in lib.tann_last_error()
    short = _write(tmp_path, "short", "weights = 1,2\nfeature_means = 1,2\nfeature_inv_stds = 1,2\n")
    assert lib.tann_rerank_learned_stop_load(short.encode(), 64, 10, C.byref(out)) == 1
    assert b"length 13 or 12" in lib.tann_last_error()


def _hand_case():
    """One query at the origin, 1-d float vectors v[i] = i + 1 (distance (i+1)^2), candidate list = nodes
    23, 22, ..., 0: every window of four ranks improves the best-2 list."""
    n = 24
    vectors = (np.arange(n, dtype=np.float32) + 1).reshape(n, 1)
    pages, vpp, vb = pipeline.vectors_to_pages(vectors)
    cand = np.zeros((1, n, 2), np.uint32)
    cand[0, :, 0] = np.arange(n, dtype=np.float32).view(np.uint32)   # approximate distances, unused without bounds
    cand[0, :, 1] = np.arange(n - 1, -1, -1, dtype=np.uint32)
    return cand, np.zeros((1, 1), np.float32), pages, vpp, vb


def _stop(stages, bootstrap, weights, bias, threshold, top_k=2, budget=24):
    m = orc.RerankStop()
    m.enabled, m.num_stages, m.top_k, m.bootstrap_prefix = 1, len(stages), top_k, bootstrap
    for i, p in enumerate(stages):
        m.stage_prefixes[i] = p
    while m.initial_stage_index < m.num_stages and m.stage_prefixes[m.initial_stage_index] <= bootstrap:
        m.initial_stage_index += 1
    for i, w in weights.items():
        m.linear_weights[i] = w
    m.bias, m.threshold_logit = bias, threshold
    m.budget_log2 = np.log2(np.float32(budget))
    m.inv_budget_top_n, m.inv_top_k = np.float32(1) / np.float32(budget), np.float32(1) / np.float32(top_k)
    return m


def test_checker_rule_on_a_hand_made_case():
    cand, q, pages, vpp, vb = _hand_case()
    kw = dict(top_n=24, top_k=2, tile=4, vectors_per_page=vpp, page_bytes=4096, vector_bytes=vb)
    # logit = 1 - 4 * prefix_frac: 1/3 at prefix 4 (bootstrap, no stage), -1/3 at prefix 8, -1 at 12 ...
    m = _stop([8, 12, 16], 4, {1: -4.0}, 1.0, -0.5)
    r = orc.rerank_learned(cand, q, pages, np.float32, model=m, **kw)
    assert (int(r["stop_prefixes"][0]), int(r["checkpoint_counts"][0]), int(r["stop_flags"][0])) == (12, 2, 1)
    assert r["n_exact"] == 12
    assert r["ids"][0].tolist() == [12, 13] and r["dists"][0].tolist() == [169.0, 196.0]
    # a threshold nothing reaches: all stages evaluated, then plain tiles to the end of the budget
    m = _stop([8, 12, 16], 4, {1: -4.0}, 1.0, -100.0)
    r = orc.rerank_learned(cand, q, pages, np.float32, model=m, **kw)
    assert (int(r["stop_prefixes"][0]), int(r["checkpoint_counts"][0]), int(r["stop_flags"][0])) == (24, 3, 0)
    assert r["ids"][0].tolist() == [0, 1] and r["n_exact"] == 24
    # entered-ratio feature: both list entries are replaced by every window, ratio 1 -> logit = -1 + 2 = 1
    m = _stop([8], 4, {6: 2.0}, -1.0, 0.5)
    r = orc.rerank_learned(cand, q, pages, np.float32, model=m, **kw)
    assert int(r["stop_flags"][0]) == 0 and int(r["checkpoint_counts"][0]) == 1
    # replay: the model is not evaluated, the query stops at the first window end >= its recorded prefix
    m = _stop([8, 12, 16], 4, {1: -4.0}, 1.0, -0.5)
    r = orc.rerank_learned(cand, q, pages, np.float32, model=m, replay=np.array([14], np.uint32), **kw)
    assert (int(r["stop_prefixes"][0]), int(r["checkpoint_counts"][0]), int(r["stop_flags"][0])) == (16, 0, 1)
    # no model: plain tiles, same best-2 as the full rerank
    r = orc.rerank_learned(cand, q, pages, np.float32, **kw)
    assert r["ids"][0].tolist() == [0, 1] and int(r["stop_prefixes"][0]) == 24


# ---- GPU: kernel against the checker -------------------------------------------------------------

def _gpu_imports():
    import torch
    from topoanns_b200 import capi, search
    import gpu_support as gs
    return torch, capi, search, gs


def _as_capi(model, capi):
    out = capi.RerankLearnedStop()
    C.memmove(C.byref(out), C.byref(model), C.sizeof(out))
    return out


def _compare(got, want, gs):
    assert np.array_equal(gs.np_u32(got["ids"]), want["ids"])
    assert np.array_equal(got["dists"].cpu().numpy().view(np.uint32), want["dists"].view(np.uint32))
    assert np.array_equal(gs.np_u32(got["stop_prefixes"]), want["stop_prefixes"])
    assert np.array_equal(gs.np_u32(got["checkpoint_counts"]), want["checkpoint_counts"])
    assert np.array_equal(gs.np_u32(got["stop_flags"]), want["stop_flags"])
    assert (got["n_exact"], got["n_filtered"]) == (want["n_exact"], want["n_filtered"])


@pytest.mark.gpu
def test_hand_made_case_on_the_gpu():
    torch, capi, search, gs = _gpu_imports()
    cand, q, pages, vpp, vb = _hand_case()
    n = 24
    vectors = (np.arange(n, dtype=np.float32) + 1).reshape(n, 1)
    ix = search.device_index_from_arrays(
        adjacency=np.full((n, 64), INVALID, np.uint32), codes=np.zeros((n, 1), np.uint8), vectors=vectors,
        pq_tables_row_major=np.zeros((256, 1), np.float32), pq_centroid=np.zeros(1, np.float32),
        pq_chunk_offsets=np.array([0, 1], np.uint32))
    dcand = torch.from_numpy(cand.view(np.int32)).cuda()
    dq = torch.from_numpy(q).cuda()
    rp = search.RerankExactParams(top_k=2, top_n=24, rank_tile_size=4)
    for m, replay in ((_stop([8, 12, 16], 4, {1: -4.0}, 1.0, -0.5), None),
                      (_stop([8, 12, 16], 4, {1: -4.0}, 1.0, -100.0), None),
                      (_stop([8], 4, {6: 2.0}, -1.0, 0.5), None),
                      (_stop([8, 12, 16], 4, {1: -4.0}, 1.0, -0.5), np.array([14], np.uint32)),
                      (None, None)):
        want = orc.rerank_learned(cand, q, pages, np.float32, top_n=24, top_k=2, tile=4, vectors_per_page=vpp,
                                  page_bytes=4096, vector_bytes=vb, model=m, replay=replay)
        got = search.rerank_exact_learned_stop(
            ix, rp, dcand, dq, model=_as_capi(m, capi) if m is not None else None,
            replay_stop_prefixes=torch.from_numpy(replay.view(np.int32)).cuda() if replay is not None else None)
        _compare(got, want, gs)


@pytest.mark.gpu
@pytest.mark.parametrize("model_text,threshold", [(MODEL_NO_NEXT_WINDOW, -0.2), (MODEL_NO_NEXT_WINDOW, 0.4),
                                                  (MODEL_12, -0.3), (MODEL_12, 0.3)])
def test_learned_stop_uint8_index(tmp_path, model_text, threshold):
    """uint8 index, no bound filter: models without next-window features; stop prefixes differ between
    queries; record -> replay gives the same lists."""
    torch, capi, search, gs = _gpu_imports()
    s, host = gs.small_index()
    ix = gs.device_index(s)
    Q = s.queries.shape[0]
    eo, ei = gs.fixed_entries(Q, [s.medoid])
    top_n = 128
    p = search.TopologySearchParams(top_l=top_n, search_width=2, max_expansions=4096)
    q = s.queries.cuda().to(torch.uint8).contiguous()
    cand, _ = search.beam_search(ix, p, eo, ei, queries=q, capacity=p.capacity(top_n))
    pages, vpp, vb = pipeline.vectors_to_pages(host["vectors"])
    path = _write(tmp_path, "model", model_text.format(threshold=threshold))
    model = search.load_rerank_learned_stop(path, top_n, 10)
    ref_model = orc.load_rerank_stop_model(path, top_n, 10)
    assert model.enabled == 1
    kw = dict(top_n=top_n, top_k=10, tile=16, vectors_per_page=vpp, page_bytes=4096, vector_bytes=vb)
    for early in (False, True):
        rp = search.RerankExactParams(top_k=10, top_n=top_n, rank_tile_size=16, use_early_stop=early,
                                      early_stop_min_prefix=48, early_stop_patience_tiles=2)
        for qt in (q, q.float().contiguous()):
            got = search.rerank_exact_learned_stop(ix, rp, cand, qt, model=model)
            want = orc.rerank_learned(gs.np_u32(cand), qt.cpu().numpy(), pages, np.uint8, model=ref_model,
                                      use_early_stop=early, early_stop_min_prefix=48, early_stop_patience_tiles=2, **kw)
            _compare(got, want, gs)
    prefixes = gs.np_u32(got["stop_prefixes"])
    assert int(got["checkpoint_counts"].sum()) > 0
    # replay of the recorded prefixes: same windows, no model evaluation, same lists
    rp = search.RerankExactParams(top_k=10, top_n=top_n, rank_tile_size=16)
    first = search.rerank_exact_learned_stop(ix, rp, cand, q, model=model)
    again = search.rerank_exact_learned_stop(ix, rp, cand, q, model=model, replay_stop_prefixes=first["stop_prefixes"])
    want = orc.rerank_learned(gs.np_u32(cand), q.cpu().numpy(), pages, np.uint8, model=ref_model,
                              replay=gs.np_u32(first["stop_prefixes"]), **kw)
    _compare(again, want, gs)
    assert torch.equal(again["ids"], first["ids"]) and torch.equal(again["stop_prefixes"], first["stop_prefixes"])
    assert int(again["checkpoint_counts"].sum()) == 0
    assert prefixes.min() >= 16 and prefixes.max() <= top_n
    # model off (file without bootstrap prefix): plain tiles over the whole budget = top-k of the full rerank
    off = capi.RerankLearnedStop()
    plain = search.rerank_exact_learned_stop(ix, rp, cand, q, model=off)
    d_full, i_full, _, _ = search.rerank_exact(ix, rp, cand, q)
    assert torch.equal(plain["ids"], i_full[:, :10]) and torch.equal(plain["dists"], d_full[:, :10])


@pytest.mark.gpu
@pytest.mark.parametrize("model_text,threshold", [(MODEL_13, -0.2), (MODEL_13, 0.5), (MODEL_SIX, 0.0),
                                                  (MODEL_SIX, 0.6)])
def test_learned_stop_float_index_with_bound_filter(tmp_path, model_text, threshold):
    """float32 index with residual pq2 and error bounds: bound filter on, next-window features in use."""
    torch, capi, search, gs = _gpu_imports()
    s, host = gs.small_index(name="cfg3", num_nodes=12000, components=60, num_queries=128)
    ix = gs.device_index(s)
    q = s.queries.cuda().contiguous()
    Q = q.shape[0]
    eo, ei = gs.fixed_entries(Q, [s.medoid])
    p = search.TopologySearchParams(top_l=128, search_width=2, max_expansions=2048)
    cand, stats = search.beam_search(ix, p, eo, ei, queries=q)
    off = ix.pq_chunk_offsets
    t2 = s.pq2_tables.cuda().contiguous()
    c2 = s.pq2_centroid.cuda().contiguous()
    lut2 = search.lut_build(ix, q, tables_col_major=t2.t().contiguous(), centroid=c2, chunk_offsets=off)
    cross = search.pq2_cross_terms(off, s.pq_tables.cuda().contiguous(), ix.pq_centroid, t2, c2)
    refined = search.pq2_refine(cand, stats, 128, s.pq2_codes.cuda().contiguous(), lut2, base_codes=ix.codes,
                                cross_terms=cross)
    err = s.pq2_error_bounds.cuda().contiguous()
    pages, vpp, vb = pipeline.vectors_to_pages(host["vectors"])
    path = _write(tmp_path, "model", model_text.format(threshold=threshold))
    for top_n in (128, 100):
        model = search.load_rerank_learned_stop(path, top_n, 10)
        ref_model = orc.load_rerank_stop_model(path, top_n, 10)
        rp = search.RerankExactParams(top_k=10, top_n=top_n, rank_tile_size=16, use_pq2_bound_filter=True)
        got = search.rerank_exact_learned_stop(ix, rp, refined, q, model=model, error_bounds=err)
        want = orc.rerank_learned(gs.np_u32(refined), s.queries.cpu().numpy(), pages, np.float32, top_n=top_n,
                                  top_k=10, tile=16, vectors_per_page=vpp, page_bytes=4096, vector_bytes=vb,
                                  model=ref_model, error_bounds=host["pq2_error_bounds"])
        _compare(got, want, gs)
        assert got["n_filtered"] > 0
    # a model with next-window features needs the lower bounds
    rp = search.RerankExactParams(top_k=10, top_n=128, rank_tile_size=16)
    with pytest.raises(RuntimeError, match="next-window features"):
        search.rerank_exact_learned_stop(ix, rp, refined, q, model=model)


@pytest.mark.gpu
def test_searcher_with_learned_stop_equals_the_staged_calls(tmp_path):
    """tann_searcher_set_rerank_learned_stop: the whole path with the learned stop gives what beam search +
    tann_rerank_exact_learned_stop give when called one after the other."""
    torch, capi, search, gs = _gpu_imports()
    s, host = gs.small_index()
    ix = gs.device_index(s)
    Q = s.queries.shape[0]
    top_n = 128
    tp = search.TopologySearchParams(top_l=top_n, search_width=2, max_expansions=4096)
    rp = search.RerankExactParams(top_k=10, top_n=top_n, rank_tile_size=16)
    q = s.queries.cuda().contiguous()
    eo, ei = gs.fixed_entries(Q, [s.medoid])
    cand, _ = search.beam_search(ix, tp, eo, ei, queries=q, capacity=tp.capacity(top_n))
    model = search.load_rerank_learned_stop(_write(tmp_path, "m", MODEL_NO_NEXT_WINDOW.format(threshold=0.1)), top_n, 10)
    want = search.rerank_exact_learned_stop(ix, rp, cand, q, model=model)
    sr = search.Searcher(ix, Q, tp.capacity(top_n), top_n, 4)
    sr.set_rerank_learned_stop(model)
    ids, dists, _ = sr.run_host(s.queries.cpu().numpy(), tp, rp, fixed_entries=np.array([s.medoid], np.uint32))
    assert np.array_equal(ids, gs.np_u32(want["ids"]))
    assert np.array_equal(dists.view(np.uint32), want["dists"].cpu().numpy().view(np.uint32))
    sr.set_rerank_learned_stop(None)
    ids2, _, _ = sr.run_host(s.queries.cpu().numpy(), tp, rp, fixed_entries=np.array([s.medoid], np.uint32))
    d_full, i_full, _, _ = search.rerank_exact(ix, rp, cand, q)
    assert np.array_equal(ids2, gs.np_u32(i_full[:, :10]))
    assert int(want["stop_prefixes"].float().mean()) < top_n
    sr.close()
