"""The reference's own implementation (its sources compiled in place into oracle/_ref by
oracle/ref_build.sh) run on the GPU against the CPU checker and the CUDA path, on the same index
files. Skipped when the reference build is not present."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from oracle import pipeline
from topoanns_b200 import capi, formats, search, synth

from gpu_support import np_u32, small_index

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
INVALID = 0xFFFFFFFF


def _write_index(tmp, s, host, entries):
    formats.write_topology(tmp / "topology.bin", formats.pad_degree(host["adjacency"], 64))
    formats.write_pq(tmp / "_pq_pivots.bin", tmp / "_pq_compressed.bin", host["pq_tables"], host["pq_centroid"],
                     host["pq_chunk_offsets"], host["codes"])
    formats.write_vector_store(tmp / "vectors.ssd", host["vectors"])
    formats.write_fbin(tmp / "queries.fbin", s.queries.cpu().numpy())
    e = np.ascontiguousarray(entries, np.uint32)
    with open(tmp / "entries.bin", "wb") as f:
        f.write(np.array(e.shape, np.uint32).tobytes())
        f.write(e.tobytes())
    if host.get("pq2_tables") is not None:
        formats.write_pq(tmp / "_pq2_pivots.bin", tmp / "_pq2_compressed.bin", host["pq2_tables"], host["pq2_centroid"],
                         host["pq_chunk_offsets"], host["pq2_codes"])
        formats.write_error_bounds(tmp / "_pq2_error.bin", host["pq2_error_bounds"])


def _run(tmp, tag, mode, *args, env=None):
    cmd = [DRIVER, str(tmp), str(tmp / tag), mode] + [str(a) for a in args]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=dict(os.environ, **(env or {})))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def _load(tmp, tag, name, dtype):
    return np.fromfile(tmp / f"{tag}.{name}.bin", dtype=dtype)


def _report(name, payload):
    """Appends one JSON record per case to $TANN_REPORT_DIR/reference_pin.jsonl when that variable is set."""
    out = os.environ.get("TANN_REPORT_DIR")
    if not out:
        return
    os.makedirs(out, exist_ok=True)
    with open(os.path.join(out, "reference_pin.jsonl"), "a") as f:
        f.write(json.dumps({"case": name, **payload}) + "\n")


@pytest.fixture(scope="module")
def ref_case(tmp_path_factory):
    if not os.path.exists(DRIVER):
        pytest.skip("oracle/_ref/ref_driver is not built (needs a reference checkout)")
    s, host = small_index(name="cfg2", num_nodes=40000, components=40, num_queries=300)
    tmp = tmp_path_factory.mktemp("refidx")
    Q = s.queries.shape[0]
    clusters, _, _ = orc.rvq_clusters(s.queries.cpu().numpy(), host["rvq_coarse"], host["rvq_fine"], host["rvq_sizes"])
    entries = orc.rvq_gather(clusters, host["rvq_offsets"], host["rvq_ids"], 128)
    _write_index(tmp, s, host, entries)
    return s, host, tmp, entries


def test_reference_tables_equal_checker(ref_case):
    s, host, tmp, _ = ref_case
    _run(tmp, "lut", "lut", 64, 2, 4096, 10, 32)
    Q, M = s.queries.shape[0], host["codes"].shape[1]
    ref = _load(tmp, "lut", "lut", np.float32).reshape(Q, M, 256)
    want = orc.lut_build(s.queries.cpu().numpy(), host["pq_tables"], host["pq_centroid"], host["pq_chunk_offsets"])
    np.testing.assert_allclose(ref, want, rtol=1e-5)
    exact = float((ref.view(np.uint32) == want.view(np.uint32)).mean())
    _report("lut", {"bit_exact_fraction": exact})
    assert exact == 1.0


@pytest.mark.parametrize("top_l,width", [(64, 2), (16, 1), (200, 4)])
def test_reference_traversal_against_checker_and_cuda(ref_case, top_l, width):
    s, host, tmp, entries = ref_case
    Q = s.queries.shape[0]
    top_n = 32
    tag = f"s{top_l}_{width}"
    _run(tmp, tag, "search", top_l, width, 4096, 10, top_n, "linear", 16, 0, 0, 3)
    limit = max(top_l, top_n)
    cap = orc.candidate_capacity(top_l, 0, top_n)
    lut = orc.lut_build(s.queries.cpu().numpy(), host["pq_tables"], host["pq_centroid"], host["pq_chunk_offsets"])
    eo = np.arange(Q + 1, dtype=np.uint32) * entries.shape[1]

    def packed(cand):
        out = cand[:, :limit].copy()
        inval = out[..., 1] == INVALID
        out[..., 0][inval] = 0
        return out

    refs = []
    for rep in range(3):
        ids = _load(tmp, tag, f"search{rep}_ids", np.uint32).reshape(Q, limit)
        dist = _load(tmp, tag, f"search{rep}_dist", np.float32).reshape(Q, limit)
        stats = _load(tmp, tag, f"search{rep}_stats", np.uint32).reshape(Q, 3)
        refs.append((np.stack([dist.view(np.uint32), ids], axis=2), stats))
    agree = {}
    for name, two_phase in (("two_phase", True), ("sequential", False)):
        cand, st = orc.beam_search(host["adjacency"], host["codes"], lut, eo, entries.reshape(-1), top_l=top_l,
                                   search_width=width, max_expansions=4096, capacity=cap, two_phase=two_phase)
        same = (packed(cand) == refs[0][0]).reshape(Q, -1).all(1) & (st[:, [0, 1, 3]] == refs[0][1]).all(1)
        agree[name] = float(same.mean())
        top10 = (orc.cand_raw_id(cand)[:, :10] == (refs[0][0][:, :10, 1] & 0x7FFFFFFF)).all(1)
        agree[name + "_top10"] = float(top10.mean())
    self_agree = float(np.mean([(refs[0][0] == r[0]).reshape(Q, -1).all(1).mean() for r in refs[1:]]))
    # the CUDA path against the reference kernel
    ix = search.device_index_from_synth(s)
    p = search.TopologySearchParams(top_l=top_l, search_width=width, max_expansions=4096)
    dc, ds = search.beam_search(ix, p, torch.from_numpy(eo.view(np.int32)).cuda(),
                                torch.from_numpy(entries.reshape(-1).view(np.int32)).cuda(),
                                queries=s.queries.cuda().contiguous(), capacity=cap)
    cuda_same = (packed(np_u32(dc)) == refs[0][0]).reshape(Q, -1).all(1) & (np_u32(ds)[:, [0, 1, 3]] == refs[0][1]).all(1)
    _report("traversal", {"top_l": top_l, "width": width, **agree, "reference_self_agreement": self_agree,
                          "cuda_vs_reference": float(cuda_same.mean())})
    assert max(agree["two_phase"], agree["sequential"]) >= 0.95
    assert float(cuda_same.mean()) >= 0.95


def test_reference_uint8_rerank_and_fused_path(ref_case):
    s, host, tmp, entries = ref_case
    Q = s.queries.shape[0]
    _run(tmp, "u8", "e2e_u8", 64, 2, 4096, 10, 32)
    rid = _load(tmp, "u8", "rerank_ids", np.uint32).reshape(Q, 32)
    rdist = _load(tmp, "u8", "rerank_dist", np.float32).reshape(Q, 32)
    ref = pipeline.run(host, s.queries.cpu().numpy().astype(np.uint8), top_l=64, search_width=2, max_expansions=4096,
                       top_n=32, top_k=10, entry_count=128)
    same_ids = float((rid[:, :10] == ref["topk_ids"]).all(1).mean())
    same_rows = (rid == ref["ids"]).all(1)
    assert np.array_equal(rdist[same_rows].view(np.uint32), ref["dists"][same_rows].view(np.uint32))  # bit-exact distances
    # the CUDA path end to end (host buffers) against the reference's top-10
    ix = search.device_index_from_synth(s)
    sr = search.Searcher(ix, Q, 64, 32, 128)
    sr.set_rvq(search.rvq_model_from_synth(s), 128)
    ids, dists, _ = sr.run_host(s.queries.cpu().numpy().astype(np.uint8), search.TopologySearchParams(top_l=64, search_width=2, max_expansions=4096),
                                search.RerankExactParams(top_k=10, top_n=32))
    cuda_same = float((ids == rid[:, :10]).all(1).mean())
    gt = s.gt_ids.cpu().numpy()
    _report("e2e_u8", {"checker_top10_identical": same_ids, "cuda_top10_identical": cuda_same,
                       "recall_reference": synth.recall_at_k(rid[:, :10], gt, 10), "recall_cuda": synth.recall_at_k(ids, gt, 10)})
    assert same_ids >= 0.99 and cuda_same >= 0.99
    assert abs(synth.recall_at_k(rid[:, :10], gt, 10) - synth.recall_at_k(ids, gt, 10)) <= 0.002
    sr.close()
    # fused modes of the reference give the same rerank as its materialised path
    for mode, tile in (("linear", 16), ("tiled", 8), ("page", 1)):
        _run(tmp, "f_" + mode, "fused", 64, 2, 4096, 10, 32, mode, tile, 0, 0)
        fid = _load(tmp, "f_" + mode, "rerank_ids", np.uint32).reshape(Q, 32)
        fref = pipeline.run(host, s.queries.cpu().numpy(), top_l=64, search_width=2, max_expansions=4096, top_n=32,
                            top_k=10, entry_count=128)
        assert float((fid[:, :10] == fref["topk_ids"]).all(1).mean()) >= 0.99


@pytest.mark.parametrize("chunks", [32, 48])
def test_reference_pq2_refine_and_bound_filter(tmp_path, chunks):
    """pq2 refine, bound filter and float32 rerank against the reference.

    With 48 chunks the reference's refine kernel copies only the first 32 residual codes of a node
    (its vectorised copy checks 16-byte alignment but moves bytes/32 32-byte words, src/search/rerank_exact.cu:108-133
    used at :806-807) and reads the other 16 from shared memory it never wrote. On the test GPU that memory reads as
    zero, so the reference is compared with the checker run on residual codes zeroed from chunk 32 on; with a
    multiple of 32 chunks the comparison is direct."""
    if not os.path.exists(DRIVER):
        pytest.skip("oracle/_ref/ref_driver is not built (needs a reference checkout)")
    s, host = small_index(name="cfg3", num_nodes=12000, components=60, num_queries=128, pq_chunks=chunks)
    Q = s.queries.shape[0]
    entries = np.full((Q, 1), s.medoid, np.uint32)
    _write_index(tmp_path, s, host, entries)
    q = s.queries.cpu().numpy()
    emu = dict(host)
    emu.pop("pages", None)
    if chunks % 32:
        emu["pq2_codes"] = host["pq2_codes"].copy()
        emu["pq2_codes"][:, 32:] = 0
    # traversal (M = 48: two tree groups) and the refined lists themselves
    _run(tmp_path, "rf", "pq2refine", 64, 2, 2048, 10, 64, "linear", 16, 1, 0)
    rf_ids = _load(tmp_path, "rf", "refined_ids", np.uint32).reshape(Q, 64)
    rf_dist = _load(tmp_path, "rf", "refined_dist", np.float32).reshape(Q, 64)
    base = pipeline.run(emu, q, top_l=64, search_width=2, max_expansions=2048, top_n=64, top_k=10,
                        fixed_entries=[s.medoid], use_pq2=True, refine_top_l=64)
    refined_same = float(((rf_ids == base["refined"][..., 1]) & (rf_dist.view(np.uint32) == base["refined"][..., 0])).all(1).mean())
    _report("pq2_refined_lists", {"chunks": chunks, "identical": refined_same})
    failures = []
    if refined_same < 0.99:
        failures.append(f"refined lists {refined_same}")
    for mode, tile, pq2, bound in (("linear", 16, 0, 0), ("tiled", 16, 1, 0), ("tiled", 16, 1, 1), ("page", 1, 1, 1)):
        tag = f"pq2_{mode}_{pq2}_{bound}"
        _run(tmp_path, tag, "fused", 64, 2, 2048, 10, 64, mode, tile, pq2, bound)
        rid = _load(tmp_path, tag, "rerank_ids", np.uint32).reshape(Q, 64)
        rdist = _load(tmp_path, tag, "rerank_dist", np.float32).reshape(Q, 64)
        rstats = _load(tmp_path, tag, "rerank_stats", np.uint64)
        ref = pipeline.run(emu, q, top_l=64, search_width=2, max_expansions=2048, top_n=64, top_k=10,
                           fixed_entries=[s.medoid], use_pq2=bool(pq2), refine_top_l=64, bound_filter=bool(bound),
                           tile=0 if mode == "linear" else tile)
        same = (rid == ref["ids"]).all(1)
        dist_same = float((rdist[same].view(np.uint32) == ref["dists"][same].view(np.uint32)).mean()) if same.any() else 0.0
        _report("pq2", {"chunks": chunks, "mode": mode, "pq2": pq2, "bound": bound, "rows_identical": float(same.mean()),
                        "dist_bits_identical": dist_same, "ref_exact": int(rstats[1]), "ref_filtered": int(rstats[2]),
                        "checker_exact": ref["n_exact"], "checker_filtered": ref["n_filtered"]})
        if float(same.mean()) < 0.99 or dist_same < 1.0 or int(rstats[2]) != ref["n_filtered"]:
            failures.append(f"{tag}: rows identical {float(same.mean()):.3f}, filtered {int(rstats[2])} vs {ref['n_filtered']}")
    assert not failures, failures


def _rvq_buckets(host):
    """Posting lists [coarse][fine] of the synthetic RVQ model (capped lists, as the entry gather reads them)."""
    nc, nf = host["rvq_coarse"].shape[0], host["rvq_fine"].shape[0]
    off, ids = host["rvq_offsets"], host["rvq_ids"]
    return [[ids[off[c * nf + f]:off[c * nf + f + 1]].astype(np.int32) for f in range(nf)] for c in range(nc)]


def test_reference_rvq_entry_selection(ref_case):
    """RVQ entry selection by the reference's own RVQ::search (src/legacy_rvq/gas_legacy/anns/RVQ/RVQ.cu:792-882:
    cuBLAS scores, functions/distance_kernel.cu:229-323, argmin kernels functions/selectMin1.cu:9-81) and its
    entry gather (src/search/rvq_device_entries.cu) against the checker and the CUDA kernel. cuBLAS sums in an
    order of its own, so a query may flip between two centroids whose scores tie to rounding: at least 99.9 % of
    the queries must get identical entry lists and every other one must be such a tie (< 1e-4 relative)."""
    s, host, tmp, _ = ref_case
    formats.write_rvq_model(tmp / "rvq_model.bin", host["rvq_coarse"], host["rvq_fine"], _rvq_buckets(host))
    more = synth.more_queries(s.cfg, s.extras["centres"], 3700, 4242).cpu().numpy()
    q = np.concatenate([s.queries.cpu().numpy(), more])
    Q, E = q.shape[0], 128
    formats.write_fbin(tmp / "queries.fbin", q)
    try:
        _run(tmp, "rvq", "rvq", 64, 2, 4096, 10, E)
    finally:
        formats.write_fbin(tmp / "queries.fbin", s.queries.cpu().numpy())
    ref_off = _load(tmp, "rvq", "rvq_dev_offsets", np.uint32)
    ref_ids = _load(tmp, "rvq", "rvq_dev_ids", np.uint32)
    host_ids = _load(tmp, "rvq", "rvq_host_ids", np.uint32).reshape(Q, E)
    host_cnt = _load(tmp, "rvq", "rvq_host_counts", np.uint32)
    assert ref_off.size == Q + 1
    # checker and CUDA
    clusters, _, _ = orc.rvq_clusters(q, host["rvq_coarse"], host["rvq_fine"], host["rvq_sizes"])
    want = orc.rvq_gather(clusters, host["rvq_offsets"], host["rvq_ids"], E)
    model = search.rvq_model_from_synth(s)
    offs, ids, cl = model.device_entry_batch(torch.from_numpy(q).cuda(), E)
    assert np.array_equal(np_u32(ids), want) and np.array_equal(cl.cpu().numpy(), clusters)
    # the reference's device batch: ragged CSR or fixed stride, compare query by query
    same = np.zeros(Q, bool)
    for i in range(Q):
        r = ref_ids[ref_off[i]:ref_off[i + 1]]
        w = want[i][want[i] != INVALID] if (want[i] != INVALID).any() else want[i][:1]
        r_valid = r[r != INVALID] if (r != INVALID).any() else r[:1]
        same[i] = r_valid.size == w.size and np.array_equal(r_valid, w)
        h = host_ids[i, :host_cnt[i]]
        assert np.array_equal(h, r_valid) or host_cnt[i] == 1   # the reference's host and device forms agree
    nf = host["rvq_fine"].shape[0]
    bad = np.nonzero(~same)[0]
    ties = 0
    c64, f64 = host["rvq_coarse"].astype(np.float64), host["rvq_fine"].astype(np.float64)
    cluster_of = {}
    for i in bad:
        r = ref_ids[ref_off[i]:ref_off[i + 1]]
        first = int(r[0])
        if not cluster_of:
            off = host["rvq_offsets"]
            for c in range(off.size - 1):
                for node in host["rvq_ids"][off[c]:off[c + 1]]:
                    cluster_of[int(node)] = c
        rc = cluster_of.get(first)
        if rc is None:
            continue
        x = q[i].astype(np.float64)
        mine, theirs = int(clusters[i]), int(rc)
        if mine // nf != theirs // nf:
            a, b = ((x - c64[mine // nf]) ** 2).sum(), ((x - c64[theirs // nf]) ** 2).sum()
        else:
            res = x - c64[mine // nf]
            a, b = ((res - f64[mine % nf]) ** 2).sum(), ((res - f64[theirs % nf]) ** 2).sum()
        ties += int(abs(a - b) <= 1e-4 * max(a, b))
    frac = float(same.mean())
    _report("rvq_entries", {"queries": int(Q), "identical_entry_lists": frac, "disagreements": int(bad.size),
                            "disagreements_that_are_ties": int(ties)})
    assert frac >= 0.999, (frac, bad[:10])
    assert ties == bad.size


def _write_learned_stop_model(path, stages, weights, bias, threshold, churn="ratio", next64="frac", mask=None,
                              means=None, inv_stds=None, per_l=None, top_k=10):
    with open(path, "w") as f:
        f.write("# synthetic learned traversal-stop model\n")
        f.write("stage_prefixes = " + ",".join(str(x) for x in stages) + "\n")
        f.write("feature_means = " + ",".join(repr(float(x)) for x in (means if means is not None else [0.0] * 12)) + "\n")
        f.write("feature_inv_stds = " + ",".join(repr(float(x)) for x in (inv_stds if inv_stds is not None else [1.0] * 12)) + "\n")
        f.write("weights = " + ",".join(repr(float(x)) for x in weights) + "\n")
        f.write(f"bias = {bias!r}\nthreshold_logit = {threshold!r}\ntop_k = {top_k}\n")
        f.write(f"topk_churn_mode = {churn}\nnext64_mode = {next64}\n")
        if mask is not None:
            f.write("feature_mask = " + ",".join(str(int(x)) for x in mask) + "\n")
        for L, t in (per_l or {}).items():
            f.write(f"threshold_logit_top_l_{L} = {t!r}\n")


def _stop_model_numbers():
    """A synthetic model that stops some queries and not others: the logit falls with the share of the list that
    has been expanded and visited and rises with top-k churn; the distance features carry small weights so that
    the decision differs from query to query."""
    rng = np.random.default_rng(5)
    weights = np.zeros(12, np.float32)
    weights[0], weights[1], weights[2] = -0.010, -0.020, -0.0004       # stage prefix, expanded, visited (per top_l)
    weights[3], weights[4], weights[5] = 0.010, 0.004, 0.004           # best unexpanded rank, unexpanded shares
    weights[6:11] = (rng.normal(size=5) * 2e-8).astype(np.float32)     # distances and their changes
    weights[11] = 0.02                                                 # top-k churn
    means = (rng.normal(size=12) * 0.05).astype(np.float32)
    means[6:11] = 0.0
    inv_stds = (1.0 + rng.random(12)).astype(np.float32)
    return weights, means, inv_stds


@pytest.mark.parametrize("churn,next64,mask,shadow", [("ratio", "frac", None, False),
                                                       ("flag", "flag", [0, 0, 1, 1, 0, 0, 1, 1, 1, 0, 1, 1], False),
                                                       ("ratio", "frac", None, True)])
def test_reference_learned_traversal_stop(ref_case, churn, next64, mask, shadow):
    """The learned traversal stop of the compiled reference (TOPOANNS_LEARNED_STOP_MODEL read at
    src/search/topology_search_kernel.cu:3482, model parsed at :248-380, evaluated at :953-1137) against the checker
    and the CUDA kernel on the same model file: candidate lists, flags and visited / expanded / iteration counts."""
    s, host, tmp, entries = ref_case
    Q = s.queries.shape[0]
    top_l, width, top_n = 64, 2, 32
    weights, means, inv_stds = _stop_model_numbers()
    model_path = tmp / f"stop_{churn}_{next64}_{int(shadow)}.txt"
    _write_learned_stop_model(model_path, [8, 16, 24, 32, 48, 64, 80], weights, 0.02, 0.0, churn, next64, mask,
                              means, inv_stds, per_l={64: 0.01, 128: -5.0})
    tag = f"ls_{churn}_{int(shadow)}"
    env = {"TOPOANNS_LEARNED_STOP_MODEL": str(model_path)}
    if shadow:
        env["TOPOANNS_LEARNED_STOP_SHADOW"] = "1"
    _run(tmp, tag, "search", top_l, width, 4096, 10, top_n, "linear", 16, 0, 0, 1, env=env)
    limit = max(top_l, top_n)
    cap = orc.candidate_capacity(top_l, 0, top_n)
    ids = _load(tmp, tag, "search0_ids", np.uint32).reshape(Q, limit)
    dist = _load(tmp, tag, "search0_dist", np.float32).reshape(Q, limit)
    rstats = _load(tmp, tag, "search0_stats", np.uint32).reshape(Q, 3)
    ref = np.stack([dist.view(np.uint32), ids], axis=2)
    ls = search.load_learned_stop(model_path, top_l, 10, shadow=shadow)
    assert ls.enabled == 1 and ls.num_stages == 5 and abs(ls.threshold_logit - 0.01) < 1e-9
    ols = orc.LearnedStop()
    for name, _ in capi.LearnedStop._fields_:
        setattr(ols, name, getattr(ls, name))
    lut = orc.lut_build(s.queries.cpu().numpy(), host["pq_tables"], host["pq_centroid"], host["pq_chunk_offsets"])
    eo = np.arange(Q + 1, dtype=np.uint32) * entries.shape[1]
    cand, st = orc.beam_search(host["adjacency"], host["codes"], lut, eo, entries.reshape(-1), top_l=top_l,
                               search_width=width, max_expansions=4096, capacity=cap, learned_stop=ols)

    def packed(c):
        out = c[:, :limit].copy()
        out[..., 0][out[..., 1] == INVALID] = 0
        return out

    checker_same = (packed(cand) == ref).reshape(Q, -1).all(1) & (st[:, [0, 1, 3]] == rstats).all(1)
    ix = search.device_index_from_synth(s)
    p = search.TopologySearchParams(top_l=top_l, search_width=width, max_expansions=4096, learned_stop=ls)
    dc, ds = search.beam_search(ix, p, torch.from_numpy(eo.view(np.int32)).cuda(),
                                torch.from_numpy(entries.reshape(-1).view(np.int32)).cuda(),
                                queries=s.queries.cuda().contiguous(), capacity=cap)
    cuda_same = (packed(np_u32(dc)) == ref).reshape(Q, -1).all(1) & (np_u32(ds)[:, [0, 1, 3]] == rstats).all(1)
    # the stop has to bite, otherwise this pins nothing: compare with the traversal without a model
    _, st_plain = orc.beam_search(host["adjacency"], host["codes"], lut, eo, entries.reshape(-1), top_l=top_l,
                                  search_width=width, max_expansions=4096, capacity=cap)
    stopped_early = float((st[:, 1] < st_plain[:, 1]).mean())
    _report("learned_traversal_stop", {"churn": churn, "next64": next64, "shadow": shadow,
                                       "checker_vs_reference": float(checker_same.mean()),
                                       "cuda_vs_reference": float(cuda_same.mean()), "queries_stopped_early": stopped_early})
    if shadow:
        assert stopped_early == 0.0
    else:
        assert stopped_early > 0.05
    assert float(checker_same.mean()) >= 0.999 and float(cuda_same.mean()) >= 0.999


def test_reference_hpq_refine(tmp_path):
    """Hybrid-PQ refine of the compiled reference (hpq_refine_bitonic_sort_kernel, src/search/rerank_exact.cu:667-771,
    driven by detail::RunHpqRefineBatchDevice :2457-2531, index loaded by HpqIndex::Load, src/io/hpq_index.cpp) against
    the checker and the CUDA kernel, on index files both sides read."""
    if not os.path.exists(DRIVER):
        pytest.skip("oracle/_ref/ref_driver is not built (needs a reference checkout)")
    s, host = small_index(name="cfg3", num_nodes=12000, components=60, num_queries=128, pq_chunks=32)
    Q = s.queries.shape[0]
    entries = np.full((Q, 1), s.medoid, np.uint32)
    _write_index(tmp_path, s, host, entries)
    N, M = host["codes"].shape
    rng = np.random.default_rng(11)
    bits = rng.integers(0, 2, size=(N, M), dtype=np.uint8)
    hybrid = np.where(bits == 1, host["pq2_codes"], host["codes"]).astype(np.uint8)
    selectors = np.packbits(bits, axis=1, bitorder="little")
    formats.write_pq(tmp_path / "_hpq_outlier_pivots.bin", tmp_path / "_hpq_codes.bin", host["pq2_tables"],
                     host["pq2_centroid"], host["pq_chunk_offsets"], hybrid)
    formats.write_hpq_selector_bits(tmp_path / "_hpq_selector.bin", selectors)
    assert np.array_equal(formats.read_hpq_selector_bits(tmp_path / "_hpq_selector.bin", N, M), selectors)
    _run(tmp_path, "hpq", "hpq", 64, 2, 2048, 10, 64)
    rf_ids = _load(tmp_path, "hpq", "refined_ids", np.uint32).reshape(Q, 64)
    rf_dist = _load(tmp_path, "hpq", "refined_dist", np.float32).reshape(Q, 64)
    q = s.queries.cpu().numpy()
    lut = orc.lut_build(q, host["pq_tables"], host["pq_centroid"], host["pq_chunk_offsets"])
    lut_out = orc.lut_build(q, host["pq2_tables"], host["pq2_centroid"], host["pq_chunk_offsets"])
    eo = np.arange(Q + 1, dtype=np.uint32)
    cap = orc.candidate_capacity(64, 0, 64)
    cand, st = orc.beam_search(host["adjacency"], host["codes"], lut, eo, entries.reshape(-1), top_l=64, search_width=2,
                               max_expansions=2048, capacity=cap)
    want = orc.hpq_refine(cand, st, 64, hybrid, selectors, lut, lut_out)
    checker_same = float(((rf_ids == want[..., 1]) & (rf_dist.view(np.uint32) == want[..., 0])).all(1).mean())
    ix = search.device_index_from_synth(s)
    qd = s.queries.cuda().contiguous()
    p = search.TopologySearchParams(top_l=64, search_width=2, max_expansions=2048)
    dc, ds = search.beam_search(ix, p, torch.from_numpy(eo.view(np.int32)).cuda(),
                                torch.from_numpy(entries.reshape(-1).view(np.int32)).cuda(), queries=qd, capacity=cap)
    base_lut = search.lut_build(ix, qd)
    outlier_lut = search.lut_build(ix, qd, tables_col_major=s.pq2_tables.cuda().t().contiguous(),
                                   centroid=s.pq2_centroid.cuda().contiguous(), chunk_offsets=ix.pq_chunk_offsets)
    got = np_u32(search.hpq_refine(dc, ds, 64, torch.from_numpy(hybrid).cuda(), torch.from_numpy(selectors).cuda(),
                                   base_lut, outlier_lut))
    cuda_same = float(((rf_ids == got[..., 1]) & (rf_dist.view(np.uint32) == got[..., 0])).all(1).mean())
    _report("hpq_refine", {"checker_vs_reference": checker_same, "cuda_vs_reference": cuda_same})
    assert checker_same >= 0.999 and cuda_same >= 0.999


def test_reference_config1_at_full_size(tmp_path):
    """The first benchmark configuration at its stated size: 100 000 x 128 uint8 vectors, R = 32 (24 nearest + 8 random
    edges), PQ M = 32, 1 000 queries, top_k = 10, L = 64, search width 2, rerank_top_n = 32 with integer exact L2, a
    single medoid entry, uint8 queries through the reference's RunBatchUint8 entry point
    (src/search/topoanns_search.cpp:377-401): reference, checker and CUDA path, rerank lists and distances bit for bit."""
    if not os.path.exists(DRIVER):
        pytest.skip("oracle/_ref/ref_driver is not built (needs a reference checkout)")
    import dataclasses
    cfg = dataclasses.replace(synth.CONFIGS["cfg1"])
    s = synth.build(cfg, "cuda")
    host = pipeline.index_from_synth(s)
    Q = s.queries.shape[0]
    assert (s.vectors.shape[0], Q, s.adjacency.shape[1]) == (100_000, 1000, 32)
    entries = np.full((Q, 1), s.medoid, np.uint32)
    _write_index(tmp_path, s, host, entries)
    _run(tmp_path, "cfg1", "e2e_u8", 64, 2, 1024, 10, 32)
    rid = _load(tmp_path, "cfg1", "rerank_ids", np.uint32).reshape(Q, 32)
    rdist = _load(tmp_path, "cfg1", "rerank_dist", np.float32).reshape(Q, 32)
    q8 = s.queries.cpu().numpy().astype(np.uint8)
    ref = pipeline.run(host, q8, top_l=64, search_width=2, max_expansions=1024, top_n=32, top_k=10,
                       fixed_entries=[s.medoid])
    checker_rows = (rid == ref["ids"]).all(1) & (rdist.view(np.uint32) == ref["dists"].view(np.uint32)).all(1)
    ix = search.device_index_from_synth(s)
    sr = search.Searcher(ix, Q, 64, 32, 8)
    ids, dists, _ = sr.run_host(q8, search.TopologySearchParams(top_l=64, search_width=2, max_expansions=1024),
                                search.RerankExactParams(top_k=10, top_n=32), fixed_entries=np.array([s.medoid], np.uint32))
    sr.close()
    cuda_rows = (ids == rid[:, :10]).all(1) & (dists.view(np.uint32) == rdist[:, :10].view(np.uint32)).all(1)
    gt = s.gt_ids.cpu().numpy()
    rec_ref, rec_cuda = synth.recall_at_k(rid[:, :10], gt, 10), synth.recall_at_k(ids, gt, 10)
    _report("config1_full_size", {"queries": int(Q), "checker_lists_identical": float(checker_rows.mean()),
                                  "cuda_top10_identical": float(cuda_rows.mean()), "recall_reference": rec_ref,
                                  "recall_cuda": rec_cuda})
    assert float(checker_rows.mean()) >= 0.999 and float(cuda_rows.mean()) >= 0.999
    assert abs(rec_ref - rec_cuda) <= 0.002
