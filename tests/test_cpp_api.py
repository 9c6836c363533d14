"""Runs the C++ API tests (tests/cpp) built by topoanns_b200/host/Makefile."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "build")


def _build():
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "topoanns_b200", "csrc"), "-j8"], stdout=subprocess.DEVNULL)
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "topoanns_b200", "host"), "-j8"], stdout=subprocess.DEVNULL)


def _run(name, tmp_path):
    _build()
    env = dict(os.environ, TANN_TEST_TMP=str(tmp_path))
    r = subprocess.run([os.path.join(BIN, name)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert f"{name} passed" in r.stdout


def test_cpp_host_only_api(tmp_path):
    _run("test_api_host", tmp_path)


@pytest.mark.gpu
def test_cpp_search_api(tmp_path):
    _run("test_api_search", tmp_path)


def _write_index_dir(tmp_path, name="cfg2", num_nodes=40000, components=40):
    """A small RVQ-entry index written in the reference's file layouts; returns what the tests need."""
    import numpy as np

    from gpu_support import small_index
    from topoanns_b200 import formats

    s, host = small_index(name=name, num_nodes=num_nodes, components=components, num_queries=300)
    d = tmp_path / "index"
    d.mkdir()
    if host.get("pq2_tables") is not None:
        formats.write_pq(tmp_path / "pq2_pivots.bin", tmp_path / "pq2_codes.bin", host["pq2_tables"], host["pq2_centroid"],
                         host["pq_chunk_offsets"], host["pq2_codes"])
        formats.write_error_bounds(tmp_path / "pq2_eps.bin", host["pq2_error_bounds"])
    formats.write_topology(d / "topology.bin", host["adjacency"])
    formats.write_pq(d / "_pq_pivots.bin", d / "_pq_compressed.bin", host["pq_tables"], host["pq_centroid"],
                     host["pq_chunk_offsets"], host["codes"])
    formats.write_vector_store(d / "vectors.ssd", host["vectors"])
    q = s.queries.cpu().numpy()
    gt = s.gt_ids.cpu().numpy()
    formats.write_fbin(tmp_path / "queries.fbin", q)
    formats.write_gt(tmp_path / "gt.bin", gt.astype(np.int32))
    sizes, offsets, ids = (t.cpu().numpy() for t in s.rvq_buckets)
    nc, nf = s.rvq_coarse.shape[0], s.rvq_fine.shape[0]
    buckets = [[ids[offsets[c * nf + f]:offsets[c * nf + f + 1]] for f in range(nf)] for c in range(nc)]
    formats.write_rvq_model(tmp_path / "rvq.bin", s.rvq_coarse.cpu().numpy(), s.rvq_fine.cpu().numpy(), buckets)
    base_cmd = [os.path.join(ROOT, "topoanns_b200", "topoanns_eval_sift"), "--index-dir", str(d), "--rvq-model",
                str(tmp_path / "rvq.bin"), "--query-bin", str(tmp_path / "queries.fbin"), "--gt-bin", str(tmp_path / "gt.bin"),
                "--num-queries", str(q.shape[0]), "--search-width", "2", "--max-expansions", "4096",
                "--rvq-entry-count", "128", "--batch-size", "128"]
    return s, q, gt, base_cmd


_SUMMARY = (r"\[topoanns_eval\] frontier_pq_mode=\S+ top_l=(\d+) rerank_top_n=(\d+) rerank_mode=\S+ queries=(\d+) "
            r"elapsed_sec=\S+ wall_elapsed_sec=\S+ qps=(\S+) wall_qps=\S+ recall@10=(\S+) avg_io_pages=\S+ "
            r"avg_exact=(\S+) avg_bound_filtered=\S+ avg_visited=(\S+) avg_expanded=(\S+)$")


def _summaries(stdout):
    import re
    out = {}
    for line in stdout.splitlines():
        m = re.match(_SUMMARY, line)
        if m:
            out[int(m.group(1))] = dict(top_n=int(m.group(2)), queries=int(m.group(3)), qps=float(m.group(4)),
                                        recall=float(m.group(5)), avg_exact=float(m.group(6)),
                                        avg_visited=float(m.group(7)), avg_expanded=float(m.group(8)))
    return out


@pytest.mark.gpu
def test_eval_driver_lines_and_recall(tmp_path):
    """The evaluation driver (flags and output lines of the reference's tools/topoanns_eval_sift.cpp) on an
    index directory written by the Python generators: its recall@10 per sweep point must equal the Python
    path's on the same files, and the Pareto lines must be printed."""
    from topoanns_b200 import search, synth

    _build()
    s, q, gt, base_cmd = _write_index_dir(tmp_path)
    Q = q.shape[0]
    r = subprocess.run(base_cmd + ["--top-l-values", "16,64", "--rerank-top-n", "32", "--bam-queue-depth", "64"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    summary = _summaries(r.stdout)
    assert set(summary) == {16, 64}, r.stdout
    assert any(line.startswith("[topoanns_pareto] ") for line in r.stdout.splitlines())
    assert "--bam-queue-depth is ignored" in r.stderr
    ix = search.device_index_from_synth(s)
    model = search.rvq_model_from_synth(s)
    sr = search.Searcher(ix, Q, 128, 64, 128)
    sr.set_rvq(model, 128)
    for L in (16, 64):
        got_ids, _, stats = sr.run_host(q, search.TopologySearchParams(top_l=L, search_width=2, max_expansions=4096),
                                        search.RerankExactParams(top_k=10, top_n=32), want_stats=True)
        assert abs(summary[L]["recall"] - synth.recall_at_k(got_ids, gt, 10)) < 1e-6
        assert abs(summary[L]["avg_visited"] - float(stats[:, 0].mean())) < 1e-3 * max(1.0, float(stats[:, 0].mean()))
        assert summary[L]["queries"] == Q and summary[L]["qps"] > 0
    sr.close()


@pytest.mark.gpu
def test_learned_stop_model_file_and_early_stop_through_the_driver(tmp_path):
    """TOPOANNS_LEARNED_STOP_MODEL names a key=value model file (src/search/topology_search_kernel.cu:248-380);
    the C++ layer folds mean / inverse-std into weights and bias. The driver's traversal statistics must equal
    the Python path's with the same folded model, and the model must really cut the traversal short. The rerank
    early-stop flags must reduce the exact distances per query."""
    import numpy as np

    from topoanns_b200 import capi, search

    _build()
    s, q, gt, base_cmd = _write_index_dir(tmp_path)
    Q = q.shape[0]
    rng = np.random.default_rng(5)
    # feature 1 (expanded / L) decides: logit = 2 - 4 * expanded / 64 after folding, so with the per-L threshold
    # 0.1 the stage at prefix 32 stops every traversal that has expanded 32 nodes; the other features carry
    # small weights so that the folding of means and inverse deviations is exercised without deciding anything
    w = (rng.normal(size=12) * 0.1).astype(np.float32)
    means = rng.normal(size=12).astype(np.float32)
    inv_stds = np.full(12, 1e-7, np.float32)
    w[1], means[1], inv_stds[1] = -8.0, 0.25, 0.5
    mask = [1, 1, 1, 1, 0, 1, 1, 1, 1, 1, 1, 1]
    bias, threshold, threshold_64 = np.float32(1.0), np.float32(5.0), np.float32(0.1)

    def fmt(a):
        return ",".join("%.9g" % float(x) for x in a)
    model = tmp_path / "stop.model"
    model.write_text("# synthetic model\nstage_prefixes=16,32,48\nfeature_means=%s\nfeature_inv_stds=%s\nweights=%s\n"
                     "bias=%.9g\nthreshold_logit=%.9g\nthreshold_logit_top_l_64=%.9g\ntop_k=10\ntopk_churn_mode=ratio\n"
                     "next64_mode=flag\nfeature_mask=%s\n" % (fmt(means), fmt(inv_stds), fmt(w), bias, threshold, threshold_64,
                                                              ",".join(str(m) for m in mask)))
    env = dict(os.environ, TOPOANNS_LEARNED_STOP_MODEL=str(model))
    r = subprocess.run(base_cmd + ["--top-l-values", "64", "--rerank-top-n", "32"], capture_output=True, text=True,
                       timeout=600, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    with_model = _summaries(r.stdout)[64]
    r0 = subprocess.run(base_cmd + ["--top-l-values", "64", "--rerank-top-n", "32"], capture_output=True, text=True, timeout=600)
    plain = _summaries(r0.stdout)[64]
    # the same folding in float32 (host/search.cpp), then the Python path
    ls = capi.LearnedStop()
    ls.enabled, ls.num_stages, ls.top_k, ls.shadow_mode = 1, 3, 10, 0
    ls.topk_churn_flag_mode, ls.next64_flag_mode = 0, 1
    for i, pfx in enumerate((16, 32, 48)):
        ls.stage_prefixes[i] = pfx
    folded_bias = np.float32(bias)
    for i in range(12):
        ls.feature_mask[i] = mask[i]
        wi = np.float32(w[i] if mask[i] else 0.0) * inv_stds[i]
        ls.weights[i] = float(wi)
        folded_bias = np.float32(folded_bias - np.float32(means[i] * wi))
    ls.bias, ls.threshold_logit, ls.inv_top_l = float(folded_bias), float(threshold_64), float(np.float32(1.0) / np.float32(64))
    ix = search.device_index_from_synth(s)
    rvq = search.rvq_model_from_synth(s)
    sr = search.Searcher(ix, Q, 128, 64, 128)
    sr.set_rvq(rvq, 128)
    _, _, stats = sr.run_host(q, search.TopologySearchParams(top_l=64, search_width=2, max_expansions=4096, learned_stop=ls),
                              search.RerankExactParams(top_k=10, top_n=32), want_stats=True)
    sr.close()
    assert abs(with_model["avg_visited"] - float(stats[:, 0].mean())) < 1e-3 * float(stats[:, 0].mean())
    assert abs(with_model["avg_expanded"] - float(stats[:, 1].mean())) < 1e-3 * float(stats[:, 1].mean())
    assert with_model["avg_expanded"] < plain["avg_expanded"]          # the model stops some traversals early
    # rerank early stop through the driver's flags
    r2 = subprocess.run(base_cmd + ["--top-l-values", "64", "--rerank-top-n", "64", "--rerank-use-early-stop",
                                    "--rerank-early-stop-min-prefix", "16", "--rerank-early-stop-patience-tiles", "1",
                                    "--rerank-rank-tile-size", "8"], capture_output=True, text=True, timeout=600)
    assert r2.returncode == 0, r2.stdout + r2.stderr
    assert _summaries(r2.stdout)[64]["avg_exact"] < 64.0


@pytest.mark.gpu
def test_learned_rerank_stop_through_the_driver(tmp_path):
    """--rerank-use-learned-stop / --rerank-learned-stop-model on a float index with residual pq2 and error
    bounds: the summary line carries the learned-stop keys, a model that stops early scores fewer candidates,
    and a model whose threshold nothing reaches gives the recall of the plain persistent rerank."""
    import re

    _build()
    s, q, gt, base_cmd = _write_index_dir(tmp_path, name="cfg3", num_nodes=12000, components=60)
    pq2 = ["--pq2-pivots", str(tmp_path / "pq2_pivots.bin"), "--pq2-codes", str(tmp_path / "pq2_codes.bin"),
           "--pq2-error-bounds", str(tmp_path / "pq2_eps.bin"), "--rerank-use-pq2", "--rerank-use-pq2-bound-filter",
           "--rerank-mode", "persistent", "--rerank-rank-tile-size", "16", "--top-l-values", "128", "--rerank-top-n", "128"]

    def model(name, threshold):
        path = tmp_path / name
        path.write_text("stage_prefixes = 16, 32, 64, 96\nbootstrap_prefix = 16\n"
                        "feature_means = 0,0,0,0,0,0,0,0,0,0,0,0,0\nfeature_inv_stds = 1,1,1,1,1,1,1,1,1,1,1,1,1\n"
                        "weights = 0,-4,0,0,0,0,1,0,0,0,0,0,0\nbias = 1\nthreshold_logit = %g\n" % threshold)
        return str(path)

    def run(extra):
        r = subprocess.run(base_cmd + pq2 + extra, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout + r.stderr
        line = [l for l in r.stdout.splitlines() if " elapsed_sec=" in l][-1]
        return dict(kv.split("=", 1) for kv in line.split()[1:] if "=" in kv)

    plain = run([])
    stop = run(["--rerank-use-learned-stop", "--rerank-learned-stop-model", model("stop.model", 0.0)])
    never = run(["--rerank-use-learned-stop", "--rerank-learned-stop-model", model("never.model", -1000.0)])
    assert "learned_stop_queries" not in plain
    assert int(stop["learned_stop_queries"]) == q.shape[0]
    assert 16 <= int(stop["learned_stop_prefix_min"]) <= int(stop["learned_stop_prefix_max"]) <= 128
    assert float(stop["avg_learned_stop_prefix"]) < 128 and float(stop["avg_learned_checkpoints"]) >= 1
    assert float(stop["avg_exact"]) < float(never["avg_exact"])
    assert float(never["avg_learned_stop_prefix"]) == 128.0 and float(never["avg_learned_checkpoints"]) == 3.0
    assert abs(float(never["recall@10"]) - float(plain["recall@10"])) < 1e-9
    assert re.match(r"^\d+(\.\d+)?$", stop["avg_learned_stop_prefix"])
