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


@pytest.mark.gpu
def test_eval_driver_lines_and_recall(tmp_path):
    """The evaluation driver (flags and output lines of the reference's tools/topoanns_eval_sift.cpp) on an
    index directory written by the Python generators: its recall@10 per sweep point must equal the Python
    path's on the same files, and the Pareto lines must be printed."""
    import re

    import numpy as np

    from gpu_support import small_index
    from topoanns_b200 import formats, search, synth

    _build()
    s, host = small_index(name="cfg2", num_nodes=40000, components=40, num_queries=300)
    d = tmp_path / "index"
    d.mkdir()
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
    tool = os.path.join(ROOT, "topoanns_b200", "topoanns_eval_sift")
    Q = q.shape[0]
    r = subprocess.run([tool, "--index-dir", str(d), "--rvq-model", str(tmp_path / "rvq.bin"), "--query-bin",
                        str(tmp_path / "queries.fbin"), "--gt-bin", str(tmp_path / "gt.bin"), "--num-queries", str(Q),
                        "--top-l-values", "16,64", "--rerank-top-n", "32", "--search-width", "2", "--max-expansions", "4096",
                        "--rvq-entry-count", "128", "--batch-size", "128", "--bam-queue-depth", "64"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    summary = {}
    for line in r.stdout.splitlines():
        m = re.match(r"\[topoanns_eval\] frontier_pq_mode=\S+ top_l=(\d+) rerank_top_n=(\d+) rerank_mode=\S+ queries=(\d+) "
                     r"elapsed_sec=\S+ wall_elapsed_sec=\S+ qps=(\S+) wall_qps=\S+ recall@10=(\S+) avg_io_pages=\S+ "
                     r"avg_exact=(\S+) avg_bound_filtered=\S+ avg_visited=(\S+) avg_expanded=(\S+)$", line)
        if m:
            summary[int(m.group(1))] = dict(top_n=int(m.group(2)), queries=int(m.group(3)), qps=float(m.group(4)),
                                            recall=float(m.group(5)), avg_visited=float(m.group(7)))
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
