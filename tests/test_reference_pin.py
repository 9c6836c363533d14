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
from topoanns_b200 import formats, search, synth

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
