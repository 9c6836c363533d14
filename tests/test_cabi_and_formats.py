"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, its
parameter checks answer before any CUDA work, and the index file layouts round-trip byte for byte."""
import ctypes as C
import os
import re
import struct

import numpy as np
import pytest

from topoanns_b200 import capi, formats

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "topoanns_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tann_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    declared = _header_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(capi.SIGNATURES) == declared      # the binding covers exactly the header
    assert b"sm_100a" in lib.tann_version()


def test_struct_sizes_match_the_header():
    # sizes follow from the C declarations (natural alignment, 8 shards)
    assert C.sizeof(capi.Shards) == 16 + 8 * capi.MAX_SHARDS
    assert C.sizeof(capi.LearnedStop) == 6 * 4 + 32 * 4 + 12 * 4 + 12 * 4 + 3 * 4
    assert C.sizeof(capi.BeamParams) == 8 * 4 + C.sizeof(capi.LearnedStop)
    assert C.sizeof(capi.RerankParams) == 32
    assert C.sizeof(capi.IndexView) == 8 + 16 + 24 + 3 * C.sizeof(capi.Shards) + 16 + 24 + C.sizeof(capi.Shards)


def test_parameter_checks_answer_without_a_gpu():
    lib = capi.load()
    v, p = capi.IndexView(), capi.BeamParams()
    assert lib.tann_beam_search(C.byref(v), C.byref(p), None, None, 0, 0, None, None, None, None, None, None) == 1
    assert b"top_l must be positive" in lib.tann_last_error()
    p.top_l, p.search_width, p.max_expansions, p.candidate_capacity = 8, 40, 16, 8
    assert lib.tann_beam_search(C.byref(v), C.byref(p), None, None, 0, 0, None, None, None, None, None, None) == 1
    assert b"search_width must be at most 32" in lib.tann_last_error()
    p.search_width, p.candidate_capacity = 2, 12
    assert lib.tann_beam_search(C.byref(v), C.byref(p), None, None, 0, 0, None, None, None, None, None, None) == 1
    assert b"power of two" in lib.tann_last_error()
    assert lib.tann_rvq_entries(None, 4, 8, None, None, None, 1, None, None, 1, None, None, None, 0, 0, None, None,
                                None, None) == 1
    assert b"entry_count must be positive" in lib.tann_last_error()
    r = capi.RerankParams(2, 1, 1, 1)
    v.vector_bytes, v.vectors_per_page = 8, 512
    v.vectors.num_shards = 1
    v.vectors.base[0] = 4096
    assert lib.tann_rerank_exact(C.byref(v), C.byref(r), 4096, 2, 1, 4096, 2, None, 4096, 4096, None, None, None) == 1
    assert b"error bounds" in lib.tann_last_error()


def test_misaligned_tables_and_code_rows_are_rejected_before_any_launch():
    """Query tables, PQ code rows and neighbour-code rows are read with 16-byte loads: a base pointer off a
    16-byte boundary is answered with an error status on the host, nothing is launched."""
    lib = capi.load()
    v, p = capi.IndexView(), capi.BeamParams()
    p.top_l, p.search_width, p.max_expansions, p.candidate_capacity = 8, 2, 16, 8
    v.num_nodes, v.degree, v.num_chunks, v.dim = 100, 32, 32, 128
    v.adjacency.num_shards = v.codes.num_shards = 1
    v.adjacency.base[0] = 4096
    v.codes.base[0] = 8192
    args = (0, 4, 4096, 4096, 4096, 4096, None, None)     # kind, Q, offsets, ids, out, stats, status, stream
    assert lib.tann_beam_search(C.byref(v), C.byref(p), 4096 + 4, None, *args) == 1      # table at base + 4 bytes
    assert b"query tables must be 16-byte aligned" in lib.tann_last_error()
    v.codes.base[0] = 8192 + 4
    assert lib.tann_beam_search(C.byref(v), C.byref(p), 4096, None, *args) == 1
    assert b"codes shard 0 must be 16-byte aligned" in lib.tann_last_error()
    v.codes.base[0] = 8192
    v.neighbor_codes.num_shards = 1
    v.neighbor_codes.base[0] = 16384 + 8
    assert lib.tann_beam_search(C.byref(v), C.byref(p), 4096, None, *args) == 1
    assert b"neighbor_codes shard 0 must be 16-byte aligned" in lib.tann_last_error()


def test_owner_rerank_entry_points_reject_bad_sizes_before_any_launch():
    """Owner counts, slots and shard sizes of the rerank-by-owner helpers are checked on the host."""
    lib = capi.load()
    x = 4096
    assert lib.tann_partition_candidates(x, 64, 32, 10, 0, 8, 16, x, x, None) == 1          # rows_per_shard = 0
    assert b"tann_partition_candidates" in lib.tann_last_error()
    assert lib.tann_partition_candidates(x, 64, 32, 10, 1000, 65, 16, x, x, None) == 1      # more than 64 owners
    assert lib.tann_partition_candidates(x, 64, 32, 10, 1000, 8, 0, x, x, None) == 1        # empty slot
    assert lib.tann_partition_candidates(x, 64, 32, 10, 1000, 8, 16, x, None, None) == 1    # no overflow word
    assert lib.tann_merge_topk_lists(x, x, 8, 10, 40, 1000, x, x, None) == 1                # top_k above 32
    assert b"tann_merge_topk_lists" in lib.tann_last_error()
    assert lib.tann_merge_topk_lists(x, x, 8, 10, 10, 1 << 30, x, x, None) == 1             # ids beyond 31 bits
    assert lib.tann_merge_topk_lists(x, x, 0, 10, 10, 1000, x, x, None) == 1                # no list
    assert lib.tann_partition_candidates(x, 64, 32, 0, 1000, 8, 16, x, x, None) == 0        # empty batch: no-op
    assert lib.tann_merge_topk_lists(x, x, 8, 0, 10, 1000, x, x, None) == 0


def test_capacity_rule():
    # nextpow2(max(top_l, candidate_queue_size, rerank top_n))
    assert capi.candidate_capacity(4, 0, 5) == 8
    assert capi.candidate_capacity(64, 0, 32) == 64
    assert capi.candidate_capacity(100, 0, 32) == 128
    assert capi.candidate_capacity(16, 300, 32) == 512


def test_topology_file_layout(tmp_path):
    # tests/test_topology_layout.cpp: padding with 0xffffffff to 64 slots, 4 KB header, offsets
    lists = [[1, 2], [3], [], [0, 1, 2]]
    adj = np.full((4, 3), formats.INVALID, np.uint32)
    for i, l in enumerate(lists):
        adj[i, :len(l)] = l
    padded = formats.pad_degree(adj, 64)
    assert padded.shape == (4, 64) and padded[0, 2] == formats.INVALID and padded[3, 2] == 2
    path = tmp_path / "topology.bin"
    formats.write_topology(path, padded)
    raw = path.read_bytes()
    assert len(raw) == 4096 + 4 * 64 * 4 and raw[:8] == b"TOPOANNS"
    assert struct.unpack_from("<IIQQQ", raw, 8) == (1, 64, 4, 4096, 4 * 64 * 4)
    assert np.array_equal(formats.read_topology(path), padded)
    with open(path, "r+b") as f:
        f.write(b"XOPOANNS")
    with pytest.raises(ValueError, match="magic"):
        formats.read_topology(path)
    with pytest.raises(ValueError, match="more than 64"):
        formats.pad_degree(np.zeros((1, 65), np.uint32))


def test_vector_page_layout_and_store(tmp_path):
    # tests/test_vector_page_layout.cpp: 512-byte vectors -> 8 per page, 100-byte -> 40 per page, > 4 KB throws
    assert formats.VectorPageLayout(512).vectors_per_page == 8
    assert formats.VectorPageLayout(100).vectors_per_page == 40
    with pytest.raises(ValueError):
        formats.VectorPageLayout(5000)
    lay = formats.VectorPageLayout(384)   # float32 d = 96: 10 per page, 256 bytes of padding
    assert lay.vectors_per_page == 10 and lay.resolve(23) == (2, 3, 4096 + 2 * 4096 + 3 * 384)
    rng = np.random.default_rng(0)
    for dt, d in ((np.uint8, 128), (np.float32, 96), (np.int8, 100), (np.float32, 768)):
        v = (rng.normal(size=(77, d)) * 50).astype(dt)
        path = tmp_path / f"v_{d}.ssd"
        formats.write_vector_store(path, v)
        hdr, back = formats.read_vector_store(path)
        assert np.array_equal(back, v) and hdr["dim"] == d and hdr["num_vectors"] == 77
        vpp = 4096 // (d * v.dtype.itemsize)
        assert os.path.getsize(path) == 4096 + ((77 + vpp - 1) // vpp) * 4096
        raw = path.read_bytes()
        _, _, off = formats.VectorPageLayout(d * v.dtype.itemsize).resolve(50)
        assert raw[off:off + d * v.dtype.itemsize] == v[50].tobytes()


def test_pq_and_aux_files(tmp_path):
    rng = np.random.default_rng(1)
    tables = rng.normal(size=(256, 12)).astype(np.float32)
    cen = rng.normal(size=12).astype(np.float32)
    offs = np.array([0, 4, 8, 12], np.uint32)
    codes = rng.integers(0, 256, size=(31, 3)).astype(np.uint8)
    formats.write_pq(tmp_path / "_pq_pivots.bin", tmp_path / "_pq_compressed.bin", tables, cen, offs, codes)
    raw = (tmp_path / "_pq_pivots.bin").read_bytes()
    assert struct.unpack_from("<ii", raw, 0) == (4, 1)                    # offsets block at byte 0
    assert struct.unpack_from("<Q", raw, 8)[0] == 4096                    # tables at the metadata offset
    assert struct.unpack_from("<ii", raw, 4096) == (256, 12)
    t, c, o, k = formats.read_pq(tmp_path / "_pq_pivots.bin", tmp_path / "_pq_compressed.bin")
    assert np.array_equal(t, tables) and np.array_equal(c, cen) and np.array_equal(o, offs) and np.array_equal(k, codes)
    eps = rng.random(31).astype(np.float32)
    formats.write_error_bounds(tmp_path / "eps.bin", eps)
    assert np.array_equal(formats.read_error_bounds(tmp_path / "eps.bin"), eps)
    buckets = [[np.arange(3, dtype=np.int32), np.zeros(0, np.int32)], [np.arange(300, dtype=np.int32), np.array([7], np.int32)]]
    coarse, fine = rng.normal(size=(2, 12)).astype(np.float32), rng.normal(size=(2, 12)).astype(np.float32)
    formats.write_rvq_model(tmp_path / "rvq.bin", coarse, fine, buckets)
    c2, f2, b2 = formats.read_rvq_model(tmp_path / "rvq.bin")
    assert np.array_equal(c2, coarse) and np.array_equal(f2, fine)
    sizes, offsets, ids = formats.flatten_rvq_postings(b2)
    assert sizes.tolist() == [3, 0, 300, 1] and offsets.tolist() == [0, 3, 3, 259, 260] and ids.size == 260
    q = rng.normal(size=(5, 12)).astype(np.float32)
    formats.write_fbin(tmp_path / "q.fbin", q)
    assert np.array_equal(formats.read_fbin(tmp_path / "q.fbin"), q)
    formats.write_gt(tmp_path / "gt.bin", np.arange(10, dtype=np.int32).reshape(5, 2), np.ones((5, 2), np.float32))
    gi, gd = formats.read_gt(tmp_path / "gt.bin")
    assert gi.shape == (5, 2) and gd.shape == (5, 2)


def test_hpq_selector_file_and_learned_stop_model_file(tmp_path):
    # selector bits: int32 rows, int32 cols, rows x cols bytes (src/io/hpq_index.cpp:69-86); shape checks as the loader's
    rng = np.random.default_rng(3)
    bits = rng.integers(0, 256, size=(37, 6), dtype=np.uint8)
    formats.write_hpq_selector_bits(tmp_path / "sel.bin", bits)
    raw = (tmp_path / "sel.bin").read_bytes()
    assert struct.unpack_from("<ii", raw, 0) == (37, 6) and len(raw) == 8 + 37 * 6
    assert np.array_equal(formats.read_hpq_selector_bits(tmp_path / "sel.bin", 37, 48), bits)
    with pytest.raises(ValueError, match="shape does not match"):
        formats.read_hpq_selector_bits(tmp_path / "sel.bin", 37, 64)
    # learned traversal-stop model file folded for one top_l (src/search/topology_search_kernel.cu:248-380)
    from topoanns_b200 import search
    path = tmp_path / "stop.txt"
    path.write_text("# comment\nstage_prefixes = 0, 8,16, 64,200\nfeature_means = " + ",".join(["0.5"] * 12) + "\n"
                    "feature_inv_stds = " + ",".join(["2.0"] * 12) + "\nweights = " + ",".join(str(i) for i in range(12)) + "\n"
                    "bias = 1.0\nthreshold_logit = 0.25\nthreshold_logit_top_l_64 = -0.5\ntopk_churn_mode = flag\n"
                    "feature_mask = 1,1,0,1\n")
    ls = search.load_learned_stop(path, 64, 10)
    assert ls.enabled == 1 and ls.top_k == 10 and ls.topk_churn_flag_mode == 1 and ls.next64_flag_mode == 0
    assert [ls.stage_prefixes[i] for i in range(ls.num_stages)] == [8, 16]          # 0, 64 >= top_l and 200 are dropped
    assert ls.threshold_logit == -0.5 and abs(ls.inv_top_l - 1.0 / 64) < 1e-9
    assert ls.weights[1] == 2.0 and ls.weights[2] == 0.0 and ls.weights[5] == 10.0  # weight / std, masked feature -> 0
    assert abs(ls.bias - (1.0 - 0.5 * sum(2.0 * i for i in range(12) if i != 2))) < 1e-4
    assert search.load_learned_stop(path, 128, 10).threshold_logit == 0.25
    path.write_text("weights = 1,2\nfeature_means = 1\nfeature_inv_stds = 1\n")
    with pytest.raises(ValueError, match="length 12"):
        search.load_learned_stop(path, 64, 10)
