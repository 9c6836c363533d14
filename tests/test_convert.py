"""Index converters (tools/topoanns_build_sift_subset.cpp, src/io/diskann_disk_index.cpp of the reference):
a synthetic DiskANN disk index in both node layouts plus a .bvecs base, converted and read back."""
import json
import struct

import numpy as np
import pytest

from topoanns_b200 import convert, formats

INVALID = 0xFFFFFFFF


def _write_diskann(path, coords, lists, capacity, medoid=3):
    n, dim = coords.shape
    node_len = dim * 4 + 4 + capacity * 4
    nps = 4096 // node_len                      # 0: a node spans several sectors
    spn = (node_len + 4095) // 4096
    meta = [n, dim, medoid, node_len, nps, 0, 0, 0, 0]
    with open(path, "wb") as f:
        head = bytearray(4096)
        struct.pack_into("<II9Q", head, 0, 9, 1, *meta)
        f.write(head)
        sector = bytearray(4096)
        for i in range(n):
            rec = coords[i].astype("<f4").tobytes() + struct.pack("<I", len(lists[i]))
            rec += np.asarray(lists[i] + [0xDEADBEEF] * (capacity - len(lists[i])), "<u4").tobytes()
            assert len(rec) == node_len
            if nps > 0:
                k = i % nps
                sector[k * node_len:(k + 1) * node_len] = rec
                if k == nps - 1 or i == n - 1:
                    f.write(sector)
                    sector = bytearray(4096)
            else:
                f.write(rec + bytes(spn * 4096 - node_len))
    return nps


def _write_bvecs(path, x):
    with open(path, "wb") as f:
        for row in x:
            f.write(struct.pack("<I", x.shape[1]) + row.tobytes())


def _expected_adjacency(lists, num_vectors):
    adj = np.full((num_vectors, 64), INVALID, np.uint32)
    filtered = 0
    for i in range(num_vectors):
        for j, v in enumerate(lists[i][:64]):
            if v < num_vectors:
                adj[i, j] = v
            else:
                filtered += 1
    return adj, filtered


@pytest.mark.parametrize("dim,capacity", [(8, 70), (960, 64)])
def test_diskann_subset_conversion(tmp_path, dim, capacity):
    rng = np.random.default_rng(7)
    n, keep = 300, 211
    base = rng.integers(0, 256, size=(n, dim), dtype=np.uint8)
    lists = [rng.choice(n, size=int(rng.integers(0, capacity + 1)), replace=False).tolist() for _ in range(n)]
    nps = _write_diskann(tmp_path / "disk.index", base.astype(np.float32), lists, capacity)
    assert (nps > 0) == (dim == 8)
    _write_bvecs(tmp_path / "base.bvecs", base)
    codes = rng.integers(0, 256, size=(n, 4), dtype=np.uint8)
    formats.write_pq(tmp_path / "pivots.bin", tmp_path / "codes.bin", rng.normal(size=(256, dim)).astype(np.float32),
                     np.zeros(dim, np.float32), np.array([0, dim // 4, dim // 2, 3 * dim // 4, dim], np.uint32), codes)
    layout = convert.DiskannLayout.load(tmp_path / "disk.index")
    assert (layout.num_nodes, layout.vector_dim, layout.medoid_id, layout.neighbor_capacity) == (n, dim, 3, capacity)
    assert layout.node_offset(0) == 4096
    if nps > 0:
        assert layout.node_offset(nps + 1) == 4096 + 4096 + layout.max_node_len
    else:
        assert layout.node_offset(2) == 4096 + 2 * layout.sectors_per_node * 4096
    out = tmp_path / "out"
    rc = convert.main(["--base-bvecs", str(tmp_path / "base.bvecs"), "--disk-index", str(tmp_path / "disk.index"),
                       "--pq-pivots", str(tmp_path / "pivots.bin"), "--pq-compressed", str(tmp_path / "codes.bin"),
                       "--output-dir", str(out), "--num-vectors", str(keep)])
    assert rc == 0
    want_adj, want_filtered = _expected_adjacency(lists, keep)
    assert np.array_equal(formats.read_topology(out / "topology.bin"), want_adj)
    header, vectors = formats.read_vector_store(out / "vectors.ssd")
    assert vectors.dtype == np.float32 and header["num_vectors"] == keep
    assert np.array_equal(vectors, base[:keep].astype(np.float32))
    tables, centroid, offsets, got_codes = formats.read_pq(out / "_pq_pivots.bin", out / "_pq_compressed.bin")
    assert np.array_equal(got_codes, codes[:keep])
    manifest = json.loads((out / "manifest.json").read_text())
    assert manifest["num_vectors"] == keep and manifest["diskann_medoid"] == 3
    assert manifest["diskann_neighbor_capacity"] == capacity and manifest["topology_degree"] == 64
    _, filtered = convert.extract_topology(tmp_path / "disk.index", layout, keep, chunk_nodes=50)
    assert filtered == want_filtered and want_filtered > 0
    # uint8 kept as uint8
    convert.build_subset(tmp_path / "base.bvecs", tmp_path / "disk.index", tmp_path / "out8", keep, keep_scalar=True,
                         log=lambda *_: None)
    _, v8 = formats.read_vector_store(tmp_path / "out8" / "vectors.ssd")
    assert v8.dtype == np.uint8 and np.array_equal(v8, base[:keep])


def test_converter_errors(tmp_path):
    base = np.zeros((4, 8), np.uint8)
    _write_bvecs(tmp_path / "base.bvecs", base)
    _write_diskann(tmp_path / "small.index", base.astype(np.float32), [[1], [2], [3], [0]], 10)   # < 64 neighbours
    assert convert.main(["--base-bvecs", str(tmp_path / "base.bvecs"), "--disk-index", str(tmp_path / "small.index"),
                         "--output-dir", str(tmp_path / "o"), "--num-vectors", "4"]) == 1
    with open(tmp_path / "bad.index", "wb") as f:
        f.write(struct.pack("<II", 8, 1) + bytes(4096))
    with pytest.raises(ValueError, match="Unexpected DiskANN metadata header"):
        convert.DiskannLayout.load(tmp_path / "bad.index")
    with pytest.raises(ValueError, match="exceeds"):
        convert.read_vecs(tmp_path / "base.bvecs", 0, 5, np.uint8)
    with open(tmp_path / "ragged.bvecs", "wb") as f:
        f.write(struct.pack("<I", 8) + bytes(8) + struct.pack("<I", 7) + bytes(8))
    with pytest.raises(ValueError, match="dimension mismatch"):
        convert.read_vecs(tmp_path / "ragged.bvecs", 0, 2, np.uint8)
