"""Index file layouts of the reference, byte for byte (numpy readers and writers).

* ``topology.bin``  - include/topoanns/topology_layout.hpp:12-23, src/io/topology_layout.cpp:10-195:
  4096-byte header {"TOPOANNS", u32 version = 1, u32 degree, u64 num_nodes, u64 header_bytes,
  u64 payload_bytes}, then num_nodes x degree uint32. The reference reader accepts degree 64 only;
  this reader accepts any degree and ``pad_degree`` writes reference-readable 64-slot rows.
* ``vectors.ssd``   - include/topoanns/vector_store_builder.hpp:13-27, src/builder/vector_store_builder.cpp:
  4096-byte header {"TPVECTOR", u32 version = 1, u32 scalar_kind, u32 dim, u32 reserved, u64
  num_vectors, u64 page_size, u64 vector_bytes, u64 vectors_per_page}, then 4096-byte pages holding
  floor(4096 / vector_bytes) vectors each (src/io/vector_page_layout.cpp:15-57).
* ``_pq_pivots.bin`` / ``_pq_compressed.bin`` - DiskANN layout read by src/io/pq_index.cpp:116-243.
* error bounds      - {i32 N, i32 1} + N float32 (src/search/search_resources.cpp:153-159).
* RVQ model         - src/legacy_rvq/gas_legacy/anns/RVQ/RVQ.cu:884-924,977-1033.
* queries / ground truth - tools/topoanns_eval_sift.cpp:517-568.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

PAGE = 4096
KIND_CODE = {"int8": 0, "uint8": 1, "float32": 2}
KIND_DTYPE = {0: np.int8, 1: np.uint8, 2: np.float32}
INVALID = 0xFFFFFFFF


# ---- topology.bin ---------------------------------------------------------------------------

def pad_degree(adjacency: np.ndarray, degree: int = 64) -> np.ndarray:
    n, r = adjacency.shape
    if r > degree:
        raise ValueError("MakePadded: A node has more than 64 neighbors.")
    out = np.full((n, degree), INVALID, np.uint32)
    out[:, :r] = adjacency.astype(np.uint32, copy=False)
    return out


def write_topology(path, adjacency: np.ndarray) -> None:
    adj = np.ascontiguousarray(adjacency).view(np.uint32) if adjacency.dtype != np.uint32 else np.ascontiguousarray(adjacency)
    n, deg = adj.shape
    header = bytearray(PAGE)
    header[0:8] = b"TOPOANNS"
    struct.pack_into("<IIQQQ", header, 8, 1, deg, n, PAGE, adj.size * 4)
    with open(path, "wb") as f:
        f.write(header)
        f.write(adj.tobytes())


def read_topology(path) -> np.ndarray:
    with open(path, "rb") as f:
        header = f.read(PAGE)
        if len(header) < PAGE:
            raise ValueError("ReadFile: Topology file is smaller than the header.")
        if header[0:8] != b"TOPOANNS":
            raise ValueError("ReadFile: Unexpected topology magic.")
        version, deg, n, hbytes, pbytes = struct.unpack_from("<IIQQQ", header, 8)
        if version != 1:
            raise ValueError("ReadFile: Unexpected topology version.")
        data = f.read()
    if len(data) != n * deg * 4:
        raise ValueError("ReadFile: Topology file size does not match metadata.")
    return np.frombuffer(data, np.uint32).reshape(n, deg)


# ---- vectors.ssd ----------------------------------------------------------------------------

@dataclass
class VectorPageLayout:
    """src/io/vector_page_layout.cpp:15-57"""
    vector_bytes: int
    page_bytes: int = PAGE

    def __post_init__(self):
        if self.vector_bytes == 0 or self.vector_bytes > self.page_bytes:
            raise ValueError("VectorPageLayout: vector does not fit in one page.")

    @property
    def vectors_per_page(self) -> int:
        return self.page_bytes // self.vector_bytes

    def page_count(self, n: int) -> int:
        vpp = self.vectors_per_page
        return (n + vpp - 1) // vpp

    def resolve(self, node_id: int):
        vpp = self.vectors_per_page
        page, slot = node_id // vpp, node_id % vpp
        return page, slot, PAGE + page * self.page_bytes + slot * self.vector_bytes


def vectors_to_pages(vectors: np.ndarray, page_bytes: int = PAGE) -> np.ndarray:
    """[N, d] -> flat uint8 page array (no file header)."""
    v = np.ascontiguousarray(vectors)
    n = v.shape[0]
    vb = v.shape[1] * v.dtype.itemsize
    layout = VectorPageLayout(vb, page_bytes)
    vpp = layout.vectors_per_page
    pages = np.zeros((layout.page_count(n), page_bytes), np.uint8)
    raw = v.view(np.uint8).reshape(n, vb)
    full = (n // vpp) * vpp
    if full:
        pages[: n // vpp, : vpp * vb] = raw[:full].reshape(n // vpp, vpp * vb)
    if n > full:
        pages[n // vpp, : (n - full) * vb] = raw[full:].reshape(-1)
    return pages.reshape(-1)


def write_vector_store(path, vectors: np.ndarray) -> None:
    v = np.ascontiguousarray(vectors)
    n, d = v.shape
    vb = d * v.dtype.itemsize
    layout = VectorPageLayout(vb)
    header = bytearray(PAGE)
    header[0:8] = b"TPVECTOR"
    struct.pack_into("<IIIIQQQQ", header, 8, 1, KIND_CODE[str(v.dtype)], d, 0, n, PAGE, vb, layout.vectors_per_page)
    with open(path, "wb") as f:
        f.write(header)
        f.write(vectors_to_pages(v).tobytes())


def read_vector_store(path):
    """Returns (header dict, vectors [N, d])."""
    with open(path, "rb") as f:
        header = f.read(PAGE)
        if header[0:8] != b"TPVECTOR":
            raise ValueError("ReadHeader: Unexpected vector store magic.")
        version, kind, d, _, n, page, vb, vpp = struct.unpack_from("<IIIIQQQQ", header, 8)
        pages = np.frombuffer(f.read(), np.uint8).reshape(-1, page)
    dt = KIND_DTYPE[kind]
    rows = pages[:, : vpp * vb].reshape(-1, vb)[:n]
    return dict(version=version, scalar_kind=kind, dim=d, num_vectors=n, page_size_bytes=page,
                vector_bytes=vb, vectors_per_page=vpp), rows.view(dt).reshape(n, d)


# ---- PQ files -----------------------------------------------------------------------------------

def _bin_block(rows: int, cols: int, data: np.ndarray) -> bytes:
    return struct.pack("<ii", rows, cols) + np.ascontiguousarray(data).tobytes()


def write_pq(pivots_path, compressed_path, tables_row_major, centroid, chunk_offsets, codes) -> None:
    t = np.ascontiguousarray(tables_row_major, np.float32)
    d = t.shape[1]
    c = np.ascontiguousarray(centroid, np.float32)
    o = np.ascontiguousarray(chunk_offsets, np.uint32)
    t_off = PAGE
    c_off = t_off + 8 + t.nbytes
    o_off = c_off + 8 + c.nbytes
    end = o_off + 8 + o.nbytes
    offsets = np.array([t_off, c_off, o_off, end], np.uint64)
    buf = bytearray(end)
    buf[0:8 + 32] = _bin_block(4, 1, offsets)
    buf[t_off:t_off + 8 + t.nbytes] = _bin_block(256, d, t)
    buf[c_off:c_off + 8 + c.nbytes] = _bin_block(d, 1, c)
    buf[o_off:o_off + 8 + o.nbytes] = _bin_block(o.size, 1, o)
    with open(pivots_path, "wb") as f:
        f.write(buf)
    codes = np.ascontiguousarray(codes, np.uint8)
    with open(compressed_path, "wb") as f:
        f.write(struct.pack("<ii", codes.shape[0], codes.shape[1]))
        f.write(codes.tobytes())


def read_pq(pivots_path, compressed_path):
    """Returns (tables [256, d], centroid [d], chunk_offsets [M+1], codes [N, M])."""
    raw = open(pivots_path, "rb").read()
    rows, cols = struct.unpack_from("<ii", raw, 0)
    if rows not in (4, 5):
        raise ValueError("PqIndex::LoadFromSeparatePaths: Unexpected PQ offset count.")
    offs = np.frombuffer(raw, np.uint64, rows * cols, 8)
    t_off, c_off, o_off = int(offs[0]), int(offs[1]), int(offs[3 if rows == 5 else 2])
    tr, tc = struct.unpack_from("<ii", raw, t_off)
    if tr != 256:
        raise ValueError("PqIndex::LoadFromSeparatePaths: Unexpected PQ centroid count.")
    tables = np.frombuffer(raw, np.float32, tr * tc, t_off + 8).reshape(tr, tc)
    cr, cc = struct.unpack_from("<ii", raw, c_off)
    centroid = np.frombuffer(raw, np.float32, cr * cc, c_off + 8)
    orows, ocols = struct.unpack_from("<ii", raw, o_off)
    chunk_offsets = np.frombuffer(raw, np.uint32, orows * ocols, o_off + 8)
    craw = open(compressed_path, "rb").read()
    n, m = struct.unpack_from("<ii", craw, 0)
    if chunk_offsets.size != m + 1:
        raise ValueError("PqIndex::LoadFromSeparatePaths: Unexpected PQ chunk offsets shape.")
    codes = np.frombuffer(craw, np.uint8, n * m, 8).reshape(n, m)
    return tables, centroid, chunk_offsets, codes


def write_error_bounds(path, eps: np.ndarray) -> None:
    e = np.ascontiguousarray(eps, np.float32)
    with open(path, "wb") as f:
        f.write(_bin_block(e.size, 1, e))


def read_error_bounds(path) -> np.ndarray:
    raw = open(path, "rb").read()
    rows, cols = struct.unpack_from("<ii", raw, 0)
    if cols != 1:
        raise ValueError("LoadPq2Index: Residual error-bound file shape does not match PQ2 point count.")
    return np.frombuffer(raw, np.float32, rows, 8)


# ---- RVQ model ----------------------------------------------------------------------------------

def write_rvq_model(path, coarse, fine, buckets) -> None:
    """buckets[c][f] = int32 id array of the (uncapped) posting list."""
    coarse = np.ascontiguousarray(coarse, np.float32)
    fine = np.ascontiguousarray(fine, np.float32)
    with open(path, "wb") as f:
        f.write(struct.pack("<iii", coarse.shape[1], coarse.shape[0], fine.shape[0]))
        f.write(coarse.tobytes())
        f.write(fine.tobytes())
        f.write(struct.pack("<Q", len(buckets)))
        for inner in buckets:
            f.write(struct.pack("<Q", len(inner)))
            for ids in inner:
                ids = np.ascontiguousarray(ids, np.int32)
                f.write(struct.pack("<Q", ids.size))
                f.write(ids.tobytes())


def write_hpq_selector_bits(path, bits) -> None:
    """Selector-bit file of a hybrid-PQ index (src/io/hpq_index.cpp:69-86): int32 rows, int32 cols, then
    rows x cols bytes; bit m & 7 of byte m >> 3 of a node's row picks the outlier codebook for chunk m."""
    bits = np.ascontiguousarray(bits, np.uint8)
    with open(path, "wb") as f:
        f.write(struct.pack("<ii", bits.shape[0], bits.shape[1]))
        f.write(bits.tobytes())


def read_hpq_selector_bits(path, num_points=None, num_chunks=None):
    raw = open(path, "rb").read()
    rows, cols = struct.unpack_from("<ii", raw, 0)
    if rows < 0 or cols <= 0 or len(raw) < 8 + rows * cols:
        raise ValueError("HpqIndex::Load: Invalid selector-bit metadata.")
    if (num_points is not None and rows != num_points) or (num_chunks is not None and cols != (num_chunks + 7) // 8):
        raise ValueError("HpqIndex::Load: Selector-bit shape does not match HPQ codes.")
    return np.frombuffer(raw, np.uint8, rows * cols, 8).reshape(rows, cols)


def read_rvq_model(path):
    raw = open(path, "rb").read()
    d, nc, nf = struct.unpack_from("<iii", raw, 0)
    if d <= 0 or nc <= 0 or nf <= 0:
        raise ValueError("ReadRvqModelHeader: Invalid RVQ model header in " + str(path))
    pos = 12
    coarse = np.frombuffer(raw, np.float32, nc * d, pos).reshape(nc, d)
    pos += nc * d * 4
    fine = np.frombuffer(raw, np.float32, nf * d, pos).reshape(nf, d)
    pos += nf * d * 4
    (outer,) = struct.unpack_from("<Q", raw, pos)
    pos += 8
    buckets = []
    for _ in range(outer):
        (inner,) = struct.unpack_from("<Q", raw, pos)
        pos += 8
        row = []
        for _ in range(inner):
            (n,) = struct.unpack_from("<Q", raw, pos)
            pos += 8
            row.append(np.frombuffer(raw, np.int32, n, pos))
            pos += 4 * n
        buckets.append(row)
    return coarse, fine, buckets


def flatten_rvq_postings(buckets, limit: int = 256):
    """src/search/rvq_entry_provider.cpp:115-144: sizes (uncapped), CSR offsets / ids capped at 256."""
    sizes, offsets, ids = [], [0], []
    for inner in buckets:
        for b in inner:
            sizes.append(len(b))
            ids.append(np.asarray(b[:limit], np.uint32))
            offsets.append(offsets[-1] + min(len(b), limit))
    flat = np.concatenate(ids) if ids else np.zeros(0, np.uint32)
    return np.array(sizes, np.int32), np.array(offsets, np.uint32), flat.astype(np.uint32)


# ---- queries / ground truth ---------------------------------------------------------------------

def write_fbin(path, x: np.ndarray) -> None:
    x = np.ascontiguousarray(x, np.float32)
    with open(path, "wb") as f:
        f.write(struct.pack("<II", x.shape[0], x.shape[1]))
        f.write(x.tobytes())


def read_fbin(path) -> np.ndarray:
    raw = open(path, "rb").read()
    r, c = struct.unpack_from("<II", raw, 0)
    return np.frombuffer(raw, np.float32, r * c, 8).reshape(r, c)


def write_gt(path, ids: np.ndarray, dists: np.ndarray | None = None) -> None:
    ids = np.ascontiguousarray(ids, np.int32)
    with open(path, "wb") as f:
        f.write(struct.pack("<II", ids.shape[0], ids.shape[1]))
        f.write(ids.tobytes())
        if dists is not None:
            f.write(np.ascontiguousarray(dists, np.float32).tobytes())


def read_gt(path):
    raw = open(path, "rb").read()
    r, c = struct.unpack_from("<II", raw, 0)
    ids = np.frombuffer(raw, np.int32, r * c, 8).reshape(r, c)
    dists = None
    if len(raw) >= 8 + 2 * r * c * 4:
        dists = np.frombuffer(raw, np.float32, r * c, 8 + r * c * 4).reshape(r, c)
    return ids, dists
