"""Index converters: a DiskANN disk index plus the base vectors it was built from become the files the
search path loads (`topology.bin`, `vectors.ssd`, `_pq_pivots.bin`, `_pq_compressed.bin`, `manifest.json`).

Same inputs, flags and outputs as the reference's `tools/topoanns_build_sift_subset.cpp` (vectors :153-228,
topology :230-322, PQ files and manifest :324-343) with its DiskANN layout reader
(`src/io/diskann_disk_index.cpp`, `include/topoanns/diskann_disk_index.hpp`); the work is done with array
slicing instead of per-record loops. Also reads `.fvecs` / `.fbin` / `.u8bin` bases, which the reference's tool
does not.

    python -m topoanns_b200.convert --base-bvecs base.bvecs --disk-index index_disk.index \\
        --pq-pivots index_pq_pivots.bin --pq-compressed index_pq_compressed.bin \\
        --output-dir out --num-vectors 1000000
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import struct
import sys
from dataclasses import dataclass

import numpy as np

from . import formats

SECTOR = 4096
INVALID = 0xFFFFFFFF
DEGREE = 64


# ---- base vectors ---------------------------------------------------------------------------------
def vecs_metadata(path, scalar_bytes: int):
    """(dim, record_bytes, num_vectors) of a .bvecs (scalar_bytes = 1) or .fvecs / .ivecs (4) file: every
    record is a uint32 dimension followed by dim scalars (include/topoanns/bvecs_io.hpp:12-18)."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(4)
    if len(head) != 4:
        raise ValueError("ReadBvecsMetadata: file is too short: %s" % path)
    dim = struct.unpack("<I", head)[0]
    record = 4 + dim * scalar_bytes
    if dim == 0 or size % record != 0:
        raise ValueError("ReadBvecsMetadata: file size is not a whole number of records: %s" % path)
    return dim, record, size // record


def read_vecs(path, start: int, count: int, dtype) -> np.ndarray:
    """Rows [start, start + count) of a .bvecs / .fvecs / .ivecs file as [count, dim] of dtype; every
    record's dimension field is checked."""
    dt = np.dtype(dtype)
    dim, record, total = vecs_metadata(path, dt.itemsize)
    if start + count > total:
        raise ValueError("Requested range exceeds the file: %s" % path)
    raw = np.fromfile(path, np.uint8, count=count * record, offset=start * record).reshape(count, record)
    dims = raw[:, :4].copy().view("<u4").reshape(-1)
    if np.any(dims != dim):
        raise ValueError("Per-record dimension mismatch in %s" % path)
    return raw[:, 4:].copy().view(dt).reshape(count, dim)


def read_base(path, count: int) -> np.ndarray:
    """Base vectors by file extension: .bvecs (uint8), .fvecs (float32), .fbin / .u8bin / .i8bin
    (uint32 rows, uint32 cols, then the rows)."""
    ext = os.path.splitext(str(path))[1].lower()
    if ext == ".bvecs":
        return read_vecs(path, 0, count, np.uint8)
    if ext == ".fvecs":
        return read_vecs(path, 0, count, np.float32)
    if ext in (".fbin", ".u8bin", ".i8bin", ".bin"):
        dt = {".fbin": np.float32, ".u8bin": np.uint8, ".i8bin": np.int8, ".bin": np.float32}[ext]
        with open(path, "rb") as f:
            rows, cols = struct.unpack("<II", f.read(8))
        if count > rows:
            raise ValueError("Requested num_vectors exceeds source dataset size.")
        return np.fromfile(path, dt, count=count * cols, offset=8).reshape(count, cols)
    raise ValueError("Unknown base vector format: %s" % path)


# ---- DiskANN disk index ---------------------------------------------------------------------------
@dataclass
class DiskannLayout:
    """The nine metadata words of a DiskANN disk index (include/topoanns/diskann_disk_index.hpp:10-20) and
    the node addressing derived from them (src/io/diskann_disk_index.cpp:45-73)."""
    num_nodes: int
    vector_dim: int
    medoid_id: int
    max_node_len: int
    nodes_per_sector: int
    num_frozen_points: int
    file_num_frozen_points: int
    append_reorder: int
    reorder_data_start: int

    @staticmethod
    def load(path) -> "DiskannLayout":
        with open(path, "rb") as f:
            head = f.read(8 + 9 * 8)
        if len(head) < 80:
            raise ValueError("DiskannDiskIndexLayout::Load: Failed to read metadata payload.")
        count, dim = struct.unpack_from("<II", head, 0)
        if count != 9 or dim != 1:
            raise ValueError("DiskannDiskIndexLayout::Load: Unexpected DiskANN metadata header.")
        return DiskannLayout(*struct.unpack_from("<9Q", head, 8))

    @property
    def coord_bytes(self) -> int:
        return self.vector_dim * 4

    @property
    def neighbor_capacity(self) -> int:
        if self.max_node_len < self.coord_bytes + 4:
            raise ValueError("DiskannDiskIndexLayout::neighbor_capacity: Invalid max_node_len.")
        return (self.max_node_len - self.coord_bytes - 4) // 4

    @property
    def sectors_per_node(self) -> int:
        return (self.max_node_len + SECTOR - 1) // SECTOR

    def node_offset(self, node_id: int) -> int:
        if node_id >= self.num_nodes:
            raise ValueError("DiskannDiskIndexLayout::NodeOffsetBytes: node_id is out of bounds.")
        if self.nodes_per_sector > 0:
            return SECTOR + (node_id // self.nodes_per_sector) * SECTOR + (node_id % self.nodes_per_sector) * self.max_node_len
        return SECTOR + node_id * self.sectors_per_node * SECTOR


def extract_topology(disk_index_path, layout: DiskannLayout, num_vectors: int, chunk_nodes: int = 1 << 18):
    """Adjacency [num_vectors, 64] uint32 of the first num_vectors nodes: the first min(degree, 64) stored
    neighbours of every node in their slots, neighbours >= num_vectors replaced by the invalid id in place,
    the rest invalid (tools/topoanns_build_sift_subset.cpp:230-322). Returns (adjacency, filtered count)."""
    if layout.neighbor_capacity < DEGREE:
        raise ValueError("DiskANN index has fewer than 64 neighbors per node.")
    adjacency = np.full((num_vectors, DEGREE), INVALID, np.uint32)
    filtered = 0
    node_len = layout.max_node_len
    nps = layout.nodes_per_sector
    with open(disk_index_path, "rb") as f:
        done = 0
        while done < num_vectors:
            n = min(chunk_nodes, num_vectors - done)
            if nps > 0:
                first_sector = done // nps
                last_sector = (done + n - 1) // nps
                f.seek(SECTOR + first_sector * SECTOR)
                want = (last_sector - first_sector + 1) * SECTOR
                buf = np.frombuffer(f.read(want), np.uint8)
                if buf.size != want:
                    raise ValueError("Short read while extracting DiskANN sectors.")
                sectors = buf.reshape(-1, SECTOR)[:, : nps * node_len].reshape(-1, node_len)
                nodes = sectors[done - first_sector * nps: done - first_sector * nps + n]
            else:
                stride = layout.sectors_per_node * SECTOR
                f.seek(SECTOR + done * stride)
                buf = np.frombuffer(f.read(n * stride), np.uint8)
                if buf.size != n * stride:
                    raise ValueError("Short read while extracting multi-sector DiskANN nodes.")
                nodes = buf.reshape(n, stride)[:, :node_len]
            tail = np.ascontiguousarray(nodes[:, layout.coord_bytes: layout.coord_bytes + 4 + DEGREE * 4]).view("<u4")
            degree = np.minimum(tail[:, 0], DEGREE)
            neigh = tail[:, 1:1 + DEGREE]
            in_list = np.arange(DEGREE, dtype=np.uint32)[None, :] < degree[:, None]
            in_range = neigh < num_vectors
            filtered += int(np.count_nonzero(in_list & ~in_range))
            adjacency[done:done + n] = np.where(in_list & in_range, neigh, INVALID)
            done += n
    return adjacency, filtered


def slice_pq_compressed(src, dst, num_vectors: int) -> None:
    """First num_vectors rows of a PQ code file (int32 rows, int32 cols, then the rows)."""
    with open(src, "rb") as f:
        rows, cols = struct.unpack("<ii", f.read(8))
        if num_vectors > rows:
            raise ValueError("Requested num_vectors exceeds the PQ code file.")
        body = f.read(num_vectors * cols)
    if len(body) != num_vectors * cols:
        raise ValueError("Short read while slicing PQ codes.")
    with open(dst, "wb") as f:
        f.write(struct.pack("<ii", num_vectors, cols))
        f.write(body)


def build_subset(base_path, disk_index_path, output_dir, num_vectors: int, pq_pivots=None, pq_compressed=None,
                 keep_scalar: bool = False, log=print) -> dict:
    """Writes the index directory; returns the manifest. Vectors are stored as float32 like the reference's
    tool unless keep_scalar is set (uint8 bases then stay uint8: a quarter of the bytes per rerank row)."""
    os.makedirs(output_dir, exist_ok=True)
    layout = DiskannLayout.load(disk_index_path)
    base = read_base(base_path, num_vectors)
    if base.shape[1] != layout.vector_dim:
        raise ValueError("bvecs dim and DiskANN vector dim do not match.")
    if num_vectors > layout.num_nodes:
        raise ValueError("Requested num_vectors exceeds source dataset size.")
    vectors = base if keep_scalar else base.astype(np.float32)
    formats.write_vector_store(os.path.join(output_dir, "vectors.ssd"), vectors)
    log("[topoanns_build] converted vectors %d / %d" % (num_vectors, num_vectors))
    adjacency, filtered = extract_topology(disk_index_path, layout, num_vectors)
    formats.write_topology(os.path.join(output_dir, "topology.bin"), adjacency)
    log("[topoanns_build] extracted topology %d / %d" % (num_vectors, num_vectors))
    log("[topoanns_build] filtered out-of-range neighbors: %d" % filtered)
    if pq_pivots:
        shutil.copyfile(pq_pivots, os.path.join(output_dir, "_pq_pivots.bin"))
    if pq_compressed:
        slice_pq_compressed(pq_compressed, os.path.join(output_dir, "_pq_compressed.bin"), num_vectors)
    vb = vectors.shape[1] * vectors.dtype.itemsize
    manifest = {
        "num_vectors": int(num_vectors), "dim": int(vectors.shape[1]), "vector_scalar": str(vectors.dtype),
        "topology_degree": DEGREE, "vectors_per_page": formats.VectorPageLayout(vb).vectors_per_page,
        "source_base_bvecs": str(base_path), "source_disk_index": str(disk_index_path),
        "diskann_medoid": int(layout.medoid_id), "diskann_neighbor_capacity": int(layout.neighbor_capacity),
    }
    with open(os.path.join(output_dir, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=2)
        f.write("\n")
    log("[topoanns_build] done")
    return manifest


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--base-bvecs", required=True, help=".bvecs / .fvecs / .fbin / .u8bin base vectors")
    ap.add_argument("--disk-index", required=True)
    ap.add_argument("--pq-pivots")
    ap.add_argument("--pq-compressed")
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--num-vectors", type=int, required=True)
    ap.add_argument("--chunk-vectors", type=int, default=0, help="accepted for compatibility; unused")
    ap.add_argument("--keep-scalar", action="store_true", help="store uint8 bases as uint8 instead of float32")
    a = ap.parse_args(argv)
    try:
        build_subset(a.base_bvecs, a.disk_index, a.output_dir, a.num_vectors, a.pq_pivots, a.pq_compressed, a.keep_scalar)
    except (ValueError, OSError) as e:
        print("[topoanns_build] %s" % e, file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
