"""Generates tests/golden/reference_small.npz: a tiny seeded index together with what the REFERENCE
ITSELF (its own sources, built in place by oracle/ref_build.sh into oracle/_ref/ref_driver) computed
for it on a B200: query tables, traversal candidate lists and statistics for two parameter sets, and
the uint8 rerank lists. Needs a GPU and the reference build; the committed .npz lets the CPU tests pin
the checker (and the GPU tests the CUDA path) against the reference without either.

    python tests/golden/make_reference_fixtures.py [out.npz]  # default: rewrites reference_small.npz
"""
import dataclasses
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import pipeline  # noqa: E402
from topoanns_b200 import formats, synth  # noqa: E402

DRIVER = ROOT / "oracle" / "_ref" / "ref_driver"
CASES = [dict(top_l=32, width=2), dict(top_l=16, width=1)]
TOP_N, TOP_K, MAX_EXP = 16, 10, 4096


def run_driver(tmp, tag, mode, *args):
    cmd = [str(DRIVER), str(tmp), str(tmp / tag), mode] + [str(a) for a in args]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if r.returncode != 0:
        raise RuntimeError(r.stdout[-2000:] + r.stderr[-2000:])


def load(tmp, tag, name, dtype):
    return np.fromfile(tmp / f"{tag}.{name}.bin", dtype=dtype)


def main():
    cfg = dataclasses.replace(synth.CONFIGS["cfg1"], num_nodes=1024, components=8, num_queries=24, dim=64,
                              pq_chunks=16, knn_edges=48, random_edges=16, train_sample=1024, kmeans_iters=6, seed=77)
    s = synth.build(cfg, "cuda")
    host = pipeline.index_from_synth(s)
    Q = s.queries.shape[0]
    rng = np.random.default_rng(5)
    entries = np.tile(rng.integers(0, cfg.num_nodes, size=4, dtype=np.uint32), (Q, 1))   # the same 4 entry nodes for every query
    out = {
        "vectors": host["vectors"], "adjacency": host["adjacency"], "codes": host["codes"],
        "pq_tables": host["pq_tables"], "pq_centroid": host["pq_centroid"],
        "pq_chunk_offsets": host["pq_chunk_offsets"], "queries": s.queries.cpu().numpy(), "entries": entries,
        "top_n": np.int64(TOP_N), "top_k": np.int64(TOP_K), "max_expansions": np.int64(MAX_EXP),
    }
    with tempfile.TemporaryDirectory() as d:
        tmp = Path(d)
        formats.write_topology(tmp / "topology.bin", formats.pad_degree(host["adjacency"], 64))
        formats.write_pq(tmp / "_pq_pivots.bin", tmp / "_pq_compressed.bin", host["pq_tables"], host["pq_centroid"],
                         host["pq_chunk_offsets"], host["codes"])
        formats.write_vector_store(tmp / "vectors.ssd", host["vectors"])
        formats.write_fbin(tmp / "queries.fbin", out["queries"])
        with open(tmp / "entries.bin", "wb") as f:
            f.write(np.array(entries.shape, np.uint32).tobytes())
            f.write(entries.tobytes())
        M = host["codes"].shape[1]
        run_driver(tmp, "lut", "lut", 32, 2, MAX_EXP, TOP_K, TOP_N)
        out["ref_lut"] = load(tmp, "lut", "lut", np.float32).reshape(Q, M, 256)[:4].copy()   # first 4 queries
        for c in CASES:
            tag = f"s{c['top_l']}_{c['width']}"
            limit = max(c["top_l"], TOP_N)
            run_driver(tmp, tag, "search", c["top_l"], c["width"], MAX_EXP, TOP_K, TOP_N, "linear", 16, 0, 0, 1)
            out[f"ref_{tag}_ids"] = load(tmp, tag, "search0_ids", np.uint32).reshape(Q, limit)
            out[f"ref_{tag}_dist"] = load(tmp, tag, "search0_dist", np.float32).reshape(Q, limit)
            out[f"ref_{tag}_stats"] = load(tmp, tag, "search0_stats", np.uint32).reshape(Q, 3)
        run_driver(tmp, "u8", "e2e_u8", 32, 2, MAX_EXP, TOP_K, TOP_N)
        out["ref_rerank_ids"] = load(tmp, "u8", "rerank_ids", np.uint32).reshape(Q, TOP_N)
        out["ref_rerank_dist"] = load(tmp, "u8", "rerank_dist", np.float32).reshape(Q, TOP_N)
    path = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).with_name("reference_small.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
