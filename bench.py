#!/usr/bin/env python
"""Benchmark of the batched graph-search path.

  python bench.py --gpus N --steps K --warmup W            # this library (CUDA)
  python bench.py --impl reference --gpus N --steps K ...   # the CPU implementation, host cores
  python bench.py --stages --config cfg3 --nodes ...        # per-stage CUDA-event timings (for profilers)

One "step" is one pass of the whole path (RVQ entry selection -> table build + beam search ->
exact rerank -> top-k) over one batch of 10 000 synthetic queries on the 10 M-vector uint8 d=128
configuration (R = 64, M = 32, two-level RVQ entries). Every step takes its own seeded query batch
(generated before the timed region). The operating point (top_l, rerank top_n) is picked before the
timed region by a sweep over the configuration's L values: the fastest point with recall@10 >= 0.95,
or the highest-recall point when none reaches it (stated in `config`).

Prints ONE JSON line: `value` = device-resident QPS over all ranks, `e2e` = QPS through the host
buffer entry point (H2D of the queries and D2H of ids/distances inside the timed region),
`roofline` for the beam-search kernel (algorithmic gather bytes / its own launch time, against the
measured HBM copy bandwidth), `cpu_baseline` = the CPU implementation timed on this box's cores,
`parity` = the CUDA results against that CPU implementation on the same queries at the timed
operating point. With N > 1 ranks the line also carries `sharded`: the same path over an index split
by node-id range across the GPUs (remote rows read over NVLink inside the kernels, the top-k lists
collected on rank 0 with one NCCL gather inside the end-to-end region).
"""
import argparse
import ctypes as C
import dataclasses
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

os.environ.setdefault("NCCL_DEBUG", "WARN")  # keeps NCCL's version banner off stdout: one JSON line only

import numpy as np  # noqa: E402
import torch  # noqa: E402

# one string for both arms: the driver divides the two lines only when their metrics are the same
METRIC = "QPS at recall@10>=0.95 (10M uint8 d=128, 1 batch of 10k queries per GPU)"
L_SWEEP = (16, 32, 64, 128, 256, 512, 1024)
TOPN_SWEEP = (32, 128, 192, 256, 512)
DEFAULT_POINT = (16, 192)   # (top_l, rerank_top_n): fastest sweep point with recall@10 >= 0.95 on the seeded cfg2 data
# candidates for the degree-32 sharded index (its recall falls as the index grows with the number of GPUs)
SHARDED_POINTS = ((16, 256), (32, 256), (32, 512), (64, 512), (64, 1024), (128, 1024), (128, 2048))
# DRAM traffic of one beam_search_kernel launch (10 k queries, 10 M nodes), ncu dram__bytes_read.sum +
# dram__bytes_write.sum, keyed by (top_l, candidate capacity) - the kernel does not depend on rerank_top_n
# beyond the capacity it implies; summarised under profiles/.
NCU_BEAM_TRAFFIC_BYTES_PLAIN = {(16, 256): 749.9e6}
NCU_BEAM_TRAFFIC_BYTES_NEIGHBOR_CODES = {(16, 256): 489.7e6}
RECALL_TARGET = 0.95
MAX_DISTINCT_BATCHES = 64
NVLINK_INGRESS_GBS = 900.0   # nominal NVLink 5 bandwidth per direction per GPU


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="cfg2", help="synthetic configuration (cfg1..cfg5); the metric is quoted on cfg2")
    ap.add_argument("--nodes", type=int, default=0, help="base vectors (default: cfg2's 10 M; other configs: their own size)")
    ap.add_argument("--queries", type=int, default=10_000)
    ap.add_argument("--top-l", type=int, default=0, help="skip the sweep and use this top_l")
    ap.add_argument("--top-n", type=int, default=0, help="with --top-l: rerank top_n (default 32)")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the CPU baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true",
                    help="--impl reference: skip the timed run of the reference's own GPU kernels (oracle/_ref)")
    ap.add_argument("--streams", type=int, default=4,
                    help="searchers (each on its own stream) that the steps alternate between; 1 = one batch at a time")
    ap.add_argument("--no-neighbor-codes", action="store_true",
                    help="do not build the neighbour-code layout (degree * M bytes per node of extra HBM)")
    ap.add_argument("--shard-nodes", type=int, default=10_000_000,
                    help="N > 1: rows per GPU of the node-id-range-sharded leg (R = 32 records as in the 1 B-vector configuration)")
    ap.add_argument("--no-sharded-leg", action="store_true", help="N > 1: skip the node-id-range-sharded leg")
    ap.add_argument("--shard-rvq-side", type=int, default=0,
                    help="centroids per level of the sharded index's entry model (0: 256, doubled while a bucket "
                         "would hold more than 640 nodes)")
    ap.add_argument("--shard-gt-stride", type=int, default=1,
                    help="N > 1: brute-force ground truth of the sharded leg for every n-th query only (very large shards)")
    ap.add_argument("--sharded-only", action="store_true",
                    help="N > 1: run only the sharded leg and print its record as the line (very large shards)")
    ap.add_argument("--stages", action="store_true",
                    help="per-stage CUDA-event timings of one synthetic case (1 GPU), one line per stage; for profilers")
    ap.add_argument("--top-l-values", default="", help="--stages: comma-separated top_l values timed on one index build")
    ap.add_argument("--search-width", type=int, default=2)
    ap.add_argument("--entries", type=int, default=128)
    ap.add_argument("--reps", type=int, default=5, help="--stages: timed calls per stage")
    ap.add_argument("--staged-table", action="store_true", help="--stages: build the query tables with tann_lut_build first")
    ap.add_argument("--topology", default="hbm", choices=["hbm", "pinned-host"],
                    help="--stages: where the adjacency lists live (pinned-host = mapped host memory read over PCIe)")
    ap.add_argument("--vectors", default="hbm", choices=["hbm", "pinned-host"],
                    help="--stages: where the vector pages live")
    ap.add_argument("--cached-fractions", default="", help="--stages: comma-separated cached fractions timed on one index build")
    ap.add_argument("--cached-fraction", type=float, default=0.0,
                    help="--stages --topology pinned-host: fraction of the rows (an id prefix) cached in HBM")
    return ap.parse_args()


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def host_threads():
    """Host threads this process may run on (the launcher's OMP_NUM_THREADS does not count)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        try:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        except Exception:
            pass
        try:
            self.out.close()
            rows = [r.split(", ") for r in open(self.path).read().strip().splitlines() if r.strip()]
            os.unlink(self.path)
            sm = [float(r[1]) for r in rows if len(r) >= 9]
            if sm:
                out["sm_mhz"] = float(np.median(sm))
                out["sm_max_mhz"] = float(rows[0][2])
                names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
                for i, n in enumerate(names):
                    if any(r[5 + i].strip().lower() == "active" for r in rows if len(r) >= 9):
                        out["reasons"].append(n)
                out["samples"] = len(sm)
        except Exception:
            pass
        return out


def build_index(args, device):
    from topoanns_b200 import synth
    base = synth.CONFIGS[args.config]
    nodes = args.nodes or base.num_nodes
    cfg = dataclasses.replace(base, num_nodes=nodes, num_queries=args.queries, components=max(1, nodes // 1000))
    t0 = time.time()
    s = synth.build(cfg, device)
    if device != "cpu":
        torch.cuda.synchronize()
    return s, time.time() - t0


def algorithmic_bytes(stats, degree, M, top_n, vector_bytes):
    """Per-query gather bytes: E * 4 * degree (adjacency rows) + V * M (code rows) for the traversal,
    + top_n * vector_bytes for the rerank."""
    E = stats[:, 1].astype(np.float64)
    V = stats[:, 0].astype(np.float64)
    beam = float((E * 4 * degree + V * M).sum())
    rerank = float(stats.shape[0] * top_n * vector_bytes)
    return beam, rerank


def cpu_leg(s, L, top_n, seconds, cuda_ids=None, cuda_dists=None):
    """Times the CPU implementation (the checker's restatement, OpenMP over queries, every host thread this
    process may use) on the same index and parameters, on as many of the batch's queries as fit the time
    budget; with the CUDA results of the same queries given, also compares the two lists query by query."""
    from oracle import oracle as orc
    from oracle import pipeline
    from topoanns_b200 import synth
    orc.set_num_threads(host_threads())    # a launcher may have exported OMP_NUM_THREADS=1
    host = pipeline.index_from_synth(s)
    q = s.queries.cpu().numpy()
    kw = dict(top_l=L, search_width=2, max_expansions=4096, top_n=top_n, top_k=10, entry_count=128)
    n = min(q.shape[0], 500)
    tm = {}
    pipeline.run(host, q[:n], timings=tm, **kw)          # warm-up + rate estimate
    rate = n / max(tm["total"], 1e-6)
    n = int(min(q.shape[0], max(500, rate * seconds / 3)))
    best = None
    reps = 0
    t_begin = time.perf_counter()
    while reps < 3 or (time.perf_counter() - t_begin < seconds and reps < 50):
        tm = {}
        r = pipeline.run(host, q[:n], timings=tm, **kw)
        best = tm["total"] if best is None else min(best, tm["total"])
        reps += 1
    gt = s.gt_ids.cpu().numpy()[:n]
    recall = synth.recall_at_k(r["topk_ids"], gt, 10)
    res = dict(value=n / best, unit="queries/s", cores=orc.num_threads(), kind="port",
               sample=f"{n} of {q.shape[0]} queries x {reps} passes (best pass), top_l={L}, rerank_top_n={top_n}, "
                      f"recall@10={recall:.3f}")
    parity = None
    if cuda_ids is not None:
        same_ids = (np.asarray(cuda_ids[:n]).view(np.uint32) == r["topk_ids"].view(np.uint32)).all(1)
        same_bits = (np.asarray(cuda_dists[:n]).view(np.uint32) == r["topk_dists"].view(np.uint32)).all(1)
        parity = dict(queries=int(n), top10_identical_frac=float(same_ids.mean()),
                      dist_bits_identical_frac=float(same_bits.mean()),
                      recall_cuda=round(synth.recall_at_k(np.asarray(cuda_ids[:n]), gt, 10), 4),
                      recall_cpu=round(recall, 4), top_l=L, rerank_top_n=top_n,
                      against="CPU restatement of the reference path (oracle/), same index, same queries")
    return res, parity


def reference_gpu_leg(s, host, L, top_n, cpu_ids=None):
    """The reference's own CUDA kernels (its sources compiled in place for sm_100a by oracle/ref_build.sh) on the
    same index, queries and parameters, beside the CPU baseline: its fused entry point RunBatchFloat32Fused with
    the entry lists given, timed per batch as a caller sees it (its query upload, kernels, result download and
    host materialisation). Returns None when that build or a GPU is absent."""
    driver = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
    if not (os.path.exists(driver) and torch.cuda.is_available()) or host["adjacency"].shape[1] > 64:
        return None
    from oracle import oracle as orc
    from topoanns_b200 import formats
    q = s.queries.cpu().numpy()
    with tempfile.TemporaryDirectory() as tmp:
        formats.write_topology(os.path.join(tmp, "topology.bin"), formats.pad_degree(host["adjacency"], 64))
        formats.write_pq(os.path.join(tmp, "_pq_pivots.bin"), os.path.join(tmp, "_pq_compressed.bin"), host["pq_tables"],
                         host["pq_centroid"], host["pq_chunk_offsets"], host["codes"])
        formats.write_vector_store(os.path.join(tmp, "vectors.ssd"), host["vectors"])
        formats.write_fbin(os.path.join(tmp, "queries.fbin"), q)
        clusters, _, _ = orc.rvq_clusters(q, host["rvq_coarse"], host["rvq_fine"], host["rvq_sizes"])
        entries = np.ascontiguousarray(orc.rvq_gather(clusters, host["rvq_offsets"], host["rvq_ids"], 128), np.uint32)
        with open(os.path.join(tmp, "entries.bin"), "wb") as f:
            f.write(np.array(entries.shape, np.uint32).tobytes())
            f.write(entries.tobytes())
        r = subprocess.run([driver, tmp, os.path.join(tmp, "out"), "time", str(L), "2", "4096", "10", str(top_n), "linear",
                            "16", "0", "0", "3"], capture_output=True, text=True, timeout=1200)
        if r.returncode != 0:
            return {"error": (r.stdout + r.stderr)[-300:]}
        fields = {}
        for line in r.stdout.splitlines():
            if line.startswith("ref_time"):
                fields = dict(kv.split("=") for kv in line.split()[1:])
        ids = np.fromfile(os.path.join(tmp, "out.time_topk_ids.bin"), np.uint32).reshape(q.shape[0], 10)
    from topoanns_b200 import synth
    out = {"value": q.shape[0] / (float(fields["best_ms"]) * 1e-3), "unit": "queries/s",
           "ms_per_batch": float(fields["best_ms"]), "traversal_kernel_ms": float(fields["traversal_kernel_ms"]),
           "recall_at_10": round(synth.recall_at_k(ids, s.gt_ids.cpu().numpy(), 10), 4),
           "what": "the reference's CUDA kernels compiled in place for sm_100a, RunBatchFloat32Fused on the same index files "
                   f"({q.shape[0]} queries, top_l={L}, rerank_top_n={top_n}, linear rerank, entry lists given), best of 3 batches, "
                   "wall clock around the call; RVQ entry selection is not in its timed call and its persistent rerank "
                   "needs the NVMe provider"}
    if cpu_ids is not None:
        n = min(cpu_ids.shape[0], ids.shape[0])
        out["top10_identical_to_cpu_port_frac"] = float((ids[:n] == cpu_ids[:n]).all(1).mean())
    return out


def reference_arm(args, s, workload):
    """The reference's path on the host cores (CPU restatement; the reference ships no CPU implementation of the
    batched path of its own), and beside it - one GPU, first rank only - the reference's own GPU kernels."""
    Q = s.queries.shape[0]
    L = args.top_l or DEFAULT_POINT[0]       # the operating point the CUDA arm's sweep settles on for this seeded workload
    top_n = args.top_n or DEFAULT_POINT[1]
    res, _ = cpu_leg(s, L, top_n, args.cpu_seconds)
    line = {"impl": "reference", "metric": METRIC,
            "value": res["value"], "unit": "queries/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * Q / res["value"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": workload, "top_l": L, "rerank_top_n": top_n,
                       "note": "host cores only; one process whatever --gpus says"},
            "cpu_baseline": res,
            "e2e": {"value": res["value"], "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if args.gpus == 1 and not args.no_reference_gpu:
        try:
            from oracle import pipeline
            rg = reference_gpu_leg(s, pipeline.index_from_synth(s), L, top_n)
            if rg is not None:
                line["reference_gpu"] = rg
        except Exception as e:   # an aid beside the baseline: never takes the line down
            line["reference_gpu"] = {"error": f"{type(e).__name__}: {e}"}
    print(json.dumps(line))


def _time_calls(fn, reps):
    """One warm-up call, then `reps` calls back to back between two CUDA events; (last result, mean ms)."""
    out = fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        out = fn()
    stop.record()
    torch.cuda.synchronize()
    return out, start.elapsed_time(stop) / reps


def stage_timings(args):
    """The stages of the path, each timed alone with CUDA events on one synthetic case (any configuration, any
    size); prints one line per stage and a closing JSON line per case. Small cases of this mode are what profiler
    captures run. One index build serves every value of --top-l-values and --cached-fractions."""
    from topoanns_b200 import capi, search, synth
    lib = capi.load()
    s, build_s = build_index(args, "cuda")
    cfg = s.cfg
    base_ix = search.device_index_from_synth(s)
    q = s.queries.cuda().contiguous()
    Qn = q.shape[0]
    top_n = args.top_n or 32
    top_ls = [int(x) for x in args.top_l_values.split(",") if x] or [args.top_l or 64]
    gt = s.gt_ids.cpu().numpy()
    if not args.no_neighbor_codes and args.topology == "hbm" and base_ix.num_nodes * base_ix.degree * base_ix.num_chunks <= 40e9:
        search.inline_neighbor_codes(base_ix)
        print(f"neighbour-code layout: {base_ix.neighbor_codes.numel() / 1e9:.2f} GB")
    host_allocs = []

    def to_mapped_host(t):
        nbytes = t.numel() * t.element_size()
        hp, dp = C.c_void_p(), C.c_void_p()
        capi.check(lib.tann_host_alloc_mapped(nbytes, C.byref(hp), C.byref(dp)))
        host_allocs.append(hp)
        step = 1 << 28
        flat = t.contiguous().view(torch.uint8).view(-1)
        for b in range(0, nbytes, step):   # through bounded host staging copies
            part = flat[b:b + step].cpu().numpy()
            C.memmove(hp.value + b, part.ctypes.data, part.nbytes)
        return dp.value, nbytes

    adj_mapped = vec_mapped = None
    if args.topology == "pinned-host":
        adj_mapped, nbytes = to_mapped_host(base_ix.adjacency)
        print(f"topology: {nbytes / 1e9:.2f} GB in mapped pinned host memory")
    if args.vectors == "pinned-host":
        vec_mapped, nbytes = to_mapped_host(base_ix.vector_pages)
        print(f"vector pages: {nbytes / 1e9:.2f} GB in mapped pinned host memory")
        base_ix.vector_pages = None    # the HBM copy is not needed any more
        torch.cuda.empty_cache()
    model = search.rvq_model_from_synth(s) if cfg.rvq else None
    pq2 = None
    if s.pq2_tables is not None:
        t2 = s.pq2_tables.cuda().contiguous()
        pq2 = dict(t2=t2, c2=s.pq2_centroid.cuda().contiguous(), codes2=s.pq2_codes.cuda().contiguous(), t2_cm=t2.t().contiguous(),
                   eps=s.pq2_error_bounds.cuda().contiguous())
        pq2["cross"] = search.pq2_cross_terms(base_ix.pq_chunk_offsets, s.pq_tables.cuda().contiguous(), base_ix.pq_centroid,
                                              t2, pq2["c2"])

    def time_case(ix, top_l, label):
        out = {"config": args.config, "nodes": int(ix.num_nodes), "queries": Qn, "top_l": top_l, "top_n": top_n,
               "residency": label, "index_build_s": round(build_s, 1), "stages_ms": {}}
        if model is not None:
            (offs, ids, _), ms = _time_calls(lambda: model.device_entry_batch(q, args.entries), args.reps)
            out["stages_ms"]["rvq_entries"] = ms
            print(f"rvq_entries {ms:.3f} ms")
        else:
            offs = torch.arange(Qn + 1, dtype=torch.int32, device="cuda")
            ids = torch.full((Qn,), int(s.medoid), dtype=torch.int32, device="cuda")
        p = search.TopologySearchParams(top_l=top_l, search_width=args.search_width, max_expansions=4096)
        cap = p.capacity(top_n)
        lut = None
        if args.staged_table:
            lut, ms = _time_calls(lambda: search.lut_build(ix, q), args.reps)
            out["stages_ms"]["lut_build"] = ms
            print(f"lut_build {ms:.3f} ms")
        (cand, stats), ms = _time_calls(lambda: search.beam_search(ix, p, offs, ids, queries=None if lut is not None else q,
                                                                   lut=lut, capacity=cap), args.reps)
        st = stats.cpu().numpy()
        e, v = float(st[:, 1].mean()), float(st[:, 0].mean())
        gbytes = Qn * (e * 4 * ix.degree + v * ix.num_chunks) / 1e9
        smem, bps, _ = search.beam_occupancy(ix, p, cap)
        out["stages_ms"]["beam_search"] = ms
        out["beam"] = dict(expanded=e, visited=v, algorithmic_gb=gbytes, gbs=gbytes / ms * 1e3, smem_bytes=smem, blocks_per_sm=bps)
        print(f"beam_search {ms:.3f} ms  nodes={ix.num_nodes} queries={Qn} L={top_l} C={cap} expanded/query={e:.1f} "
              f"visited/query={v:.1f} algorithmic={gbytes:.3f} GB -> {gbytes / ms * 1e3:.1f} GB/s  ({bps} blocks/SM, {smem} B smem)")
        rp = search.RerankExactParams(top_k=10, top_n=top_n)
        (_, rr_ids, _, _), ms = _time_calls(lambda: search.rerank_exact(ix, rp, cand, q), args.reps)
        gb = Qn * top_n * ix.vector_bytes / 1e9
        out["stages_ms"]["rerank_exact_f32_queries"] = ms
        out["recall_at_10"] = round(synth.recall_at_k(rr_ids.cpu().numpy().view(np.uint32), gt, 10), 4)
        print(f"rerank_exact {ms:.3f} ms  top_n={top_n}  (float32 queries) {gb / ms * 1e3:.1f} GB/s  recall@10={out['recall_at_10']}")
        if s.vectors.dtype == torch.uint8:
            q8 = q.to(torch.uint8).contiguous()   # the searcher makes this copy on the device when the values allow it
            _, ms = _time_calls(lambda: search.rerank_exact(ix, rp, cand, q8), args.reps)
            out["stages_ms"]["rerank_exact_u8_queries"] = ms
            print(f"rerank_exact {ms:.3f} ms  top_n={top_n}  (uint8 queries, integer path) {gb / ms * 1e3:.1f} GB/s")
        if model is not None and pq2 is None:
            sr = search.Searcher(ix, Qn, cap, top_n, args.entries)
            sr.set_rvq(model, args.entries)
            _, ms = _time_calls(lambda: sr.run_device(q, p, rp), args.reps)
            out["stages_ms"]["searcher_whole_path"] = ms
            out["qps_whole_path"] = Qn / ms * 1e3
            print(f"searcher whole path (rvq, beam, rerank, top-k) {ms:.3f} ms = {Qn / ms * 1e3:.0f} queries/s")
            sr.close()
        if pq2 is not None:
            # residual pq2 refine + bound filter (float configurations): second table build, refine, tiled rerank
            lr = min(top_l, cap)
            rp2 = search.RerankExactParams(top_k=10, top_n=min(top_n, lr), rank_tile_size=16, use_pq2_bound_filter=True)
            if Qn * ix.num_chunks * 1024 <= 2e9:
                lut2, ms = _time_calls(lambda: search.lut_build(ix, q, tables_col_major=pq2["t2_cm"], centroid=pq2["c2"]), args.reps)
                out["stages_ms"]["lut_build_pq2"] = ms
                print(f"lut_build (pq2) {ms:.3f} ms  {lut2.numel() * 4 / 1e6:.0f} MB written")
                refined, ms = _time_calls(lambda: search.pq2_refine(cand, stats, lr, pq2["codes2"], lut2, base_codes=ix.codes,
                                                                    cross_terms=pq2["cross"]), args.reps)
                out["stages_ms"]["pq2_refine"] = ms
                print(f"pq2_refine {ms:.3f} ms  refine_top_l={lr}")
                (_, _, n_exact, n_flt), ms = _time_calls(lambda: search.rerank_exact(ix, rp2, refined, q, pq2["eps"]), args.reps)
                out["stages_ms"]["rerank_exact_tiled_bound_filter"] = ms
                print(f"rerank_exact (tiled, bound filter) {ms:.3f} ms  exact={n_exact} filtered={n_flt}")
                # persistent rerank with a learned stop: a synthetic model on the share of ranks scored and the top-k
                # churn (logit = 1 - 2.5 * prefix / budget + entered / k, threshold 0)
                ls = capi.RerankLearnedStop()
                budget = rp2.top_n
                stages = [pfx for pfx in (16, 32, 48, 64, 96, 128, 192, 256, 384, 512) if pfx < budget]
                ls.enabled, ls.num_stages, ls.top_k, ls.bootstrap_prefix = 1, len(stages), 10, 16
                for i, pfx in enumerate(stages):
                    ls.stage_prefixes[i] = pfx
                while ls.initial_stage_index < ls.num_stages and ls.stage_prefixes[ls.initial_stage_index] <= 16:
                    ls.initial_stage_index += 1
                ls.linear_weights[1], ls.linear_weights[6], ls.bias, ls.threshold_logit = -2.5, 1.0, 1.0, 0.0
                ls.inv_budget_top_n, ls.inv_top_k = 1.0 / budget, 0.1
                if ls.initial_stage_index < ls.num_stages:
                    res, ms = _time_calls(lambda: search.rerank_exact_learned_stop(ix, rp2, refined, q, model=ls,
                                                                                   error_bounds=pq2["eps"]), args.reps)
                    out["stages_ms"]["rerank_exact_learned_stop"] = ms
                    print(f"rerank_exact_learned_stop {ms:.3f} ms  exact={res['n_exact']} filtered={res['n_filtered']} "
                          f"mean_stop_prefix={float(res['stop_prefixes'].float().mean()):.1f} of {budget}")
            if model is not None:
                sr = search.Searcher(ix, Qn, cap, min(top_n, lr), args.entries)
                sr.set_rvq(model, args.entries)
                sr.set_pq2(search.Pq2Resources(codes=pq2["codes2"], tables_col_major=pq2["t2_cm"], centroid=pq2["c2"],
                                               chunk_offsets=ix.pq_chunk_offsets, cross_terms=pq2["cross"],
                                               error_bounds=pq2["eps"]), lr)
                (oi, _, _), ms = _time_calls(lambda: sr.run_device(q, p, rp2), args.reps)
                out["stages_ms"]["searcher_whole_path"] = ms
                out["qps_whole_path"] = Qn / ms * 1e3
                ids_k = _device_view(oi, Qn * 10, torch.int32).view(Qn, 10).cpu().numpy().view(np.uint32)
                out["recall_at_10_whole_path"] = round(synth.recall_at_k(ids_k, gt, 10), 4)
                print(f"searcher whole path (rvq, beam, table-free pq2 refine, bound-filtered rerank, top-k) {ms:.3f} ms "
                      f"= {Qn / ms * 1e3:.0f} queries/s  recall@10={out['recall_at_10_whole_path']}")
                sr.close()
        return out

    all_out = []
    fractions = [float(x) for x in args.cached_fractions.split(",") if x] or [args.cached_fraction]
    for frac in (fractions if adj_mapped is not None else [None]):
        ix, label = base_ix, "adjacency + codes + vector pages in HBM"
        if adj_mapped is not None or vec_mapped is not None:
            kw = dict(num_nodes=base_ix.num_nodes, degree=base_ix.degree, dim=base_ix.dim, vector_kind=base_ix.vector_kind,
                      codes=base_ix.codes, pq_tables_col_major=base_ix.pq_tables_col_major, pq_centroid=base_ix.pq_centroid,
                      pq_chunk_offsets=base_ix.pq_chunk_offsets, vector_bytes=base_ix.vector_bytes,
                      vectors_per_page=base_ix.vectors_per_page)
            label = ""
            if adj_mapped is not None:
                cached = int(base_ix.num_nodes * frac)
                kw.update(adjacency_bases=[adj_mapped], adjacency_cache=base_ix.adjacency[:cached] if cached else None,
                          adjacency_cached_rows=cached)
                label = f"adjacency in mapped pinned host memory, {cached} rows ({frac:.0%}) cached in HBM"
                print(f"topology: {cached} rows ({frac:.0%}) cached in HBM")
            else:
                kw.update(adjacency=base_ix.adjacency)
                label = "adjacency in HBM"
            if vec_mapped is not None:
                kw.update(vector_bases=[vec_mapped])
                label += "; vector pages in mapped pinned host memory"
            else:
                kw.update(vector_pages=base_ix.vector_pages)
                label += "; vector pages in HBM"
            ix = search.DeviceIndex(**kw)
        for top_l in top_ls:
            all_out.append(time_case(ix, top_l, label))
    torch.cuda.synchronize()
    for hp in host_allocs:
        capi.check(lib.tann_host_free(hp))
    for o in all_out:
        print(json.dumps(o))


def _device_view(ptr, count, dtype):
    """torch view of `count` elements of a device buffer owned by a searcher."""
    from topoanns_b200 import sharding
    return sharding._tensor_from_ptr(ptr, count * torch.empty((), dtype=dtype).element_size()).view(dtype)


def sharded_leg(args, rank, world, local, device):
    """The path over an index split by node-id range across the ranks (R = 32 records, RVQ entries, as the
    1 B-vector configuration prescribes, at --shard-nodes rows per GPU): every rank searches its own 10 k-query
    batch, its kernels read (N-1)/N of all rows from the peers over NVLink with ordinary loads, and rank 0
    collects the [Q, k] lists of every rank with one NCCL gather that sits inside the end-to-end region."""
    import torch.distributed as dist
    from topoanns_b200 import capi, search, sharding, synth, synth_sharded
    lib = capi.load()
    Q = args.queries
    t0 = time.time()
    # Mixture components of 1000 nodes whatever the size of the index: larger components of this isotropic mixture
    # cannot be ranked by 32-byte PQ codes (4000-node components gave recall@10 0.58 with 2048 candidates reranked).
    # The entry model follows the index: its posting lists stop at 256 ids and 128 of them are the entries, so a
    # bucket of many more nodes hands out a thin sample of the query's region (256 x 256 on 82 M nodes, 1250 nodes
    # per bucket: recall@10 levelled off at 0.946).
    total = args.shard_nodes * world
    side = 256 if args.shard_rvq_side == 0 else args.shard_rvq_side
    while args.shard_rvq_side == 0 and side * side * 640 < total and side < 4096:
        side *= 2
    cfg = dataclasses.replace(synth.CONFIGS["cfg4"], num_nodes=total, num_queries=Q * world,
                              components=max(world, total // 1000), kmeans_iters=5, train_sample=max(65536, 64 * side),
                              rvq_coarse=side, rvq_fine=side)
    s = synth_sharded.build(cfg, device, gt_stride=max(1, args.shard_gt_stride))   # this rank's shard + all queries + ground truth
    torch.cuda.synchronize()
    build_s = time.time() - t0
    b, e = sharding.query_shard(s.queries.shape[0], world, rank)
    gt_all = s.gt_ids.cpu().numpy()[b:e]
    has_gt = gt_all[:, 0] >= 0            # with a ground-truth stride only these rows count for recall
    gt = gt_all[has_gt]
    my_queries = s.queries[b:e].contiguous()
    degree, M = s.adjacency.shape[1], s.pq_codes.shape[1]
    ix, peer_buffers = sharding.peer_index_from_sharded(s)
    whole_bytes = s.total_nodes * (degree * 4 + M + ix.vector_bytes)
    if whole_bytes > 60e9:     # no unsharded self-check at this size: the generator's copies of the shard can go
        s.vectors, s.adjacency = s.vectors[:0], s.adjacency[:0]
        torch.cuda.empty_cache()
    model = search.RvqModel(dim=s.cfg.dim, coarse=s.rvq_coarse.contiguous(), fine=s.rvq_fine.contiguous(),
                            bucket_sizes=s.rvq_buckets[0], cluster_offsets=s.rvq_buckets[1], cluster_ids=s.rvq_buckets[2])
    max_top_n = max(tn for _, tn in SHARDED_POINTS)
    sr = search.Searcher(ix, Q, max_top_n, max_top_n, 128)
    sr.set_rvq(model, 128)
    q_pinned = my_queries.cpu().pin_memory()
    # operating point: the fastest candidate whose recall@10 over ALL ranks' queries reaches the target
    sweep = []
    for L, tn in SHARDED_POINTS:
        tp = search.TopologySearchParams(top_l=L, search_width=2, max_expansions=4096)
        rp = search.RerankExactParams(top_k=10, top_n=tn)
        sr.run_host(q_pinned.numpy(), tp, rp)
        dist.barrier()
        t1 = time.perf_counter()
        ids, _, _ = sr.run_host(q_pinned.numpy(), tp, rp)
        dt = time.perf_counter() - t1
        n_gt = int(has_gt.sum())
        agg = torch.tensor([synth.recall_at_k(ids[has_gt], gt, 10) * n_gt, float(n_gt), 0.0], dtype=torch.float64, device=device)
        dist.all_reduce(agg)
        worst = torch.tensor([dt], dtype=torch.float64, device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        sweep.append(dict(top_l=L, rerank_top_n=tn, recall_at_10=round(float(agg[0] / agg[1]), 4),
                          qps_e2e=round(Q * world / float(worst), 1)))
    ok = [p for p in sweep if p["recall_at_10"] >= RECALL_TARGET]
    if not ok:   # recall has levelled off below the target: the fastest point within 0.005 of the best one
        top = max(p["recall_at_10"] for p in sweep)
        ok = [p for p in sweep if p["recall_at_10"] >= top - 0.005]
    chosen = max(ok, key=lambda p: p["qps_e2e"])
    L, top_n = chosen["top_l"], chosen["rerank_top_n"]
    tp = search.TopologySearchParams(top_l=L, search_width=2, max_expansions=4096)
    rp = search.RerankExactParams(top_k=10, top_n=top_n)
    # distinct query batches of this rank's slice
    nb = max(1, min(args.steps + args.warmup, 16))
    batches = [my_queries] + [synth.more_queries(s.cfg, s.centres, Q, 7000 + 131 * rank + i) for i in range(1, nb)]
    q_devs = [t.to(device).contiguous() for t in batches]
    q_pins = [t.cpu().pin_memory() for t in batches]
    stream = torch.cuda.current_stream()

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident -----------------------------------------------------------------------
    for i in range(args.warmup):
        sr.run_device(q_devs[i % nb], tp, rp)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for i in range(args.steps):
        sr.run_device(q_devs[i % nb], tp, rp)
    ev1.record(stream)
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    # ---- end to end: H2D of the queries, the five kernels, ONE NCCL gather of the [Q, k] lists to rank 0,
    # D2H of the gathered lists there --------------------------------------------------------------
    q_in = torch.empty_like(q_devs[0])
    packed = torch.empty((Q, 20), dtype=torch.int32, device=device)
    gathered = [torch.empty_like(packed) for _ in range(world)] if rank == 0 else None
    out_pinned = torch.empty((world, Q, 20), dtype=torch.int32).pin_memory() if rank == 0 else None

    def e2e_step(i):
        q_in.copy_(q_pins[i % nb], non_blocking=True)
        oi, od, _ = sr.run_device(q_in, tp, rp)
        packed[:, :10] = _device_view(oi, Q * 10, torch.int32).view(Q, 10)
        packed[:, 10:] = _device_view(od, Q * 10, torch.int32).view(Q, 10)
        dist.gather(packed, gathered, dst=0)
        if rank == 0:
            for r in range(world):
                out_pinned[r].copy_(gathered[r], non_blocking=True)
        torch.cuda.current_stream().synchronize()     # the caller holds the results of this batch

    for i in range(args.warmup):
        e2e_step(i)
    barrier()
    t1 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t1
    barrier()
    # ---- the beam kernel alone: local and remote algorithmic bytes ----------------------------------
    offs, eids, _ = model.device_entry_batch(q_devs[0], 128)
    cap = tp.capacity(top_n)
    view = ix.view()
    bp = tp.to_c(cap)
    cand = torch.empty((Q, cap, 2), dtype=torch.int32, device=device)
    stats_d = torch.empty((Q, 8), dtype=torch.int32, device=device)

    def beam_once():
        capi.check(lib.tann_beam_search(C.byref(view), C.byref(bp), None, C.c_void_p(q_devs[0].data_ptr()),
                                        capi.KIND_FLOAT32, Q, C.c_void_p(offs.data_ptr()), C.c_void_p(eids.data_ptr()),
                                        C.c_void_p(cand.data_ptr()), C.c_void_p(stats_d.data_ptr()), None,
                                        C.c_void_p(stream.cuda_stream)))
    for _ in range(max(3, args.warmup)):
        beam_once()
    barrier()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record(stream)
    for _ in range(args.steps):
        beam_once()
    k1.record(stream)
    barrier()
    beam_ms = k0.elapsed_time(k1) / args.steps
    stats = stats_d.cpu().numpy().view(np.uint32)
    beam_bytes, rerank_bytes = algorithmic_bytes(stats, degree, M, top_n, ix.vector_bytes)
    smem, blocks_per_sm, _ = search.beam_occupancy(ix, tp, cap)
    # ---- self-check: a sample of queries against the same index searched unsharded on one GPU ---------
    ids_sh, d_sh, _ = sr.run_host(q_pinned.numpy(), tp, rp)
    all_ids, all_d = sharding.gather_topk(torch.from_numpy(ids_sh.view(np.int32)).to(device),
                                          torch.from_numpy(d_sh).to(device), Q * world)
    ids_identical, checked = None, 0
    if whole_bytes <= 60e9:
        whole = synth_sharded.gather_whole(s)
        if rank == 0:
            full_ix = search.device_index_from_synth(whole, device)
            full_model = search.rvq_model_from_synth(whole, device)
            checked = min(Q * world, 4000)
            pick = np.linspace(0, Q * world - 1, checked).astype(np.int64)     # queries of every rank
            sr2 = search.Searcher(full_ix, checked, cap, top_n, 128)
            sr2.set_rvq(full_model, 128)
            ids2, d2, _ = sr2.run_host(np.ascontiguousarray(s.queries.cpu().numpy()[pick]), tp, rp)
            got_i = all_ids.cpu().numpy().view(np.uint32)[pick]
            got_d = all_d.cpu().numpy().view(np.uint32)[pick]
            ids_identical = bool(np.array_equal(got_i, ids2) and np.array_equal(got_d, d2.view(np.uint32)))
            sr2.close()
            del full_ix, full_model
        del whole
    torch.cuda.empty_cache()
    # ---- the same shards with the PQ codes replicated on every GPU (M bytes per node: 32 GB at one billion nodes,
    # which 180 GB of HBM affords next to a 52 GB shard): code rows - most of the gather bytes - become local reads,
    # adjacency rows and vector pages stay sharded ------------------------------------------------------------
    rep_ms = rep_beam_ms = 0.0
    rep_same = True
    own_ms = own_e2e_ms = 0.0
    own_same, own_slot, own_over = True, 0, False
    if s.total_nodes * M <= 40e9:
        parts = [torch.empty_like(s.pq_codes) for _ in range(world)]
        dist.all_gather(parts, s.pq_codes.contiguous())
        all_codes = torch.cat(parts)
        del parts
        ix_r = dataclasses.replace(ix, codes=all_codes, codes_bases=None)
        sr_r = search.Searcher(ix_r, Q, max_top_n, max_top_n, 128)
        sr_r.set_rvq(model, 128)
        ids_r, d_r, _ = sr_r.run_host(q_pinned.numpy(), tp, rp)
        rep_same = bool(np.array_equal(ids_r, ids_sh) and np.array_equal(d_r.view(np.uint32), d_sh.view(np.uint32)))
        for i in range(args.warmup):
            sr_r.run_device(q_devs[i % nb], tp, rp)
        barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record(stream)
        for i in range(args.steps):
            sr_r.run_device(q_devs[i % nb], tp, rp)
        r1.record(stream)
        barrier()
        rep_ms = r0.elapsed_time(r1)
        view_r = ix_r.view()

        def beam_r():
            capi.check(lib.tann_beam_search(C.byref(view_r), C.byref(bp), None, C.c_void_p(q_devs[0].data_ptr()),
                                            capi.KIND_FLOAT32, Q, C.c_void_p(offs.data_ptr()), C.c_void_p(eids.data_ptr()),
                                            C.c_void_p(cand.data_ptr()), C.c_void_p(stats_d.data_ptr()), None,
                                            C.c_void_p(stream.cuda_stream)))
        for _ in range(3):
            beam_r()
        barrier()
        r0.record(stream)
        for _ in range(args.steps):
            beam_r()
        r1.record(stream)
        barrier()
        rep_beam_ms = r0.elapsed_time(r1) / args.steps
        sr_r.close()
        # ---- the same, and the exact rerank done by the owner of the rows: the candidate lists are split by owner
        # and exchanged (all-to-all), every GPU scores what it received against its own shard, the [Q, 10] lists
        # travel back and are merged - no vector row crosses NVLink ------------------------------------------------
        local_ix = dataclasses.replace(ix, num_nodes=s.rows_per_shard, codes=None, rows_per_shard=0,
                                       adjacency_bases=[ix.adjacency_bases[rank]], codes_bases=[ix.codes_bases[rank]],
                                       vector_bases=[ix.vector_bases[rank]])
        orr = sharding.OwnerRerank(local_ix, s.rows_per_shard, Q, top_n, 10, q_devs[0].dtype)
        own_slot = orr.slot
        cap_o = tp.capacity(top_n)

        def owner_step(qd):
            eo, ei, _ = model.device_entry_batch(qd, 128)
            cand_o, _ = search.beam_search(ix_r, tp, eo, ei, queries=qd, capacity=cap_o)
            return orr.run(cand_o, qd)

        oi, od = owner_step(q_devs[0])
        torch.cuda.synchronize()
        own_same = bool(np.array_equal(oi.cpu().numpy().view(np.uint32), ids_sh.view(np.uint32)) and
                        np.array_equal(od.cpu().numpy().view(np.uint32), d_sh.view(np.uint32)))
        for i in range(args.warmup):
            owner_step(q_devs[i % nb])
        barrier()
        r0.record(stream)
        for i in range(args.steps):
            owner_step(q_devs[i % nb])
        r1.record(stream)
        barrier()
        own_ms = r0.elapsed_time(r1)

        def owner_e2e_step(i):
            q_in.copy_(q_pins[i % nb], non_blocking=True)
            oi, od = owner_step(q_in)
            packed[:, :10] = oi
            packed[:, 10:] = od.view(torch.int32)
            dist.gather(packed, gathered, dst=0)
            if rank == 0:
                for r in range(world):
                    out_pinned[r].copy_(gathered[r], non_blocking=True)
            torch.cuda.current_stream().synchronize()

        for i in range(args.warmup):
            owner_e2e_step(i)
        barrier()
        t1 = time.perf_counter()
        for i in range(args.steps):
            owner_e2e_step(i)
        torch.cuda.synchronize()
        own_e2e_ms = (time.perf_counter() - t1) * 1000.0
        barrier()
        own_over = orr.overflowed()
        del orr, local_ix
        del all_codes, ix_r
        torch.cuda.empty_cache()
    times = torch.tensor([dev_ms, e2e_s * 1000.0, beam_ms, rep_ms, rep_beam_ms, 0.0 if rep_same else 1.0, own_ms, own_e2e_ms,
                          0.0 if own_same else 1.0, 1.0 if own_over else 0.0], dtype=torch.float64, device=device)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, beam_ms, rep_ms, rep_beam_ms, rep_bad, own_ms, own_e2e_ms, own_bad, own_overflow = \
        [float(x) for x in times.cpu()]
    sums = torch.tensor([beam_bytes, rerank_bytes], dtype=torch.float64, device=device)
    dist.all_reduce(sums)
    rec_t = torch.tensor([synth.recall_at_k(ids_sh[has_gt], gt, 10) * int(has_gt.sum()), float(has_gt.sum())],
                         dtype=torch.float64, device=device)
    dist.all_reduce(rec_t)
    sr.close()
    dist.barrier()
    for pb in peer_buffers.values():
        pb.close()
    if rank != 0:
        return None
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm_peak = float(json.load(open(peaks_path))["hbm_gbs"]) if os.path.exists(peaks_path) else 6650.0
    remote_frac = 1.0 - 1.0 / world
    per_gpu_beam_bytes = float(sums[0]) / world
    remote_gbs = per_gpu_beam_bytes * remote_frac / (beam_ms * 1e-3) / 1e9
    local_gbs = per_gpu_beam_bytes * (1.0 - remote_frac) / (beam_ms * 1e-3) / 1e9
    total_q = Q * world * args.steps
    return {
        "workload": (f"cfg4-style shards: {s.total_nodes} x {cfg.dim} uint8 over {world} GPUs ({s.rows_per_shard} per GPU), "
                     f"R={degree}, PQ M={M}x256, RVQ {side}x{side} entries=128, {cfg.components} mixture components, {Q} queries/batch per GPU, k=10, W=2; node ids scattered "
                     f"so that {world - 1}/{world} of the row gathers are NVLink peer loads"),
        "top_l": L, "rerank_top_n": top_n, "recall_at_10": round(float(rec_t[0] / rec_t[1]), 4),
        "recall_target_met": bool(float(rec_t[0] / rec_t[1]) >= RECALL_TARGET), "recall_queries": int(rec_t[1]), "sweep": sweep,
        "value": total_q / (dev_ms * 1e-3), "unit": "queries/s", "ms_per_step": dev_ms / args.steps,
        "e2e": {"value": total_q / (e2e_ms * 1e-3), "unit": "queries/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": int(Q * cfg.dim * 4), "d2h_bytes_per_step": int(world * Q * 10 * 8),
                "collective": f"one NCCL gather of the [Q, 10] id + distance lists ({Q * 80} B per rank) to rank 0 per step, inside the timed region"},
        "beam_kernel": {"ms": round(beam_ms, 4), "smem_bytes": smem, "blocks_per_sm": blocks_per_sm,
                        "bytes_per_query": per_gpu_beam_bytes / Q, "remote_fraction": remote_frac,
                        "remote_gbs_per_gpu": remote_gbs, "nvlink_frac": remote_gbs / NVLINK_INGRESS_GBS,
                        "nvlink_peak_gbs": NVLINK_INGRESS_GBS, "local_gbs_per_gpu": local_gbs,
                        "local_hbm_frac": local_gbs / hbm_peak},
        "codes_replicated": (None if rep_ms == 0.0 else {
            "what": f"the same shards with the PQ codes ({M} B per node) replicated on every GPU: code rows are read from local "
                    "HBM, adjacency rows and vector pages stay sharded",
            "value": total_q / (rep_ms * 1e-3), "unit": "queries/s", "ms_per_step": rep_ms / args.steps,
            "beam_kernel_ms": round(rep_beam_ms, 4), "results_identical_to_sharded_codes": rep_bad == 0.0}),
        "codes_replicated_rerank_by_owner": (None if own_ms == 0.0 else {
            "what": "PQ codes replicated as above, and the exact rerank done by the owner of the rows: candidate lists split "
                    "by owner and exchanged (NCCL all-to-all), scored against the local shard, [Q, 10] lists returned "
                    "(all-to-all) and merged; no vector row crosses NVLink",
            "value": total_q / (own_ms * 1e-3), "unit": "queries/s", "ms_per_step": own_ms / args.steps,
            "e2e": {"value": total_q / (own_e2e_ms * 1e-3), "unit": "queries/s", "ms_per_step": own_e2e_ms / args.steps},
            "slot_per_query_and_owner": own_slot, "slot_overflowed": own_overflow != 0.0,
            "results_identical_to_peer_reads": own_bad == 0.0}),
        "ids_identical": ids_identical, "ids_checked_queries": checked,
        "ids_check": "sample of every rank's queries against the whole index searched unsharded on rank 0"
                     if ids_identical is not None else "skipped: the whole index does not fit one GPU beside the shards",
        "index_build_s": round(build_s, 1), "distinct_batches": nb,
    }


def main():
    args = parse_args()
    rank, world, local = dist_env()
    if args.impl == "reference" and rank != 0:
        return 0
    use_cuda = torch.cuda.is_available()
    if args.impl == "b200" and not use_cuda:
        raise SystemExit("bench.py: the CUDA path needs a GPU (there is no CPU fallback); use --impl reference "
                         "for the host-core baseline.")
    if use_cuda:
        torch.cuda.set_device(local)
    if args.stages:
        stage_timings(args)
        return 0
    if world > 1 and args.impl == "b200":
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    device = f"cuda:{local}" if use_cuda else "cpu"

    from topoanns_b200 import synth
    if args.sharded_only and world > 1 and args.impl == "b200":
        rec = sharded_leg(args, rank, world, local, device)
        if rank == 0:
            print(json.dumps({"metric": "QPS at recall@10>=0.95 (uint8 d=128 index sharded by node-id range, 1 batch of 10k queries per GPU)",
                              "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "sharded": rec}))
        import torch.distributed as dist
        dist.destroy_process_group()
        return 0
    s, build_s = build_index(args, device)
    gt = s.gt_ids.cpu().numpy()
    degree, M = s.adjacency.shape[1], s.pq_codes.shape[1]
    workload = (f"{args.config}: {s.vectors.shape[0]} x {s.cfg.dim} {s.cfg.kind}, R={degree}, PQ M={M}x256, RVQ 256x256 entries=128, "
                f"{s.queries.shape[0]} queries/batch, k=10, W=2, max_expansions=4096")
    Q = s.queries.shape[0]

    if args.impl == "reference":
        reference_arm(args, s, workload)
        return 0

    from topoanns_b200 import capi, search
    lib = capi.load()
    ix = search.device_index_from_synth(s, device)
    model = search.rvq_model_from_synth(s, device)
    if not args.no_neighbor_codes:
        # HBM is plentiful for this configuration: also keep every node's neighbours' PQ codes next to each
        # other (degree * M bytes per node), so that an expansion needs one memory round trip, not two
        search.inline_neighbor_codes(ix)
    max_cap = 1024
    sr = search.Searcher(ix, Q, max_cap, max(TOPN_SWEEP), 128)
    sr.set_rvq(model, 128)
    # distinct seeded query batches: batch 0 is the one with ground truth, the others come from the same mixture
    nb = max(1, min(args.steps + args.warmup, MAX_DISTINCT_BATCHES))
    batches = [s.queries] + [synth.more_queries(s.cfg, s.extras["centres"], Q, 9000 + 977 * rank + i, s.extras["basis"])
                             for i in range(1, nb)]
    q_devs = [t.to(device).contiguous() for t in batches]
    q_pins = [t.cpu().pin_memory() for t in batches]
    q_nps = [t.numpy() for t in q_pins]
    q_host_bytes = int(q_nps[0].nbytes)

    def run_point(L, top_n):
        tp = search.TopologySearchParams(top_l=L, search_width=2, max_expansions=4096)
        rp = search.RerankExactParams(top_k=10, top_n=top_n)
        t0 = time.perf_counter()
        ids, dists, stats = sr.run_host(q_nps[0], tp, rp, want_stats=True)
        dt = time.perf_counter() - t0
        return ids, stats, dt, tp, rp

    # ---- operating point ---------------------------------------------------------------------
    sweep = []
    if args.top_l:
        points = [(args.top_l, args.top_n or 32)]
    else:
        points = [(L, 32) for L in L_SWEEP] + [(L, tn) for tn in TOPN_SWEEP[1:] for L in (16, 32, 64)]
    for L, tn in points:
        run_point(L, tn)  # warm
        ids, stats, dt, _, _ = run_point(L, tn)
        for _ in range(2):   # best of three: the choice between close points should not hinge on one timing
            dt = min(dt, run_point(L, tn)[2])
        rec = synth.recall_at_k(ids, gt, 10)
        sweep.append(dict(top_l=L, rerank_top_n=tn, recall_at_10=round(rec, 4), qps_e2e=round(Q / dt, 1),
                          mean_expanded=float(stats[:, 1].mean()), mean_visited=float(stats[:, 0].mean())))
    ok = [p for p in sweep if p["recall_at_10"] >= RECALL_TARGET]
    chosen = max(ok, key=lambda p: p["qps_e2e"]) if ok else max(sweep, key=lambda p: (p["recall_at_10"], p["qps_e2e"]))
    L, top_n = chosen["top_l"], chosen["rerank_top_n"]
    if world > 1:  # every rank runs rank 0's operating point
        import torch.distributed as dist
        pt = torch.tensor([L, top_n], dtype=torch.int64, device=device)
        dist.broadcast(pt, 0)
        L, top_n = int(pt[0]), int(pt[1])
    tp = search.TopologySearchParams(top_l=L, search_width=2, max_expansions=4096)
    rp = search.RerankExactParams(top_k=10, top_n=top_n)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream()
    # ---- device-resident leg: `value` ----------------------------------------------------------
    for i in range(args.warmup):
        sr.run_device(q_devs[i % nb], tp, rp)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for i in range(args.steps):
        sr.run_device(q_devs[i % nb], tp, rp)
    ev1.record(stream)
    barrier()
    dev_one_stream_ms = ev0.elapsed_time(ev1)
    # The same K steps through several searchers on their own streams, submitted in turn: the short kernels of one
    # batch (entry selection, rerank, top-k) and the ragged last wave of its beam search run beside another batch's
    # beam search. Timed with events: every stream starts after ev0, ev1 follows the end of all of them.
    n_lanes = max(1, args.streams)
    searchers, streams = [sr], [torch.cuda.Stream(device)]
    for _ in range(n_lanes - 1):
        extra = search.Searcher(ix, Q, max_cap, max(TOPN_SWEEP), 128)
        extra.set_rvq(model, 128)
        searchers.append(extra)
        streams.append(torch.cuda.Stream(device))

    def many_streams(steps):
        for i in range(steps):
            with torch.cuda.stream(streams[i % n_lanes]):
                searchers[i % n_lanes].run_device(q_devs[i % nb], tp, rp)

    many_streams(max(args.warmup, n_lanes))
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(streams[0])
    for st in streams[1:]:
        st.wait_event(ev0)
    many_streams(args.steps)
    for st in streams[1:]:
        done = torch.cuda.Event()
        done.record(st)
        streams[0].wait_event(done)
    ev1.record(streams[0])
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    # ---- host-buffer leg: `e2e` ----------------------------------------------------------------
    # caller-side buffers of a serving process: page-locked queries in, page-locked results out
    out_ids_pinned = torch.empty((Q, 10), dtype=torch.int32).pin_memory()
    out_dists_pinned = torch.empty((Q, 10), dtype=torch.float32).pin_memory()
    out_ids_np, out_dists_np = out_ids_pinned.numpy().view(np.uint32), out_dists_pinned.numpy()
    for i in range(args.warmup):
        sr.run_host(q_nps[i % nb], tp, rp, out_ids=out_ids_np, out_dists=out_dists_np)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        # every rank serves its own batch and reads its own results back: no data-path collective
        sr.run_host(q_nps[i % nb], tp, rp, out_ids=out_ids_np, out_dists=out_dists_np)
    torch.cuda.synchronize()
    e2e_serial_s = time.perf_counter() - t0
    barrier()
    # The same through the searchers on their streams, submitted in turn: batch i's copies overlap the kernels of
    # the batches before it. Every step still copies its queries in and its results out inside the timed region.
    lanes = [(sr, streams[0], out_ids_np, out_dists_np)]
    for k in range(1, n_lanes):
        lanes.append((searchers[k], streams[k],
                      torch.empty((Q, 10), dtype=torch.int32).pin_memory().numpy().view(np.uint32),
                      torch.empty((Q, 10), dtype=torch.float32).pin_memory().numpy()))
    last_batch = [0] * n_lanes

    def pipelined(steps):
        for i in range(steps):
            srx, st, oi, od = lanes[i % n_lanes]
            srx.wait()
            srx.submit_host(q_nps[i % nb], tp, rp, oi, od, stream=st)
            last_batch[i % n_lanes] = i % nb
        for srx, *_ in lanes:
            srx.wait()

    torch.cuda.synchronize()
    pipelined(args.warmup)
    barrier()
    t0 = time.perf_counter()
    pipelined(args.steps)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop() if rank == 0 else {}
    # what every lane returned last equals a blocking call on the same batch
    for k, (_, _, oi, od) in enumerate(lanes):
        if args.steps > k:
            ci, cd, _ = sr.run_host(q_nps[last_batch[k]], tp, rp)
            assert np.array_equal(oi, ci) and np.array_equal(od.view(np.uint32), cd.view(np.uint32)), \
                "pipelined and blocking calls disagree"
    for extra in searchers[1:]:
        extra.close()
    ids, dists, _ = sr.run_host(q_nps[0], tp, rp)      # batch 0: the one with ground truth
    ids, dists = ids.copy(), dists.copy()
    # ---- the beam-search kernel alone, for the roofline -----------------------------------------
    offs, eids, _ = model.device_entry_batch(q_devs[0], 128)
    cap = tp.capacity(top_n)
    view = ix.view()
    bp = tp.to_c(cap)
    cand = torch.empty((Q, cap, 2), dtype=torch.int32, device=device)
    stats_d = torch.empty((Q, 8), dtype=torch.int32, device=device)

    def beam_once():
        capi.check(lib.tann_beam_search(C.byref(view), C.byref(bp), None, C.c_void_p(q_devs[0].data_ptr()),
                                        capi.KIND_FLOAT32, Q, C.c_void_p(offs.data_ptr()), C.c_void_p(eids.data_ptr()),
                                        C.c_void_p(cand.data_ptr()), C.c_void_p(stats_d.data_ptr()), None,
                                        C.c_void_p(stream.cuda_stream)))
    for _ in range(max(3, args.warmup)):
        beam_once()
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record(stream)
    for _ in range(args.steps):
        beam_once()
    k1.record(stream)
    torch.cuda.synchronize()
    beam_ms = k0.elapsed_time(k1) / args.steps
    stats = stats_d.cpu().numpy().view(np.uint32)
    beam_bytes, rerank_bytes = algorithmic_bytes(stats, degree, M, top_n, ix.vector_bytes)
    smem, blocks_per_sm, grid = search.beam_occupancy(ix, tp, cap)
    # one dependent random load of the adjacency array after another: the round trip a push cannot go below
    round_trip_ns = None
    if hasattr(lib, "tann_dependent_load_ns"):
        ns = C.c_float(0.0)
        capi.check(lib.tann_dependent_load_ns(C.c_void_p(ix.adjacency.data_ptr()), ix.adjacency.numel() * 4, 2000,
                                              C.byref(ns), C.c_void_p(stream.cuda_stream)))
        round_trip_ns = float(ns.value)

    # ---- max over ranks --------------------------------------------------------------------------
    times = torch.tensor([dev_ms, e2e_s * 1000.0, beam_ms, e2e_serial_s * 1000.0, dev_one_stream_ms], dtype=torch.float64,
                         device=device)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, beam_ms, e2e_serial_ms, dev_one_stream_ms = [float(x) for x in times.cpu()]
    sr.close()
    sharded = None
    if world > 1 and not args.no_sharded_leg:
        del sr, searchers, ix, model, q_devs, cand
        torch.cuda.empty_cache()
        try:
            sharded = sharded_leg(args, rank, world, local, device)
        except Exception as e:   # the replica numbers must survive a failure of this leg
            sharded = {"error": f"{type(e).__name__}: {e}"} if rank == 0 else None
    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return 0

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    achieved = beam_bytes / (beam_ms * 1e-3) / 1e9
    have_nc = not args.no_neighbor_codes
    table = NCU_BEAM_TRAFFIC_BYTES_NEIGHBOR_CODES if have_nc else NCU_BEAM_TRAFFIC_BYTES_PLAIN
    traffic = table.get((L, cap)) if (s.vectors.shape[0], Q, args.config) == (10_000_000, 10_000, "cfg2") else None
    rec = synth.recall_at_k(ids, gt, 10)
    total_q = Q * world * args.steps
    pushes = float(stats[:, 3].mean()) + (128 + 2 * degree - 1) // (2 * degree)      # iterations + entry batches
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "frac_of_nominal_8tbs": achieved / 8000.0, "traffic": traffic, "peak_source": peak_src,
                "kernel": "beam_search_kernel",
                "whole_step_gbs": (beam_bytes + rerank_bytes) * args.steps / (dev_ms * 1e-3) / 1e9}
    if round_trip_ns:
        # what the resident queries could move if a push cost exactly one dependent DRAM round trip
        resident = grid
        bytes_per_push = beam_bytes / Q / max(pushes, 1.0)
        roofline["dependent_load_round_trip_ns"] = round_trip_ns
        roofline["latency_ceiling_gbs"] = resident * bytes_per_push / round_trip_ns
        roofline["latency_ceiling_note"] = (f"{resident} resident queries x {bytes_per_push:.0f} B per push / one dependent "
                                            f"random load ({round_trip_ns:.0f} ns); a query's pushes are sequential")
    line = {
        "metric": METRIC,
        "value": total_q / (dev_ms * 1e-3), "unit": "queries/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": workload, "top_l": L, "rerank_top_n": top_n, "recall_at_10": round(rec, 4),
                   "recall_target_met": bool(rec >= RECALL_TARGET),
                   "parallelism": f"replica x{world}, queries sharded",
                   "query_batches": f"{nb} distinct seeded batches, one per step in turn (batch 0 carries the ground truth)",
                   "l2_policy": "index (4.2 GB) and per-step gathers exceed the 126 MB L2; no flush",
                   "streams": f"{n_lanes}: steps alternate between {n_lanes} searchers, each on its own stream; one stream alone: "
                              f"{total_q / (dev_one_stream_ms * 1e-3):.0f} queries/s, {dev_one_stream_ms / args.steps:.4f} ms per step",
                   "layout": ("adjacency + PQ codes + vector pages in HBM"
                              + (f" + neighbour codes next to each node ({s.vectors.shape[0] * degree * M / 1e9:.1f} GB)"
                                 if have_nc else "")),
                   "index_build_s": round(build_s, 1), "sweep": sweep,
                   "beam_kernel": {"smem_bytes": smem, "blocks_per_sm": blocks_per_sm, "resident_blocks": grid, "grid": "one block per query",
                                   "ms": round(beam_ms, 4), "mean_expanded": float(stats[:, 1].mean()),
                                   "mean_visited": float(stats[:, 0].mean()), "mean_pushes": pushes,
                                   "bytes_per_query": beam_bytes / Q}},
        "e2e": {"value": total_q / (e2e_ms * 1e-3), "unit": "queries/s",
                "h2d_bytes_per_step": q_host_bytes, "d2h_bytes_per_step": int(Q * 10 * 8),
                "pipeline": f"{n_lanes} searchers on {n_lanes} streams, batches submitted in turn (copies of one overlap kernels of the others)",
                "one_batch_at_a_time": total_q / (e2e_serial_ms * 1e-3)},
        "gpu_launches": 5 * args.steps,  # rvq, beam, float->uint8 check, rerank, top-k pack
        "clocks": clocks,
        "roofline": roofline,
    }
    if sharded is not None:
        line["sharded"] = sharded
    if not args.no_cpu_baseline:
        # rank 0 alone; under a launcher the pool is sized here, not by the launcher's OMP_NUM_THREADS
        try:
            line["cpu_baseline"], line["parity"] = cpu_leg(s, L, top_n, args.cpu_seconds, ids, dists)
        except Exception as e:  # the baseline must not take the GPU numbers down with it
            line["cpu_baseline"] = {"value": None, "error": str(e)}
    print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
