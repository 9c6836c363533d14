#!/usr/bin/env python
"""Benchmark of the batched graph-search path.

  python bench.py --gpus N --steps K --warmup W            # this library (CUDA)
  python bench.py --impl reference --gpus N --steps K ...   # the CPU implementation, host cores

One "step" is one pass of the whole path (RVQ entry selection -> table build + beam search ->
exact rerank -> top-k) over one batch of 10 000 synthetic queries on the 10 M-vector uint8 d=128
configuration (R = 64, M = 32, two-level RVQ entries). The operating point (top_l, rerank top_n) is
picked before the timed region by a sweep over the configuration's L values: the fastest point with
recall@10 >= 0.95, or the highest-recall point when none reaches it (stated in `config`).

Prints ONE JSON line: `value` = device-resident QPS over all ranks, `e2e` = QPS through the host
buffer entry point (H2D of the queries and D2H of ids/distances inside the timed region),
`roofline` for the beam-search kernel (algorithmic gather bytes / its own launch time, against the
measured HBM copy bandwidth), `cpu_baseline` = the CPU implementation timed on this box's cores.
"""
import argparse
import ctypes as C
import dataclasses
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

os.environ.setdefault("NCCL_DEBUG", "WARN")  # keeps NCCL's version banner off stdout: one JSON line only

import numpy as np  # noqa: E402
import torch  # noqa: E402

L_SWEEP = (16, 32, 64, 128, 256, 512, 1024)
TOPN_SWEEP = (32, 128, 192, 256, 512)
DEFAULT_POINT = (16, 192)   # (top_l, rerank_top_n): fastest sweep point with recall@10 >= 0.95 on the seeded cfg2 data
# DRAM traffic of one beam_search_kernel launch (10 k queries, 10 M nodes), ncu dram__bytes_read.sum +
# dram__bytes_write.sum, keyed by (top_l, candidate capacity) - the kernel does not depend on rerank_top_n
# beyond the capacity it implies; summarised under profiles/.
NCU_BEAM_TRAFFIC_BYTES_PLAIN = {(16, 256): 749.9e6}
NCU_BEAM_TRAFFIC_BYTES_NEIGHBOR_CODES = {(16, 256): 489.7e6}
RECALL_TARGET = 0.95


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--nodes", type=int, default=10_000_000, help="base vectors (default: configuration 2)")
    ap.add_argument("--queries", type=int, default=10_000)
    ap.add_argument("--top-l", type=int, default=0, help="skip the sweep and use this top_l")
    ap.add_argument("--top-n", type=int, default=0, help="with --top-l: rerank top_n (default 32)")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the CPU baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--streams", type=int, default=4,
                    help="searchers (each on its own stream) that the steps alternate between; 1 = one batch at a time")
    ap.add_argument("--no-neighbor-codes", action="store_true",
                    help="do not build the neighbour-code layout (degree * M bytes per node of extra HBM)")
    ap.add_argument("--sharded", action="store_true",
                    help="N > 1 only: instead of replicas, split the index by node-id range over the GPUs (--nodes per "
                         "GPU, R = 32 records as in the 1 B-vector configuration); every rank searches its own 10 k "
                         "queries and reads (N-1)/N of all rows from its peers over NVLink")
    return ap.parse_args()


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


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
    cfg = dataclasses.replace(synth.CONFIGS["cfg2"], num_nodes=args.nodes, num_queries=args.queries,
                              components=max(1, args.nodes // 1000))
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


def cpu_leg(s, L, top_n, seconds, host=None):
    """Times the CPU implementation (the checker's restatement, OpenMP over queries) on the same
    index and parameters, on as many queries as fit the time budget."""
    from oracle import oracle as orc
    from oracle import pipeline
    from topoanns_b200 import synth
    host = host or pipeline.index_from_synth(s)
    q = s.queries.cpu().numpy()
    pipeline.vectors_to_pages  # noqa: B018
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
    recall = synth.recall_at_k(r["topk_ids"], s.gt_ids.cpu().numpy()[:n], 10)
    return dict(value=n / best, unit="queries/s", cores=orc.num_threads(), kind="port",
                sample=f"{n} of {q.shape[0]} queries x {reps} passes (best pass), top_l={L}, rerank_top_n={top_n}, "
                       f"recall@10={recall:.3f}"), host


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
    if world > 1 and args.impl == "b200":
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    device = f"cuda:{local}" if use_cuda else "cpu"

    from topoanns_b200 import synth
    sharded = args.sharded and world > 1 and args.impl == "b200"
    peer_buffers = None
    if sharded:
        from topoanns_b200 import sharding, synth_sharded
        t0 = time.time()
        cfg = dataclasses.replace(synth.CONFIGS["cfg4"], num_nodes=args.nodes * world, num_queries=args.queries * world,
                                  components=max(world, args.nodes * world // 1000), kmeans_iters=5, train_sample=65536)
        s = synth_sharded.build(cfg, device)       # this rank's shard + the whole query set and ground truth
        build_s = time.time() - t0
        b, e = sharding.query_shard(s.queries.shape[0], world, rank)
        queries_all, gt = s.queries, s.gt_ids.cpu().numpy()[b:e]
        s.queries = queries_all[b:e].contiguous()  # every rank serves its own slice
        degree, M = s.adjacency.shape[1], s.pq_codes.shape[1]
        workload = (f"cfg4-style shards: {s.total_nodes} x {cfg.dim} uint8 over {world} GPUs ({s.rows_per_shard} per GPU), "
                    f"R={degree}, PQ M={M}x256, RVQ entries=128, {args.queries} queries/batch per GPU, k=10, W=2, "
                    f"{world - 1}/{world} of the row gathers remote (NVLink peer loads)")
    else:
        s, build_s = build_index(args, device)
        gt = s.gt_ids.cpu().numpy()
        degree, M = s.adjacency.shape[1], s.pq_codes.shape[1]
        workload = (f"cfg2: {s.vectors.shape[0]} x {s.cfg.dim} uint8, R={degree}, PQ M={M}x256, RVQ 256x256 entries=128, "
                    f"{s.queries.shape[0]} queries/batch, k=10, W=2, max_expansions=4096")
    Q = s.queries.shape[0]

    if args.impl == "reference":
        # the operating point the CUDA arm's sweep settles on for this seeded workload
        L = args.top_l or DEFAULT_POINT[0]
        top_n = args.top_n or DEFAULT_POINT[1]
        res, _ = cpu_leg(s, L, top_n, args.cpu_seconds)
        line = {"impl": "reference", "metric": "QPS at recall@10>=0.95 (10M uint8 d=128, 1 batch of 10k queries)",
                "value": res["value"], "unit": "queries/s", "n_gpus": 0, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": 1000.0 * Q / res["value"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                "config": {"workload": workload, "top_l": L, "rerank_top_n": top_n},
                "cpu_baseline": res,
                "e2e": {"value": res["value"], "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    from topoanns_b200 import capi, search
    lib = capi.load()
    if sharded:
        ix, peer_buffers = sharding.peer_index_from_sharded(s)
        model = search.RvqModel(dim=s.cfg.dim, coarse=s.rvq_coarse.contiguous(), fine=s.rvq_fine.contiguous(),
                                bucket_sizes=s.rvq_buckets[0], cluster_offsets=s.rvq_buckets[1], cluster_ids=s.rvq_buckets[2])
    else:
        ix = search.device_index_from_synth(s, device)
        model = search.rvq_model_from_synth(s, device)
        if not args.no_neighbor_codes:
            # HBM is plentiful for this configuration: also keep every node's neighbours' PQ codes next to each
            # other (degree * M bytes per node), so that an expansion needs one memory round trip, not two
            search.inline_neighbor_codes(ix)
    max_cap = 1024
    sr = search.Searcher(ix, Q, max_cap, max(TOPN_SWEEP), 128)
    sr.set_rvq(model, 128)
    q_host = s.queries.cpu().numpy()
    q_pinned = torch.from_numpy(q_host).pin_memory()
    q_dev = s.queries.to(device).contiguous()

    def run_point(L, top_n):
        tp = search.TopologySearchParams(top_l=L, search_width=2, max_expansions=4096)
        rp = search.RerankExactParams(top_k=10, top_n=top_n)
        t0 = time.perf_counter()
        ids, dists, stats = sr.run_host(q_pinned.numpy(), tp, rp, want_stats=True)
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
    for _ in range(args.warmup):
        sr.run_device(q_dev, tp, rp)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        sr.run_device(q_dev, tp, rp)
    ev1.record(stream)
    barrier()
    dev_one_stream_ms = ev0.elapsed_time(ev1)
    # The same K steps through two searchers on two streams, submitted alternately: the short kernels of one batch
    # (entry selection, rerank, top-k) and the ragged last wave of its beam search run beside the other batch's
    # beam search. Timed with events: both streams start after ev0, ev1 follows the end of both.
    n_lanes = max(1, args.streams)
    searchers, streams, q_devs = [sr], [torch.cuda.Stream(device)], [q_dev]
    for _ in range(n_lanes - 1):
        extra = search.Searcher(ix, Q, max_cap, max(TOPN_SWEEP), 128)
        extra.set_rvq(model, 128)
        searchers.append(extra)
        streams.append(torch.cuda.Stream(device))
        q_devs.append(q_dev.clone())

    def many_streams(steps):
        for i in range(steps):
            with torch.cuda.stream(streams[i % n_lanes]):
                searchers[i % n_lanes].run_device(q_devs[i % n_lanes], tp, rp)

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
    q_np = q_pinned.numpy()
    for _ in range(args.warmup):
        sr.run_host(q_np, tp, rp, out_ids=out_ids_np, out_dists=out_dists_np)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        # every rank serves its own batch and reads its own results back: no data-path collective
        ids, dists, _ = sr.run_host(q_np, tp, rp, out_ids=out_ids_np, out_dists=out_dists_np)
    torch.cuda.synchronize()
    e2e_serial_s = time.perf_counter() - t0
    barrier()
    # The same through two searchers on two streams, submitted alternately: batch i's copies overlap batch
    # i-1's kernels. Every step still copies its queries in and its results out inside the timed region.
    lanes = [(sr, streams[0], q_np, out_ids_np, out_dists_np)]
    for k in range(1, n_lanes):
        lanes.append((searchers[k], streams[k], torch.from_numpy(q_host).pin_memory().numpy(),
                      torch.empty((Q, 10), dtype=torch.int32).pin_memory().numpy().view(np.uint32),
                      torch.empty((Q, 10), dtype=torch.float32).pin_memory().numpy()))

    def pipelined(steps):
        for i in range(steps):
            srx, st, qx, oi, od = lanes[i % n_lanes]
            srx.wait()
            srx.submit_host(qx, tp, rp, oi, od, stream=st)
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
    for _, _, _, oi, od in lanes[1:]:
        assert np.array_equal(oi, out_ids_np) and np.array_equal(od, out_dists_np)
    for extra in searchers[1:]:
        extra.close()
    clocks = sampler.stop() if rank == 0 else {}
    # ---- the beam-search kernel alone, for the roofline -----------------------------------------
    offs, eids, _ = model.device_entry_batch(q_dev, 128)
    cap = tp.capacity(top_n)
    view = ix.view()
    bp = tp.to_c(cap)
    cand = torch.empty((Q, cap, 2), dtype=torch.int32, device=device)
    stats_d = torch.empty((Q, 8), dtype=torch.int32, device=device)

    def beam_once():
        capi.check(lib.tann_beam_search(C.byref(view), C.byref(bp), None, C.c_void_p(q_dev.data_ptr()),
                                        capi.KIND_FLOAT32, Q, C.c_void_p(offs.data_ptr()), C.c_void_p(eids.data_ptr()),
                                        C.c_void_p(cand.data_ptr()), C.c_void_p(stats_d.data_ptr()), None,
                                        C.c_void_p(stream.cuda_stream)))
    for _ in range(args.warmup):
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

    # ---- max over ranks --------------------------------------------------------------------------
    times = torch.tensor([dev_ms, e2e_s * 1000.0, beam_ms, e2e_serial_s * 1000.0, dev_one_stream_ms], dtype=torch.float64,
                         device=device)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, beam_ms, e2e_serial_ms, dev_one_stream_ms = [float(x) for x in times.cpu()]
    if rank != 0:
        sr.close()
        if world > 1:
            import torch.distributed as dist
            if peer_buffers is not None:
                dist.barrier()
                for pb in peer_buffers.values():
                    pb.close()
            dist.destroy_process_group()
        return 0

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    achieved = beam_bytes / (beam_ms * 1e-3) / 1e9
    table = NCU_BEAM_TRAFFIC_BYTES_NEIGHBOR_CODES if ix.neighbor_codes is not None else NCU_BEAM_TRAFFIC_BYTES_PLAIN
    traffic = table.get((L, cap)) if (args.nodes, Q) == (10_000_000, 10_000) and not sharded else None
    rec = synth.recall_at_k(ids, gt, 10)
    total_q = Q * world * args.steps
    line = {
        "metric": ("QPS at recall@10>=0.95 (uint8 d=128 index sharded by node-id range, 1 batch of 10k queries per GPU)"
                   if sharded else "QPS at recall@10>=0.95 (10M uint8 d=128, 1 batch of 10k queries per GPU)"),
        "value": total_q / (dev_ms * 1e-3), "unit": "queries/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": workload, "top_l": L, "rerank_top_n": top_n, "recall_at_10": round(rec, 4),
                   "recall_target_met": bool(rec >= RECALL_TARGET),
                   "parallelism": (f"node-id-range shards x{world}, queries sharded" if sharded
                                   else f"replica x{world}, queries sharded"),
                   "l2_policy": "index (4.2 GB) and per-step gathers exceed the 126 MB L2; no flush",
                   "streams": f"{n_lanes}: steps alternate between {n_lanes} searchers, each on its own stream; one stream alone: "
                              f"{total_q / (dev_one_stream_ms * 1e-3):.0f} queries/s, {dev_one_stream_ms / args.steps:.4f} ms per step",
                   "layout": ("adjacency + PQ codes + vector pages in HBM"
                              + (f" + neighbour codes next to each node ({ix.neighbor_codes.numel() / 1e9:.1f} GB)"
                                 if ix.neighbor_codes is not None else "")),
                   "index_build_s": round(build_s, 1), "sweep": sweep,
                   "beam_kernel": {"smem_bytes": smem, "blocks_per_sm": blocks_per_sm, "resident_blocks": grid, "grid": "one block per query",
                                   "ms": round(beam_ms, 4), "mean_expanded": float(stats[:, 1].mean()),
                                   "mean_visited": float(stats[:, 0].mean()),
                                   "bytes_per_query": beam_bytes / Q}},
        "e2e": {"value": total_q / (e2e_ms * 1e-3), "unit": "queries/s",
                "h2d_bytes_per_step": int(q_host.nbytes), "d2h_bytes_per_step": int(Q * 10 * 8),
                "pipeline": f"{n_lanes} searchers on {n_lanes} streams, batches submitted in turn (copies of one overlap kernels of the others)",
                "one_batch_at_a_time": total_q / (e2e_serial_ms * 1e-3)},
        "gpu_launches": 5 * args.steps,  # rvq, beam, float->uint8 check, rerank, top-k pack
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "frac_of_nominal_8tbs": achieved / 8000.0, "traffic": traffic, "peak_source": peak_src, "kernel": "beam_search_kernel",
                     "whole_step_gbs": (beam_bytes + rerank_bytes) * args.steps / (dev_ms * 1e-3) / 1e9},
    }
    if world == 1 and not args.no_cpu_baseline:
        try:
            line["cpu_baseline"], _ = cpu_leg(s, L, top_n, args.cpu_seconds)
        except Exception as e:  # the baseline must not take the GPU numbers down with it
            line["cpu_baseline"] = {"value": None, "error": str(e)}
    print(json.dumps(line))
    sr.close()
    if world > 1:
        import torch.distributed as dist
        if peer_buffers is not None:
            dist.barrier()
            for pb in peer_buffers.values():
                pb.close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
