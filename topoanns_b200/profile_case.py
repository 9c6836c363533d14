"""Run the stages of the search path a few times on a small synthetic index, for use under a profiler
(`ncu -k regex:beam_search ... python -m topoanns_b200.profile_case --nodes 1000000 --queries 4000`).
The index is the bench workload's generator at a reduced size: large enough that gathers miss L2, small
enough that a multi-pass capture saves and restores little device memory. Prints one line per stage
with its CUDA-event time.
"""
from __future__ import annotations

import argparse
import dataclasses

import torch

from . import capi, search, synth


def _time(fn, reps):
    """One warm-up call, then `reps` calls back to back between two CUDA events (the queue stays full, so
    the host's launch latency is not part of the figure); returns (last result, mean ms per call)."""
    out = fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        out = fn()
    stop.record()
    torch.cuda.synchronize()
    return out, start.elapsed_time(stop) / reps


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--config", default="cfg2", choices=sorted(synth.CONFIGS))
    ap.add_argument("--nodes", type=int, default=1_000_000)
    ap.add_argument("--queries", type=int, default=4000)
    ap.add_argument("--top-l", type=int, default=64)
    ap.add_argument("--search-width", type=int, default=2)
    ap.add_argument("--top-n", type=int, default=32)
    ap.add_argument("--entries", type=int, default=128)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--staged-table", action="store_true", help="build the query tables with tann_lut_build first")
    ap.add_argument("--inline-neighbor-codes", action="store_true",
                    help="also store every node's neighbours' PQ codes next to each other (degree * M bytes per node)")
    ap.add_argument("--topology", default="hbm", choices=["hbm", "pinned-host"],
                    help="where the adjacency lists live (pinned-host = mapped host memory read over PCIe)")
    ap.add_argument("--cached-fraction", type=float, default=0.0,
                    help="with --topology pinned-host: fraction of the rows (an id prefix) cached in HBM")
    a = ap.parse_args()
    cfg = dataclasses.replace(synth.CONFIGS[a.config], num_nodes=a.nodes, components=max(1, a.nodes // 1000),
                              num_queries=a.queries, kmeans_iters=5)
    s = synth.build(cfg, "cuda")
    ix = search.device_index_from_synth(s)
    q = s.queries.cuda().contiguous()
    if a.inline_neighbor_codes:
        search.inline_neighbor_codes(ix)
        print(f"neighbour-code layout: {ix.neighbor_codes.numel() / 1e9:.2f} GB")
    host_alloc = None
    if a.topology == "pinned-host":
        import ctypes as C

        lib = capi.load()
        nbytes = ix.adjacency.numel() * 4
        hp, dp = C.c_void_p(), C.c_void_p()
        capi.check(lib.tann_host_alloc_mapped(nbytes, C.byref(hp), C.byref(dp)))
        host_alloc = hp
        adj_host = ix.adjacency.cpu().numpy()   # keep the array alive across the copy
        C.memmove(hp.value, adj_host.ctypes.data, nbytes)
        del adj_host
        cached = int(ix.num_nodes * a.cached_fraction)
        ix = search.DeviceIndex(
            num_nodes=ix.num_nodes, degree=ix.degree, dim=ix.dim, vector_kind=ix.vector_kind, codes=ix.codes,
            vector_pages=ix.vector_pages, pq_tables_col_major=ix.pq_tables_col_major, pq_centroid=ix.pq_centroid,
            pq_chunk_offsets=ix.pq_chunk_offsets, vector_bytes=ix.vector_bytes, vectors_per_page=ix.vectors_per_page,
            adjacency_bases=[dp.value], adjacency_cache=ix.adjacency[:cached].clone() if cached else None,
            adjacency_cached_rows=cached)
        print(f"topology: {nbytes / 1e9:.2f} GB in mapped pinned host memory, {cached} rows ({a.cached_fraction:.0%}) cached in HBM")
    if cfg.rvq:
        model = search.rvq_model_from_synth(s)
        (offs, ids, _), ms = _time(lambda: model.device_entry_batch(q, a.entries), a.reps)
        print(f"rvq_entries {ms:.3f} ms")
    else:
        offs = torch.arange(a.queries + 1, dtype=torch.int32, device="cuda")
        ids = torch.full((a.queries,), int(s.medoid), dtype=torch.int32, device="cuda")
    p = search.TopologySearchParams(top_l=a.top_l, search_width=a.search_width, max_expansions=4096)
    cap = p.capacity(a.top_n)
    lut = None
    if a.staged_table:
        lut, ms = _time(lambda: search.lut_build(ix, q), a.reps)
        print(f"lut_build {ms:.3f} ms")
    (cand, stats), ms = _time(lambda: search.beam_search(ix, p, offs, ids, queries=None if lut is not None else q,
                                                         lut=lut, capacity=cap), a.reps)
    st = stats.cpu().numpy()
    e, v = float(st[:, 1].mean()), float(st[:, 0].mean())
    gbytes = a.queries * (e * 4 * ix.degree + v * ix.num_chunks) / 1e9
    print(f"beam_search {ms:.3f} ms  nodes={a.nodes} queries={a.queries} L={a.top_l} C={cap} expanded/query={e:.1f} "
          f"visited/query={v:.1f} algorithmic={gbytes:.3f} GB -> {gbytes / ms * 1e3:.1f} GB/s")
    rp = search.RerankExactParams(top_k=10, top_n=a.top_n)
    _, ms = _time(lambda: search.rerank_exact(ix, rp, cand, q), a.reps)
    print(f"rerank_exact {ms:.3f} ms  top_n={a.top_n}  (float32 queries)")
    if s.vectors.dtype == torch.uint8:
        q8 = q.to(torch.uint8).contiguous()   # the searcher makes this copy on the device when the values allow it
        _, ms = _time(lambda: search.rerank_exact(ix, rp, cand, q8), a.reps)
        gb = a.queries * a.top_n * s.vectors.shape[1] / 1e9
        print(f"rerank_exact {ms:.3f} ms  top_n={a.top_n}  (uint8 queries, integer path) {gb / ms * 1e3:.1f} GB/s")
    if getattr(s, "pq2_tables", None) is not None:
        # residual pq2 refine + bound filter (float configurations): second table build, refine, tiled rerank
        t2 = s.pq2_tables.cuda().contiguous()
        c2 = s.pq2_centroid.cuda().contiguous()
        codes2 = s.pq2_codes.cuda().contiguous()
        cross = search.pq2_cross_terms(ix.pq_chunk_offsets, s.pq_tables.cuda().contiguous(), ix.pq_centroid, t2, c2)
        t2_cm = t2.t().contiguous()
        lut2, ms = _time(lambda: search.lut_build(ix, q, tables_col_major=t2_cm, centroid=c2), a.reps)
        print(f"lut_build (pq2) {ms:.3f} ms  {lut2.numel() * 4 / 1e6:.0f} MB written")
        lr = min(a.top_l, cap)
        refined, ms = _time(lambda: search.pq2_refine(cand, stats, lr, codes2, lut2, base_codes=ix.codes, cross_terms=cross), a.reps)
        print(f"pq2_refine {ms:.3f} ms  refine_top_l={lr}")
        eps = s.pq2_error_bounds.cuda().contiguous()
        rp2 = search.RerankExactParams(top_k=10, top_n=min(a.top_n, lr), rank_tile_size=16, use_pq2_bound_filter=True)
        (_, _, n_exact, n_flt), ms = _time(lambda: search.rerank_exact(ix, rp2, refined, q, eps), a.reps)
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
            res, ms = _time(lambda: search.rerank_exact_learned_stop(ix, rp2, refined, q, model=ls, error_bounds=eps), a.reps)
            print(f"rerank_exact_learned_stop {ms:.3f} ms  exact={res['n_exact']} filtered={res['n_filtered']} "
                  f"mean_stop_prefix={float(res['stop_prefixes'].float().mean()):.1f} of {budget}")
        if cfg.rvq:
            sr = search.Searcher(ix, a.queries, cap, min(a.top_n, lr), a.entries)
            sr.set_rvq(model, a.entries)
            sr.set_pq2(search.Pq2Resources(codes=codes2, tables_col_major=t2_cm, centroid=c2, chunk_offsets=ix.pq_chunk_offsets,
                                           cross_terms=cross, error_bounds=eps), lr)
            _, ms = _time(lambda: sr.run_device(q, p, rp2), a.reps)
            print(f"searcher whole path (rvq, beam, table-free pq2 refine, bound-filtered rerank, top-k) {ms:.3f} ms")
            sr.close()
    if host_alloc is not None:
        torch.cuda.synchronize()
        capi.check(lib.tann_host_free(host_alloc))


if __name__ == "__main__":
    main()
