"""Synthetic index split by node-id range over the ranks of one box (the 1 B-vector configuration
at one eighth per GPU). Every rank generates the mixture components it is responsible for, builds
their kNN edges locally, then node ids are scattered over the whole id space by an affine
permutation and every row (vector, adjacency list, PQ code) is sent to the rank that owns its new
id. After that a node's kNN neighbours live on all ranks with equal probability, so (G-1)/G of the
adjacency / code / vector gathers of a search are remote reads.

Uses only point-to-point sends plus all_gather / broadcast, so it runs on NCCL (GPU) and gloo (CPU).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from . import synth


@dataclass
class ShardedSynth:
    cfg: synth.SynthConfig
    world: int
    rank: int
    total_nodes: int
    rows_per_shard: int
    vectors: torch.Tensor          # [rows_per_shard, d] local shard
    adjacency: torch.Tensor        # [rows_per_shard, degree] int32, global ids
    pq_codes: torch.Tensor         # [rows_per_shard, M] uint8
    pq_tables: torch.Tensor
    pq_centroid: torch.Tensor
    pq_chunk_offsets: torch.Tensor
    queries: torch.Tensor          # [Q, d] identical on every rank
    gt_ids: torch.Tensor           # [Q, k] global ids, identical on every rank
    rvq_coarse: Optional[torch.Tensor] = None
    rvq_fine: Optional[torch.Tensor] = None
    rvq_buckets: Optional[list] = None   # (sizes, offsets, ids) over the whole index, identical on every rank
    centres: Optional[torch.Tensor] = None   # mixture centres (identical on every rank), for drawing further queries


def _coprime_multiplier(n: int) -> int:
    a = 2_147_483_629  # a large prime; step down until coprime with n
    while math.gcd(a, n) != 1:
        a -= 2
    return a


def exchange_rows(chunks: List[torch.Tensor]) -> List[torch.Tensor]:
    """chunks[j] goes to rank j; returns what every rank sent to this one (index = source rank)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = chunks[0].device
    counts = torch.tensor([c.shape[0] for c in chunks], dtype=torch.int64, device=dev)
    all_counts = [torch.empty_like(counts) for _ in range(world)]
    dist.all_gather(all_counts, counts)
    out: List[Optional[torch.Tensor]] = [None] * world
    out[rank] = chunks[rank]
    ops = []
    for j in range(world):
        if j == rank:
            continue
        n_in = int(all_counts[j][rank])
        out[j] = torch.empty((n_in,) + tuple(chunks[0].shape[1:]), dtype=chunks[0].dtype, device=dev)
        if chunks[j].shape[0] > 0:
            ops.append(dist.P2POp(dist.isend, chunks[j].contiguous(), j))
        if n_in > 0:
            ops.append(dist.P2POp(dist.irecv, out[j], j))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return out  # type: ignore[return-value]


def _scatter_by_owner(rows: torch.Tensor, owner: torch.Tensor, local_row: torch.Tensor, n_loc: int):
    """Send every row to its owner and place it at its local row there."""
    world = dist.get_world_size()
    order = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=world).tolist()
    rows_s, lr_s = rows[order], local_row[order]
    chunks, lr_chunks, pos = [], [], 0
    for j in range(world):
        chunks.append(rows_s[pos:pos + counts[j]])
        lr_chunks.append(lr_s[pos:pos + counts[j]])
        pos += counts[j]
    got = torch.cat(exchange_rows(chunks))
    got_lr = torch.cat(exchange_rows(lr_chunks))
    out = torch.empty((n_loc,) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    out[got_lr] = got
    return out


def build(cfg: synth.SynthConfig, device="cpu", gt_stride: int = 1) -> ShardedSynth:
    """cfg.num_nodes is the size of the WHOLE index; it is rounded down so that shards are equal and
    page-aligned. Must be called by every rank of the process group. With gt_stride > 1 the brute-force
    ground truth is computed for every gt_stride-th query only (the other rows of gt_ids are -1): at a
    billion vectors the exact neighbours of all queries cost more than the index."""
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device(device)
    if dev.type == "cuda":
        torch.backends.cuda.matmul.allow_tf32 = False
    d = cfg.dim
    comps_total = max(world, cfg.components // world * world)
    comps_loc = comps_total // world
    n_per = max(cfg.knn_edges + 1, cfg.num_nodes // comps_total)
    n_per = (n_per + 31) // 32 * 32                     # keeps shards page-aligned for any vector size <= 4 KB / 32
    n_loc = n_per * comps_loc
    n_tot = n_loc * world
    common = synth._gen(dev, cfg.seed)                  # same stream on every rank
    if cfg.kind == "uint8":
        centres = torch.rand((comps_total, d), generator=common, device=dev) * 255.0
    else:
        centres = torch.randn((comps_total, d), generator=common, device=dev)
        centres = centres / centres.norm(dim=1, keepdim=True)
    qcomp = torch.randint(0, comps_total, (cfg.num_queries,), generator=common, device=dev)
    queries = synth._sample_component(cfg, centres, qcomp, common).float()
    own = synth._gen(dev, cfg.seed * 1000 + 17 + rank)  # this rank's stream
    out_dtype = torch.uint8 if cfg.kind == "uint8" else torch.float32
    grouped = torch.empty((n_loc, d), dtype=out_dtype, device=dev)
    step = max(1, (1 << 22) // n_per) * n_per
    for s in range(0, n_loc, step):
        e = min(n_loc, s + step)
        comp_ids = rank * comps_loc + torch.arange(s, e, device=dev) // n_per
        grouped[s:e] = synth._sample_component(cfg, centres, comp_ids, own).to(out_dtype)
    a, b = _coprime_multiplier(n_tot), 12345 % n_tot

    def perm(x):  # old global id -> new global id
        return (x.to(torch.int64) * a + b) % n_tot

    old = rank * n_loc + torch.arange(n_loc, device=dev, dtype=torch.int64)
    new = perm(old)
    if n_loc <= (1 << 25):
        knn = synth.build_knn_graph(grouped, n_per, cfg.knn_edges)              # local row numbers
        rand_edges = torch.randint(0, n_tot, (n_loc, cfg.random_edges), generator=own, device=dev)
        adjacency = torch.cat([perm(rank * n_loc + knn), rand_edges], 1).to(torch.int32)
        del knn, rand_edges
    else:
        # very large shards: slices of whole components, so that only a slice's 64-bit tables exist at a time
        kk = min(cfg.knn_edges, n_per - 1)
        adjacency = torch.empty((n_loc, kk + cfg.random_edges), dtype=torch.int32, device=dev)
        slice_rows = max(1, (1 << 22) // n_per) * n_per
        for lo in range(0, n_loc, slice_rows):
            hi = min(n_loc, lo + slice_rows)
            knn = synth.build_knn_graph(grouped[lo:hi], n_per, cfg.knn_edges) + lo
            rnd = torch.randint(0, n_tot, (hi - lo, cfg.random_edges), generator=own, device=dev)
            adjacency[lo:hi] = torch.cat([perm(rank * n_loc + knn), rnd], 1).to(torch.int32)
            del knn, rnd
    # training sample drawn from every rank's components (a rank holds its own components only at this point);
    # rank 0 trains the PQ pivots and the entry model on it and shares them
    take = min(n_loc, max(1, cfg.train_sample // world))
    sample = torch.randperm(n_loc, generator=own, device=dev)[:take]
    mine = grouped[sample].contiguous()
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    xs = torch.cat(parts).float()
    del parts, mine
    if rank == 0:
        tables, centroid, offs = synth.train_pq(xs, cfg.pq_chunks, cfg.kmeans_iters, own)
    else:
        tables = torch.empty((256, d), device=dev)
        centroid = torch.empty(d, device=dev)
        offs = torch.empty(cfg.pq_chunks + 1, dtype=torch.int32, device=dev)
    for t in (tables, centroid, offs):
        dist.broadcast(t, 0)
    codes = synth.encode_pq(grouped, tables, centroid, offs)
    coarse = fine = None
    if cfg.rvq:
        if rank == 0:
            coarse = synth.kmeans(xs, min(cfg.rvq_coarse, xs.shape[0]), cfg.kmeans_iters, own)
            ca = synth._sqdist(xs, coarse).argmin(1)
            fine = synth.kmeans(xs - coarse[ca], min(cfg.rvq_fine, xs.shape[0]), cfg.kmeans_iters, own)
            shape = torch.tensor([coarse.shape[0], fine.shape[0]], device=dev)
        else:
            shape = torch.zeros(2, dtype=torch.int64, device=dev)
        dist.broadcast(shape, 0)
        if rank != 0:
            coarse = torch.empty((int(shape[0]), d), device=dev)
            fine = torch.empty((int(shape[1]), d), device=dev)
        dist.broadcast(coarse, 0)
        dist.broadcast(fine, 0)
    # scatter rows to the owners of their new ids
    owner, local_row = new // n_loc, new % n_loc
    vectors = _scatter_by_owner(grouped, owner, local_row, n_loc)
    del grouped
    adjacency = _scatter_by_owner(adjacency, owner, local_row, n_loc)
    codes = _scatter_by_owner(codes, owner, local_row, n_loc)
    # ground truth: local brute force, merged over ranks
    gt_rows = torch.arange(0, queries.shape[0], max(1, gt_stride), device=dev)
    loc_i, loc_d = synth.brute_force_topk(vectors, queries[gt_rows], cfg.top_k)
    loc_i = loc_i + rank * n_loc
    all_i = [torch.empty_like(loc_i) for _ in range(world)]
    all_d = [torch.empty_like(loc_d) for _ in range(world)]
    dist.all_gather(all_i, loc_i)
    dist.all_gather(all_d, loc_d)
    cat_d, cat_i = torch.cat(all_d, 1), torch.cat(all_i, 1)
    order = torch.argsort(cat_d, dim=1, stable=True)[:, :cfg.top_k]
    gt = cat_i.gather(1, order)
    if gt_stride > 1:
        full = torch.full((queries.shape[0], cfg.top_k), -1, dtype=gt.dtype, device=dev)
        full[gt_rows] = gt
        gt = full
    out = ShardedSynth(cfg, world, rank, n_tot, n_loc, vectors, adjacency, codes, tables, centroid, offs, queries, gt)
    out.centres = centres
    if cfg.rvq:
        nc, nf = coarse.shape[0], fine.shape[0]
        cluster = torch.empty(n_loc, dtype=torch.int64, device=dev)
        for s in range(0, n_loc, 262144):
            xb = vectors[s:s + 262144].float()
            ca = synth._sqdist(xb, coarse).argmin(1)
            cluster[s:s + 262144] = ca * nf + synth._sqdist(xb - coarse[ca], fine).argmin(1)
        sizes = torch.bincount(cluster, minlength=nc * nf)
        dist.all_reduce(sizes)
        gid = rank * n_loc + torch.arange(n_loc, device=dev, dtype=torch.int64)
        order = torch.argsort(cluster, stable=True)               # ascending id inside a bucket
        lsz = torch.bincount(cluster, minlength=nc * nf)
        starts = torch.cumsum(lsz, 0) - lsz
        keep = (torch.arange(n_loc, device=dev) - starts[cluster[order]]) < 256
        cand = torch.stack([cluster[order][keep], gid[order][keep]], 1)    # this rank's first 256 per bucket
        count = torch.tensor([cand.shape[0]], device=dev)
        counts = [torch.empty_like(count) for _ in range(world)]
        dist.all_gather(counts, count)
        longest = int(max(int(c) for c in counts))
        padded = torch.full((longest, 2), -1, dtype=torch.int64, device=dev)
        padded[:cand.shape[0]] = cand
        gathered = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(gathered, padded)
        merged = torch.cat([g[:int(c)] for g, c in zip(gathered, counts)])
        key = merged[:, 0] * n_tot + merged[:, 1]                          # sort by (bucket, id)
        merged = merged[torch.argsort(key)]
        msz = torch.bincount(merged[:, 0], minlength=nc * nf)
        mstart = torch.cumsum(msz, 0) - msz
        mkeep = (torch.arange(merged.shape[0], device=dev) - mstart[merged[:, 0]]) < 256
        capped = torch.clamp(sizes, max=256)
        offsets = torch.zeros(nc * nf + 1, dtype=torch.int64, device=dev)
        offsets[1:] = torch.cumsum(capped, 0)
        out.rvq_coarse, out.rvq_fine = coarse, fine
        out.rvq_buckets = [sizes.to(torch.int32), offsets.to(torch.int32), merged[mkeep, 1].to(torch.int32)]
    return out


def gather_whole(s: ShardedSynth) -> synth.SynthIndex:
    """All shards concatenated on every rank (tests only: the whole index must fit one process)."""
    def allcat(t):
        parts = [torch.empty_like(t) for _ in range(s.world)]
        dist.all_gather(parts, t.contiguous())
        return torch.cat(parts)
    idx = synth.SynthIndex(s.cfg, allcat(s.vectors), allcat(s.adjacency), s.pq_tables, s.pq_centroid,
                           s.pq_chunk_offsets, allcat(s.pq_codes), s.queries, s.gt_ids, 0)
    idx.rvq_coarse, idx.rvq_fine, idx.rvq_buckets = s.rvq_coarse, s.rvq_fine, s.rvq_buckets
    return idx
