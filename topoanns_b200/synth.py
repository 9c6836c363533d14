"""Seeded synthetic indices with the shapes and value distributions of the benchmark
configurations (Gaussian-mixture base vectors, kNN + random-edge graph, k-means PQ, optional
residual pq2 with error bounds, two-level RVQ entry model, brute-force ground truth).

The generator is not on the hot path; it uses torch ops on whatever device it is given so that
the 10 M-vector configuration builds on the GPU in well under a minute.

Approximation used for the kNN edges: the k nearest neighbours are searched among the points of
the same mixture component (components are far apart compared with their spread, so this equals
the exact kNN for all but a vanishing fraction of nodes; the unit tests measure the agreement
with brute force). Node ids are then shuffled by a random permutation so that neighbours are not
id-contiguous and every gather is a random access.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch


@dataclass
class SynthConfig:
    name: str
    num_nodes: int
    dim: int
    kind: str                 # "uint8" or "float32"
    components: int
    sigma: float = 20.0
    knn_edges: int = 24
    random_edges: int = 8
    pq_chunks: int = 32
    num_queries: int = 1000
    top_k: int = 10
    rvq: bool = False
    rvq_coarse: int = 256
    rvq_fine: int = 256
    pq2: bool = False
    normalise: bool = False   # float32 configurations: L2-normalised vectors
    low_rank: int = 0         # > 0: rank of the component covariance (embedding-like workload)
    iso_sigma: float = 0.05
    kmeans_iters: int = 25
    train_sample: int = 262144
    seed: int = 1234

    @property
    def degree(self) -> int:
        return self.knn_edges + self.random_edges


# The five benchmark configurations (sizes can be scaled down by the callers for tests).
CONFIGS = {
    "cfg1": SynthConfig("cfg1", 100_000, 128, "uint8", 1000, knn_edges=24, random_edges=8, pq_chunks=32,
                        num_queries=1000),
    "cfg2": SynthConfig("cfg2", 10_000_000, 128, "uint8", 10_000, knn_edges=48, random_edges=16,
                        pq_chunks=32, num_queries=10_000, rvq=True),
    "cfg3": SynthConfig("cfg3", 100_000_000, 96, "float32", 50_000, sigma=0.05, knn_edges=48,
                        random_edges=16, pq_chunks=48, num_queries=10_000, pq2=True, normalise=True,
                        rvq=True),
    "cfg4": SynthConfig("cfg4", 1_000_000_000, 128, "uint8", 100_000, knn_edges=24, random_edges=8,
                        pq_chunks=32, num_queries=10_000, rvq=True),
    # sigma scales the rank-64 part: 0.05 per latent dim keeps a component's spread (~0.4) below the distance
    # between unit-norm centres (~1.4), so that components stay separate after normalisation
    "cfg5": SynthConfig("cfg5", 10_000_000, 768, "float32", 10_000, sigma=0.05, knn_edges=48, random_edges=16,
                        pq_chunks=96, num_queries=10_000, normalise=True, low_rank=64, rvq=True),
}


@dataclass
class SynthIndex:
    cfg: SynthConfig
    vectors: torch.Tensor            # [N, d] uint8 or float32
    adjacency: torch.Tensor          # [N, degree] int32
    pq_tables: torch.Tensor          # [256, d] f32, row-major as in the pivots file
    pq_centroid: torch.Tensor        # [d]
    pq_chunk_offsets: torch.Tensor   # [M + 1] int32
    pq_codes: torch.Tensor           # [N, M] uint8
    queries: torch.Tensor            # [Q, d] float32 (integer-valued for uint8 data)
    gt_ids: torch.Tensor             # [Q, top_k] int64
    medoid: int = 0
    rvq_coarse: Optional[torch.Tensor] = None
    rvq_fine: Optional[torch.Tensor] = None
    rvq_buckets: Optional[list] = None          # (sizes [nc*nf] int32, offsets [nc*nf+1] int32, ids int32), capped lists
    pq2_tables: Optional[torch.Tensor] = None
    pq2_centroid: Optional[torch.Tensor] = None
    pq2_codes: Optional[torch.Tensor] = None
    pq2_error_bounds: Optional[torch.Tensor] = None
    extras: dict = field(default_factory=dict)


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _sqdist(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """[n, d] x [m, d] -> [n, m] squared distances (fp32, no TF32)."""
    an = (a * a).sum(1, keepdim=True)
    bn = (b * b).sum(1).unsqueeze(0)
    return an + bn - 2.0 * (a @ b.t())


def kmeans(x: torch.Tensor, k: int, iters: int, gen) -> torch.Tensor:
    """Plain Lloyd iterations from a seeded sample of the data; empty clusters keep their centre."""
    n = x.shape[0]
    idx = torch.randperm(n, generator=gen, device=x.device)[:k]
    c = x[idx].clone()
    if c.shape[0] < k:  # fewer points than centres: repeat
        c = c.repeat((k + c.shape[0] - 1) // c.shape[0], 1)[:k].clone()
    for _ in range(iters):
        assign = torch.empty(n, dtype=torch.long, device=x.device)
        for s in range(0, n, 65536):
            assign[s:s + 65536] = _sqdist(x[s:s + 65536], c).argmin(1)
        sums = torch.zeros_like(c).index_add_(0, assign, x)
        cnt = torch.zeros(k, device=x.device, dtype=x.dtype).index_add_(0, assign, torch.ones(n, device=x.device, dtype=x.dtype))
        nz = cnt > 0
        c[nz] = sums[nz] / cnt[nz].unsqueeze(1)
    return c


def _sample_component(cfg: SynthConfig, centres, comp_ids, gen, basis=None):
    """Draw one point per entry of comp_ids from its mixture component."""
    dev = centres.device
    n = comp_ids.shape[0]
    if cfg.low_rank > 0:
        z = torch.randn((n, cfg.low_rank), generator=gen, device=dev)
        x = centres[comp_ids]
        step = 8192   # the gathered bases are [step, rank, dim] floats: bounded, whatever n is
        for b in range(0, n, step):
            e = min(n, b + step)
            x[b:e] += (z[b:e].unsqueeze(1) @ basis[comp_ids[b:e] % basis.shape[0]]).squeeze(1) * cfg.sigma
        x = x + torch.randn((n, cfg.dim), generator=gen, device=dev) * cfg.iso_sigma
    else:
        x = centres[comp_ids] + torch.randn((n, cfg.dim), generator=gen, device=dev) * cfg.sigma
    if cfg.kind == "uint8":
        x = x.round().clamp_(0, 255)
    if cfg.normalise:
        x = x / x.norm(dim=1, keepdim=True).clamp_min(1e-12)
    return x


def train_pq(x_float: torch.Tensor, chunks: int, iters: int, gen):
    """DiskANN-style pivots: global centroid, per-chunk k-means of the centred data.
    Returns (tables [256, d] row-major, centroid [d], chunk_offsets [M+1])."""
    d = x_float.shape[1]
    centroid = x_float.mean(0)
    xc = x_float - centroid
    offs = [round(i * d / chunks) for i in range(chunks + 1)]
    tables = torch.zeros((256, d), dtype=torch.float32, device=x_float.device)
    for m in range(chunks):
        lo, hi = offs[m], offs[m + 1]
        tables[:, lo:hi] = kmeans(xc[:, lo:hi].contiguous(), 256, iters, gen)
    return tables, centroid, torch.tensor(offs, dtype=torch.int32, device=x_float.device)


def encode_pq(x: torch.Tensor, tables, centroid, offs, batch: int = 262144) -> torch.Tensor:
    n = x.shape[0]
    M = offs.numel() - 1
    codes = torch.empty((n, M), dtype=torch.uint8, device=x.device)
    o = offs.tolist()
    for s in range(0, n, batch):
        xc = x[s:s + batch].float() - centroid
        for m in range(M):
            lo, hi = o[m], o[m + 1]
            codes[s:s + batch, m] = _sqdist(xc[:, lo:hi], tables[:, lo:hi]).argmin(1).to(torch.uint8)
    return codes


def decode_pq(codes: torch.Tensor, tables, centroid, offs) -> torch.Tensor:
    n, M = codes.shape
    out = torch.empty((n, tables.shape[1]), dtype=torch.float32, device=codes.device)
    o = offs.tolist()
    for m in range(M):
        lo, hi = o[m], o[m + 1]
        out[:, lo:hi] = tables[codes[:, m].long(), lo:hi]
    return out + centroid


def build_knn_graph(x: torch.Tensor, n_per: int, k: int, mem_budget: int = 1 << 30) -> torch.Tensor:
    """x is grouped by component: rows [c * n_per, (c+1) * n_per) belong to component c.
    Returns [N, k] int64 neighbour ids (nearest first, self excluded)."""
    n = x.shape[0]
    comps = n // n_per
    k = min(k, n_per - 1)
    out = torch.empty((n, k), dtype=torch.int64, device=x.device)
    per = max(1, mem_budget // (n_per * n_per * 4 * 3))
    for c0 in range(0, comps, per):
        c1 = min(comps, c0 + per)
        xb = x[c0 * n_per:c1 * n_per].float().view(c1 - c0, n_per, -1)
        nrm = (xb * xb).sum(2)
        dist = nrm.unsqueeze(2) + nrm.unsqueeze(1) - 2.0 * torch.bmm(xb, xb.transpose(1, 2))
        dist.diagonal(dim1=1, dim2=2).fill_(float("inf"))
        idx = dist.topk(k, dim=2, largest=False).indices  # [b, n_per, k]
        base = (torch.arange(c0, c1, device=x.device) * n_per).view(-1, 1, 1)
        out[c0 * n_per:c1 * n_per] = (idx + base).view(-1, k)
    return out


def brute_force_topk(base: torch.Tensor, queries: torch.Tensor, k: int, batch: int = 0):
    """Exact top-k by (distance, id); returns ids [Q, k] int64 and squared distances [Q, k]."""
    Q = queries.shape[0]
    if batch <= 0:  # keep each [Q, batch] distance block near 512 MB
        batch = max(4096, (1 << 27) // max(Q, 1))
    dev = base.device
    best_d = torch.full((Q, k), float("inf"), device=dev)
    best_i = torch.full((Q, k), -1, dtype=torch.int64, device=dev)
    qf = queries.float()
    for s in range(0, base.shape[0], batch):
        d = _sqdist(qf, base[s:s + batch].float())
        kk = min(k, d.shape[1])
        dd, ii = d.topk(kk, dim=1, largest=False)
        cat_d = torch.cat([best_d, dd], 1)
        cat_i = torch.cat([best_i, ii + s], 1)
        order = torch.argsort(cat_d, dim=1, stable=True)[:, :k]
        best_d = cat_d.gather(1, order)
        best_i = cat_i.gather(1, order)
    return best_i, best_d


def build(cfg: SynthConfig, device="cpu") -> SynthIndex:
    dev = torch.device(device)
    if dev.type == "cuda":
        torch.backends.cuda.matmul.allow_tf32 = False
    gen = _gen(dev, cfg.seed)
    N, d = cfg.num_nodes, cfg.dim
    comps = max(1, min(cfg.components, N))
    n_per = N // comps
    N = n_per * comps  # equal-sized components
    if cfg.kind == "uint8":
        centres = torch.rand((comps, d), generator=gen, device=dev) * 255.0
    else:
        centres = torch.randn((comps, d), generator=gen, device=dev)
        centres = centres / centres.norm(dim=1, keepdim=True)
    basis = None
    if cfg.low_rank > 0:
        basis = torch.randn((min(comps, 64), cfg.low_rank, d), generator=gen, device=dev) / (d ** 0.5)
    out_dtype = torch.uint8 if cfg.kind == "uint8" else torch.float32
    grouped = torch.empty((N, d), dtype=out_dtype, device=dev)
    step = max(1, (1 << 22) // n_per) * n_per
    for s in range(0, N, step):
        e = min(N, s + step)
        comp_ids = torch.arange(s, e, device=dev) // n_per
        grouped[s:e] = _sample_component(cfg, centres, comp_ids, gen, basis).to(out_dtype)
    # graph in grouped order, then shuffle ids
    if N <= (1 << 25):
        knn = build_knn_graph(grouped, n_per, cfg.knn_edges)
        perm = torch.randperm(N, generator=gen, device=dev)          # new id of grouped row i
        rand_edges = torch.randint(0, N, (N, cfg.random_edges), generator=gen, device=dev)
        adjacency = torch.empty((N, knn.shape[1] + cfg.random_edges), dtype=torch.int32, device=dev)
        adjacency[perm] = torch.cat([perm[knn], rand_edges], 1).to(torch.int32)
        del knn, rand_edges
    else:
        # very large indices: the same construction in slices of whole components, so that the 64-bit
        # neighbour tables of a slice (not of the whole index) exist at any time
        perm = torch.randperm(N, generator=gen, device=dev)
        kk = min(cfg.knn_edges, n_per - 1)
        adjacency = torch.empty((N, kk + cfg.random_edges), dtype=torch.int32, device=dev)
        slice_rows = max(1, (1 << 22) // n_per) * n_per
        for b in range(0, N, slice_rows):
            e = min(N, b + slice_rows)
            knn = build_knn_graph(grouped[b:e], n_per, cfg.knn_edges) + b
            rnd = torch.randint(0, N, (e - b, cfg.random_edges), generator=gen, device=dev)
            adjacency[perm[b:e]] = torch.cat([perm[knn], rnd], 1).to(torch.int32)
            del knn, rnd
    vectors = torch.empty_like(grouped)
    if N <= (1 << 25):
        vectors[perm] = grouped
    else:
        for b in range(0, N, 1 << 24):
            vectors[perm[b:b + (1 << 24)]] = grouped[b:b + (1 << 24)]
    component_of = torch.empty(N, dtype=torch.int32, device=dev)
    component_of[perm] = (torch.arange(N, device=dev) // n_per).to(torch.int32)
    del grouped
    # PQ
    sample = torch.randperm(N, generator=gen, device=dev)[:min(N, cfg.train_sample)]
    xs = vectors[sample].float()
    tables, centroid, offs = train_pq(xs, cfg.pq_chunks, cfg.kmeans_iters, gen)
    codes = encode_pq(vectors, tables, centroid, offs)
    # queries from the same mixture
    qcomp = torch.randint(0, comps, (cfg.num_queries,), generator=gen, device=dev)
    queries = _sample_component(cfg, centres, qcomp, gen, basis).float()
    gt_ids, _ = brute_force_topk(vectors, queries, cfg.top_k)
    mean = xs.mean(0, keepdim=True)
    medoid = int(_sqdist(mean, xs).argmin(1).item())
    medoid = int(sample[medoid].item())
    idx = SynthIndex(cfg, vectors, adjacency, tables, centroid, offs, codes, queries, gt_ids, medoid)
    idx.extras["component_of"] = component_of
    idx.extras["query_component"] = qcomp
    idx.extras["centres"], idx.extras["basis"] = centres, basis
    if cfg.pq2:
        recon = torch.empty((N, d), dtype=torch.float32, device=dev) if N <= (1 << 24) else None
        res_sample = xs - decode_pq(codes[sample], tables, centroid, offs)
        t2, c2, _ = train_pq(res_sample, cfg.pq_chunks, cfg.kmeans_iters, gen)
        codes2 = torch.empty_like(codes)
        err = torch.empty(N, dtype=torch.float32, device=dev)
        for s in range(0, N, 262144):
            xb = vectors[s:s + 262144].float()
            r = xb - decode_pq(codes[s:s + 262144], tables, centroid, offs)
            codes2[s:s + 262144] = encode_pq(r, t2, c2, offs)
            r2 = decode_pq(codes2[s:s + 262144], t2, c2, offs)
            err[s:s + 262144] = (r - r2).norm(dim=1)   # |x - (b^ + r^)|_2, the reference's bound
        del recon
        idx.pq2_tables, idx.pq2_centroid, idx.pq2_codes, idx.pq2_error_bounds = t2, c2, codes2, err
    if cfg.rvq:
        coarse = kmeans(xs, min(cfg.rvq_coarse, xs.shape[0]), cfg.kmeans_iters, gen)
        ca = _sqdist(xs, coarse).argmin(1)
        fine = kmeans(xs - coarse[ca], min(cfg.rvq_fine, xs.shape[0]), cfg.kmeans_iters, gen)
        nc, nf = coarse.shape[0], fine.shape[0]
        cluster = torch.empty(N, dtype=torch.int64, device=dev)
        for s in range(0, N, 262144):
            xb = vectors[s:s + 262144].float()
            a = _sqdist(xb, coarse).argmin(1)
            f = _sqdist(xb - coarse[a], fine).argmin(1)
            cluster[s:s + 262144] = a * nf + f
        order = torch.argsort(cluster, stable=True)          # ascending id inside a bucket
        sizes = torch.bincount(cluster, minlength=nc * nf)
        starts = torch.cumsum(sizes, 0) - sizes
        rank_in_bucket = torch.arange(N, device=dev) - starts[cluster[order]]
        keep = rank_in_bucket < 256                           # posting lists capped at 256 ids
        capped = torch.clamp(sizes, max=256)
        offsets = torch.zeros(nc * nf + 1, dtype=torch.int64, device=dev)
        offsets[1:] = torch.cumsum(capped, 0)
        idx.rvq_coarse, idx.rvq_fine = coarse, fine
        idx.rvq_buckets = [sizes.to(torch.int32), offsets.to(torch.int32), order[keep].to(torch.int32)]
    return idx


def more_queries(cfg: SynthConfig, centres: torch.Tensor, count: int, seed: int, basis=None) -> torch.Tensor:
    """`count` further queries from the mixture an index was drawn from (its centres are kept in
    SynthIndex.extras["centres"]), from their own seeded stream; float32 [count, dim]."""
    gen = _gen(centres.device, seed)
    qcomp = torch.randint(0, centres.shape[0], (count,), generator=gen, device=centres.device)
    return _sample_component(cfg, centres, qcomp, gen, basis).float()


def recall_at_k(result_ids: np.ndarray, gt_ids: np.ndarray, k: int) -> float:
    """Reference definition (tools/topoanns_eval_sift.cpp:570-590): every returned id among the first
    k that is in the first k ground-truth ids counts, duplicates included."""
    hits = 0
    for r, g in zip(result_ids[:, :k], gt_ids[:, :k]):
        gs = set(int(x) for x in g)
        hits += sum(1 for x in r if int(x) in gs)
    return hits / float(result_ids.shape[0] * k)
