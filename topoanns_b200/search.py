"""Host side of the path over the C ABI, for Python callers (tests, benchmark, examples).

Device memory and streams come from torch; every computation is a call into
``libtopoanns_b200.so``. Names follow the reference's API: ``SearchResources``-like ``DeviceIndex``,
``TopologySearchParams`` / ``RerankExactParams`` fields, ``DeviceEntryBatch``-style CSR entries.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from . import capi

_KIND_OF_DTYPE = {torch.int8: capi.KIND_INT8, torch.uint8: capi.KIND_UINT8, torch.float32: capi.KIND_FLOAT32}
_NP_KIND = {"int8": capi.KIND_INT8, "uint8": capi.KIND_UINT8, "float32": capi.KIND_FLOAT32}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def make_shards(bases: Sequence[int], rows_per_shard: int = 0) -> capi.Shards:
    s = capi.Shards()
    s.num_shards = len(bases)
    s.rows_per_shard = rows_per_shard
    for i, b in enumerate(bases):
        s.base[i] = b
    return s


@dataclass
class TopologySearchParams:
    """include/topoanns/topology_search.hpp:17-32 (the fields this path uses)."""
    top_k: int = 10
    top_l: int = 32
    candidate_queue_size: int = 0
    search_width: int = 1
    max_expansions: int = 1024
    stop_prefix: int = 0          # 0 = top_l
    stop_use_expanded: bool = False
    learned_stop: Optional[capi.LearnedStop] = None

    def capacity(self, rerank_top_n: int = 0) -> int:
        return capi.candidate_capacity(self.top_l, self.candidate_queue_size, rerank_top_n)

    def to_c(self, capacity: int) -> capi.BeamParams:
        p = capi.BeamParams()
        p.top_l = self.top_l
        p.search_width = self.search_width
        p.max_expansions = self.max_expansions
        p.candidate_capacity = capacity
        p.stop_prefix = self.stop_prefix or self.top_l
        p.stop_use_expanded = int(self.stop_use_expanded)
        if self.learned_stop is not None:
            p.learned_stop = self.learned_stop
        return p


def load_learned_stop(path, top_l: int, top_k: int, shadow: bool = False) -> capi.LearnedStop:
    """Reads a learned traversal-stop model file (`key = value` lines: stage_prefixes, feature_means,
    feature_inv_stds, weights, bias, threshold_logit, top_k, topk_churn_mode, next64_mode, feature_mask,
    threshold_logit_top_l_<L>) and folds it for one top_l the way the reference does
    (src/search/topology_search_kernel.cu:248-380): weight_i / std_i per feature, the means folded into the bias,
    stages outside (0, top_l) dropped, the per-top_l threshold preferred."""
    vals = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            if "=" not in line:
                raise ValueError("LoadLearnedStopConfigFromFile: Invalid learned-stop config line: " + line)
            k, v = line.split("=", 1)
            vals[k.strip()] = v.strip()

    def floats(key):
        return [np.float32(x) for x in vals.get(key, "").split(",") if x.strip()]

    means, inv_stds, weights = floats("feature_means"), floats("feature_inv_stds"), floats("weights")
    if not (len(means) == len(inv_stds) == len(weights) == 12):
        raise ValueError("LoadLearnedStopConfigFromFile: learned-stop feature vectors must all have length 12.")
    mask = [int(x) for x in vals.get("feature_mask", "").split(",") if x.strip()]
    ls = capi.LearnedStop()
    ls.top_k = int(vals.get("top_k", "0")) or top_k
    ls.inv_top_l = float(np.float32(1.0) / np.float32(top_l)) if top_l else 0.0
    ls.shadow_mode = int(shadow)
    ls.topk_churn_flag_mode = int(vals.get("topk_churn_mode", "") == "flag")
    ls.next64_flag_mode = int(vals.get("next64_mode", "") == "flag")
    key = f"threshold_logit_top_l_{top_l}"
    ls.threshold_logit = float(np.float32(vals[key] if key in vals else vals.get("threshold_logit", "0")))
    bias = np.float32(vals.get("bias", "0"))
    for i in range(12):
        ls.feature_mask[i] = mask[i] if i < len(mask) else 1
        w = (weights[i] if ls.feature_mask[i] else np.float32(0.0)) * inv_stds[i]
        ls.weights[i] = float(w)
        bias = np.float32(bias - means[i] * w)
    ls.bias = float(bias)
    n = 0
    for pfx in (int(x) for x in vals.get("stage_prefixes", "").split(",") if x.strip()):
        if pfx == 0 or pfx >= top_l:
            continue
        if n >= 32:
            break
        ls.stage_prefixes[n] = pfx
        n += 1
    ls.num_stages = n
    ls.enabled = int(n > 0 and 0 < ls.top_k <= 32)
    return ls


@dataclass
class RerankExactParams:
    """include/topoanns/rerank_exact.hpp:21-37 (the fields this path uses)."""
    top_k: int = 10
    top_n: int = 100
    rank_tile_size: int = 0       # 0 = one tile (linear mode); 1 = page-by-page
    use_pq2_refine: bool = False
    use_pq2_bound_filter: bool = False
    pq2_refine_top_l: int = 0
    use_early_stop: bool = False
    early_stop_min_prefix: int = 32
    early_stop_patience_tiles: int = 1

    def to_c(self) -> capi.RerankParams:
        return capi.RerankParams(self.top_n, self.top_k, self.rank_tile_size, int(self.use_pq2_bound_filter),
                                 int(self.use_early_stop), self.early_stop_min_prefix, self.early_stop_patience_tiles, 0)


@dataclass
class DeviceIndex:
    """What SearchResources hands to the kernels, as torch tensors on one device (or views of
    peer / mapped-host memory given as raw base pointers in ``*_bases``)."""
    num_nodes: int
    degree: int
    dim: int
    vector_kind: int
    adjacency: Optional[torch.Tensor] = None      # [N, degree] int32 (bit pattern of uint32)
    codes: Optional[torch.Tensor] = None          # [N, M] uint8
    vector_pages: Optional[torch.Tensor] = None   # uint8, page layout without the file header
    pq_tables_col_major: Optional[torch.Tensor] = None   # [dim, 256] f32
    pq_centroid: Optional[torch.Tensor] = None
    pq_chunk_offsets: Optional[torch.Tensor] = None      # [M+1] int32
    vector_bytes: int = 0
    vectors_per_page: int = 0
    page_bytes: int = 4096
    # several shards: raw base pointers + rows per shard replace the single tensors above
    adjacency_bases: Optional[Sequence[int]] = None
    codes_bases: Optional[Sequence[int]] = None
    vector_bases: Optional[Sequence[int]] = None
    rows_per_shard: int = 0
    adjacency_cache: Optional[torch.Tensor] = None
    adjacency_cached_rows: int = 0
    # optional [N, degree, M] uint8: every node's neighbours' PQ codes in adjacency order (see inline_neighbor_codes)
    neighbor_codes: Optional[torch.Tensor] = None
    neighbor_codes_bases: Optional[Sequence[int]] = None
    keepalive: list = field(default_factory=list)

    @property
    def num_chunks(self) -> int:
        return int(self.pq_chunk_offsets.numel()) - 1

    def view(self) -> capi.IndexView:
        v = capi.IndexView()
        v.num_nodes = self.num_nodes
        v.degree = self.degree
        v.num_chunks = self.num_chunks
        v.dim = self.dim
        v.vector_kind = self.vector_kind
        v.vector_bytes = self.vector_bytes
        v.vectors_per_page = self.vectors_per_page
        v.page_bytes = self.page_bytes
        v.adjacency = make_shards(self.adjacency_bases or [self.adjacency.data_ptr()], self.rows_per_shard)
        v.codes = make_shards(self.codes_bases or [self.codes.data_ptr()], self.rows_per_shard)
        if self.vector_bases or self.vector_pages is not None:
            v.vectors = make_shards(self.vector_bases or [self.vector_pages.data_ptr()], self.rows_per_shard)
        if self.adjacency_cache is not None:
            v.adjacency_cache = self.adjacency_cache.data_ptr()
            v.adjacency_cached_rows = self.adjacency_cached_rows
        v.pq_tables_col_major = self.pq_tables_col_major.data_ptr()
        v.pq_centroid = self.pq_centroid.data_ptr()
        v.pq_chunk_offsets = self.pq_chunk_offsets.data_ptr()
        if self.neighbor_codes_bases or self.neighbor_codes is not None:
            v.neighbor_codes = make_shards(self.neighbor_codes_bases or [self.neighbor_codes.data_ptr()], self.rows_per_shard)
        return v


def inline_neighbor_codes(index: DeviceIndex) -> DeviceIndex:
    """Adds the neighbour-code layout to an index held by this device: neighbor_codes[n, j] = codes[adjacency[n, j]]
    (zeros for padding slots), built by the library's gather kernel. degree * M bytes per node; the search
    results do not change."""
    dev = index.pq_centroid.device
    out = torch.empty((index.num_nodes, index.degree, index.num_chunks), dtype=torch.uint8, device=dev)
    view = index.view()
    capi.check(capi.load().tann_neighbor_codes_build(C.byref(view), 0, index.num_nodes, _ptr(out), _stream_ptr()))
    index.neighbor_codes = out
    return index


def kind_of(t: torch.Tensor) -> int:
    return _KIND_OF_DTYPE[t.dtype]


def lut_build(index: DeviceIndex, queries: torch.Tensor, *, tables_col_major=None, centroid=None,
              chunk_offsets=None) -> torch.Tensor:
    """PqQueryDistanceTables::From*Queries: returns the device tables [Q, M, 256]."""
    t = index.pq_tables_col_major if tables_col_major is None else tables_col_major
    c = index.pq_centroid if centroid is None else centroid
    o = index.pq_chunk_offsets if chunk_offsets is None else chunk_offsets
    Q = queries.shape[0]
    M = o.numel() - 1
    out = torch.empty((Q, M, 256), dtype=torch.float32, device=queries.device)
    capi.check(capi.load().tann_lut_build(_ptr(t), _ptr(c), _ptr(o), index.dim, M, _ptr(queries),
                                          kind_of(queries), Q, _ptr(out), _stream_ptr()))
    return out


def beam_search(index: DeviceIndex, params: TopologySearchParams, entry_offsets: torch.Tensor,
                entry_ids: torch.Tensor, *, lut: Optional[torch.Tensor] = None,
                queries: Optional[torch.Tensor] = None, capacity: Optional[int] = None,
                status: Optional[torch.Tensor] = None):
    """Returns (candidates [Q, C, 2] int32 {dist bits, packed id}, stats [Q, 8] int32). `status`: an int32 device
    tensor of one element the kernel ors its TANN_STATUS_* bits into (ids outside the index are skipped)."""
    Q = entry_offsets.numel() - 1
    cap = capacity or params.capacity()
    dev = entry_offsets.device
    cand = torch.empty((Q, cap, 2), dtype=torch.int32, device=dev)
    stats = torch.empty((Q, 8), dtype=torch.int32, device=dev)
    view = index.view()
    p = params.to_c(cap)
    capi.check(capi.load().tann_beam_search(
        C.byref(view), C.byref(p), _ptr(lut), _ptr(queries),
        kind_of(queries) if queries is not None else capi.KIND_FLOAT32, Q, _ptr(entry_offsets),
        _ptr(entry_ids), _ptr(cand), _ptr(stats), _ptr(status), _stream_ptr()))
    return cand, stats


def beam_occupancy(index: DeviceIndex, params: TopologySearchParams, capacity: Optional[int] = None):
    view = index.view()
    p = params.to_c(capacity or params.capacity())
    smem, bps, grid = C.c_uint32(), C.c_uint32(), C.c_uint32()
    capi.check(capi.load().tann_beam_search_occupancy(C.byref(view), C.byref(p), 1, C.byref(smem),
                                                     C.byref(bps), C.byref(grid)))
    return smem.value, bps.value, grid.value


@dataclass
class RvqModel:
    """RvqModel of the reference (include/topoanns/rvq_entry_provider.hpp:21-58) on the device."""
    dim: int
    coarse: torch.Tensor          # [nc, dim]
    fine: torch.Tensor            # [nf, dim]
    bucket_sizes: torch.Tensor    # [nc * nf] int32, uncapped
    cluster_offsets: torch.Tensor  # [nc * nf + 1] int32, lists capped at 256 ids
    cluster_ids: torch.Tensor
    coarse_t: torch.Tensor = None
    fine_t: torch.Tensor = None
    coarse_norms: torch.Tensor = None
    fine_norms: torch.Tensor = None

    def __post_init__(self):
        lib = capi.load()
        self.coarse_t = self.coarse.t().contiguous()
        self.fine_t = self.fine.t().contiguous()
        self.coarse_norms = torch.empty(self.coarse.shape[0], dtype=torch.float32, device=self.coarse.device)
        self.fine_norms = torch.empty(self.fine.shape[0], dtype=torch.float32, device=self.fine.device)
        capi.check(lib.tann_rvq_norms(_ptr(self.coarse), self.coarse.shape[0], self.dim,
                                      _ptr(self.coarse_norms), _stream_ptr()))
        capi.check(lib.tann_rvq_norms(_ptr(self.fine), self.fine.shape[0], self.dim,
                                      _ptr(self.fine_norms), _stream_ptr()))

    def view(self, entry_count: int, fallback_entry: int = 0) -> capi.RvqModelView:
        v = capi.RvqModelView()
        v.dim, v.num_coarse, v.num_fine = self.dim, self.coarse.shape[0], self.fine.shape[0]
        v.entry_count, v.fallback_entry = entry_count, fallback_entry
        v.coarse, v.coarse_t, v.coarse_norms = self.coarse.data_ptr(), self.coarse_t.data_ptr(), self.coarse_norms.data_ptr()
        v.fine_t, v.fine_norms = self.fine_t.data_ptr(), self.fine_norms.data_ptr()
        v.bucket_sizes = self.bucket_sizes.data_ptr()
        v.cluster_offsets, v.cluster_ids = self.cluster_offsets.data_ptr(), self.cluster_ids.data_ptr()
        return v

    def device_entry_batch(self, queries: torch.Tensor, entry_count: int, fallback_entry: int = 0):
        """RvqModel::ComputeFloat32DeviceEntryBatch: (offsets [Q+1], ids [Q, entry_count], clusters [Q])."""
        if entry_count <= 0:
            raise capi.TannError(1, "RvqModel::ComputeFloat32DeviceEntryBatch: entry_count must be positive.")
        Q = queries.shape[0]
        dev = queries.device
        offsets = torch.empty(Q + 1, dtype=torch.int32, device=dev)
        ids = torch.empty((Q, entry_count), dtype=torch.int32, device=dev)
        clusters = torch.empty(Q, dtype=torch.int32, device=dev)
        capi.check(capi.load().tann_rvq_entries(
            _ptr(queries), Q, self.dim, _ptr(self.coarse), _ptr(self.coarse_t), _ptr(self.coarse_norms),
            self.coarse.shape[0], _ptr(self.fine_t), _ptr(self.fine_norms), self.fine.shape[0],
            _ptr(self.bucket_sizes), _ptr(self.cluster_offsets), _ptr(self.cluster_ids), entry_count,
            fallback_entry, _ptr(clusters), _ptr(ids), _ptr(offsets), _stream_ptr()))
        return offsets, ids, clusters


def pq2_cross_terms(chunk_offsets, t1_row_major, mu1, t2_row_major, mu2) -> torch.Tensor:
    M = chunk_offsets.numel() - 1
    d = t1_row_major.shape[1]
    out = torch.empty((M, 256, 256), dtype=torch.float32, device=t1_row_major.device)
    capi.check(capi.load().tann_pq2_cross_terms(d, M, _ptr(chunk_offsets), _ptr(t1_row_major), _ptr(mu1),
                                                _ptr(t2_row_major), _ptr(mu2), _ptr(out), _stream_ptr()))
    return out


def pq2_refine(cand, stats, refine_top_l, pq2_codes, lut2, base_codes=None, cross_terms=None):
    Q, capacity, _ = cand.shape
    M = pq2_codes.shape[1]
    out = torch.empty((Q, refine_top_l, 2), dtype=torch.int32, device=cand.device)
    p2 = make_shards([pq2_codes.data_ptr()])
    b = make_shards([base_codes.data_ptr()]) if base_codes is not None else None
    capi.check(capi.load().tann_pq2_refine(
        _ptr(cand), _ptr(stats), Q, capacity, refine_top_l, C.byref(b) if b is not None else None,
        C.byref(p2), M, _ptr(lut2), _ptr(cross_terms), _ptr(out), None, _stream_ptr()))
    return out


def hpq_refine(cand, stats, refine_top_l, hybrid_codes, selector_bits, base_lut, outlier_lut):
    """Hybrid-PQ refine and re-sort (detail::RunHpqRefineBatchDevice, src/search/rerank_exact.cu:2457-2531):
    hybrid_codes [N, M] uint8, selector_bits [N, (M + 7) // 8] uint8, the two query tables [Q, M, 256]."""
    Q, capacity, _ = cand.shape
    M = hybrid_codes.shape[1]
    out = torch.empty((Q, refine_top_l, 2), dtype=torch.int32, device=cand.device)
    codes = make_shards([hybrid_codes.data_ptr()])
    capi.check(capi.load().tann_hpq_refine(_ptr(cand), _ptr(stats), Q, capacity, refine_top_l, C.byref(codes),
                                           _ptr(selector_bits), M, _ptr(base_lut), _ptr(outlier_lut), _ptr(out), None,
                                           _stream_ptr()))
    return out


def rerank_exact(index: DeviceIndex, params: RerankExactParams, cand: torch.Tensor, queries: torch.Tensor,
                 error_bounds: Optional[torch.Tensor] = None):
    """Returns (dists [Q, top_n] f32, ids [Q, top_n] int32, n_exact, n_filtered)."""
    Q, capacity, _ = cand.shape
    dev = cand.device
    dists = torch.empty((Q, params.top_n), dtype=torch.float32, device=dev)
    ids = torch.empty((Q, params.top_n), dtype=torch.int32, device=dev)
    counts = torch.zeros(2, dtype=torch.int64, device=dev)
    view = index.view()
    p = params.to_c()
    capi.check(capi.load().tann_rerank_exact(C.byref(view), C.byref(p), _ptr(cand), capacity, Q, _ptr(queries),
                                             kind_of(queries), _ptr(error_bounds), _ptr(dists), _ptr(ids),
                                             _ptr(counts), None, _stream_ptr()))
    c = counts.cpu()
    return dists, ids, int(c[0]), int(c[1])


def load_rerank_learned_stop(path, budget_top_n: int, top_k: int) -> capi.RerankLearnedStop:
    """Reads a learned rerank-stop model file and folds it for a budget of budget_top_n ranks
    (LoadRerankLearnedStopConfigFromFile, src/io/bam_vector_provider.cu:125-279)."""
    model = capi.RerankLearnedStop()
    capi.check(capi.load().tann_rerank_learned_stop_load(str(path).encode(), budget_top_n, top_k, C.byref(model)))
    return model


def rerank_exact_learned_stop(index: DeviceIndex, params: RerankExactParams, cand: torch.Tensor,
                              queries: torch.Tensor, model: Optional[capi.RerankLearnedStop] = None,
                              replay_stop_prefixes: Optional[torch.Tensor] = None,
                              error_bounds: Optional[torch.Tensor] = None):
    """The reference's persistent rerank (src/io/bam_vector_provider.cu:721-1323): top_k list per query,
    learned stage schedule and stop, or stop-prefix replay. Returns a dict: dists / ids [Q, top_k],
    stop_prefixes / checkpoint_counts / stop_flags [Q] (device tensors), n_exact, n_filtered."""
    Q, capacity, _ = cand.shape
    dev = cand.device
    dists = torch.empty((Q, params.top_k), dtype=torch.float32, device=dev)
    ids = torch.empty((Q, params.top_k), dtype=torch.int32, device=dev)
    counts = torch.zeros(2, dtype=torch.int64, device=dev)
    stop_prefixes = torch.zeros(Q, dtype=torch.int32, device=dev)
    checkpoints = torch.zeros(Q, dtype=torch.int32, device=dev)
    flags = torch.zeros(Q, dtype=torch.int32, device=dev)
    view = index.view()
    p = params.to_c()
    capi.check(capi.load().tann_rerank_exact_learned_stop(
        C.byref(view), C.byref(p), C.byref(model) if model is not None else None, _ptr(cand), capacity, Q,
        _ptr(queries), kind_of(queries), _ptr(error_bounds), _ptr(replay_stop_prefixes), _ptr(dists), _ptr(ids),
        _ptr(counts), _ptr(stop_prefixes), _ptr(checkpoints), _ptr(flags), None, _stream_ptr()))
    c = counts.cpu()
    return dict(dists=dists, ids=ids, stop_prefixes=stop_prefixes, checkpoint_counts=checkpoints, stop_flags=flags,
                n_exact=int(c[0]), n_filtered=int(c[1]))


def topk_pack(dists, ids, top_k):
    Q, top_n = dists.shape
    od = torch.empty((Q, top_k), dtype=torch.float32, device=dists.device)
    oi = torch.empty((Q, top_k), dtype=torch.int32, device=dists.device)
    capi.check(capi.load().tann_topk_pack(_ptr(dists), _ptr(ids), Q, top_n, top_k, _ptr(od), _ptr(oi), _stream_ptr()))
    return od, oi


@dataclass
class Pq2Resources:
    codes: torch.Tensor
    tables_col_major: torch.Tensor
    centroid: torch.Tensor
    chunk_offsets: torch.Tensor
    cross_terms: Optional[torch.Tensor] = None     # given = residual refine
    error_bounds: Optional[torch.Tensor] = None


class Searcher:
    """The whole path behind one call (TopoAnnsSearch::RunBatchFloat32Fused), host buffers in and out."""

    def __init__(self, index: DeviceIndex, max_queries: int, max_capacity: int, max_top_n: int,
                 max_entries: int = 256):
        self.index = index
        self._view = index.view()
        self._h = C.c_void_p()
        capi.check(capi.load().tann_searcher_create(C.byref(self._view), max_queries, max_capacity, max_top_n,
                                                    max_entries, C.byref(self._h)))
        self._keep = []

    def set_rvq(self, model: RvqModel, entry_count: int, fallback_entry: int = 0):
        v = model.view(entry_count, fallback_entry)
        self._keep.append(model)
        capi.check(capi.load().tann_searcher_set_rvq(self._h, C.byref(v)))

    def set_pq2(self, pq2: Pq2Resources, refine_top_l: int = 0):
        v = capi.Pq2View()
        v.enabled = 1
        v.residual = int(pq2.cross_terms is not None)
        v.refine_top_l = refine_top_l
        v.codes = make_shards([pq2.codes.data_ptr()])
        v.tables_col_major = pq2.tables_col_major.data_ptr()
        v.centroid = pq2.centroid.data_ptr()
        v.chunk_offsets = pq2.chunk_offsets.data_ptr()
        v.cross_terms = pq2.cross_terms.data_ptr() if pq2.cross_terms is not None else None
        v.error_bounds = pq2.error_bounds.data_ptr() if pq2.error_bounds is not None else None
        self._keep.append(pq2)
        capi.check(capi.load().tann_searcher_set_pq2(self._h, C.byref(v)))

    def run_host(self, queries: np.ndarray, topology: TopologySearchParams, rerank: RerankExactParams,
                 fixed_entries: Optional[np.ndarray] = None, want_stats: bool = False,
                 out_ids: Optional[np.ndarray] = None, out_dists: Optional[np.ndarray] = None):
        """queries: numpy [Q, dim] (float32 / uint8 / int8). Returns (ids [Q,k] u32, dists [Q,k] f32, stats).
        Page-locked query / output arrays (e.g. views of torch pinned tensors) are copied without staging."""
        q = np.ascontiguousarray(queries)
        Q = q.shape[0]
        ids = out_ids if out_ids is not None else np.empty((Q, rerank.top_k), np.uint32)
        dists = out_dists if out_dists is not None else np.empty((Q, rerank.top_k), np.float32)
        assert ids.shape == (Q, rerank.top_k) and ids.dtype == np.uint32 and ids.flags.c_contiguous
        assert dists.shape == (Q, rerank.top_k) and dists.dtype == np.float32 and dists.flags.c_contiguous
        stats = np.empty((Q, 8), np.uint32) if want_stats else None
        cap = topology.capacity(rerank.top_n)
        bp = topology.to_c(cap)
        rp = rerank.to_c()
        fe = np.ascontiguousarray(fixed_entries, dtype=np.uint32) if fixed_entries is not None else None
        capi.check(capi.load().tann_searcher_run(
            self._h, C.byref(bp), C.byref(rp), q.ctypes.data_as(C.c_void_p), _NP_KIND[str(q.dtype)], Q,
            fe.ctypes.data_as(C.c_void_p) if fe is not None else None, 0 if fe is None else fe.size,
            ids.ctypes.data_as(C.c_void_p), dists.ctypes.data_as(C.c_void_p),
            stats.ctypes.data_as(C.c_void_p) if stats is not None else None, _stream_ptr()))
        return ids, dists, stats

    def set_rerank_learned_stop(self, model: Optional[capi.RerankLearnedStop]):
        """Reranks of this searcher use the persistent rerank with this learned-stop model (None: plain rerank)."""
        capi.check(capi.load().tann_searcher_set_rerank_learned_stop(
            self._h, C.byref(model) if model is not None else None))

    def submit_host(self, queries: np.ndarray, topology: TopologySearchParams, rerank: RerankExactParams,
                    out_ids: np.ndarray, out_dists: np.ndarray, stream: Optional[torch.cuda.Stream] = None):
        """First half of run_host: enqueues copy-in, kernels and copy-out on `stream` (default: the current
        stream) and returns at once; wait() completes the batch. Two searchers submitted alternately on two
        streams overlap one batch's copies with the other's kernels. The arrays must stay alive until wait()."""
        q = queries
        assert q.flags.c_contiguous and out_ids.flags.c_contiguous and out_dists.flags.c_contiguous
        Q = q.shape[0]
        assert out_ids.shape == (Q, rerank.top_k) and out_ids.dtype == np.uint32
        assert out_dists.shape == (Q, rerank.top_k) and out_dists.dtype == np.float32
        bp = topology.to_c(topology.capacity(rerank.top_n))
        rp = rerank.to_c()
        sp = C.c_void_p(stream.cuda_stream) if stream is not None else _stream_ptr()
        self._in_flight = (q, out_ids, out_dists)
        capi.check(capi.load().tann_searcher_submit(
            self._h, C.byref(bp), C.byref(rp), q.ctypes.data_as(C.c_void_p), _NP_KIND[str(q.dtype)], Q, None, 0,
            out_ids.ctypes.data_as(C.c_void_p), out_dists.ctypes.data_as(C.c_void_p), None, sp))

    def wait(self):
        capi.check(capi.load().tann_searcher_wait(self._h))
        self._in_flight = None

    def run_device(self, queries: torch.Tensor, topology: TopologySearchParams, rerank: RerankExactParams,
                   entry_offsets: Optional[torch.Tensor] = None, entry_ids: Optional[torch.Tensor] = None):
        """Device queries in; returns raw device pointers (ids, dists, stats) owned by the searcher."""
        Q = queries.shape[0]
        cap = topology.capacity(rerank.top_n)
        bp = topology.to_c(cap)
        rp = rerank.to_c()
        oi, od, os_ = C.c_void_p(), C.c_void_p(), C.c_void_p()
        capi.check(capi.load().tann_searcher_run_device(
            self._h, C.byref(bp), C.byref(rp), _ptr(queries), kind_of(queries), Q, _ptr(entry_offsets),
            _ptr(entry_ids), C.byref(oi), C.byref(od), C.byref(os_), _stream_ptr()))
        return oi.value, od.value, os_.value

    def close(self):
        if self._h:
            capi.load().tann_searcher_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def device_index_from_arrays(*, adjacency, codes, vectors, pq_tables_row_major, pq_centroid, pq_chunk_offsets,
                             device="cuda", page_bytes: int = 4096) -> DeviceIndex:
    """Build an HBM-resident DeviceIndex from host (numpy or torch) arrays in the file layouts:
    adjacency [N, degree] uint32/int32, codes [N, M] uint8, vectors [N, d], pivots [256, d]."""
    from . import formats

    def t(a, dtype=None):
        if isinstance(a, np.ndarray):
            if a.dtype == np.uint32:
                a = a.view(np.int32)
            a = torch.from_numpy(np.ascontiguousarray(a))
        if dtype is not None:
            a = a.to(dtype)
        return a.to(device).contiguous()

    vec_np = vectors.detach().cpu().numpy() if isinstance(vectors, torch.Tensor) else np.asarray(vectors)
    layout = formats.VectorPageLayout(vec_np.shape[1] * vec_np.dtype.itemsize, page_bytes)
    pages = torch.from_numpy(formats.vectors_to_pages(vec_np, page_bytes)).to(device)
    tables = t(pq_tables_row_major, torch.float32)
    adj = t(adjacency)
    if adj.dtype != torch.int32:
        adj = adj.to(torch.int32)
    return DeviceIndex(
        num_nodes=adj.shape[0], degree=adj.shape[1], dim=vec_np.shape[1],
        vector_kind=_NP_KIND[str(vec_np.dtype)], adjacency=adj, codes=t(codes, torch.uint8),
        vector_pages=pages, pq_tables_col_major=tables.t().contiguous(), pq_centroid=t(pq_centroid, torch.float32),
        pq_chunk_offsets=t(pq_chunk_offsets).to(torch.int32), vector_bytes=layout.vector_bytes,
        vectors_per_page=layout.vectors_per_page, page_bytes=page_bytes)


def device_index_from_synth(s, device="cuda") -> DeviceIndex:
    if isinstance(s.vectors, torch.Tensor) and s.vectors.is_cuda and torch.device(device).type == "cuda":
        # everything already lives on the device: lay the vector pages out there, no trip through host memory
        from . import sharding
        vb = s.vectors.shape[1] * s.vectors.element_size()
        adj = s.adjacency if s.adjacency.dtype == torch.int32 else s.adjacency.to(torch.int32)
        return DeviceIndex(
            num_nodes=adj.shape[0], degree=adj.shape[1], dim=s.vectors.shape[1], vector_kind=kind_of(s.vectors),
            adjacency=adj.contiguous(), codes=s.pq_codes.contiguous(), vector_pages=sharding.pages_from_rows(s.vectors),
            pq_tables_col_major=s.pq_tables.float().t().contiguous(), pq_centroid=s.pq_centroid.float().contiguous(),
            pq_chunk_offsets=s.pq_chunk_offsets.to(torch.int32).contiguous(), vector_bytes=vb,
            vectors_per_page=4096 // vb, page_bytes=4096)
    return device_index_from_arrays(adjacency=s.adjacency, codes=s.pq_codes, vectors=s.vectors,
                                    pq_tables_row_major=s.pq_tables, pq_centroid=s.pq_centroid,
                                    pq_chunk_offsets=s.pq_chunk_offsets, device=device)


def rvq_model_from_synth(s, device="cuda") -> RvqModel:
    sizes, offsets, ids = s.rvq_buckets
    return RvqModel(dim=s.cfg.dim, coarse=s.rvq_coarse.to(device).contiguous(),
                    fine=s.rvq_fine.to(device).contiguous(), bucket_sizes=sizes.to(device),
                    cluster_offsets=offsets.to(device), cluster_ids=ids.to(device))
