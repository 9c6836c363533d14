"""Partitioning of the path over the GPUs of one box (one process per GPU).

* Replicated index, queries sharded: rank r owns queries [r*Q/G, (r+1)*Q/G); no communication while
  searching; the final top-k lists go to one rank with a single gather.
* Node-id-range shards (indices larger than one GPU): node n lives on rank n // rows_per_shard;
  adjacency, codes and vector pages are split by the same ranges and every rank maps its peers'
  shard buffers (CUDA IPC), so the search kernel reads remote rows with ordinary loads over NVLink.
  Queries stay sharded by rank, so the gather above is still the only collective.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

from . import capi


def query_shard(num_queries: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous query range of `rank` (sizes differ by at most one)."""
    base, extra = divmod(num_queries, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def rows_per_shard(num_nodes: int, world_size: int, vectors_per_page: int = 1) -> int:
    """Nodes per shard, rounded up so that a vector page never straddles two shards."""
    rows = (num_nodes + world_size - 1) // world_size
    vpp = max(1, vectors_per_page)
    return (rows + vpp - 1) // vpp * vpp


def gather_topk(ids: torch.Tensor, dists: torch.Tensor, num_queries: int, dst: int = 0):
    """One gather of the per-rank [Q_r, k] id / distance lists to `dst`; returns the [Q, k] lists there
    (None elsewhere). Shards are padded to the largest shard so a single collective suffices."""
    world, rank = dist.get_world_size(), dist.get_rank()
    k = ids.shape[1]
    longest = max(query_shard(num_queries, world, r)[1] - query_shard(num_queries, world, r)[0] for r in range(world))
    packed = torch.full((longest, 2 * k), -1, dtype=torch.int32, device=ids.device)
    n = ids.shape[0]
    packed[:n, :k] = ids.to(torch.int32)
    packed[:n, k:] = dists.contiguous().view(torch.int32)
    out = [torch.empty_like(packed) for _ in range(world)] if rank == dst else None
    dist.gather(packed, out, dst=dst)
    if rank != dst:
        return None, None
    all_ids, all_d = [], []
    for r, t in enumerate(out):
        b, e = query_shard(num_queries, world, r)
        all_ids.append(t[: e - b, :k])
        all_d.append(t[: e - b, k:].contiguous().view(torch.float32))
    return torch.cat(all_ids), torch.cat(all_d)


class PeerBuffers:
    """One shard buffer per rank for one array, allocated through the C ABI and mapped into every rank."""

    def __init__(self, local_bytes: int):
        self.lib = capi.load()
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        ptr = C.c_void_p()
        capi.check(self.lib.tann_device_alloc(max(local_bytes, 256), C.byref(ptr)))
        self.local = ptr.value
        handle = C.create_string_buffer(capi.IPC_HANDLE_BYTES)
        capi.check(self.lib.tann_ipc_export(C.c_void_p(self.local), handle))
        mine = torch.tensor(list(handle.raw), dtype=torch.uint8, device="cuda")
        every = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(every, mine)
        self.bases: List[int] = []
        self._opened = []
        for r, h in enumerate(every):
            if r == self.rank:
                self.bases.append(self.local)
                continue
            p = C.c_void_p()
            capi.check(self.lib.tann_ipc_open(bytes(h.cpu().numpy().tobytes()), C.byref(p)))
            self.bases.append(p.value)
            self._opened.append(p.value)

    def local_tensor(self, nbytes: int) -> torch.Tensor:
        """uint8 view of the local shard (for filling it with torch ops)."""
        return _tensor_from_ptr(self.local, nbytes)

    def close(self):
        dist.barrier()
        for p in self._opened:
            self.lib.tann_ipc_close(C.c_void_p(p))
        self._opened = []
        dist.barrier()
        if self.local:
            self.lib.tann_device_free(C.c_void_p(self.local))
            self.local = 0


def _tensor_from_ptr(ptr: int, nbytes: int) -> torch.Tensor:
    """Wrap raw device memory as a uint8 torch tensor through the CUDA array interface."""

    class _Holder:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}

    return torch.as_tensor(_Holder(), device="cuda")


def pages_from_rows(rows: torch.Tensor, page_bytes: int = 4096) -> torch.Tensor:
    """[n, d] device tensor -> flat uint8 page array in the vector-store page layout."""
    n = rows.shape[0]
    raw = rows.contiguous().view(torch.uint8).view(n, -1)
    vb = raw.shape[1]
    vpp = page_bytes // vb
    pages = torch.zeros(((n + vpp - 1) // vpp, page_bytes), dtype=torch.uint8, device=rows.device)
    full = (n // vpp) * vpp
    if full:
        pages[: n // vpp, : vpp * vb] = raw[:full].view(n // vpp, vpp * vb)
    if n > full:
        pages[n // vpp, : (n - full) * vb] = raw[full:].reshape(-1)
    return pages.view(-1)


def peer_index_from_sharded(sh):
    """Put this rank's shard of a synth_sharded.ShardedSynth into IPC-shared device buffers and return a
    search.DeviceIndex whose adjacency / code / vector rows resolve to local or peer memory.
    Returns (index, buffers); keep `buffers` alive and close() them after the last search."""
    from . import search
    dev = sh.vectors.device
    vec_pages = pages_from_rows(sh.vectors)
    parts = {"adjacency": sh.adjacency.contiguous().view(torch.uint8).view(-1),
             "codes": sh.pq_codes.contiguous().view(-1), "vectors": vec_pages}
    buffers, bases = {}, {}
    for name, t in parts.items():
        pb = PeerBuffers(t.numel())
        pb.local_tensor(t.numel()).copy_(t)
        buffers[name] = pb
        bases[name] = pb.bases
    torch.cuda.synchronize()
    dist.barrier()
    vb = sh.vectors.shape[1] * sh.vectors.element_size()
    ix = search.DeviceIndex(
        num_nodes=sh.total_nodes, degree=sh.adjacency.shape[1], dim=sh.vectors.shape[1],
        vector_kind=search.kind_of(sh.vectors), pq_tables_col_major=sh.pq_tables.t().contiguous(),
        pq_centroid=sh.pq_centroid.contiguous(), pq_chunk_offsets=sh.pq_chunk_offsets.to(torch.int32).contiguous(),
        vector_bytes=vb, vectors_per_page=4096 // vb, page_bytes=4096, adjacency_bases=bases["adjacency"],
        codes_bases=bases["codes"], vector_bases=bases["vectors"], rows_per_shard=sh.rows_per_shard,
        keepalive=[buffers])
    _ = dev
    return ix, buffers


class _CudaOwnerOps:
    """The three device steps of OwnerRerank through the C ABI, on the current CUDA stream."""

    def __init__(self, local_index):
        from . import search
        self._kind_of = search.kind_of
        self._view = local_index.view()
        self.device = local_index.pq_centroid.device
        self.dim = local_index.dim

    @staticmethod
    def _p(t):
        return C.c_void_p(t.data_ptr())

    @staticmethod
    def _stream():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def partition(self, cand, top_n, rows, owners, slot, out, overflow):
        capi.check(capi.load().tann_partition_candidates(self._p(cand), int(cand.shape[1]), top_n, int(cand.shape[0]), rows,
                                                         owners, slot, self._p(out), self._p(overflow), self._stream()))

    def rerank_topk(self, lists, queries, slot, top_k, dists, ids, out_d, out_i):
        lib, n = capi.load(), int(queries.shape[0]) * int(queries.shape[1])
        params = capi.RerankParams(slot, top_k, 0, 0, 0, 0, 0, 0)
        capi.check(lib.tann_rerank_exact(C.byref(self._view), C.byref(params), self._p(lists), slot, n, self._p(queries),
                                         self._kind_of(queries), None, self._p(dists), self._p(ids), None, None,
                                         self._stream()))
        capi.check(lib.tann_topk_pack(self._p(dists), self._p(ids), n, slot, top_k, self._p(out_d), self._p(out_i),
                                      self._stream()))

    def merge(self, lists_d, lists_i, rows, out_d, out_i):
        W, Q, k = (int(x) for x in lists_d.shape)
        capi.check(capi.load().tann_merge_topk_lists(self._p(lists_d), self._p(lists_i), W, Q, k, rows, self._p(out_d),
                                                     self._p(out_i), self._stream()))


class OwnerRerank:
    """Exact rerank by the owner of the rows, for an index sharded by node-id range (one process per GPU).

    Reading candidates' vectors from the peers' shards is one random access into another GPU's memory per
    candidate; over shards of tens of GB those accesses spread over hundreds of GB of peer address space and
    their rate collapses. Here the candidates travel instead: every rank splits its queries' candidate lists by
    owner (`tann_partition_candidates`), one all-to-all hands every owner its lists, the owner scores them against
    its own shard (`tann_rerank_exact` + `tann_topk_pack` on a view of that shard alone), a second all-to-all
    returns the [Q, k] lists and `tann_merge_topk_lists` merges them by (distance, global id). The result is the
    unsharded one bit for bit. Every rank must call `run` with the same number of queries.

    `local_index` is a `search.DeviceIndex` over this rank's shard only (num_nodes = rows_per_shard, one base per
    array). `slot` is the room per (query, owner) list; 0 picks twice the even share plus 32, at most top_n. A list
    that outgrows its slot sets a flag that `overflowed()` reads back (the results of that call are then short of
    some candidates: build a new object with slot = top_n, which cannot overflow). `ops` replaces the three device
    steps (the CPU tests of the exchange pass plain torch code); by default they are the library's kernels."""

    def __init__(self, local_index, rows_per_shard: int, max_queries: int, top_n: int, top_k: int,
                 query_dtype: torch.dtype, slot: int = 0, group=None, ops=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows = int(rows_per_shard)
        self.top_n, self.top_k = int(top_n), int(top_k)
        if slot <= 0:
            slot = 2 * ((top_n + self.world - 1) // self.world) + 32
        self.slot = max(self.top_k, min(int(slot), self.top_n))
        self.ops = ops if ops is not None else _CudaOwnerOps(local_index)
        W, Q, dev = self.world, int(max_queries), self.ops.device
        self.max_queries = Q
        self.send = torch.empty((W, Q, self.slot, 2), dtype=torch.int32, device=dev)
        self.recv = torch.empty_like(self.send)
        self.all_q = torch.empty((W, Q, self.ops.dim), dtype=query_dtype, device=dev)
        self.dists = torch.empty((W * Q, self.slot), dtype=torch.float32, device=dev)
        self.ids = torch.empty((W * Q, self.slot), dtype=torch.int32, device=dev)
        self.pack_d = torch.empty((W, Q, self.top_k), dtype=torch.float32, device=dev)
        self.pack_i = torch.empty((W, Q, self.top_k), dtype=torch.int32, device=dev)
        self.back_d = torch.empty_like(self.pack_d)
        self.back_i = torch.empty_like(self.pack_i)
        self.out_d = torch.empty((Q, self.top_k), dtype=torch.float32, device=dev)
        self.out_i = torch.empty((Q, self.top_k), dtype=torch.int32, device=dev)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)

    def run(self, cand: torch.Tensor, queries: torch.Tensor):
        """cand: [Q, capacity, 2] candidate records (distance bits, id) of this rank's queries, ids global;
        queries: [Q, dim]. Returns (ids [Q, top_k] int32 holding global ids, dists [Q, top_k]) - buffers that the
        next call reuses."""
        if int(cand.shape[0]) != self.max_queries:
            raise ValueError("OwnerRerank.run: every call takes max_queries queries on every rank")
        self.ops.partition(cand, self.top_n, self.rows, self.world, self.slot, self.send, self.overflow)
        dist.all_to_all_single(self.recv, self.send, group=self.group)      # recv[h]: rank h's queries, my rows
        dist.all_gather_into_tensor(self.all_q.view(-1, self.all_q.shape[2]), queries.contiguous(), group=self.group)
        self.ops.rerank_topk(self.recv, self.all_q, self.slot, self.top_k, self.dists, self.ids, self.pack_d, self.pack_i)
        dist.all_to_all_single(self.back_d, self.pack_d, group=self.group)  # back[o]: my queries, owner o's rows
        dist.all_to_all_single(self.back_i, self.pack_i, group=self.group)
        self.ops.merge(self.back_d, self.back_i, self.rows, self.out_d, self.out_i)
        return self.out_i, self.out_d

    def overflowed(self) -> bool:
        """True if some (query, owner) list outgrew its slot since the object was built (synchronises)."""
        return bool(int(self.overflow.item()) != 0)
