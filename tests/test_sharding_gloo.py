"""Query sharding and the single top-k gather, as two gloo ranks on the CPU. Each rank searches its
query range with the CPU checker; rank 0 must end up with exactly the unsharded result."""
import dataclasses
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from topoanns_b200 import sharding


def test_query_shard_covers_everything():
    for Q in (0, 1, 7, 10, 10000):
        for G in (1, 2, 3, 8):
            spans = [sharding.query_shard(Q, G, r) for r in range(G)]
            assert spans[0][0] == 0 and spans[-1][1] == Q
            assert all(spans[i][1] == spans[i + 1][0] for i in range(G - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    assert sharding.rows_per_shard(1000, 8, 32) % 32 == 0 and sharding.rows_per_shard(1000, 8, 32) * 8 >= 1000
    assert sharding.rows_per_shard(10, 4) == 3


def _worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import pipeline
    from topoanns_b200 import synth
    torch.set_num_threads(1)
    cfg = dataclasses.replace(synth.CONFIGS["cfg2"], num_nodes=4000, components=20, num_queries=51,
                              train_sample=4000, kmeans_iters=3)
    s = synth.build(cfg, "cpu")                        # same seed -> same replica on every rank
    host = pipeline.index_from_synth(s)
    q = s.queries.numpy()
    b, e = sharding.query_shard(q.shape[0], world, rank)
    kw = dict(top_l=32, search_width=2, max_expansions=512, top_n=32, top_k=10, entry_count=128)
    mine = pipeline.run(host, q[b:e], **kw)
    ids, dists = sharding.gather_topk(torch.from_numpy(mine["topk_ids"].view(np.int32)),
                                      torch.from_numpy(mine["topk_dists"]), q.shape[0])
    if rank == 0:
        full = pipeline.run(host, q, **kw)
        ok = np.array_equal(ids.numpy().view(np.uint32), full["topk_ids"]) and \
            np.array_equal(dists.numpy().view(np.uint32), full["topk_dists"].view(np.uint32))
        open(out_path, "w").write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_gather_equals_unsharded(tmp_path):
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    out = tmp_path / "result.txt"
    mp.spawn(_worker, args=(2, port, str(out)), nprocs=2, join=True)
    assert out.read_text() == "ok"


def _sharded_worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import pipeline
    from topoanns_b200 import synth, synth_sharded
    torch.set_num_threads(1)
    cfg = dataclasses.replace(synth.CONFIGS["cfg4"], num_nodes=6000, components=24, num_queries=40,
                              train_sample=3000, kmeans_iters=3)
    sh = synth_sharded.build(cfg, "cpu")
    whole = synth_sharded.gather_whole(sh)
    problems = []
    N = whole.vectors.shape[0]
    if N != sh.total_nodes or sh.rows_per_shard * world != N or sh.rows_per_shard % 32:
        problems.append("shard sizes")
    if int(whole.adjacency.min()) < 0 or int(whole.adjacency.max()) >= N:
        problems.append("adjacency range")
    # kNN neighbours of a node are spread over both shards
    nbr_owner = (whole.adjacency[:, :cfg.knn_edges].long() // sh.rows_per_shard).float().mean().item()
    if not 0.3 < nbr_owner < 0.7:
        problems.append(f"neighbours not scattered ({nbr_owner})")
    x = whole.vectors.float()
    want = (torch.cdist(whole.queries, x) ** 2).topk(10, largest=False).values
    got = ((x[whole.gt_ids] - whole.queries.unsqueeze(1)) ** 2).sum(2)
    if not torch.allclose(got, want):
        problems.append("ground truth")
    sizes, offsets, ids = whole.rvq_buckets
    if int(sizes.sum()) != N or int(offsets[-1]) != ids.numel():
        problems.append("rvq buckets")
    # ground truth for every fourth query only: the same index, the same rows where they are computed, -1 elsewhere
    strided = synth_sharded.build(cfg, "cpu", gt_stride=4)
    if not (torch.equal(strided.vectors, sh.vectors) and torch.equal(strided.gt_ids[::4], sh.gt_ids[::4])
            and int(strided.gt_ids[1::4].max()) == -1 and int(strided.gt_ids[2::4].max()) == -1):
        problems.append("strided ground truth")
    if rank == 0:
        host = pipeline.index_from_synth(whole)
        r = pipeline.run(host, whole.queries.numpy(), top_l=64, search_width=2, max_expansions=2048, top_n=64,
                         top_k=10, entry_count=128)
        rec = synth.recall_at_k(r["topk_ids"], whole.gt_ids.numpy(), 10)
        if rec < 0.6:
            problems.append(f"recall {rec}")
        open(out_path, "w").write("ok" if not problems else "; ".join(problems))
    dist.barrier()
    dist.destroy_process_group()


def test_node_range_sharded_generator(tmp_path):
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    out = tmp_path / "result.txt"
    mp.spawn(_sharded_worker, args=(2, port, str(out)), nprocs=2, join=True)
    assert out.read_text() == "ok"


class _TorchOwnerOps:
    """Plain torch stand-ins for the three device steps of sharding.OwnerRerank (same contracts as the C ABI's
    tann_partition_candidates, tann_rerank_exact + tann_topk_pack, tann_merge_topk_lists), for CPU ranks."""

    def __init__(self, local_vectors):
        self.vectors = local_vectors.to(torch.int64)          # [rows, dim]
        self.device = torch.device("cpu")
        self.dim = local_vectors.shape[1]

    def partition(self, cand, top_n, rows, owners, slot, out, overflow):
        out[..., 0] = 0
        out[..., 1] = -1
        n = min(top_n, cand.shape[1])
        for q in range(cand.shape[0]):
            used = [0] * owners
            for r in range(n):
                bits, raw = int(cand[q, r, 0]), int(cand[q, r, 1]) & 0xffffffff
                if raw == 0xffffffff:
                    continue
                raw &= 0x7fffffff
                o = raw // rows
                if o >= owners:
                    continue
                if used[o] < slot:
                    out[o, q, used[o], 0] = bits
                    out[o, q, used[o], 1] = raw - o * rows
                    used[o] += 1
                else:
                    overflow[0] = 1

    def rerank_topk(self, lists, queries, slot, top_k, dists, ids, out_d, out_i):
        flat = lists.reshape(-1, slot, 2)
        qs = queries.reshape(-1, self.dim).to(torch.int64)
        for n in range(flat.shape[0]):
            keys = []
            for j in range(slot):
                row = int(flat[n, j, 1])
                if row < 0 or row >= self.vectors.shape[0]:
                    continue
                d = int(((self.vectors[row] - qs[n]) ** 2).sum())
                keys.append((float(d), row))
            keys.sort()
            keys = (keys + [(float("inf"), -1)] * top_k)[:top_k]
            out_d.view(-1, top_k)[n] = torch.tensor([k[0] for k in keys])
            out_i.view(-1, top_k)[n] = torch.tensor([k[1] for k in keys], dtype=torch.int32)

    def merge(self, lists_d, lists_i, rows, out_d, out_i):
        W, Q, k = lists_d.shape
        for q in range(Q):
            keys = []
            for l in range(W):
                for j in range(k):
                    if int(lists_i[l, q, j]) >= 0:
                        keys.append((float(lists_d[l, q, j]), int(lists_i[l, q, j]) + l * rows))
            keys.sort()
            keys = (keys + [(float("inf"), -1)] * k)[:k]
            out_d[q] = torch.tensor([x[0] for x in keys])
            out_i[q] = torch.tensor([x[1] for x in keys], dtype=torch.int32)


def _owner_worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(99)                       # the same data on every rank
    rows, dim, Q, cap, top_n, k = 96, 16, 9, 64, 40, 5
    vectors = torch.randint(0, 256, (rows * world, dim), generator=g, dtype=torch.int64).to(torch.uint8)
    queries = torch.randint(0, 256, (world, Q, dim), generator=g, dtype=torch.int64).to(torch.uint8)
    ids = torch.stack([torch.stack([torch.randperm(rows * world, generator=g)[:cap] for _ in range(Q)])
                       for _ in range(world)]).to(torch.int32)
    ids[:, :, 7] = -1                                            # an empty rank in every list
    ids[:, 0, 3] |= -0x80000000                                  # the traversal's "expanded" bit on one record
    cand = torch.stack([torch.zeros_like(ids), ids], dim=3)      # (distance bits, id); the distance is not used here
    ok = True
    for slot in (0, top_n):
        orr = sharding.OwnerRerank(None, rows, Q, top_n, k, torch.uint8, slot=slot,
                                   ops=_TorchOwnerOps(vectors[rank * rows:(rank + 1) * rows]))
        got_i, got_d = orr.run(cand[rank], queries[rank])
        # the unsharded answer: exact distances of the first top_n ranks against the whole matrix, by (distance, id)
        for q in range(Q):
            keys = []
            for r in range(top_n):
                raw = int(ids[rank, q, r])
                if raw == -1:
                    continue
                raw &= 0x7fffffff
                d = int(((vectors[raw].to(torch.int64) - queries[rank, q].to(torch.int64)) ** 2).sum())
                keys.append((float(d), raw))
            keys.sort()
            want = keys[:k]
            ok = ok and [int(x) for x in got_i[q]] == [w[1] for w in want] and \
                [float(x) for x in got_d[q]] == [w[0] for w in want]
        ok = ok and not orr.overflowed()
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        open(out_path, "w").write("ok" if int(flag) == 1 else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


def test_rerank_by_owner_exchange_on_three_ranks(tmp_path):
    """The two all-to-alls and the query all-gather of sharding.OwnerRerank, with the device steps replaced by plain
    torch code: every rank ends up with the top-k of its own queries over the rows of all ranks."""
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    out = tmp_path / "owner.txt"
    mp.spawn(_owner_worker, args=(3, port, str(out)), nprocs=3, join=True)
    assert out.read_text() == "ok"
