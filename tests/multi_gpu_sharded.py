"""Node-id-range sharding on real peers: run with
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 tests/multi_gpu_sharded.py
Every rank holds one shard (adjacency, codes, vector pages) in IPC-shared device memory, searches its
own slice of the queries reading remote rows over NVLink, and rank 0 gathers the top-k lists. The
result must equal (a) the same search on an unsharded copy of the whole index held by rank 0 and
(b) the CPU checker. Not collected by pytest (needs >= 2 GPUs); NVLS is switched off so that a rank
that dies cannot disturb its peers."""
import dataclasses
import os
import sys

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from oracle import pipeline
    from topoanns_b200 import search, sharding, synth, synth_sharded
    nodes = int(os.environ.get("TANN_NODES", "400000"))       # whole index, split evenly over the ranks
    num_queries = int(os.environ.get("TANN_QUERIES", "1000"))
    top_l, top_n = int(os.environ.get("TANN_TOP_L", "64")), int(os.environ.get("TANN_TOP_N", "32"))
    check_cpu = os.environ.get("TANN_CHECK_CPU", "1") == "1"   # the CPU checker needs the whole index on the host
    cfg = dataclasses.replace(synth.CONFIGS["cfg4"], num_nodes=nodes, components=max(world, nodes // 1000),
                              num_queries=num_queries, kmeans_iters=5, train_sample=65536)
    sh = synth_sharded.build(cfg, f"cuda:{local}")
    ix, buffers = sharding.peer_index_from_sharded(sh)
    model = search.RvqModel(dim=cfg.dim, coarse=sh.rvq_coarse.contiguous(), fine=sh.rvq_fine.contiguous(),
                            bucket_sizes=sh.rvq_buckets[0], cluster_offsets=sh.rvq_buckets[1], cluster_ids=sh.rvq_buckets[2])
    Q = sh.queries.shape[0]
    b, e = sharding.query_shard(Q, world, rank)
    tp = search.TopologySearchParams(top_l=top_l, search_width=2, max_expansions=4096)
    rp = search.RerankExactParams(top_k=10, top_n=top_n)
    cap = tp.capacity(top_n)
    sr = search.Searcher(ix, max(e - b, 1), cap, top_n, 128)
    sr.set_rvq(model, 128)
    qn = sh.queries.cpu().numpy()
    ids, dists, stats = sr.run_host(qn[b:e], tp, rp, want_stats=True)
    all_ids, all_d = sharding.gather_topk(torch.from_numpy(ids.view(np.int32)).cuda(), torch.from_numpy(dists).cuda(), Q)
    # throughput of the sharded search (every rank searches its query slice; (G-1)/G of the gathers are remote)
    steps = int(os.environ.get("TANN_STEPS", "20"))
    q_dev = sh.queries[b:e].cuda().contiguous()
    for _ in range(3):
        sr.run_device(q_dev, tp, rp)
    dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        sr.run_device(q_dev, tp, rp)
    ev1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([ev0.elapsed_time(ev1) / steps], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    sharded_ms = float(ms.item())
    whole = synth_sharded.gather_whole(sh)
    ok = True
    if rank == 0:
        got_ids, got_d = all_ids.cpu().numpy().view(np.uint32), all_d.cpu().numpy()
        full_ix = search.device_index_from_synth(whole)
        full_model = search.rvq_model_from_synth(whole)
        sr2 = search.Searcher(full_ix, Q, cap, top_n, 128)
        sr2.set_rvq(full_model, 128)
        ids2, d2, _ = sr2.run_host(qn, tp, rp)
        same_unsharded = np.array_equal(got_ids, ids2) and np.array_equal(got_d.view(np.uint32), d2.view(np.uint32))
        same_checker = "skipped"
        if check_cpu:
            ref = pipeline.run(pipeline.index_from_synth(whole), qn, top_l=top_l, search_width=2, max_expansions=4096,
                               top_n=top_n, top_k=10, entry_count=128)
            same_checker = np.array_equal(got_ids, ref["topk_ids"]) and np.array_equal(got_d.view(np.uint32), ref["topk_dists"].view(np.uint32))
        rec = synth.recall_at_k(got_ids, whole.gt_ids.cpu().numpy(), 10)
        remote = 1.0 - 1.0 / world
        q_all = sh.queries.cuda().contiguous()
        for _ in range(3):
            sr2.run_device(q_all, tp, rp)
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(steps):
            sr2.run_device(q_all, tp, rp)
        ev1.record()
        torch.cuda.synchronize()
        single_ms = ev0.elapsed_time(ev1) / steps
        print(f"sharded x{world}: nodes={sh.total_nodes} queries={Q} L={top_l} top_n={top_n} identical_to_unsharded={same_unsharded} identical_to_checker={same_checker} "
              f"recall@10={rec:.3f} expected_remote_fraction={remote:.3f} "
              f"sharded_ms_per_batch={sharded_ms:.3f} ({Q / sharded_ms * 1e3:.0f} QPS over {world} GPUs) "
              f"one_gpu_whole_index_ms={single_ms:.3f} ({Q / single_ms * 1e3:.0f} QPS)")
        ok = same_unsharded and same_checker in (True, "skipped")
        sr2.close()
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.broadcast(flag, 0)
    sr.close()
    for pb in buffers.values():
        pb.close()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
