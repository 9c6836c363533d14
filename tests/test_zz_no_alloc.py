"""tann_rerank_topk_static (rerank + top-k in the library's fixed device array, no allocation) against
tann_rerank_exact + tann_topk_pack on the same candidates. Collected last on purpose: it has to pass
both after every other test has used the library and alone in a fresh process."""
import ctypes as C

import numpy as np
import pytest
import torch

from topoanns_b200 import capi, search

import gpu_support as gs

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _static_topk(ix, params, cand, queries, out_d, out_i):
    view = ix.view()
    p = params.to_c()
    Q, capacity, _ = cand.shape
    return capi.load().tann_rerank_topk_static(C.byref(view), C.byref(p), _ptr(cand), capacity, Q, _ptr(queries),
                                               search.kind_of(queries), None, _ptr(out_d), _ptr(out_i),
                                               search._stream_ptr())


@pytest.mark.parametrize("float_queries", [True, False])
def test_static_rerank_equals_allocating_path_twice(float_queries):
    s, _host = gs.small_index()
    ix = gs.device_index(s)
    q = s.queries.cuda().contiguous()
    if not float_queries:
        q = q.to(torch.uint8).contiguous()
    Q = q.shape[0]
    offs, ids = gs.fixed_entries(Q, [s.medoid])
    tp = search.TopologySearchParams(top_l=64, search_width=2, max_expansions=4096)
    rp = search.RerankExactParams(top_k=10, top_n=48)
    cand, _stats = search.beam_search(ix, tp, offs, ids, queries=q, capacity=tp.capacity(rp.top_n))
    want_d, want_i, _, _ = search.rerank_exact(ix, rp, cand, q)
    want_d, want_i = search.topk_pack(want_d, want_i, rp.top_k)
    torch.cuda.synchronize()
    for call in range(2):  # two calls in a row reuse the same static area
        got_d = torch.full((Q, rp.top_k), -1.0, dtype=torch.float32, device="cuda")
        got_i = torch.full((Q, rp.top_k), -1, dtype=torch.int32, device="cuda")
        capi.check(_static_topk(ix, rp, cand, q, got_d, got_i))
        torch.cuda.synchronize()
        assert np.array_equal(gs.np_u32(got_i), gs.np_u32(want_i)), f"ids differ on call {call}"
        assert np.array_equal(got_d.cpu().numpy().view(np.uint32), want_d.cpu().numpy().view(np.uint32)), \
            f"distances differ on call {call}"


def test_static_rerank_rejects_batches_beyond_its_area():
    s, _host = gs.small_index()
    ix = gs.device_index(s)
    q = s.queries.cuda().contiguous()
    rp = search.RerankExactParams(top_k=10, top_n=2048)
    Q = 4096  # 2 * 4096 * 2048 * 4 bytes of lists: far beyond 8 MiB; rejected before any pointer is used
    cand = torch.zeros((1, 2048, 2), dtype=torch.int32, device="cuda")
    out_d = torch.empty((1, 10), dtype=torch.float32, device="cuda")
    out_i = torch.empty((1, 10), dtype=torch.int32, device="cuda")
    view = ix.view()
    p = rp.to_c()
    st = capi.load().tann_rerank_topk_static(C.byref(view), C.byref(p), _ptr(cand), 2048, Q, _ptr(q), 2, None,
                                             _ptr(out_d), _ptr(out_i), None)
    assert st == 3  # TANN_ERR_UNSUPPORTED
    assert b"static area" in capi.load().tann_last_error()


def test_static_rerank_applies_the_checks_of_the_allocating_entry_point():
    """Rejected before any launch: early stop with a top_k beyond the kernel's 128-entry list, and a sharded
    vector view whose rows_per_shard is zero (the kernel would divide by it)."""
    s, _host = gs.small_index()
    ix = gs.device_index(s)
    q = s.queries[:4].cuda().contiguous()
    cand = torch.zeros((4, 256, 2), dtype=torch.int32, device="cuda")
    out_d = torch.empty((4, 200), dtype=torch.float32, device="cuda")
    out_i = torch.empty((4, 200), dtype=torch.int32, device="cuda")
    lib = capi.load()
    view = ix.view()
    p = search.RerankExactParams(top_k=200, top_n=256, use_early_stop=True).to_c()
    st = lib.tann_rerank_topk_static(C.byref(view), C.byref(p), _ptr(cand), 256, 4, _ptr(q), 2, None, _ptr(out_d),
                                     _ptr(out_i), None)
    assert st == 1 and b"early stop requires 1 <= top_k <= 128" in lib.tann_last_error()
    view = ix.view()
    view.vectors.num_shards = 2
    view.vectors.base[1] = view.vectors.base[0]
    view.vectors.rows_per_shard = 0
    p = search.RerankExactParams(top_k=10, top_n=32).to_c()
    st = lib.tann_rerank_topk_static(C.byref(view), C.byref(p), _ptr(cand), 256, 4, _ptr(q), 2, None, _ptr(out_d),
                                     _ptr(out_i), None)
    assert st == 1 and b"shards do not cover all rows" in lib.tann_last_error()
