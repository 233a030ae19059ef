"""coral_search_static -- the search entry point that allocates nothing.

Some callers cannot allocate device memory when they search (the GPU is owned by
their own pool, or they run where an allocation is an error), so this entry point
keeps the kernel's scratch in a fixed array inside the library.  It must return
exactly what the regular entry point returns for the same inputs: the same kernel
runs, only the scratch differs.  Two calls in a row share the array, so the second
call also checks that nothing left behind by the first one leaks into its result.
Collected last on purpose: a failure here must not hide the other tests.
"""
import ctypes as C

import numpy as np
import pytest

from coral_b200 import capi
from tests import cases

pytestmark = pytest.mark.gpu


def _static_search(lib, t_vecs, t_adj, t_start, t_q, n, dim, deg_pad, metric, L, k):
    import torch
    ids = torch.full((t_q.shape[0], k), -7, dtype=torch.int32, device="cuda")
    dists = torch.zeros((t_q.shape[0], k), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    rc = lib.coral_search_static(0, None, C.c_void_p(t_vecs.data_ptr()), C.c_void_p(t_adj.data_ptr()), n, dim, deg_pad,
                                 metric, C.c_void_p(t_start.data_ptr()), int(t_start.numel()),
                                 C.c_void_p(t_q.data_ptr()), int(t_q.shape[0]), L, k,
                                 C.c_void_p(ids.data_ptr()), C.c_void_p(dists.data_ptr()))
    return rc, ids.cpu().numpy(), dists.cpu().numpy()


@pytest.mark.parametrize("metric", ["l2", "ip"])
def test_static_entry_point_matches_regular_entry_point(metric):
    import torch
    c = cases.structured(metric)
    lib = capi.load()
    with capi.Index(c.n, c.dim, c.max_degree, c.metric) as ix:
        ix.set_vectors(c.base)
        ix.set_adjacency(c.adj)
        ix.set_start_ids(c.start)
        ix.prepare(len(c.queries), 128, 10)
        want = {L: ix.search(c.queries, L, 10)[:2] for L in (64, 128)}
    tv, ta = torch.from_numpy(c.base).cuda(), torch.from_numpy(c.adj).cuda()
    ts, tq = torch.from_numpy(c.start).cuda(), torch.from_numpy(c.queries).cuda()
    m = capi.L2 if metric == "l2" else capi.IP
    _static_search(lib, tv, ta, ts, tq, c.n, c.dim, c.adj.shape[1], m, 64, 10)   # first call: address look-up
    for L in (64, 128, 64):       # consecutive calls share the scratch array, with and without re-carving
        for _ in range(2):
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            rc, ids, dists = _static_search(lib, tv, ta, ts, tq, c.n, c.dim, c.adj.shape[1], m, L, 10)
            # the output tensors come from torch's cache or the driver; the call itself must not
            # take device memory: what is free afterwards is what was free before minus those two
            assert torch.cuda.mem_get_info()[0] >= free_before - 2 * (1 << 21)
            assert rc == capi.OK
            assert lib.coral_search_static_status(0) == 0
            assert np.array_equal(ids, want[L][0])
            assert np.array_equal(dists.view(np.uint32), want[L][1].view(np.uint32))   # bit-exact, like the other tests


def test_static_entry_point_rejects_what_does_not_fit():
    import torch
    c = cases.structured("l2")
    lib = capi.load()
    tv, ta = torch.from_numpy(c.base).cuda(), torch.from_numpy(c.adj).cuda()
    ts, tq = torch.from_numpy(c.start).cuda(), torch.from_numpy(c.queries).cuda()
    rc, _, _ = _static_search(lib, tv, ta, ts, tq, c.n, c.dim, 32, capi.L2, 1024, 10)   # 1024*32 > 16384
    assert rc == capi.ERR_LIMIT
    rc, _, _ = _static_search(lib, tv, ta, ts, tq, c.n, c.dim, 32, capi.L2, 8, 10)      # k > L
    assert rc == capi.ERR_ARG
    rc, ids, _ = _static_search(lib, tv, ta, ts, tq, c.n, c.dim, 32, capi.L2, 64, 10)   # still usable
    assert rc == capi.OK and (ids >= 0).all()


def test_static_entry_point_reports_query_status_and_refuses_bad_pointers():
    import torch
    lib = capi.load()
    c = cases.chain_case()            # ten reachable nodes: every beam ends under-full (status 1)
    tv, ta = torch.from_numpy(c.base).cuda(), torch.from_numpy(c.adj).cuda()
    ts, tq = torch.from_numpy(c.start).cuda(), torch.from_numpy(c.queries).cuda()
    rc, ids, _ = _static_search(lib, tv, ta, ts, tq, c.n, c.dim, 32, capi.L2, 64, 16)
    assert rc == capi.OK and lib.coral_search_static_status(0) == 1
    assert (ids[:, :10] >= 0).all() and (ids[:, 10:] == -1).all()
    # a start id outside [0, n) is skipped and flagged, never dereferenced
    bad = torch.tensor([0, c.n + 5, -3], dtype=torch.int32, device="cuda")
    rc, ids2, _ = _static_search(lib, tv, ta, bad, tq, c.n, c.dim, 32, capi.L2, 64, 16)
    assert rc == capi.ERR_QUERY and lib.coral_search_static_status(0) == 4
    assert np.array_equal(ids2, ids)
    # a host pointer handed in by mistake is an argument error, not a fault
    host_q = np.ascontiguousarray(c.queries)
    out = torch.empty((len(host_q), 16), dtype=torch.int32, device="cuda")
    rc = lib.coral_search_static(0, None, C.c_void_p(tv.data_ptr()), C.c_void_p(ta.data_ptr()), c.n, c.dim, 32,
                                 capi.L2, C.c_void_p(ts.data_ptr()), 1, C.c_void_p(host_q.ctypes.data),
                                 len(host_q), 64, 16, C.c_void_p(out.data_ptr()), None)
    assert rc == capi.ERR_ARG
