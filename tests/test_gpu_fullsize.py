"""The search at the full size of the headline workload (10M x 512 inner product, degree 64,
100 000 queries, L = 64, k = 10) on seeded synthetic inputs of that shape.

The oracle cannot search 100 000 queries on 10M points in test time, so this file checks what does
not depend on size: order and uniqueness of every result row, returned distances recomputed bit for
bit, the same bits from a second call, from the unscheduled order and from the small-batch
(cluster) mode, recall against exact search -- and full oracle parity (ids, distance bits,
counters) on a handful of the queries.
"""
import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu

N, DIM, DEG, Q, L, K = 10_000_000, 512, 64, 100_000, 64, 10


@pytest.fixture(scope="module")
def full():
    import torch
    from coral_b200 import capi, synth
    if torch.cuda.mem_get_info()[1] < 100e9:
        pytest.skip("needs a GPU with the headline workload's memory")
    ds = synth.make_ip_cones(N, 100_000, Q, dim=DIM, clusters=4096, seed=1, device="cuda")
    g = synth.build_graph(ds.base, ds.train, ds.metric, max_degree=DEG, k_b=100, cell_size=512)
    ix = capi.Index(N, DIM, DEG, "ip")
    ix.attach_vectors(ds.base)
    ix.set_adjacency(g.adj)
    ix.set_start_ids(g.start_ids)
    ix.prepare(Q, L, K)
    ids, d, st, hops = ix.search(ds.test, L, K, dists=True, stats=True)
    to_np = lambda x: x.cpu().numpy() if hasattr(x, "cpu") else np.asarray(x)
    yield dict(ds=ds, g=g, ix=ix, ids=to_np(ids), d=to_np(d), st=to_np(st), hops=hops, to_np=to_np, torch=torch, synth=synth)
    ix.close()


def test_every_row_is_ordered_unique_and_complete(full):
    ids, d, st = full["ids"], full["d"], full["st"]
    assert ids.shape == (Q, K) and (ids >= 0).all() and (ids < N).all()
    assert (st[:, 0] == 0).all()                                   # every query converged with a full beam
    assert (d[:, :-1] >= d[:, 1:]).all()                           # inner product: closest = largest first
    tie = d[:, :-1] == d[:, 1:]
    assert (ids[:, :-1][tie] < ids[:, 1:][tie]).all()              # equal distances: smaller id first
    s = np.sort(ids, axis=1)
    assert (s[:, :-1] != s[:, 1:]).all()                           # no id twice in a row
    assert full["hops"] == int(st[:, 4].sum())
    assert full["ix"].get_option("last_scheduled") == 1            # the batch ran in the locality order


def test_returned_distances_are_the_reference_summation_bit_for_bit(full):
    torch, ds = full["torch"], full["ds"]
    rows = np.arange(0, Q, Q // 64)[:64]
    picked = torch.from_numpy(full["ids"][rows].astype(np.int64)).cuda()
    vecs = ds.base[picked.reshape(-1)].cpu().numpy().reshape(len(rows), K, DIM)
    qs = ds.test[torch.from_numpy(rows).cuda()].cpu().numpy()
    entry = set(full["g"].start_ids.cpu().numpy().tolist())   # entry points get the lane-tree order instead
    for i, r in enumerate(rows):
        for j in range(K):
            f = oracle.dist_tree if int(full["ids"][r, j]) in entry else oracle.dist_seq
            want = np.float32(f(vecs[i, j], qs[i], "ip"))
            assert want.view(np.uint32) == full["d"][r, j].view(np.uint32)


def test_same_bits_again_unscheduled_and_in_small_batches(full):
    ix, ds, to_np = full["ix"], full["ds"], full["to_np"]
    ids2, d2, st2, _ = ix.search(ds.test, L, K, dists=True, stats=True)
    assert np.array_equal(to_np(ids2), full["ids"]) and np.array_equal(to_np(d2).view(np.uint32), full["d"].view(np.uint32))
    assert np.array_equal(to_np(st2)[:, :7], full["st"][:, :7])
    ix.set_option("schedule", -1)
    ids3, d3, st3, _ = ix.search(ds.test, L, K, dists=True, stats=True)
    assert ix.get_option("last_scheduled") == 0
    assert np.array_equal(to_np(ids3), full["ids"]) and np.array_equal(to_np(d3).view(np.uint32), full["d"].view(np.uint32))
    assert np.array_equal(to_np(st3)[:, :7], full["st"][:, :7])
    ix.set_option("schedule", 0)
    for lo, n in ((0, 1), (17, 8), (4000, 64)):                    # batches that run as thread-block clusters
        ids4, d4, st4, _ = ix.search(ds.test[lo:lo + n], L, K, dists=True, stats=True)
        assert ix.get_option("last_cluster_size") > 1
        assert np.array_equal(to_np(ids4), full["ids"][lo:lo + n])
        assert np.array_equal(to_np(d4).view(np.uint32), full["d"][lo:lo + n].view(np.uint32))
        assert np.array_equal(to_np(st4)[:, :7], full["st"][lo:lo + n, :7])


def test_recall_against_exact_search(full):
    synth, ds = full["synth"], full["ds"]
    n_gt = 1000
    gt = synth.exact_knn(ds.base, ds.test[:n_gt], K, "ip").cpu().numpy()
    hit = sum(len(set(a) & set(b)) for a, b in zip(full["ids"][:n_gt], gt))
    assert hit / (K * n_gt) >= 0.95


def test_oracle_parity_on_a_handful_of_the_queries(full):
    ds, g = full["ds"], full["g"]
    base = ds.base.cpu().numpy()
    adj = g.adj.cpu().numpy()
    rows = [0, 1, 2, 3, 49_999, 50_000, 99_998, 99_999]
    qs = ds.test.cpu().numpy()[rows]
    ref_ids, ref_d, ref_st = oracle.search(base, adj, g.start_ids.cpu().numpy(), qs, L, K, "ip")
    assert np.array_equal(full["ids"][rows], ref_ids)
    assert np.array_equal(full["d"][rows].view(np.uint32), ref_d.view(np.uint32))
    assert np.array_equal(full["st"][rows][:, :7], ref_st[:, :7])
