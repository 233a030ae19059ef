"""Parity of the CUDA path (through the C ABI) with the CPU oracle.

The bar is bit-exact: ids, distance bit patterns and the per-query counters
(distance evaluations, expansions, rounds, accepted candidates, scanned
neighbour ids, largest candidate set) must all be identical, because the kernel
reproduces the reference's fp32 summation orders and uses the oracle's fixed
(distance, id) tie order.
"""
import numpy as np
import pytest

from coral_b200 import capi
from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu


def make_index(c, max_q, max_L, max_k, options=None, device_vectors=False):
    ix = capi.Index(c.n, c.dim, c.max_degree, c.metric)
    for k, v in (options or {}).items():
        ix.set_option(k, v)
    ix.set_vectors(c.base)
    ix.set_adjacency(c.adj)
    ix.set_start_ids(c.start)
    ix.prepare(max_q, max_L, max_k)
    return ix


def assert_same(c, ix, L, k, queries=None, check_stats=True, modes=(1, 0)):
    """Search and compare with the oracle.  The test batches are small, so by default each check
    runs twice: one CTA per query (cluster_size 1) and the automatic small-batch mode in which a
    thread-block cluster shares each query.  modes=None leaves the handle's setting alone."""
    q = c.queries if queries is None else queries
    ref_ids, ref_d, ref_st = oracle.search(c.base, c.adj, c.start, q, L, k, c.metric)
    for mode in (modes or (None,)):
        if mode is not None:
            ix.set_option("cluster_size", mode)
        ids, d, st, hops = ix.search(q, L, k, dists=True, stats=True)
        tag = f"{c.name} L={L} k={k} cluster_size={mode}"
        assert np.array_equal(ids, ref_ids), f"{tag}: ids differ"
        assert np.array_equal(d.view(np.uint32), ref_d.view(np.uint32)), f"{tag}: distances differ"
        if check_stats:
            assert np.array_equal(st[:, :7], ref_st[:, :7]), f"{tag}: counters differ"
            assert hops == int(ref_st[:, 4].sum())
    return ids, d, st, ref_st


@pytest.mark.parametrize("metric", ["l2", "ip"])
def test_structured_graph_all_L(metric):
    c = cases.structured(metric)
    with make_index(c, len(c.queries), 512, 100) as ix:
        for L, k in [(64, 10), (128, 10), (256, 10), (512, 10), (128, 100), (100, 100), (33, 7)]:
            assert_same(c, ix, L, k)


@pytest.mark.parametrize("metric,dim,deg", [("l2", 200, 32), ("ip", 512, 64), ("l2", 8, 32), ("ip", 100, 64),
                                            ("l2", 36, 128), ("l2", 1024, 32)])
def test_random_graph_shapes(metric, dim, deg):
    c = cases.random_case(metric, 6000, dim, deg, 64)
    with make_index(c, 64, 256, 64) as ix:
        for L, k in [(16, 16), (64, 10), (200, 64)]:
            assert_same(c, ix, L, k)


def test_exact_ties_and_duplicate_entry_points():
    c = cases.random_case("l2", 5000, 16, 32, 80, dup_start=True, quantized=True)
    with make_index(c, 80, 128, 32) as ix:
        assert_same(c, ix, 64, 32)
        assert_same(c, ix, 128, 10)
    c = cases.random_case("ip", 5000, 16, 64, 80, dup_start=True, quantized=True)
    with make_index(c, 80, 128, 32) as ix:
        assert_same(c, ix, 64, 32)


def test_ragged_degrees_and_isolated_nodes():
    c = cases.random_case("l2", 4000, 40, 32, 50, seed=9, min_degree=0)
    assert (c.adj[:, 0] < 0).any()  # some nodes have no out-edges at all
    with make_index(c, 50, 128, 20) as ix:
        assert_same(c, ix, 128, 20)


def test_underfull_beam_is_reported_not_faulted():
    c = cases.chain_case()
    with make_index(c, 8, 64, 16) as ix:
        ids, d, st, ref_st = assert_same(c, ix, 64, 16)
        assert (st[:, 0] == 1).all() and (ref_st[:, 0] == 1).all()   # BEAM_UNDERFULL
        assert (ids[:, 10:] == -1).all() and (ids[:, :10] >= 0).all()
        assert np.all(d[:, 10:] == np.float32(3.402823466e+38))


@pytest.mark.parametrize("opts", [
    {"smem_hash_bits": 0},                         # visited set entirely in the global table
    {"smem_hash_bits": 8},                         # tiny shared table: almost everything spills
    {"warps": 1, "ctas_per_sm": 1, "stages": 1},   # no overlap at all
    {"warps": 8, "ctas_per_sm": 1, "chunk_bytes": 512},
    {"warps": 2, "ctas_per_sm": 4, "chunk_bytes": 64, "stages": 3},
    {"warps": 3, "ctas_per_sm": 1, "chunk_bytes": 2048},
    {"scout_ids": 1},                              # 32 neighbour slots per scout step (half an adjacency row)
    {"scout_ids": 3, "warps": 5},
    {"visit_cache_bits": 9},                       # shared-memory cache of recently seen ids
    {"visit_cache_bits": 3, "smem_hash_bits": 8},  # a cache that thrashes, in front of both tables
    {"gather": 0},                                 # one bulk copy per row chunk
    {"gather": 1},                                 # 16-byte unit copies, one commit group per chunk
    {"gather": 1, "stages": 3, "chunk_bytes": 128, "warps": 3},
    {"gather": 1, "chunk_bytes": 1024, "warps": 2, "ctas_per_sm": 1},   # more units per chunk than lanes
    {"gather": 0, "stages": 2},
    {"gather": 2},                                 # tensor copies that gather four rows each
    {"gather": 2, "chunk_bytes": 48, "stages": 3, "warps": 3},
    {"gather": 2, "chunk_bytes": 1008, "warps": 2, "ctas_per_sm": 1},   # the widest box: 63 units
    {"probe_carry": 0},                            # ids the first probe pair leaves open are settled at once
    {"probe_carry": 1, "ghash_entries": 4096},     # a crowded visited table: many carried probes
])
def test_tuning_knobs_do_not_change_results(opts):
    c = cases.structured("ip")
    with make_index(c, len(c.queries), 256, 10, options=opts) as ix:
        assert_same(c, ix, 64, 10)
        assert_same(c, ix, 256, 10)


@pytest.mark.parametrize("metric", ["l2", "ip"])
def test_locality_scheduling_changes_only_the_order_of_work(metric):
    # Large batches are run grouped by their best "frontier" node (the entry points' neighbours);
    # forced on here for a small batch.  Every query's result stays at its own row.
    c = cases.structured(metric)
    with make_index(c, len(c.queries), 128, 10, options={"schedule": 1}) as ix:
        assert_same(c, ix, 64, 10, modes=(1,))
        assert ix.get_option("last_scheduled") == 1 and ix.get_option("frontier_size") >= 2
        assert_same(c, ix, 128, 10, queries=c.queries[:37], modes=(1,))     # ragged tile of the pre-pass
    with make_index(c, len(c.queries), 64, 10, options={"schedule": -1}) as ix:
        assert_same(c, ix, 64, 10, modes=(1,))
        assert ix.get_option("last_scheduled") == 0
    r = cases.random_case(metric, 3000, 36, 32, 50, m=3, seed=41)             # tiny frontier, odd dim
    with make_index(r, 50, 64, 10, options={"schedule": 1}) as ix:
        assert_same(r, ix, 64, 10, modes=(1,))


@pytest.mark.parametrize("metric", ["l2", "ip"])
def test_tensor_gather_of_rows(metric):
    # gather = 2 moves the chunks of four rows with one tensor copy; the last chunk of a row runs
    # past its end (zero fill).  Rows of 144, 800 and 2048 bytes, batches that do not fill a group
    # of four, large batches and clusters that share a query.
    c = cases.structured(metric)
    with make_index(c, len(c.queries), 128, 10, options={"gather": 2}) as ix:
        assert ix.get_option("plan_chunk_bytes") % 32 == 16
        assert_same(c, ix, 64, 10)
        assert_same(c, ix, 128, 10, queries=c.queries[:3], modes=(0,))       # cluster mode
        assert ix.get_option("last_cluster_size") >= 2
    for dim, deg in ((36, 32), (200, 32), (512, 64)):
        r = cases.random_case(metric, 3000, dim, deg, 40, m=5, seed=dim)
        for opts in ({"gather": 2}, {"gather": 2, "chunk_bytes": 400, "stages": 2}):
            with make_index(r, 40, 64, 10, options=opts) as ix:
                assert_same(r, ix, 64, 10)
                assert_same(r, ix, 33, 7, queries=r.queries[:9])


def test_small_sort_tiles_take_many_fill_passes():
    # Tiny staging memory -> tiny candidate sort tiles -> a round's candidates need many
    # fill passes; every thread must agree on when a tile is full (barrier-counted).
    for metric in ("l2", "ip"):
        c = cases.structured(metric)
        with make_index(c, len(c.queries), 512, 10, options={"chunk_bytes": 16, "warps": 4}) as ix:
            for _ in range(3):
                assert_same(c, ix, 512, 10)
                assert_same(c, ix, 256, 10)


@pytest.mark.parametrize("metric", ["l2", "ip"])
def test_small_batches_share_a_query_across_a_cluster(metric):
    # Batches far below the SM count run one thread-block cluster per query; results and
    # counters must not depend on how many CTAs cooperate.
    c = cases.structured(metric)
    with make_index(c, len(c.queries), 128, 10) as ix:
        for nq in (1, 3, 8, 20, 70):
            assert_same(c, ix, 64, 10, queries=c.queries[:nq], modes=(0,))
            assert 2 <= ix.get_option("last_cluster_size") <= 16
        assert_same(c, ix, 128, 10, queries=c.queries[:5], modes=(0,))
        assert_same(c, ix, 64, 10, modes=(0,))                  # the whole batch of 96
    for size in (2, 8, 16):
        with make_index(c, len(c.queries), 128, 10, options={"cluster_size": size}) as ix:
            assert_same(c, ix, 128, 10, queries=c.queries[:9], modes=None)
            assert ix.get_option("last_cluster_size") in (size, size // 2)
    with make_index(c, len(c.queries), 128, 10, options={"cluster_size": 1}) as ix:
        assert_same(c, ix, 128, 10, queries=c.queries[:2], modes=None)
        assert ix.get_option("last_cluster_size") == 1


def test_visited_overflow_sets_status_without_fault():
    c = cases.structured("l2")
    with make_index(c, len(c.queries), 64, 10, options={"smem_hash_bits": 0, "ghash_entries": 256}) as ix:
        # a 256-entry visited table cannot hold a query's visited set: every query must still
        # come back, flagged HASH_OVERFLOW, and the handle must stay usable afterwards.
        ids, d, st, hops = ix.search(c.queries, 64, 10, stats=True)
        assert ids.shape == (len(c.queries), 10)
        assert (st[:, 0] == 2).all()
        ix.set_option("ghash_entries", 0)
        ix.set_option("smem_hash_bits", 12)
        ix.prepare(len(c.queries), 64, 10)
        assert_same(c, ix, 64, 10)


def test_device_pointers_and_repeated_calls():
    import torch
    c = cases.structured("l2")
    with make_index(c, len(c.queries), 128, 10) as ix:
        ref_ids, ref_d, _ = oracle.search(c.base, c.adj, c.start, c.queries, 128, 10, c.metric)
        dq = torch.from_numpy(c.queries).cuda()
        torch.cuda.synchronize()
        for _ in range(3):   # epochs of the global visited table advance between calls
            ids, d, st, hops = ix.search(dq, 128, 10, stats=True)
            assert np.array_equal(ids.cpu().numpy(), ref_ids)
            assert np.array_equal(d.cpu().numpy().view(np.uint32), ref_d.view(np.uint32))
        # attached (borrowed) device vectors give the same answers
        dv = torch.from_numpy(c.base).cuda()
        torch.cuda.synchronize()
        ix.attach_vectors(dv)
        ids, d, _, _ = ix.search(c.queries, 128, 10)
        assert np.array_equal(ids, ref_ids)


def test_slot_form_of_the_graph_and_deleted_bits():
    c = cases.random_case("l2", 4000, 40, 32, 50, seed=21)
    degs = (c.adj >= 0).sum(1).astype(np.int32)
    with capi.Index(c.n, c.dim, 32, "l2") as ix:
        ix.set_vectors(c.base)
        ix.set_slots(degs, c.adj)          # deg + nbrs[] rows, like the reference's Slot
        ix.set_start_ids(c.start)
        ix.prepare(50, 64, 10)
        ids, d, st, _ = assert_same(c, ix, 64, 10)
        # delete the best hit of every query: the output must skip it and keep the order
        bits = np.zeros((c.n + 31) // 32, np.uint32)
        for v in np.unique(ids[:, 0]):
            bits[v >> 5] |= np.uint32(1 << (v & 31))
        ix.set_deleted(bits)
        ids2, d2, _, _ = ix.search(c.queries, 64, 10)
        ref_ids, ref_d, _ = oracle.search(c.base, c.adj, c.start, c.queries, 64, 64, "l2")
        dead = lambda v: (bits[v >> 5] >> np.uint32(v & 31)) & 1
        for qi in range(len(c.queries)):
            keep = [v for v in ref_ids[qi] if v >= 0 and not dead(v)][:10]
            assert list(ids2[qi][:len(keep)]) == keep
        ix.set_deleted(None)
        assert_same(c, ix, 64, 10)


def test_empty_and_single_query_batches_and_limits():
    c = cases.structured("l2")
    with make_index(c, len(c.queries), 64, 10) as ix:
        ids, d, st, hops = ix.search(c.queries[:0], 64, 10, stats=True)
        assert ids.shape == (0, 10) and hops == 0
        assert_same(c, ix, 64, 10, queries=c.queries[:1])
        with pytest.raises(capi.CoralError) as e:
            ix.search(c.queries, 128, 10)            # L above what prepare sized
        assert e.value.code == capi.ERR_LIMIT
        with pytest.raises(capi.CoralError) as e:
            ix.search(c.queries, 8, 10)              # k > L
        assert e.value.code == capi.ERR_ARG
        assert_same(c, ix, 64, 10)                   # the handle is still usable


def test_count_hits_matches_reference_recall_definition():
    c = cases.structured("ip")
    import torch
    from coral_b200 import synth
    gt = synth.exact_knn(torch.from_numpy(c.base), torch.from_numpy(c.queries), 100, "ip").numpy()
    with make_index(c, len(c.queries), 128, 10) as ix:
        ids, _, _, _ = ix.search(c.queries, 128, 10)
        hits = ix.count_hits(ids, gt, 10)
        assert hits == round(oracle.recall(ids, gt, 10) * 10 * len(c.queries))
        assert hits / (10 * len(c.queries)) > 0.5     # a sane graph, not a recall benchmark


def test_merge_shards_matches_oracle():
    import torch
    rng = np.random.default_rng(1)
    G, Q, k = 8, 300, 100
    ids = rng.integers(0, 1 << 30, size=(G, Q, k)).astype(np.int32)
    d = np.sort(rng.standard_normal((G, Q, k)).astype(np.float32), axis=2)
    ids[:, :, 90:][rng.random((G, Q, 10)) < 0.3] = -1        # ragged shards
    d[0, :, 5] = d[1, :, 5]                                   # cross-shard distance ties
    c = cases.structured("l2")
    for metric in ("l2", "ip"):
        dd = d if metric == "l2" else -d
        with capi.Index(c.n, c.dim, 32, metric) as ix:
            oi, od = ix.merge_shards(torch.from_numpy(ids).cuda(), torch.from_numpy(dd).cuda())
            torch.cuda.synchronize()
        ri, rd = oracle.merge_shards(ids, dd, metric)
        assert np.array_equal(oi.cpu().numpy(), ri)
        assert np.array_equal(od.cpu().numpy().view(np.uint32), rd.view(np.uint32))


def test_committed_fixture():
    import os
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "beam_search_small.npz"))
    for tag in ("l2", "ip"):
        base, adj = z[f"{tag}_base"], z[f"{tag}_adj"]
        L, k = int(z[f"{tag}_L"]), int(z[f"{tag}_k"])
        with capi.Index(base.shape[0], base.shape[1], int(z[f"{tag}_deg"]), tag) as ix:
            ix.set_vectors(base)
            ix.set_adjacency(adj)
            ix.set_start_ids(z[f"{tag}_start"])
            ix.prepare(64, L, k)
            ids, d, st, _ = ix.search(z[f"{tag}_queries"], L, k, stats=True)
        assert np.array_equal(ids, z[f"{tag}_ids"])
        assert np.array_equal(d.view(np.uint32), z[f"{tag}_dists"].view(np.uint32))
        assert np.array_equal(st[:, :7], z[f"{tag}_stats"][:, :7])


def test_sharded_entry_point_on_one_rank_equals_search_plus_id_map():
    """coral_search_sharded with a one-rank communicator: local search, id mapping, the NCCL
    all-gather (a copy at world 1) and the slice merge must reproduce coral_search's rows with
    the ids sent through the id map."""
    import torch
    from coral_b200 import sharded
    c = cases.structured("ip")
    rng = np.random.default_rng(4)
    id_map = rng.permutation(10 * c.n)[:c.n].astype(np.int32)        # any injective local -> global map
    with make_index(c, len(c.queries), 128, 100) as ix:
        comm = sharded.Communicator.from_torch(0)
        sh = sharded.ShardedIndex(ix, torch.from_numpy(id_map).cuda(), comm)
        dq = torch.from_numpy(c.queries).cuda()
        for L, k in [(64, 10), (128, 100)]:
            want_ids, want_d, _, _ = ix.search(c.queries, L, k)
            torch.cuda.synchronize()
            ids, d, lo, hi = sh.search(dq, L, k)
            torch.cuda.synchronize()
            ix.check()
            assert (lo, hi) == (0, len(c.queries))
            assert np.array_equal(ids.cpu().numpy(), id_map[want_ids])
            assert np.array_equal(d.cpu().numpy().view(np.uint32), want_d.view(np.uint32))
        comm.close()


@pytest.mark.parametrize("metric", ["l2", "ip"])
def test_tensor_core_scheduling_keys_and_the_deterministic_order(metric):
    """The pre-pass that orders large batches: keys from the tcgen05 dense scan (exact nearest
    frontier row after the re-rank) or from the fp32 SIMT tiles; either way the order is a
    permutation, the same on every call, and results stay at their own rows."""
    import torch
    c = cases.structured(metric)
    reps = np.concatenate([c.queries] * 50)[:4500]          # > 4096 queries: the tensor-core path is set up
    ref_ids, ref_d, ref_st = oracle.search(c.base, c.adj, c.start, c.queries, 64, 10, c.metric)
    orders = {}
    for tc in (1, 0):
        with make_index(c, len(reps), 64, 10, options={"schedule": 1, "schedule_tc": tc}) as ix:
            ids, d, st, _ = ix.search(reps, 64, 10, stats=True)
            assert ix.get_option("last_scheduled") == 1
            for r in range(0, len(reps), len(c.queries)):
                m = min(len(c.queries), len(reps) - r)
                assert np.array_equal(ids[r:r + m], ref_ids[:m]) and np.array_equal(st[r:r + m, :7], ref_st[:m, :7])
            dq = torch.from_numpy(reps).cuda()
            o1 = ix.query_order(dq)
            o2 = ix.query_order(dq)
            torch.cuda.synchronize()
            o1, o2 = o1.cpu().numpy(), o2.cpu().numpy()
            assert np.array_equal(o1, o2)                                   # deterministic
            assert np.array_equal(np.sort(o1), np.arange(len(reps)))        # a permutation
            orders[tc] = o1
    # identical queries share a key, so they keep their row order (the sort is stable) in both variants
    for o in orders.values():
        pos = np.empty(len(reps), np.int64)
        pos[o] = np.arange(len(reps))
        copies = np.arange(7, len(reps), len(c.queries))                  # the copies of query 7
        assert np.array_equal(np.sort(pos[copies]), pos[copies])
