"""Delete with topology repair and insert on the GPU against the CPU restatement of the reference's
update kernels (oracle/build_oracle.c: src/update.cu:101-197,312-391,499-629,674-959): after every
operation the adjacency, the stored edge distances and the degrees must be identical, and so must
the entry points and the search results on the updated graph."""
import numpy as np
import pytest

from coral_b200 import capi, synth
from oracle import oracle

pytestmark = pytest.mark.gpu


def _equal(tag, ix, st):
    adj, dd, deg = ix.build_get_graph()
    assert np.array_equal(deg, st.deg), f"{tag}: degrees differ"
    bad = np.nonzero((adj != st.adj).any(1))[0]
    assert len(bad) == 0, f"{tag}: {len(bad)} rows differ, first {bad[:5]}"
    mask = adj >= 0
    assert np.array_equal(dd.view(np.uint32)[mask], st.ndist.view(np.uint32)[mask]), f"{tag}: edge distances differ"


@pytest.mark.parametrize("metric,n,dim,deg,kb", [("l2", 12000, 64, 32, 50), ("ip", 10000, 96, 64, 64)])
def test_delete_then_insert_matches_the_restated_reference_kernels(metric, n, dim, deg, kb):
    extra = n // 20                                   # 5 % new points, kept behind the live rows
    if metric == "l2":
        ds = synth.make_l2_mixture(n + extra, n // 4, 64, dim=dim, centers=12, seed=5, rot_dims=min(60, dim), latent_dim=8,
                                   latent_jitter=0.5)
    else:
        ds = synth.make_ip_cones(n + extra, n // 4, 64, dim=dim, clusters=8, seed=6, latent_dim=8, latent_jitter=0.5)
    base, train, test = ds.base.numpy(), ds.train.numpy(), ds.test.numpy()
    rng = np.random.default_rng(9)
    del_ids = rng.choice(n, n // 10, replace=False).astype(np.int32)      # 10 % of the points, random order
    with capi.Index(n + extra, dim, deg, metric) as ix:
        ix.set_vectors(base)
        ix.set_live(n)
        info = ix.build(train, kb=kb)
        # the oracle starts from the graph the GPU built (its build parity is tested elsewhere)
        adj0 = ix.get_adjacency()
        st = oracle.state_from_adjacency(base, adj0, deg, metric)
        ix.update_begin()
        _equal("update_begin", ix, st)
        # ---- delete with repair
        dead = np.zeros(n + extra, bool)
        ix.delete(del_ids)
        start = oracle.delete_nodes(base, st, dead, del_ids, metric, live=n)
        _equal("delete", ix, st)
        assert np.array_equal(ix.get_start_ids(), start)
        live_rows = ~dead[:n]
        assert not dead[st.adj[:n][live_rows][st.adj[:n][live_rows] >= 0]].any()    # no live row points at a deleted node
        ix.prepare(len(test), 128, 10)
        got, _, _, _ = ix.search(test, 128, 10)
        want = oracle.search_hiding(base, st.adj, start, test, 128, 10, metric, dead)
        assert np.array_equal(got, want)
        # ---- insert 5 % new points, neighbours from the search
        ix.insert(n, extra, kb, L=128, batch=256)
        start = oracle.insert_nodes(base, st, dead, n, extra, kb, metric, L=128, batch=256)
        _equal("insert", ix, st)
        assert np.array_equal(ix.get_start_ids(), start)
        assert (st.deg[n:] > 0).all()
        ix.prepare(len(test), 128, 10)
        got, _, _, _ = ix.search(test, 128, 10)
        want = oracle.search_hiding(base, st.adj, start, test, 128, 10, metric, dead)
        assert np.array_equal(got, want)
        # recall against the exact neighbours among the points that exist now
        alive = np.nonzero(~dead)[0]
        gt_local, _ = oracle.exact_knn(base[alive], test, 10, metric)
        assert oracle.recall(got, alive[gt_local].astype(np.int32), 10) >= 0.85
        ix.build_end()
