"""The GPU graph build (exact k-NN lists -> neighbourhood-aware projection -> connectivity
enhancement) against the CPU restatement of the reference's build kernels
(oracle/build_oracle.c: src/upd_gpu.cu:12-303, src/enhance.cu:136-212,344-389,528-580).
Bar: the adjacency, the stored edge distances (bit patterns) and the degrees are identical
after every stage, and so are the entry points the enhancement leaves installed."""
import numpy as np
import pytest

from coral_b200 import capi, synth
from oracle import oracle

pytestmark = pytest.mark.gpu


def _dataset(metric, n, dim, n_train, nq, seed):
    if metric == "l2":
        ds = synth.make_l2_mixture(n, n_train, nq, dim=dim, centers=max(2, n // 1000), seed=seed, rot_dims=min(60, dim),
                                   latent_dim=8, latent_jitter=0.5)
    else:
        ds = synth.make_ip_cones(n, n_train, nq, dim=dim, clusters=max(2, n // 1500), seed=seed, latent_dim=8,
                                 latent_jitter=0.5)
    return ds.base.numpy(), ds.train.numpy(), ds.test.numpy()


def _assert_graph_equal(tag, got, want):
    adj, dd, deg = got
    assert np.array_equal(deg, want.deg), f"{tag}: degrees differ"
    assert np.array_equal(adj, want.adj), f"{tag}: adjacency differs"
    mask = adj >= 0
    assert np.array_equal(dd.view(np.uint32)[mask], want.ndist.view(np.uint32)[mask]), f"{tag}: edge distances differ"


@pytest.mark.parametrize("metric,n,dim,deg,kb,n_train", [
    ("l2", 20000, 64, 32, 50, 3000),
    ("ip", 12000, 96, 64, 100, 2500),
    ("l2", 6000, 200, 32, 100, 700),
])
def test_nap_and_ce_match_the_restated_reference_kernels(metric, n, dim, deg, kb, n_train):
    base, train, test = _dataset(metric, n, dim, n_train, 64, seed=n + dim)
    with capi.Index(n, dim, deg, metric) as ix:
        ix.set_vectors(base)
        knn, _, bad = ix.exact_knn(train, kb, dists=False)
        ref_knn, _ = oracle.exact_knn(base, train, kb, metric)
        assert np.array_equal(knn, ref_knn) and bad == 0
        # ---- NAP, batch after batch, every batch compared
        ix.build_begin()
        st = oracle.BuildState(n, deg)
        batch = 256
        for s in range(0, n_train, batch):
            ix.build_nap(knn[s:s + batch], batch)
            oracle.nap_batch(base, st, knn[s:s + batch], metric)
            if s in (0, batch, (n_train // batch) * batch - batch):
                _assert_graph_equal(f"NAP batch at {s}", ix.build_get_graph(), st)
        _assert_graph_equal("NAP", ix.build_get_graph(), st)
        assert (st.deg == 0).sum() > n // 10           # plenty of isolated nodes for the enhancement
        # ---- CE with small batches so that several search batches and many update batches run
        n_iso = ix.build_connect_enhance(kb, L=128, search_batch=3000, nap_batch=500, M=16)
        iso = np.nonzero(st.deg == 0)[0].astype(np.int32)
        assert n_iso == len(iso)
        start = None
        first_connected = int(np.nonzero(st.deg > 0)[0][0])      # fixed for the whole enhancement
        for s in range(0, len(iso), 3000):
            chunk = iso[s:s + 3000]
            start = oracle.select_start_ids(st.adj, first_connected, 16)
            ids, dists, _ = oracle.search(base, st.adj, start, base[chunk], 128, kb, metric)
            for j in range(0, len(chunk), 500):
                oracle.ce_batch(base, st, chunk[j:j + 500], ids[j:j + 500], dists[j:j + 500], metric)
        got = ix.build_get_graph()
        bad_rows = np.nonzero((got[0] != st.adj).any(1))[0]
        assert len(bad_rows) == 0, (f"CE: {len(bad_rows)} rows differ, first {bad_rows[:5]}; isolated before CE: "
                                    f"{np.isin(bad_rows[:5], iso)}; positions in iso: {np.searchsorted(iso, bad_rows[:5])}")
        _assert_graph_equal("CE", got, st)
        assert (st.deg > 0).all()
        # ---- the finished graph is searchable and finds the neighbours
        ix.prepare(len(test), 128, 10)
        got, _, _, _ = ix.search(test, 128, 10)
        ref, _, _ = oracle.search(base, st.adj, start, test, 128, 10, metric)
        assert np.array_equal(got, ref)
        gt, _ = oracle.exact_knn(base, test, 10, metric)
        assert oracle.recall(got, gt, 10) >= 0.9
        ix.build_end()


def test_build_limits_are_refused():
    base, train, _ = _dataset("l2", 2000, 32, 100, 8, seed=1)
    with capi.Index(2000, 32, 32, "l2") as ix:
        ix.set_vectors(base)
        with pytest.raises(capi.CoralError) as e:
            ix.build_nap(np.zeros((4, 50), np.int32))
        assert e.value.code == capi.ERR_STATE            # build_begin first
        ix.build_begin()
        with pytest.raises(capi.CoralError) as e:
            ix.build_nap(np.zeros((4, 200), np.int32))
        assert e.value.code == capi.ERR_LIMIT            # k_b <= 128
        with pytest.raises(capi.CoralError) as e:
            ix.build_connect_enhance(50)                 # nothing is connected yet: no entry point exists
        assert e.value.code == capi.ERR_STATE
