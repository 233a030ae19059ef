"""Oracle parity at the sizes of the benchmark configurations that fit a test run.

Config 1 (1M x 200, L2, degree 32) and config 2 (1M x 512, inner product, degree 32): EVERY one of
the 10 000 queries at every configured beam capacity, ids, distance bits and the seven per-query
counters equal to the CPU oracle's; k = 10 and k = 100 for config 1 (k only cuts the output, so one
oracle pass at k = 100 checks both).  Config 4: one 12.5M x 200 shard, k = 100, L in {128, 256},
256 sampled queries, and the merge of two small shards against the oracle's merge.
"""
import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu


def _np(x):
    return x.cpu().numpy() if hasattr(x, "cpu") else np.asarray(x)


def _build(config, n=None, nq=10_000, draw_seed=None):
    """Synthetic data of a benchmark configuration and its graph, built by the library on this GPU."""
    import torch
    from coral_b200 import capi, synth
    c = synth.CONFIGS[config]
    ds = synth.make_config(config, 100_000, nq, n=n, device="cuda", draw_seed=draw_seed)
    ix = capi.Index(ds.base.shape[0], c["dim"], c["deg"], c["kind"])
    ix.attach_vectors(ds.base)
    ix.build(ds.train, kb=100)
    ds.train = None
    torch.cuda.empty_cache()
    g = synth.Graph(ix.get_adjacency_tensor("cuda"), torch.from_numpy(ix.get_start_ids()), c["deg"])
    return ds, g, ix


def _check_all(ix, ds, g, metric, Ls, ks, rows=None):
    base, adj, start = _np(ds.base), _np(g.adj), _np(g.start_ids)
    test = _np(ds.test)
    rows = np.arange(test.shape[0]) if rows is None else rows
    kmax = max(ks)
    for L in Ls:
        ref_ids, ref_d, ref_st = oracle.search(base, adj, start, test[rows], L, min(kmax, L), metric)
        for k in ks:
            if k > L:
                continue
            ids, d, st, hops = ix.search(ds.test, L, k, dists=True, stats=True)
            ids, d, st = _np(ids)[rows], _np(d)[rows], _np(st)[rows]
            tag = f"{metric} L={L} k={k}"
            assert np.array_equal(ids, ref_ids[:, :k]), f"{tag}: ids differ"
            assert np.array_equal(d.view(np.uint32), ref_d[:, :k].view(np.uint32)), f"{tag}: distance bits differ"
            assert np.array_equal(st[:, :7], ref_st[:, :7]), f"{tag}: counters differ"
            if len(rows) == test.shape[0]:
                assert hops == int(ref_st[:, 4].sum())


def test_config1_every_query_every_L_both_k():
    ds, g, ix = _build("c1")
    with ix:
        ix.prepare(10_000, 512, 100)
        _check_all(ix, ds, g, "l2", [64, 128, 256, 512], [10, 100])


def test_config2_every_query_every_L():
    ds, g, ix = _build("c2")
    with ix:
        ix.prepare(10_000, 256, 10)
        _check_all(ix, ds, g, "ip", [64, 128, 256], [10])


def test_config4_one_full_size_shard_k100():
    import torch
    if torch.cuda.mem_get_info()[1] < 100e9:
        pytest.skip("needs a GPU with the shard's memory")
    ds, g, ix = _build("c4", nq=100_000, draw_seed=20261001)
    with ix:
        ix.prepare(100_000, 256, 100)
        rows = np.arange(0, 100_000, 100_000 // 256)[:256]
        _check_all(ix, ds, g, "l2", [128, 256], [100], rows=rows)


def test_config4_merge_of_two_shards_equals_the_oracle_merge():
    """Two 200k-point shards of one mixture, every query on both, k = 100: per-shard results equal the
    oracle's, and the library's merge of the two (global ids) equals the oracle's merge."""
    import torch
    from coral_b200 import sharded
    G, n_local, nq, L, k = 2, 200_000, 512, 128, 100
    per_shard, handles = [], []
    try:
        for r in range(G):
            ds, g, ix = _build("c4", n=n_local, nq=nq, draw_seed=20261001 + r)
            handles.append(ix)
            ix.prepare(nq, L, k)
            ids, d, st, _ = ix.search(ds.test, L, k, dists=True, stats=True)
            ref_ids, ref_d, ref_st = oracle.search(_np(ds.base), _np(g.adj), _np(g.start_ids), _np(ds.test), L, k, "l2")
            assert np.array_equal(_np(ids), ref_ids) and np.array_equal(_np(d).view(np.uint32), ref_d.view(np.uint32))
            id_map = torch.from_numpy(sharded.interleaved_ids(n_local, G, r)).cuda()
            ix.map_ids(ids, id_map)
            torch.cuda.synchronize()
            gl = np.where(ref_ids >= 0, sharded.interleaved_ids(n_local, G, r)[np.maximum(ref_ids, 0)], ref_ids)
            assert np.array_equal(_np(ids), gl)
            per_shard.append((ids, d, gl, ref_d))
        all_ids = torch.stack([p[0] for p in per_shard]).contiguous()
        all_d = torch.stack([p[1] for p in per_shard]).contiguous()
        m_ids, m_d = handles[0].merge_shards(all_ids, all_d)
        torch.cuda.synchronize()
        o_ids, o_d = oracle.merge_shards(np.stack([p[2] for p in per_shard]), np.stack([p[3] for p in per_shard]), "l2")
        assert np.array_equal(_np(m_ids), o_ids) and np.array_equal(_np(m_d).view(np.uint32), o_d.view(np.uint32))
    finally:
        for h in handles:
            h.close()
