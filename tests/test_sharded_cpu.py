"""Host-side logic of the multi-GPU layer on CPU ranks (gloo, world_size 2 and 3): query
slicing, random partition + id maps, the single all-gather exchange, and the merge
definition.  The local searcher is exact brute force, so the merged answer must equal the
exact global k-NN whatever the partition -- a size-independent property of shard+merge."""
import os
import tempfile
from datetime import timedelta

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from coral_b200 import sharded
from oracle import oracle


def test_query_slices_cover_the_batch_exactly():
    for q in (0, 1, 7, 100000):
        for world in (1, 2, 3, 8):
            cuts = [sharded.query_slice(q, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == q
            assert all(cuts[i][1] == cuts[i + 1][0] for i in range(world - 1))
            assert max(h - l for l, h in cuts) - min(h - l for l, h in cuts) <= 1


def test_partition_is_balanced_and_id_maps_are_a_bijection():
    a = sharded.random_partition(10001, 8)
    counts = np.bincount(a, minlength=8)
    assert counts.max() - counts.min() <= 1
    allids = np.concatenate([sharded.shard_ids(a, r) for r in range(8)])
    assert np.array_equal(np.sort(allids), np.arange(10001))
    inter = np.concatenate([sharded.interleaved_ids(5, 4, r) for r in range(4)])
    assert np.array_equal(np.sort(inter), np.arange(20))


def _exact_local(base, metric):
    def fn(q, L, k):
        qn, bn = q.numpy(), base
        s = qn @ bn.T if metric == "ip" else -((qn[:, None, :] - bn[None, :, :]) ** 2).sum(2)
        kk = min(k, bn.shape[0])
        order = np.lexsort((np.broadcast_to(np.arange(bn.shape[0]), s.shape), -s), axis=1)[:, :kk]
        d = np.take_along_axis(s if metric == "ip" else -s, order, 1).astype(np.float32)
        ids = np.full((qn.shape[0], k), -1, np.int32)
        dd = np.full((qn.shape[0], k), -3.4e38 if metric == "ip" else 3.4e38, np.float32)
        ids[:, :kk], dd[:, :kk] = order, d
        return torch.from_numpy(ids), torch.from_numpy(dd)
    return fn


def _worker(rank, world, store, metric, out_dir):
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method=f"file://{store}",
                            timeout=timedelta(seconds=60))
    rng = np.random.default_rng(5)
    base = rng.standard_normal((900, 24)).astype(np.float32)
    q = torch.from_numpy(rng.standard_normal((40, 24)).astype(np.float32))
    assign = sharded.random_partition(len(base), world, seed=9)
    mine = sharded.shard_ids(assign, rank)

    def merge(ids, dists):
        oi, od = oracle.merge_shards(ids.numpy(), dists.numpy(), metric)
        return torch.from_numpy(oi), torch.from_numpy(od)

    ids, dists = sharded.sharded_search(_exact_local(base[mine], metric), torch.from_numpy(mine), q, 0, 10, merge)
    np.save(os.path.join(out_dir, f"ids{rank}.npy"), ids.numpy())
    np.save(os.path.join(out_dir, f"d{rank}.npy"), dists.numpy())
    dist.destroy_process_group()


@pytest.mark.parametrize("world,metric", [(2, "l2"), (3, "ip")])
def test_shard_and_merge_equals_exact_global_knn(world, metric):
    with tempfile.TemporaryDirectory() as tmp:
        store = os.path.join(tmp, "store")
        mp.spawn(_worker, args=(world, store, metric, tmp), nprocs=world, join=True)
        rng = np.random.default_rng(5)
        base = rng.standard_normal((900, 24)).astype(np.float32)
        q = torch.from_numpy(rng.standard_normal((40, 24)).astype(np.float32))
        want_ids, want_d = _exact_local(base, metric)(q, 0, 10)
        for r in range(world):          # every rank holds the same merged answer
            assert np.array_equal(np.load(os.path.join(tmp, f"ids{r}.npy")), want_ids.numpy())
            assert np.allclose(np.load(os.path.join(tmp, f"d{r}.npy")), want_d.numpy(), rtol=1e-6, atol=1e-6)


def _lonely(rank, world, store, out):
    # rank 1 never joins the collective: rank 0's all-gather must end with an error, not hang
    if rank == 1:
        dist.init_process_group("gloo", rank=rank, world_size=world, init_method=f"file://{store}",
                                timeout=timedelta(seconds=5))
        return
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method=f"file://{store}",
                            timeout=timedelta(seconds=5))
    ids = torch.zeros((4, 3), dtype=torch.int32)
    try:
        sharded.all_gather_results(ids, torch.zeros((4, 3)))
        open(out, "w").write("no error")
    except Exception as e:          # a host-side failure, reported to the caller
        open(out, "w").write("error: " + type(e).__name__)


def test_missing_rank_surfaces_as_an_error_on_the_host():
    with tempfile.TemporaryDirectory() as tmp:
        out = os.path.join(tmp, "result")
        mp.spawn(_lonely, args=(2, os.path.join(tmp, "store"), out), nprocs=2, join=True)
        assert open(out).read().startswith("error")
