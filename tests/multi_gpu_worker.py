"""Run under torchrun with 2+ GPUs (one rank per GPU): replicated-and-split and
shard-and-merge searches, both compared bit for bit with the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from coral_b200 import capi, sharded, synth  # noqa: E402
from oracle import oracle  # noqa: E402
from tests import cases  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{local}"))
    c = cases.structured("l2")
    L, k = 64, 10

    # --- replicated index, queries split: no collective on the data path
    lo, hi = sharded.query_slice(len(c.queries), world, rank)
    with capi.Index(c.n, c.dim, c.max_degree, c.metric, device=local) as ix:
        ix.set_vectors(c.base)
        ix.set_adjacency(c.adj)
        ix.set_start_ids(c.start)
        ix.prepare(len(c.queries), L, k)
        ids, d, _, _ = ix.search(c.queries[lo:hi], L, k)
    ref_ids, ref_d, _ = oracle.search(c.base, c.adj, c.start, c.queries, L, k, c.metric)
    assert np.array_equal(ids, ref_ids[lo:hi]) and np.array_equal(d.view(np.uint32), ref_d[lo:hi].view(np.uint32))

    # --- sharded index: random partition, one graph per shard, all queries on every shard
    assign = sharded.random_partition(c.n, world, seed=3)
    shards = []
    for r in range(world):
        ids_r = sharded.shard_ids(assign, r)
        base_r = torch.from_numpy(c.base[ids_r])
        g_r = synth.random_graph(len(ids_r), 32, n_start=16, seed=50 + r)     # any per-shard graph will do
        shards.append((ids_r, base_r.numpy(), g_r.adj.numpy(), g_r.start_ids.numpy()))
    ids_r, base_r, adj_r, start_r = shards[rank]
    dq = torch.from_numpy(c.queries).cuda()
    with capi.Index(len(ids_r), c.dim, 32, c.metric, device=local) as ix:
        ix.set_vectors(base_r)
        ix.set_adjacency(adj_r)
        ix.set_start_ids(start_r)
        ix.prepare(len(c.queries), L, k)
        comm = sharded.Communicator.from_torch(local)
        sh = sharded.ShardedIndex(ix, torch.from_numpy(ids_r).cuda(), comm)
        torch.cuda.synchronize()
        m_ids, m_d, s_lo, s_hi = sh.search(dq, L, k)          # this rank's slice of the merged batch
        torch.cuda.synchronize()
        ix.check()
        m_ids, m_d = m_ids.cpu().numpy(), m_d.cpu().numpy()
        assert (s_lo, s_hi) == sharded.query_slice(len(c.queries), world, rank)
        comm.close()
    per = [oracle.search(b, a, s, c.queries, L, k, c.metric) for (_, b, a, s) in shards]
    g_ids = np.stack([np.where(p[0] >= 0, shards[r][0][np.maximum(p[0], 0)], -1) for r, p in enumerate(per)])
    o_ids, o_d = oracle.merge_shards(g_ids, np.stack([p[1] for p in per]), c.metric)
    assert np.array_equal(m_ids, o_ids[s_lo:s_hi]) and np.array_equal(m_d.view(np.uint32), o_d[s_lo:s_hi].view(np.uint32))
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK world=%d" % world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
