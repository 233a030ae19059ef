"""Multi-GPU layer: one process per GPU, one index handle per process.

Two modes, as the search path allows (the reference itself is single-GPU):

* replicated index -- every rank holds the whole index and searches a contiguous slice of
  the query batch (`query_slice`); there is no collective on the data path.
* sharded index -- the base is partitioned, every rank holds one shard with its own graph
  and entry points and searches ALL queries; the per-shard top-k (global ids, distances)
  are exchanged with ONE all-gather and merged per query by (distance, id).

`torch.distributed` is the plumbing (NCCL on GPUs, gloo in the CPU tests); the merge runs in
the library's shard-merge kernel on GPUs.  The search itself is injected (`search_fn`) so the
exchange logic can be exercised on CPU ranks with any local searcher.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist


def query_slice(n_queries: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous slice [lo, hi) of the batch that `rank` searches when the index is replicated."""
    return rank * n_queries // world, (rank + 1) * n_queries // world


def random_partition(n: int, world: int, seed: int = 20260004) -> np.ndarray:
    """Balanced random assignment of base ids to `world` shards: int32 [n] of shard numbers."""
    rng = np.random.default_rng(seed)
    perm = rng.permutation(n)
    out = np.empty(n, np.int32)
    out[perm] = (np.arange(n) * world // n).astype(np.int32)
    return out


def shard_ids(assign: np.ndarray, rank: int) -> np.ndarray:
    """Global ids held by `rank`, ascending: position = shard-local id (the local->global map)."""
    return np.nonzero(assign == rank)[0].astype(np.int32)


def interleaved_ids(n_local: int, world: int, rank: int) -> np.ndarray:
    """local->global map when shard r holds global ids r, r+world, r+2*world, ... (what the
    benchmark uses: each rank synthesises its own shard of an i.i.d. mixture)."""
    return (rank + world * np.arange(n_local, dtype=np.int64)).astype(np.int32)


def all_gather_results(ids: torch.Tensor, dists: torch.Tensor, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """One all-gather of the per-shard results.  ids/dists: [Q, k] -> [G, Q, k] on every rank.
    ids and distances travel in a single int32 buffer so that exactly one collective is issued."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return ids[None].contiguous(), dists[None].contiguous()
    packed = torch.stack([ids.contiguous(), dists.contiguous().view(torch.int32)], 0).contiguous()   # [2, Q, k]
    flat = torch.empty(world * packed.numel(), dtype=torch.int32, device=packed.device)
    dist.all_gather_into_tensor(flat, packed.reshape(-1), group=group)
    out = flat.view((world,) + tuple(packed.shape))
    return out[:, 0].contiguous(), out[:, 1].contiguous().view(torch.float32)


def sharded_search(search_fn: Callable, id_map, queries, L: int, k: int, merge_fn: Callable,
                   map_fn: Optional[Callable] = None, group=None):
    """Every rank: local search over all queries -> global ids -> all-gather -> merge.

    search_fn(queries, L, k) -> (ids[Q,k] shard-local, dists[Q,k]) as torch tensors
    id_map: local->global ids (tensor on the results' device), or None when ids are global already
    map_fn(ids, id_map): in-place mapping (the library's kernel on GPUs); default = torch indexing
    merge_fn(ids[G,Q,k], dists[G,Q,k]) -> (ids[Q,k], dists[Q,k])
    """
    ids, dists = search_fn(queries, L, k)
    if id_map is not None:
        if map_fn is not None:
            map_fn(ids, id_map)
        else:
            ids = torch.where(ids >= 0, id_map[ids.clamp(min=0).long()], ids)
    all_ids, all_dists = all_gather_results(ids, dists, group)
    return merge_fn(all_ids, all_dists)


class ShardedIndex:
    """A shard's index handle plus its local->global id map, searched collectively."""

    def __init__(self, index, id_map: torch.Tensor, group=None):
        self.index, self.id_map, self.group = index, id_map.to(torch.int32).contiguous(), group

    def search(self, queries: torch.Tensor, L: int, k: int):
        """queries: CUDA tensor [Q, dim], the same on every rank.  Returns merged (ids, dists)."""
        def local(q, L_, k_):
            ids, dists, _, _ = self.index.search(q, L_, k_, dists=True)
            return ids, dists

        def mapper(ids, id_map):
            self.index.map_ids(ids, id_map)
            torch.cuda.synchronize()

        def merger(all_ids, all_dists):
            torch.cuda.synchronize()       # the gathered buffers were produced on torch's streams,
            out = self.index.merge_shards(all_ids, all_dists)   # the merge runs on the handle's
            torch.cuda.synchronize()
            return out

        return sharded_search(local, self.id_map, queries, L, k, merger, mapper, self.group)
