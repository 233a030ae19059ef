"""Multi-GPU layer: one process per GPU, one index handle per process.

Two modes, as the search path allows (the reference itself is single-GPU):

* replicated index -- every rank holds the whole index and searches a contiguous slice of
  the query batch (`query_slice`); there is no collective on the data path.
* sharded index -- the base is partitioned, every rank holds one shard with its own graph
  and entry points and searches ALL queries; the per-shard top-k (global ids, distances)
  are exchanged with ONE all-gather and merged per query by (distance, id).

On GPUs the whole sharded step is ONE call into the C library (`coral_search_sharded`: local
search, id mapping, one ncclAllGather on the caller's stream, merge of this rank's slice of the
batch); `Communicator` only carries the NCCL unique id from rank 0 to the others through
`torch.distributed`.  The pure-Python `sharded_search` states the same exchange over any
`torch.distributed` backend with an injected local searcher, so that the logic can be exercised
on CPU ranks (gloo).
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


def sorted_slice(order: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Rows of the batch `rank` searches when the index is replicated and the batch has been ordered
    for locality (`order[i]` = the i-th query to run): the rank-th contiguous range of the ORDERED
    batch, so every GPU sees 1/world of the graph regions at full multiplicity instead of all of
    them thinly.  Returns the original row numbers (results go back to those rows)."""
    lo, hi = query_slice(int(order.numel()), world, rank)
    return order[lo:hi]


class Communicator:
    """The library's NCCL communicator (coral_comm_*), one per process and GPU."""

    def __init__(self, device: int, world: int, rank: int, unique_id: bytes):
        import ctypes as C
        from . import capi
        self._lib = capi.load()
        self._c = C.c_void_p()
        buf = C.create_string_buffer(unique_id, 128)
        rc = self._lib.coral_comm_create(C.byref(self._c), int(device), int(world), int(rank), buf)
        if rc != 0:
            raise capi.CoralError(rc, self._lib.coral_comm_last_error(None).decode())
        self.world, self.rank, self.device = world, rank, device

    @staticmethod
    def unique_id() -> bytes:
        import ctypes as C
        from . import capi
        lib = capi.load()
        buf = C.create_string_buffer(128)
        rc = lib.coral_comm_unique_id(buf)
        if rc != 0:
            raise capi.CoralError(rc, lib.coral_comm_last_error(None).decode())
        return buf.raw

    @classmethod
    def from_torch(cls, device: int, group=None) -> "Communicator":
        """Collective: rank 0 makes the unique id, torch.distributed carries it to the others."""
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return cls(device, 1, 0, cls.unique_id())
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [cls.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=group)
        return cls(device, world, rank, box[0])

    def close(self):
        if self._c:
            self._lib.coral_comm_destroy(self._c)
            import ctypes as C
            self._c = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ShardedIndex:
    """A shard's index handle, its local->global id map and the communicator, searched collectively."""

    def __init__(self, index, id_map: torch.Tensor, comm: Communicator):
        self.index, self.comm = index, comm
        self.id_map = id_map.to(torch.int32).contiguous() if id_map is not None else None

    def search(self, queries: torch.Tensor, L: int, k: int, stream=None, out=None):
        """queries: CUDA tensor [Q, dim], the same on every rank.  Enqueues the whole step on `stream`
        (an int cudaStream_t; None = the legacy default stream) and returns this rank's slice of the
        merged batch: (ids[hi-lo, k], dists[hi-lo, k], lo, hi), CUDA tensors (`out` = a reusable pair)."""
        import ctypes as C
        from . import capi
        Q = int(queries.shape[0])
        lo, hi = query_slice(Q, self.comm.world, self.comm.rank)
        if out is None:
            out = (torch.empty((hi - lo, k), dtype=torch.int32, device=queries.device),
                   torch.empty((hi - lo, k), dtype=torch.float32, device=queries.device))
        ids, dists = out
        rc = self.index._lib.coral_search_sharded(
            self.index._h, self.comm._c, C.c_void_p(self.id_map.data_ptr()) if self.id_map is not None else None,
            C.c_void_p(queries.data_ptr()), Q, L, k, C.c_void_p(ids.data_ptr()), C.c_void_p(dists.data_ptr()),
            C.c_void_p(stream) if stream else None)
        if rc != 0:
            raise capi.CoralError(rc, self.index._lib.coral_comm_last_error(self.comm._c).decode())
        return ids, dists, lo, hi
