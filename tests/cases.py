"""Seeded small cases shared by the CPU and GPU tests."""
from __future__ import annotations

import functools

import numpy as np
import torch

from coral_b200 import synth


class Case:
    def __init__(self, name, base, adj, start, queries, metric, max_degree):
        self.name, self.metric, self.max_degree = name, metric, max_degree
        self.base = np.ascontiguousarray(base, dtype=np.float32)
        self.adj = np.ascontiguousarray(adj, dtype=np.int32)
        self.start = np.ascontiguousarray(start, dtype=np.int32)
        self.queries = np.ascontiguousarray(queries, dtype=np.float32)

    @property
    def n(self):
        return self.base.shape[0]

    @property
    def dim(self):
        return self.base.shape[1]


@functools.lru_cache(maxsize=None)
def structured(metric: str, n: int = 12000, dim: int | None = None, deg: int = 32, nq: int = 96) -> Case:
    """A CORAL graph -- the reference's build (exact lists -> NAP -> CE), run by its CPU restatement --
    on clustered cross-modal data with overlapping clusters."""
    from oracle import oracle
    if metric == "l2":
        d = dim or 200
        ds = synth.make_l2_mixture(n, n // 4, nq, dim=d, centers=max(2, n // 1000), seed=11, rot_dims=min(60, d),
                                   latent_dim=8, latent_jitter=0.5)
    else:
        ds = synth.make_ip_cones(n, n // 4, nq, dim=dim or 512, clusters=max(2, n // 1500), seed=12, latent_dim=8,
                                 latent_jitter=0.5)
    base = ds.base.numpy()
    knn, _ = oracle.exact_knn(base, ds.train.numpy(), 50, metric)
    st, start = oracle.build_graph(base, knn, metric, deg, batch=512, ce_L=128, ce_search_batch=4096, ce_nap_batch=1024)
    return Case(f"structured_{metric}_{n}x{base.shape[1]}_d{deg}", base, st.adj, start, ds.test.numpy(), metric, deg)


@functools.lru_cache(maxsize=None)
def random_case(metric: str, n: int, dim: int, deg: int, nq: int, m: int = 16, seed: int = 5,
                min_degree: int = 0, dup_start: bool = False, quantized: bool = False) -> Case:
    """Random vectors on a random ragged-degree graph: exercises the mechanics, not recall.
    `quantized` draws coordinates from a few integers so that many distances tie exactly."""
    rng = np.random.default_rng(seed)
    if quantized:
        base = rng.integers(-2, 3, size=(n, dim)).astype(np.float32)
        q = rng.integers(-2, 3, size=(nq, dim)).astype(np.float32)
    else:
        base = rng.standard_normal((n, dim), dtype=np.float32)
        q = rng.standard_normal((nq, dim), dtype=np.float32)
    if metric == "ip" and not quantized:
        base /= np.linalg.norm(base, axis=1, keepdims=True)
        q /= np.linalg.norm(q, axis=1, keepdims=True)
    g = synth.random_graph(n, deg, n_start=m, seed=seed + 1, min_degree=min_degree)
    start = g.start_ids.numpy().copy()
    if dup_start and m >= 2:
        start[1] = start[0]
    return Case(f"random_{metric}_{n}x{dim}_d{deg}_m{m}", base, g.adj.numpy(), start, q, metric, deg)


def chain_case(n: int = 40, dim: int = 8) -> Case:
    """A graph whose reachable set is smaller than the beam: node i -> i+1 up to node 9."""
    rng = np.random.default_rng(3)
    base = rng.standard_normal((n, dim), dtype=np.float32)
    q = rng.standard_normal((5, dim), dtype=np.float32)
    adj = np.full((n, 32), -1, np.int32)
    for i in range(9):
        adj[i, 0] = i + 1
    return Case("chain", base, adj, np.array([0], np.int32), q, "l2", 32)
