"""Entry-point selection (farthest-point sampling over BFS hop counts).

The oracle's restatement of the reference's Graph::FPS (src/start.cu:72-145) is checked on the
CPU against an independent pure-Python statement and hand-worked graphs; the device path is
checked against the oracle (ids must be identical: the hop counts are integers and equal
min-hop values resolve to the lowest node id).
"""
from collections import deque

import numpy as np
import pytest

from coral_b200 import synth
from oracle import oracle
from tests import cases

INT_MAX = 2 ** 31 - 1


def python_fps(adj, first, M):
    n = adj.shape[0]
    min_hops = [INT_MAX] * n
    chosen = [first]
    start = first
    while len(chosen) < M:
        hops = [-1] * n
        hops[start] = 0
        todo = deque([start])
        while todo:
            u = todo.popleft()
            for v in adj[u]:
                if 0 <= v < n and hops[v] == -1:
                    hops[v] = hops[u] + 1
                    todo.append(int(v))
        for i in range(n):
            if hops[i] >= 0:
                if hops[i] < min_hops[i] or min_hops[i] < 0:
                    min_hops[i] = hops[i]
            elif min_hops[i] == INT_MAX:
                min_hops[i] = -1
        start = max(range(n), key=lambda i: (min_hops[i], -i))
        chosen.append(start)
    return np.array(chosen, np.int32)


def path_graph(n, deg_pad=4):
    adj = np.full((n, deg_pad), -1, np.int32)
    for i in range(n):
        if i > 0:
            adj[i, 0] = i - 1
        if i + 1 < n:
            adj[i, 1] = i + 1
    return adj


def test_path_graph_by_hand():
    # 0-1-2-...-10, first = 3: farthest is 10 (7 hops); then 0 (3 hops from 3); then the
    # lowest id among nodes at distance 3 from {3, 10, 0}: node 6 (3 from 3) and node 7 (3 from 10).
    got = oracle.select_start_ids(path_graph(11), 3, 4)
    assert got.tolist() == [3, 10, 0, 6]


def test_unreached_nodes_count_as_minus_one_until_reached():
    # Two components {0,1,2} and {3,4}; directed edge 4 -> 0 only.  From 0 nothing reaches 3 or 4
    # (they become -1), so the picks stay inside the first component; once all of it is chosen
    # (min_hops 0) the largest value is still 0 > -1, lowest id first.
    adj = np.full((5, 2), -1, np.int32)
    adj[0] = [1, -1]
    adj[1] = [2, 0]
    adj[2] = [1, -1]
    adj[3] = [4, -1]
    adj[4] = [0, 3]
    got = oracle.select_start_ids(adj, 0, 5)
    assert got.tolist() == python_fps(adj, 0, 5).tolist() == [0, 2, 1, 0, 0]
    # Starting inside the second component reaches everything.
    assert oracle.select_start_ids(adj, 3, 3).tolist() == python_fps(adj, 3, 3).tolist() == [3, 2, 0]


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_oracle_matches_python_on_random_graphs(seed):
    g = synth.random_graph(700, 6, n_start=4, seed=seed, min_degree=0)
    adj = g.adj.numpy()
    first = int(np.flatnonzero((adj >= 0).any(axis=1))[seed])
    assert np.array_equal(oracle.select_start_ids(adj, first, 9), python_fps(adj, first, 9))


def test_oracle_rejects_bad_arguments():
    adj = path_graph(5)
    with pytest.raises(ValueError):
        oracle.select_start_ids(adj, 7, 2)
    with pytest.raises(ValueError):
        oracle.select_start_ids(adj, 0, 0)


# ---------------------------------------------------------------- device path

def _index_for(adj, dim=8):
    from coral_b200 import capi
    n = adj.shape[0]
    ix = capi.Index(n, dim, adj.shape[1], "l2")
    ix.set_vectors(np.zeros((n, dim), np.float32))
    ix.set_adjacency(adj)
    return ix


@pytest.mark.gpu
@pytest.mark.parametrize("n,deg,M,seed", [(11, 4, 4, 0), (5000, 8, 16, 1), (200000, 32, 16, 2), (30000, 3, 64, 3)])
def test_device_selection_matches_oracle(n, deg, M, seed):
    if n == 11:
        adj, first = path_graph(n, 32), 3
    else:
        adj = synth.random_graph(n, deg, n_start=4, seed=seed, min_degree=0).adj.numpy()
        first = int(np.flatnonzero((adj >= 0).any(axis=1))[17])
    ix = _index_for(adj)
    got = ix.select_start_ids(first, M)
    assert np.array_equal(got, oracle.select_start_ids(adj, first, M))


@pytest.mark.gpu
def test_device_selection_on_a_search_graph_feeds_the_search():
    c = cases.structured("l2")
    from coral_b200 import capi
    ix = capi.Index(c.n, c.dim, c.max_degree, c.metric)
    ix.set_vectors(c.base)
    ix.set_adjacency(c.adj)
    first = int(c.start[0])
    got = ix.select_start_ids(first, 16)
    want = oracle.select_start_ids(c.adj, first, 16)
    assert np.array_equal(got, want)
    ix.prepare(c.queries.shape[0], 64, 10)
    ids, d, _, _ = ix.search(c.queries, 64, 10, dists=True)
    ref_ids, ref_d, _ = oracle.search(c.base, c.adj, want, c.queries, 64, 10, c.metric)
    assert np.array_equal(ids, ref_ids)
    assert np.array_equal(d.view(np.uint32), ref_d.view(np.uint32))


@pytest.mark.gpu
def test_device_selection_rejects_what_the_reference_redraws():
    from coral_b200 import capi
    adj = path_graph(6, 32)
    adj[5] = -1                      # node 5 has no out-edges: the reference would redraw
    ix = _index_for(adj)
    with pytest.raises(capi.CoralError):
        ix.select_start_ids(5, 3)
    with pytest.raises(capi.CoralError):
        ix.select_start_ids(6, 3)
    assert ix.select_start_ids(0, 1).tolist() == [0]
