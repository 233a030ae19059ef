"""The CPU oracle against first principles (no GPU).

The reference holds no golden vectors or known-answer tests for the search path,
so the oracle is pinned here by (a) hand-computed floating-point cases that
separate its two summation orders, (b) an independent pure-Python statement of
the search semantics on small graphs, (c) committed fixtures.
"""
import math
import os

import numpy as np
import pytest

from oracle import oracle
from tests import cases

F32_MAX = np.float32(3.402823466e+38)


def test_sequential_and_tree_orders_are_the_reference_orders():
    # IP, 4 elements: the sequential fused chain loses the first "+1" to rounding
    # (2^24 + 1 -> 2^24), the lane tree adds (2^24 - 2^24) + (1 + 1).
    row = np.array([2.0 ** 24, 1.0, -(2.0 ** 24), 1.0], np.float32)
    q = np.ones(4, np.float32)
    assert oracle.dist_seq(row, q, "ip") == np.float32(1.0)
    assert oracle.dist_tree(row, q, "ip") == np.float32(2.0)
    # L2 with the same magnitudes: diffs are (2^12, 1, 2^12, 1) squared.
    row = np.array([2.0 ** 12, 1.0, 2.0 ** 12, 1.0], np.float32)
    q = np.zeros(4, np.float32)
    assert oracle.dist_seq(row, q, "l2") == np.float32(2.0 ** 25)       # 2^24+1 rounds down, twice
    assert oracle.dist_tree(row, q, "l2") == np.float32(2.0 ** 25 + 2)  # (2^24+2^24)+(1+1) is exact


def test_fused_multiply_add_is_single_rounding():
    # a*b + c where the product needs more than 24 bits: fused = one rounding.
    a = np.float32(1 + 2.0 ** -12)
    row = np.array([a], np.float32)
    q = np.array([a], np.float32)
    exact = float(a) * float(a)            # 1 + 2^-11 + 2^-24, exact in float64
    assert oracle.dist_seq(row, q, "ip") == np.float32(exact)
    # second element makes a separate rounding of the product visible
    row = np.array([a, -1.0], np.float32)
    q = np.array([a, 1.0], np.float32)
    fused = np.float32(float(np.float32(exact)) - 1.0)
    assert oracle.dist_seq(row, q, "ip") == fused


@pytest.mark.parametrize("metric", ["l2", "ip"])
@pytest.mark.parametrize("dim", [4, 36, 200, 512])
def test_distances_close_to_float64(metric, dim):
    rng = np.random.default_rng(dim)
    for _ in range(20):
        row = rng.standard_normal(dim).astype(np.float32)
        q = rng.standard_normal(dim).astype(np.float32)
        ref = float(((row.astype(np.float64) - q) ** 2).sum()) if metric == "l2" else float(row.astype(np.float64) @ q)
        scale = float(np.abs(row.astype(np.float64) * q).sum()) if metric == "ip" else ref
        for f in (oracle.dist_seq, oracle.dist_tree):
            assert abs(float(f(row, q, metric)) - ref) <= 2e-6 * max(scale, 1e-30) * math.sqrt(dim)


def python_reference_search(c, q, L, k):
    """Independent statement of the reference kernel's semantics
    (src/search_gpu.cu:347-580): plain Python containers, ties by (distance, id)."""
    closer = (lambda a, b: a > b) if c.metric == "l2" else (lambda a, b: a < b)   # b closer than a
    order = (lambda d, i: (d, i)) if c.metric == "l2" else (lambda d, i: (-d, i))
    far = float(F32_MAX) if c.metric == "l2" else -float(F32_MAX)
    visited = set()
    beam = []          # [dist, id, expanded]
    for s in c.start:
        visited.add(int(s))
        beam.append([float(oracle.dist_tree(c.base[s], q, c.metric)), int(s), False])
    worst, hops, n_dist, rounds = far, 0, len(c.start), 0
    while True:
        rounds += 1
        cands = []
        for e in beam:
            if e[2]:
                continue
            e[2] = True
            for v in c.adj[e[1]]:
                v = int(v)
                if v < 0 or v in visited:
                    continue
                visited.add(v)
                d = float(oracle.dist_seq(c.base[v], q, c.metric))
                n_dist += 1
                if closer(worst, d):
                    cands.append([d, v, False])
        if not cands:
            break
        hops += len(cands)
        if len(beam) + len(cands) <= L:
            beam += cands
        else:
            beam = sorted(beam + cands, key=lambda e: order(e[0], e[1]))[:L]
            worst = beam[-1][0]
    beam.sort(key=lambda e: order(e[0], e[1]))
    ids = [e[1] for e in beam[:k]] + [-1] * max(0, k - len(beam))
    ds = [e[0] for e in beam[:k]] + [far] * max(0, k - len(beam))
    return ids, ds, hops, n_dist, rounds


@pytest.mark.parametrize("metric,quantized", [("l2", False), ("ip", False), ("l2", True), ("ip", True)])
def test_oracle_matches_python_statement(metric, quantized):
    c = cases.random_case(metric, 1500, 16, 32, 12, m=8, seed=31, dup_start=True, quantized=quantized)
    for L, k in [(8, 8), (24, 10), (64, 10)]:
        ids, d, st = oracle.search(c.base, c.adj, c.start, c.queries, L, k, metric)
        for qi in range(len(c.queries)):
            rid, rd, hops, n_dist, rounds = python_reference_search(c, c.queries[qi], L, k)
            assert list(ids[qi]) == rid
            assert [float(x) for x in d[qi]] == rd
            assert (st[qi, 4], st[qi, 1], st[qi, 3]) == (hops, n_dist, rounds)


def test_underfull_beam_pads_and_flags():
    c = cases.chain_case()
    ids, d, st = oracle.search(c.base, c.adj, c.start, c.queries, 64, 16, "l2")
    assert (st[:, 0] == 1).all()
    assert (np.sort(ids[:, :10], axis=1) == np.arange(10)).all()
    assert (ids[:, 10:] == -1).all() and (d[:, 10:] == F32_MAX).all()


def test_bad_arguments_are_rejected():
    c = cases.chain_case()
    with pytest.raises(ValueError):
        oracle.search(c.base, c.adj, c.start, c.queries, 4, 8, "l2")          # k > L
    with pytest.raises(ValueError):
        oracle.search(c.base, c.adj, np.array([c.n], np.int32), c.queries, 8, 4, "l2")   # start id out of range


def test_full_expansion_differs_from_best_first_but_both_find_neighbours():
    import torch
    from coral_b200 import synth
    c = cases.structured("l2")
    gt = synth.exact_knn(torch.from_numpy(c.base), torch.from_numpy(c.queries), 10, "l2").numpy()
    ids, _, st = oracle.search(c.base, c.adj, c.start, c.queries, 64, 10, "l2")
    cid, _, hops, secs, kind, threads = oracle.cpu_search(c.base, c.adj, c.start, c.queries, 64, 10)
    assert oracle.recall(ids, gt, 10) > 0.9
    assert oracle.recall(cid, gt, 10) > 0.5
    assert kind in ("reference", "port") and secs > 0 and hops > 0
    # the self-contained port and the harness on the reference's own classes agree
    pid, _, phops, _, pkind, _ = oracle.cpu_search(c.base, c.adj, c.start, c.queries, 64, 10, prefer_reference=False)
    assert pkind == "port" and phops == hops
    assert (pid == cid).mean() > 0.99       # summation order differs, near-ties may swap


def test_merge_shards_definition():
    ids = np.array([[[5, 9, -1]], [[7, 3, 1]]], np.int32)          # G=2, Q=1, k=3
    d = np.array([[[0.1, 0.5, 0.0]], [[0.1, 0.2, 0.9]]], np.float32)
    oi, od = oracle.merge_shards(ids, d, "l2")
    assert list(oi[0]) == [5, 7, 3] and list(od[0]) == [np.float32(0.1), np.float32(0.1), np.float32(0.2)]
    oi, od = oracle.merge_shards(ids, d, "ip")
    assert list(oi[0]) == [1, 9, 3]


GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "beam_search_small.npz")


@pytest.mark.skipif(not os.path.exists(GOLDEN), reason="fixture not generated")
def test_oracle_reproduces_committed_fixture():
    z = np.load(GOLDEN)
    for tag in ("l2", "ip"):
        ids, d, st = oracle.search(z[f"{tag}_base"], z[f"{tag}_adj"], z[f"{tag}_start"], z[f"{tag}_queries"],
                                   int(z[f"{tag}_L"]), int(z[f"{tag}_k"]), tag)
        assert np.array_equal(ids, z[f"{tag}_ids"])
        assert np.array_equal(d.view(np.uint32), z[f"{tag}_dists"].view(np.uint32))
        assert np.array_equal(st[:, :7], z[f"{tag}_stats"][:, :7])


# ---------------------------------------------------------------------------------------------
# golden vectors recorded from the reference's OWN GPU kernel (tests/golden/make_ref_kernel_golden.py)
# ---------------------------------------------------------------------------------------------

def _ref_kernel_golden():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_kernel_small.npz")
    return np.load(path, allow_pickle=False)


REF_GOLDEN_RUNS = [("rand_l2", 48, 10), ("rand_l2", 64, 32), ("rand_ip", 64, 16), ("struct_l2", 64, 10),
                   ("struct_l2", 128, 100), ("struct_ip", 64, 10), ("struct_ip", 256, 10)]


@pytest.mark.parametrize("tag,L,k", REF_GOLDEN_RUNS)
def test_oracle_reproduces_the_reference_kernels_recorded_outputs(tag, L, k):
    """ids, distance bits and the hop total the reference's beam_search_kernel produced on a B200
    (src/search_gpu.cu:347-580, compiled unmodified) must come out of the CPU oracle bit for bit."""
    g = _ref_kernel_golden()
    metric = str(g[f"{tag}_metric"])
    base, adj, start, queries = g[f"{tag}_base"], g[f"{tag}_adj"], g[f"{tag}_start"], g[f"{tag}_queries"]
    key = f"{tag}_L{L}_k{k}"
    rows = g[key + "_rows"]
    ids, d, st = oracle.search(base, adj, start, queries[rows], L, k, metric)
    assert (st[:, 0] == 0).all()
    want_ids, want_bits = g[key + "_ids"], g[key + "_dist_bits"]
    assert np.array_equal(d.view(np.uint32), want_bits)
    for r, j in zip(*np.nonzero(ids != want_ids)):   # the reference orders exact ties by thread position
        for node in (int(ids[r, j]), int(want_ids[r, j])):
            got = {np.float32(f(base[node], queries[rows[r]], metric)).view(np.uint32)
                   for f in (oracle.dist_seq, oracle.dist_tree)}
            assert want_bits[r, j] in got, f"row {r} column {j}: id {node} is not a tie"
    assert int(st[:, 4].sum()) == int(g[key + "_hops"])
