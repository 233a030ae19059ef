"""Pins the CPU oracle (and through it the CUDA path) to the reference's OWN kernel.

``oracle/_ref/libref_gpu.so`` is the reference's search launcher and bitset
``beam_search_kernel`` (src/search_gpu.cu:347-580, :835-886) with the reference's distance
functions and types, compiled unmodified from the reference tree for sm_100a.  On cases
whose every query fills its beam (the reference kernel reads out of range otherwise) and
whose distances do not tie exactly (the reference breaks ties by thread position), the
reference kernel, the oracle and this library's kernel must return the same ids, the same
distance bits and the same hop counts.

The reference's hop count is not fully deterministic: in its replace-worst loop thread 0 clears
``s_flag`` for the next pass before the other threads have tested it for the current one
(src/search_gpu.cu:530-532), so a thread can leave the loop a pass early; on a B200 this shifts the
hop total of a batch by one now and then (ids and distances were never seen to move).  The hop
check therefore accepts the reference's value when any of three runs reproduces the oracle's.
"""
import numpy as np
import pytest

from coral_b200 import capi
from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu

if not oracle.have_ref_gpu():
    pytest.skip("oracle/_ref/libref_gpu.so was not built (needs the reference tree at build time)",
                allow_module_level=True)


def _full_beam_queries(c, L, k):
    ids, d, st = oracle.search(c.base, c.adj, c.start, c.queries, L, k, c.metric)
    keep = st[:, 0] == 0
    assert keep.sum() >= len(c.queries) // 2, "case does not fill enough beams to be a useful pin"
    return c.queries[keep], ids[keep], d[keep], st[keep]


def _assert_rows_equal(tag, ids, d, ref_ids, ref_d, c=None, q=None):
    """Distance bits must be equal everywhere.  Ids must be equal except where two different nodes
    have bit-identical distances to the query (the reference orders such ties by thread position):
    there the other side's id must really have that distance."""
    assert np.array_equal(d.view(np.uint32), ref_d.view(np.uint32)), f"{tag}: distance bits differ"
    for r, j in zip(*np.nonzero(ids != ref_ids)):
        assert c is not None, f"{tag}: ids differ in row {r}"
        for node in (int(ids[r, j]), int(ref_ids[r, j])):
            got = {np.float32(f(c.base[node], q[r], c.metric)).view(np.uint32) for f in (oracle.dist_seq, oracle.dist_tree)}
            assert d[r, j].view(np.uint32) in got, f"{tag}: row {r} column {j}: id {node} is not a tie"


CASES = [
    ("structured_l2", lambda: cases.structured("l2"), [(64, 10), (128, 10), (128, 100), (256, 10)]),
    ("structured_ip", lambda: cases.structured("ip"), [(64, 10), (128, 10), (256, 10)]),
    ("structured_ip_deg64", lambda: cases.structured("ip", n=20000, deg=64, nq=128), [(64, 10), (128, 10)]),
    ("random_l2", lambda: cases.random_case("l2", 6000, 200, 32, 64), [(64, 10), (200, 64)]),
    ("random_ip", lambda: cases.random_case("ip", 6000, 512, 64, 64), [(64, 10), (128, 100)]),
    ("random_l2_dup_start", lambda: cases.random_case("l2", 6000, 40, 32, 64, dup_start=True), [(64, 10)]),
]


@pytest.mark.parametrize("name,make,Lk", CASES, ids=[c[0] for c in CASES])
def test_reference_kernel_oracle_and_library_agree(name, make, Lk):
    c = make()
    with capi.Index(c.n, c.dim, c.max_degree, c.metric) as ix:
        ix.set_vectors(c.base)
        ix.set_adjacency(c.adj)
        ix.set_start_ids(c.start)
        ix.prepare(len(c.queries), max(L for L, _ in Lk), max(k for _, k in Lk))
        for L, k in Lk:
            q, o_ids, o_d, o_st = _full_beam_queries(c, L, k)
            r_ids, r_d, r_hops, _ = oracle.ref_gpu_search(c.base, c.adj, c.start, q, L, k, c.metric, c.max_degree)
            tag = f"{name} L={L} k={k}"
            _assert_rows_equal(tag + " reference kernel vs oracle", r_ids, r_d, o_ids, o_d, c, q)
            want_hops = int(o_st[:, 4].sum())
            seen = [r_hops]
            while seen[-1] != want_hops and len(seen) < 3:
                seen.append(oracle.ref_gpu_search(c.base, c.adj, c.start, q, L, k, c.metric, c.max_degree)[2])
            assert want_hops in seen, f"{tag}: reference hops {seen} never equal the oracle's {want_hops}"
            ids, d, st, hops = ix.search(q, L, k, dists=True, stats=True)
            _assert_rows_equal(tag + " library vs reference kernel", ids, d, r_ids, r_d, c, q)
            assert hops == want_hops


def test_per_query_hops_match_the_reference_kernel():
    c = cases.structured("l2")
    L, k = 64, 10
    q, o_ids, o_d, o_st = _full_beam_queries(c, L, k)
    for i in range(8):
        seen = []
        while int(o_st[i, 4]) not in seen and len(seen) < 3:
            r_ids, r_d, r_hops, _ = oracle.ref_gpu_search(c.base, c.adj, c.start, q[i:i + 1], L, k, c.metric, c.max_degree)
            seen.append(r_hops)
        assert int(o_st[i, 4]) in seen
        assert np.array_equal(r_d.view(np.uint32), o_d[i:i + 1].view(np.uint32))
