"""The tensor-core dense scan (tcgen05, tf32 split in three passes) behind coral_exact_knn against
the brute-force CPU oracle: ids and distance bits of the k nearest rows must be identical -- the
tensor cores only select candidates, the returned distances come from the exact fp32 re-rank in the
reference's summation order (include/utils.cuh:254-275, :307-323)."""
import numpy as np
import pytest

from coral_b200 import capi
from oracle import oracle

pytestmark = pytest.mark.gpu


def _data(n, dim, nq, metric, seed, clusters=20):
    rng = np.random.default_rng(seed)
    ctr = rng.standard_normal((clusters, dim)).astype(np.float32)
    base = (ctr[rng.integers(0, clusters, n)] + 0.3 * rng.standard_normal((n, dim))).astype(np.float32)
    q = (ctr[rng.integers(0, clusters, nq)] + 0.3 * rng.standard_normal((nq, dim))).astype(np.float32)
    if metric == "ip":
        base /= np.linalg.norm(base, axis=1, keepdims=True)
        q /= np.linalg.norm(q, axis=1, keepdims=True)
    return base, q


def _check(base, q, k, metric, passes=3, max_bad=0):
    with capi.Index(base.shape[0], base.shape[1], 32, metric) as ix:
        ix.set_option("dense_passes", passes)
        ix.set_vectors(base)
        ids, d, bad = ix.exact_knn(q, k)
        tf = ix.last_dense_tflops
    ref_ids, ref_d = oracle.exact_knn(base, q, k, metric)
    wrong = int((ids != ref_ids).any(1).sum())
    assert wrong <= max_bad, f"{wrong} of {len(q)} rows differ from brute force (uncertified: {bad})"
    if max_bad == 0:
        assert np.array_equal(d.view(np.uint32), ref_d.view(np.uint32))
    if passes == 3:
        assert bad <= len(q) // 100, f"{bad} uncertified queries"
    return tf


@pytest.mark.parametrize("metric", ["ip", "l2"])
def test_one_tile(metric):
    base, q = _data(256, 32, 128, metric, 1)
    _check(base, q, 10, metric)


@pytest.mark.parametrize("metric,n,dim,nq,k", [
    ("ip", 5000, 64, 300, 10),
    ("l2", 5000, 200, 300, 100),      # 200 floats: the last k-block is ragged (TMA zero fill)
    ("ip", 3001, 512, 77, 100),       # ragged row and column tiles
    ("l2", 20000, 512, 1000, 10),
    ("ip", 700, 36, 5, 200),
])
def test_shapes(metric, n, dim, nq, k):
    base, q = _data(n, dim, nq, metric, n + dim)
    _check(base, q, k, metric)


def test_duplicate_rows_order_by_id():
    base, q = _data(2000, 64, 64, "l2", 5)
    base[1000:1500] = base[:500]          # exact ties between row i and row 1000 + i
    _check(base, q, 50, "l2")


def test_several_base_chunks_and_query_chunks():
    # more rows than one scan launch takes (2^28 / dim) and more queries than one wave of query tiles
    base, q = _data(600_000, 512, 256, "ip", 9, clusters=300)
    _check(base, q, 100, "ip")
    base, q = _data(4_000, 64, 20_000, "l2", 10)
    _check(base, q[:20_000], 10, "l2")


def test_single_pass_tf32_selects_almost_as_well():
    base, q = _data(50_000, 512, 512, "ip", 11, clusters=50)
    _check(base, q, 10, "ip", passes=1, max_bad=5)


def test_throughput_is_reported():
    base, q = _data(200_000, 512, 4096, "ip", 12, clusters=200)
    with capi.Index(base.shape[0], base.shape[1], 32, "ip") as ix:
        ix.set_vectors(base)
        ix.exact_knn(q, 100)
        ids, d, bad = ix.exact_knn(q, 100)
        assert ix.last_dense_tflops > 1.0
        print("dense scan: %.1f TFLOP/s (tf32 x3)" % ix.last_dense_tflops)
