"""Writes tests/golden/beam_search_small.npz: two small seeded cases (inputs and the
CPU oracle's outputs).  The reference ships no golden vectors for this path, so the
fixture pins the oracle (and, on a GPU, the kernels) against regressions only.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle  # noqa: E402
from tests import cases  # noqa: E402

out = {}
for tag, dim, deg, L, k in (("l2", 40, 32, 48, 10), ("ip", 64, 64, 64, 16)):
    c = cases.random_case(tag, 1000, dim, deg, 24, m=16, seed=77, dup_start=(tag == "ip"))
    ids, d, st = oracle.search(c.base, c.adj, c.start, c.queries, L, k, tag)
    out.update({f"{tag}_base": c.base, f"{tag}_adj": c.adj, f"{tag}_start": c.start, f"{tag}_queries": c.queries,
                f"{tag}_L": np.int32(L), f"{tag}_k": np.int32(k), f"{tag}_deg": np.int32(deg),
                f"{tag}_ids": ids, f"{tag}_dists": d, f"{tag}_stats": st})
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "beam_search_small.npz"), **out)
print("written")
