"""Writes ref_kernel_small.npz: outputs of the REFERENCE's own GPU kernel on small seeded cases.

Runs the reference's search launcher and bitset beam_search_kernel (src/search_gpu.cu:347-580,
:835-886; compiled unmodified from the reference tree into oracle/_ref/libref_gpu.so) on a CUDA
device and records ids, distance bits and total hops.  tests/test_oracle.py then holds the CPU
oracle to these vectors without a GPU.  Only queries whose beam fills are kept (the reference
kernel reads out of range otherwise, src/search_gpu.cu:444,466-467).

    python tests/golden/make_ref_kernel_golden.py [out.npz]      # needs a GPU and libref_gpu.so
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle  # noqa: E402
from tests import cases  # noqa: E402

SPECS = (
    # tag, case factory, (L, k) pairs, store the inputs in the fixture?
    ("rand_l2", lambda: cases.random_case("l2", 1000, 40, 32, 24, m=16, seed=77), [(48, 10), (64, 32)], True),
    ("rand_ip", lambda: cases.random_case("ip", 1000, 64, 64, 24, m=16, seed=77, dup_start=True), [(64, 16)], True),
    ("struct_l2", lambda: cases.structured("l2", n=3000, dim=64, deg=32, nq=48), [(64, 10), (128, 100)], True),
    ("struct_ip", lambda: cases.structured("ip", n=3000, dim=48, deg=64, nq=48), [(64, 10), (256, 10)], True),
)


def digest(c) -> str:
    h = hashlib.sha256()
    for a in (c.base, c.adj, c.start, c.queries):
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                                   "ref_kernel_small.npz")
    out = {}
    for tag, make, pairs, store in SPECS:
        c = make()
        out[f"{tag}_sha256"] = np.array(digest(c))
        out[f"{tag}_metric"] = np.array(c.metric)
        out[f"{tag}_max_degree"] = np.int32(c.max_degree)
        if store:
            out.update({f"{tag}_base": c.base, f"{tag}_adj": c.adj, f"{tag}_start": c.start,
                        f"{tag}_queries": c.queries})
        for L, k in pairs:
            _, _, st = oracle.search(c.base, c.adj, c.start, c.queries, L, k, c.metric)
            rows = np.nonzero(st[:, 0] == 0)[0].astype(np.int32)
            # The reference's merge loop has a race (thread 0 clears s_flag for the next pass before the
            # other threads have tested it, src/search_gpu.cu:530-532) that now and then shifts the hop
            # count by one: record the value two runs agree on.
            runs = [oracle.ref_gpu_search(c.base, c.adj, c.start, c.queries[rows], L, k, c.metric, c.max_degree)
                    for _ in range(3)]
            hop_values = [r[2] for r in runs]
            ids, d, hops, _ = next(r for r in runs if hop_values.count(r[2]) >= 2)
            assert all(np.array_equal(r[1].view(np.uint32), d.view(np.uint32)) for r in runs)
            key = f"{tag}_L{L}_k{k}"
            out.update({key + "_rows": rows, key + "_ids": ids, key + "_dist_bits": d.view(np.uint32),
                        key + "_hops": np.int64(hops)})
            print(key, "rows", len(rows), "hops", hops)
    np.savez_compressed(out_path, **out)
    print("written", out_path)


if __name__ == "__main__":
    main()
