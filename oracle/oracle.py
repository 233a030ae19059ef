"""ctypes access to the CPU checkers (test infrastructure, not product code).

Only tests, the smoke check and the benchmark's baseline legs may import this
module.  ``liboracle.so`` holds the restatement of the reference GPU kernel's
semantics (``beam_search_oracle.c``) and the self-contained CPU best-first port
(``search_in_cpu_port.c``); ``_ref/libref_cpu.so`` is the same best-first loop
driving the reference's own queue and AVX-512 distance classes;
``_ref/libref_gpu.so`` is the reference's own search launcher and kernel, compiled
unmodified from the reference tree for sm_100a (``ref_gpu_driver.cu``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
L2, IP = 0, 1
STATS_W = 8
STAT_NAMES = ("status", "n_dist", "n_exp", "rounds", "hops", "n_scan", "max_cand", "n_visited")

_lib = None
_ref = None
_ref_gpu = None


def reference_dir() -> str:
    """Where the reference tree lies: $CORAL_REFERENCE_DIR, else a directory named
    ``reference`` beside the repository; '' when neither exists."""
    cand = os.environ.get("CORAL_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "include", "efanna2e")) else ""


def build(quiet: bool = True) -> None:
    """Compile the checkers (and ``_ref`` when the reference tree is present)."""
    env = dict(os.environ, CORAL_REFERENCE_DIR=reference_dir())
    for var in ("CC", "CXX"):
        env.pop(var, None)
    subprocess.run(["make", "-C", _HERE], check=True, env=env,
                   stdout=subprocess.DEVNULL if quiet else None)


def _load():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        _lib = C.CDLL(path)
        f32p, i32p = C.POINTER(C.c_float), C.POINTER(C.c_int32)
        _lib.coral_oracle_search.restype = C.c_int
        _lib.coral_oracle_search.argtypes = [
            f32p, C.c_int64, C.c_int, i32p, C.c_int, i32p, C.c_int, f32p, C.c_int, C.c_int, C.c_int,
            C.c_int, C.c_int, i32p, f32p, i32p, C.c_int]
        _lib.coral_oracle_dist_seq.restype = C.c_float
        _lib.coral_oracle_dist_seq.argtypes = [f32p, f32p, C.c_int, C.c_int]
        _lib.coral_oracle_dist_tree.restype = C.c_float
        _lib.coral_oracle_dist_tree.argtypes = [f32p, f32p, C.c_int, C.c_int]
        _lib.coral_oracle_merge_shards.restype = C.c_int
        _lib.coral_oracle_merge_shards.argtypes = [i32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int, i32p, f32p]
        _lib.coral_oracle_select_start_ids.restype = C.c_int
        _lib.coral_oracle_select_start_ids.argtypes = [i32p, C.c_int64, C.c_int, C.c_int, C.c_int, i32p]
        _lib.coral_oracle_exact_knn.restype = C.c_int
        _lib.coral_oracle_exact_knn.argtypes = [f32p, C.c_int64, C.c_int, f32p, C.c_int, C.c_int, C.c_int, i32p, f32p]
        _lib.coral_oracle_nap_batch.restype = C.c_int
        _lib.coral_oracle_nap_batch.argtypes = [f32p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, i32p, f32p, i32p,
                                                i32p, C.c_int, C.c_int]
        _lib.coral_oracle_ce_batch.restype = C.c_int
        _lib.coral_oracle_ce_batch.argtypes = [f32p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, i32p, f32p, i32p,
                                               i32p, C.c_int, i32p, f32p, C.c_int]
        _lib.coral_oracle_delete_batch.restype = C.c_int
        _lib.coral_oracle_delete_batch.argtypes = [f32p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, i32p, f32p, i32p,
                                                   C.POINTER(C.c_uint32), i32p, i32p, C.c_int]
        _lib.coral_oracle_insert_batch.restype = C.c_int
        _lib.coral_oracle_insert_batch.argtypes = [f32p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, i32p, f32p, i32p,
                                                   i32p, C.c_int, i32p, C.c_int]
        _lib.coral_oracle_edge_dists.restype = C.c_int
        _lib.coral_oracle_edge_dists.argtypes = [f32p, C.c_int64, C.c_int, C.c_int, i32p, C.c_int, f32p, i32p]
        _lib.coral_oracle_recall.restype = C.c_double
        _lib.coral_oracle_recall.argtypes = [i32p, i32p, C.c_int, C.c_int, C.c_int]
        _set_cpu_sig(_lib)
    return _lib


def _set_cpu_sig(lib):
    f32p, i32p = C.POINTER(C.c_float), C.POINTER(C.c_int32)
    lib.coral_cpu_search.restype = C.c_int
    lib.coral_cpu_search.argtypes = [
        f32p, C.c_int64, C.c_int, i32p, C.c_int, i32p, C.c_int, f32p, C.c_int, C.c_int, C.c_int,
        i32p, f32p, C.POINTER(C.c_int64), C.POINTER(C.c_double), C.c_int]
    lib.coral_cpu_search_kind.restype = C.c_int


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _i32(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(C.POINTER(C.c_int32))


def metric_id(metric) -> int:
    if metric in (L2, "l2", "L2"):
        return L2
    if metric in (IP, "ip", "IP"):
        return IP
    raise ValueError(f"unknown metric {metric!r}")


def search(base, adj, start_ids, queries, L, k, metric, order=0, threads=0):
    """Full-expansion beam search as the reference GPU kernel defines it.

    Returns (ids[Q,k] int32, dists[Q,k] float32, stats[Q,8] int32).
    """
    lib = _load()
    base, bp = _f32(base)
    adj, ap = _i32(adj)
    start_ids, sp = _i32(start_ids)
    queries, qp = _f32(queries)
    n, dim = base.shape
    Q = queries.shape[0]
    ids = np.empty((Q, k), np.int32)
    dists = np.empty((Q, k), np.float32)
    stats = np.zeros((Q, STATS_W), np.int32)
    rc = lib.coral_oracle_search(bp, n, dim, ap, adj.shape[1], sp, len(start_ids), qp, Q, L, k,
                                 metric_id(metric), order,
                                 ids.ctypes.data_as(C.POINTER(C.c_int32)),
                                 dists.ctypes.data_as(C.POINTER(C.c_float)),
                                 stats.ctypes.data_as(C.POINTER(C.c_int32)), threads)
    if rc != 0:
        raise ValueError("coral_oracle_search: bad arguments")
    return ids, dists, stats


def dist_seq(row, q, metric):
    lib = _load()
    row, rp = _f32(row)
    q, qp = _f32(q)
    return np.float32(lib.coral_oracle_dist_seq(rp, qp, row.size, metric_id(metric)))


def dist_tree(row, q, metric):
    lib = _load()
    row, rp = _f32(row)
    q, qp = _f32(q)
    return np.float32(lib.coral_oracle_dist_tree(rp, qp, row.size, metric_id(metric)))


def merge_shards(ids, dists, metric):
    """ids/dists: [G,Q,k] -> merged ([Q,k], [Q,k]) by (distance, id)."""
    lib = _load()
    ids, ip_ = _i32(ids)
    dists, dp = _f32(dists)
    G, Q, k = ids.shape
    oi = np.empty((Q, k), np.int32)
    od = np.empty((Q, k), np.float32)
    rc = lib.coral_oracle_merge_shards(ip_, dp, G, Q, k, metric_id(metric),
                                       oi.ctypes.data_as(C.POINTER(C.c_int32)),
                                       od.ctypes.data_as(C.POINTER(C.c_float)))
    if rc != 0:
        raise ValueError("coral_oracle_merge_shards: bad arguments")
    return oi, od


def select_start_ids(adj, first, M):
    """Farthest-point sampling over BFS hop counts from `first`; returns int32 [M]."""
    lib = _load()
    adj, ap = _i32(adj)
    out = np.empty(M, dtype=np.int32)
    rc = lib.coral_oracle_select_start_ids(ap, adj.shape[0], adj.shape[1], int(first), int(M),
                                           out.ctypes.data_as(C.POINTER(C.c_int32)))
    if rc != M:
        raise ValueError("coral_oracle_select_start_ids rejected its arguments")
    return out


def exact_knn(base, queries, k, metric):
    """Brute-force k nearest rows by (sequential fp32 distance, id): (ids[Q,k], dists[Q,k])."""
    lib = _load()
    base, bp = _f32(base)
    queries, qp = _f32(queries)
    Q = queries.shape[0]
    ids = np.empty((Q, k), np.int32)
    dists = np.empty((Q, k), np.float32)
    rc = lib.coral_oracle_exact_knn(bp, base.shape[0], base.shape[1], qp, Q, k, metric_id(metric),
                                    ids.ctypes.data_as(C.POINTER(C.c_int32)),
                                    dists.ctypes.data_as(C.POINTER(C.c_float)))
    if rc != 0:
        raise ValueError("coral_oracle_exact_knn: bad arguments")
    return ids, dists


class BuildState:
    """Graph under construction as the CUDA library holds it: adj / ndist [n, deg_pad], deg [n]."""

    def __init__(self, n, max_degree):
        self.max_degree = int(max_degree)
        self.deg_pad = 32 if max_degree <= 32 else (64 if max_degree <= 64 else 128)
        self.adj = np.full((n, self.deg_pad), -1, np.int32)
        self.ndist = np.zeros((n, self.deg_pad), np.float32)
        self.deg = np.zeros(n, np.int32)


def nap_batch(base, state, lists, metric):
    """One batch of the neighbourhood-aware projection (src/upd_gpu.cu:260-303) in place."""
    lib = _load()
    base, bp = _f32(base)
    lists, lp = _i32(lists)
    i32p, f32p = C.POINTER(C.c_int32), C.POINTER(C.c_float)
    rc = lib.coral_oracle_nap_batch(bp, base.shape[0], base.shape[1], metric_id(metric), state.max_degree,
                                    state.deg_pad, state.adj.ctypes.data_as(i32p), state.ndist.ctypes.data_as(f32p),
                                    state.deg.ctypes.data_as(i32p), lp, lists.shape[0], lists.shape[1])
    if rc != 0:
        raise ValueError(f"coral_oracle_nap_batch failed with {rc}")


def ce_batch(base, state, iso_ids, res_ids, res_dists, metric):
    """One batch of the connectivity enhancement (src/enhance.cu:640-668) in place."""
    lib = _load()
    base, bp = _f32(base)
    iso_ids, ip_ = _i32(iso_ids)
    res_ids, rp = _i32(res_ids)
    res_dists, dp = _f32(res_dists)
    i32p, f32p = C.POINTER(C.c_int32), C.POINTER(C.c_float)
    rc = lib.coral_oracle_ce_batch(bp, base.shape[0], base.shape[1], metric_id(metric), state.max_degree,
                                   state.deg_pad, state.adj.ctypes.data_as(i32p), state.ndist.ctypes.data_as(f32p),
                                   state.deg.ctypes.data_as(i32p), ip_, len(iso_ids), rp, dp, res_ids.shape[1])
    if rc != 0:
        raise ValueError(f"coral_oracle_ce_batch failed with {rc}")


def state_from_adjacency(base, adj, max_degree, metric):
    """BuildState of a finished graph: edge distances recomputed, degrees counted."""
    lib = _load()
    base, bp = _f32(base)
    st = BuildState(base.shape[0], max_degree)
    st.adj = np.ascontiguousarray(adj, np.int32).copy()
    i32p, f32p = C.POINTER(C.c_int32), C.POINTER(C.c_float)
    lib.coral_oracle_edge_dists(bp, base.shape[0], base.shape[1], metric_id(metric), st.adj.ctypes.data_as(i32p),
                                st.deg_pad, st.ndist.ctypes.data_as(f32p), st.deg.ctypes.data_as(i32p))
    return st


def _first_usable(st, dead, live):
    ok = (st.deg[:live] > 0) & ~dead[:live]
    return int(np.nonzero(ok)[0][0])


def delete_nodes(base, st, dead, del_ids, metric, n_start=16, live=None, innbr_batch=4096 * 32):
    """IndexGPU::Delete (src/index_gpu.cpp:138-206): marks, repairs the live in-neighbours in batches,
    re-chooses the entry points.  `dead` (bool [n]) is updated in place.  Returns the start ids."""
    lib = _load()
    base, bp = _f32(base)
    n = base.shape[0]
    live = n if live is None else live
    del_ids = np.ascontiguousarray(del_ids, np.int32)
    dead[del_ids] = True
    bits = np.packbits(dead, bitorder="little")
    bits = np.concatenate([bits, np.zeros((-len(bits)) % 4, np.uint8)]).view(np.uint32).copy()
    # live in-neighbours of every deleted node of this call, ascending
    rows, cols = np.nonzero((st.adj >= 0) & (np.arange(st.deg_pad)[None, :] < st.deg[:, None]) & ~dead[:, None])
    tgt = st.adj[rows, cols]
    pos_of = np.full(n, -1, np.int64)
    pos_of[del_ids] = np.arange(len(del_ids))
    sel = pos_of[tgt] >= 0
    rows, tgt = rows[sel], tgt[sel]
    order = np.lexsort((rows, pos_of[tgt]))
    piv_in, piv_pos = rows[order].astype(np.int32), pos_of[tgt][order]
    counts = np.bincount(piv_pos, minlength=len(del_ids))
    offsets = np.concatenate([[0], np.cumsum(counts)])
    i32p, f32p = C.POINTER(C.c_int32), C.POINTER(C.c_float)
    b0 = 0
    while b0 < len(del_ids):
        b1, num = b0, 0
        while b1 < len(del_ids) and (num == 0 or num + counts[b1] <= innbr_batch):
            num += counts[b1]
            b1 += 1
        if num > 0:
            lo, hi = offsets[b0], offsets[b1]
            pin = np.ascontiguousarray(piv_in[lo:hi])
            pdel = np.ascontiguousarray(del_ids[piv_pos[lo:hi]])
            rc = lib.coral_oracle_delete_batch(bp, n, base.shape[1], metric_id(metric), st.max_degree, st.deg_pad,
                                               st.adj.ctypes.data_as(i32p), st.ndist.ctypes.data_as(f32p),
                                               st.deg.ctypes.data_as(i32p), bits.ctypes.data_as(C.POINTER(C.c_uint32)),
                                               pdel.ctypes.data_as(i32p), pin.ctypes.data_as(i32p), int(hi - lo))
            if rc != 0:
                raise ValueError("coral_oracle_delete_batch failed")
        b0 = b1
    return select_start_ids(st.adj, _first_usable(st, dead, live), n_start)


def search_hiding(base, adj, start, queries, L, k, metric, dead):
    """The search with the deleted bitset (src/search_gpu.cu:716): the beam's ids with deleted ones dropped."""
    ids, d, stt = search(base, adj, start, queries, L, L, metric)
    out = np.full((len(queries), k), -1, np.int32)
    for r in range(len(queries)):
        keep = ids[r][(ids[r] >= 0)]
        keep = keep[~dead[keep]][:k]
        out[r, :len(keep)] = keep
    return out


def insert_nodes(base, st, dead, first_id, count, kb, metric, L=512, batch=2048, n_start=16):
    """IndexGPU::Insert with neighbours from the search (src/index_gpu.cpp:207-224, src/update.cu:880-959)."""
    lib = _load()
    base, bp = _f32(base)
    n = base.shape[0]
    i32p, f32p = C.POINTER(C.c_int32), C.POINTER(C.c_float)
    start, live = None, first_id
    for s in range(0, count, batch):
        nb = min(batch, count - s)
        ins = np.arange(first_id + s, first_id + s + nb, dtype=np.int32)
        start = select_start_ids(st.adj, _first_usable(st, dead, live), n_start)
        res = search_hiding(base, st.adj, start, base[ins], L, kb, metric, dead)
        rc = lib.coral_oracle_insert_batch(bp, n, base.shape[1], metric_id(metric), st.max_degree, st.deg_pad,
                                           st.adj.ctypes.data_as(i32p), st.ndist.ctypes.data_as(f32p),
                                           st.deg.ctypes.data_as(i32p), ins.ctypes.data_as(i32p), nb,
                                           np.ascontiguousarray(res).ctypes.data_as(i32p), kb)
        if rc != 0:
            raise ValueError("coral_oracle_insert_batch failed")
        live = first_id + s + nb
    return start


def build_graph(base, train_knn, metric, max_degree, batch=1024, ce=True, ce_L=256, ce_search_batch=524288,
                ce_nap_batch=4096, n_start=16, log=None):
    """The reference's build on the CPU: NAP over the training lists in batches (src/index_gpu.cpp:501-580,
    config.json:5), then CE of the isolated nodes (src/enhance.cu:728-812): per search batch entry
    points by farthest-point sampling from the lowest-numbered node with an out-edge, the full
    expansion search with L = 256 and k = k_b, then batches of reverse edges and pruned rows.
    Returns (BuildState, start_ids)."""
    base = np.ascontiguousarray(base, np.float32)
    train_knn = np.ascontiguousarray(train_knn, np.int32)
    st = BuildState(base.shape[0], max_degree)
    for s in range(0, train_knn.shape[0], batch):
        nap_batch(base, st, train_knn[s:s + batch], metric)
    start = None
    if ce:
        kb = train_knn.shape[1]
        iso = np.nonzero(st.deg == 0)[0].astype(np.int32)
        if log:
            log(f"oracle build: {len(iso)} isolated nodes after NAP")
        first_connected = int(np.nonzero(st.deg > 0)[0][0])
        for s in range(0, len(iso), ce_search_batch):
            chunk = iso[s:s + ce_search_batch]
            start = select_start_ids(st.adj, first_connected, n_start)
            ids, dists, _ = search(base, st.adj, start, base[chunk], ce_L, kb, metric)
            for j in range(0, len(chunk), ce_nap_batch):
                ce_batch(base, st, chunk[j:j + ce_nap_batch], ids[j:j + ce_nap_batch], dists[j:j + ce_nap_batch], metric)
    if start is None:
        start = select_start_ids(st.adj, int(np.nonzero(st.deg > 0)[0][0]), n_start)
    return st, start


def recall(res, gt, k):
    lib = _load()
    res, rp = _i32(res)
    gt, gp = _i32(gt)
    return float(lib.coral_oracle_recall(rp, gp, res.shape[0], k, gt.shape[1]))


def _cpu_has(flag: str) -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return flag in line.split()
    except OSError:
        pass
    return False


def cpu_search_lib(prefer_reference: bool = True):
    """Return (lib, kind): kind 'reference' when the harness on the reference's own
    headers is built and this CPU has the AVX-512 it needs, else 'port'."""
    global _ref
    path = os.path.join(_HERE, "_ref", "libref_cpu.so")
    if prefer_reference and os.path.exists(path) and _cpu_has("avx512f") and _cpu_has("avx512dq"):
        if _ref is None:
            _ref = C.CDLL(path)
            _set_cpu_sig(_ref)
        return _ref, "reference"
    return _load(), "port"


def cpu_search(base, adj, start_ids, queries, L, k, threads=0, prefer_reference=True):
    """The reference's CPU best-first search (always squared L2, first M start ids).

    Returns (ids, dists, total_hops, seconds, kind, threads_used).
    """
    lib, kind = cpu_search_lib(prefer_reference)
    base, bp = _f32(base)
    adj, ap = _i32(adj)
    start_ids, sp = _i32(start_ids)
    queries, qp = _f32(queries)
    n, dim = base.shape
    Q = queries.shape[0]
    ids = np.empty((Q, k), np.int32)
    dists = np.empty((Q, k), np.float32)
    hops = C.c_int64(0)
    secs = C.c_double(0.0)
    if threads <= 0:
        threads = os.cpu_count() or 1
    rc = lib.coral_cpu_search(bp, n, dim, ap, adj.shape[1], sp, len(start_ids), qp, Q, L, k,
                              ids.ctypes.data_as(C.POINTER(C.c_int32)),
                              dists.ctypes.data_as(C.POINTER(C.c_float)),
                              C.byref(hops), C.byref(secs), threads)
    if rc != 0:
        raise ValueError("coral_cpu_search: bad arguments")
    return ids, dists, int(hops.value), float(secs.value), kind, threads


def have_ref_gpu() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libref_gpu.so"))


def _ref_gpu_lib():
    global _ref_gpu
    if _ref_gpu is None:
        _ref_gpu = C.CDLL(os.path.join(_HERE, "_ref", "libref_gpu.so"))
        f32p, i32p = C.POINTER(C.c_float), C.POINTER(C.c_int32)
        _ref_gpu.coral_ref_gpu_open.restype = C.c_void_p
        _ref_gpu.coral_ref_gpu_open.argtypes = [f32p, C.c_int64, C.c_int, i32p, C.c_int, C.c_int, C.c_int, i32p, C.c_int]
        _ref_gpu.coral_ref_gpu_close.restype = None
        _ref_gpu.coral_ref_gpu_close.argtypes = [C.c_void_p]
        _ref_gpu.coral_ref_gpu_run.restype = C.c_int
        _ref_gpu.coral_ref_gpu_run.argtypes = [C.c_void_p, f32p, C.c_int, C.c_int, C.c_int, i32p, f32p,
                                               C.POINTER(C.c_int64), C.POINTER(C.c_double)]
    return _ref_gpu


class RefGpuIndex:
    """The reference's device-side index (Slot records + row array) on the current CUDA device, for
    repeated calls of the reference's own GPUFuncs::search_gpu + beam_search_kernel (bitset
    overload).  Every query must fill its beam (oracle status 0): the reference kernel reads out of
    range otherwise."""

    def __init__(self, base, adj, start_ids, metric, max_degree=None):
        lib = _ref_gpu_lib()
        base, bp = _f32(base)
        adj, ap = _i32(adj)
        start_ids, sp = _i32(start_ids)
        n, dim = base.shape
        if max_degree is None:
            max_degree = int((adj >= 0).sum(1).max())
        self.dim = dim
        self._h = lib.coral_ref_gpu_open(bp, n, dim, ap, adj.shape[1], max_degree, metric_id(metric), sp, len(start_ids))
        if not self._h:
            raise RuntimeError("coral_ref_gpu_open failed")

    def search(self, queries, L, k):
        """Returns (ids, dists, total_hops, seconds of the reference's own timed window)."""
        queries, qp = _f32(queries)
        Q = queries.shape[0]
        ids = np.empty((Q, k), np.int32)
        dists = np.empty((Q, k), np.float32)
        hops = C.c_int64(0)
        secs = C.c_double(0.0)
        rc = _ref_gpu_lib().coral_ref_gpu_run(self._h, qp, Q, L, k, ids.ctypes.data_as(C.POINTER(C.c_int32)),
                                              dists.ctypes.data_as(C.POINTER(C.c_float)), C.byref(hops), C.byref(secs))
        if rc != 0:
            raise RuntimeError(f"coral_ref_gpu_run failed with {rc}")
        return ids, dists, int(hops.value), float(secs.value)

    def close(self):
        if self._h:
            _ref_gpu_lib().coral_ref_gpu_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def ref_gpu_search(base, adj, start_ids, queries, L, k, metric, max_degree=None):
    """One search through a temporary RefGpuIndex.  Returns (ids, dists, total_hops, seconds)."""
    with RefGpuIndex(base, adj, start_ids, metric, max_degree) as r:
        return r.search(queries, L, k)
