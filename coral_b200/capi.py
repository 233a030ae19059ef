"""ctypes binding of the C ABI declared in include/coral_b200.h.

The binding is a thin convenience for Python callers (tests, the benchmark); the
product is the shared library.  It never computes results itself: when the
library is missing or no B200 is present, calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

L2, IP = 0, 1
STATS_W = 8
STAT_NAMES = ("status", "n_dist", "n_exp", "rounds", "hops", "n_scan", "max_cand", "n_spill")
OK, ERR_ARG, ERR_STATE, ERR_CUDA, ERR_NOGPU, ERR_KERNEL, ERR_LIMIT, ERR_QUERY = range(8)

EXPORTS = (
    "coral_version", "coral_compiled_sm", "coral_plan", "coral_index_create", "coral_index_destroy",
    "coral_index_set_vectors", "coral_index_write_vectors", "coral_index_attach_vectors", "coral_index_set_slots",
    "coral_index_set_adjacency", "coral_index_set_start_ids", "coral_index_select_start_ids",
    "coral_index_get_adjacency", "coral_index_get_start_ids", "coral_index_stream",
    "coral_index_set_deleted",
    "coral_search_prepare", "coral_search_free", "coral_search", "coral_search_async",
    "coral_search_check", "coral_query_order", "coral_last_kernel_ms", "coral_last_total_ms", "coral_launch_count",
    "coral_set_option", "coral_get_option", "coral_count_hits", "coral_exact_knn", "coral_last_dense_ms",
    "coral_last_dense_flops", "coral_build_begin", "coral_build_nap", "coral_build_connect_enhance",
    "coral_build_get_graph", "coral_build_set_graph", "coral_build_end", "coral_index_set_live",
    "coral_build_begin_from_graph", "coral_delete", "coral_insert", "coral_merge_shards",
    "coral_merge_shards_strided", "coral_comm_unique_id", "coral_comm_create", "coral_comm_create_all",
    "coral_comm_set_id_map", "coral_comm_destroy", "coral_comm_world", "coral_comm_rank", "coral_comm_last_error", "coral_query_slice",
    "coral_search_sharded",
    "coral_map_ids", "coral_last_error", "coral_search_static", "coral_search_static_status",
)

_lib = None


class CoralError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"coral_b200 error {code}: {msg}")
        self.code = code


def lib_path() -> str:
    return _build.LIB


def load():
    """Load libcoral_b200.so (building it first when the sources are newer)."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.build(checked=os.environ.get("CORAL_B200_CHECKED", "0") == "1")
    lib = C.CDLL(path)
    vp, i32p, f32p, i64p = C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)
    sig = {
        "coral_version": (C.c_int, []),
        "coral_compiled_sm": (C.c_int, []),
        "coral_plan": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]),
        "coral_index_create": (C.c_int, [C.POINTER(vp), C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int]),
        "coral_index_destroy": (C.c_int, [vp]),
        "coral_index_set_vectors": (C.c_int, [vp, f32p]),
        "coral_index_attach_vectors": (C.c_int, [vp, f32p]),
        "coral_index_write_vectors": (C.c_int, [vp, C.c_int64, C.c_int64, f32p]),
        "coral_index_set_slots": (C.c_int, [vp, i32p, C.c_size_t, i32p, C.c_size_t]),
        "coral_index_set_adjacency": (C.c_int, [vp, i32p, C.c_int]),
        "coral_index_set_start_ids": (C.c_int, [vp, i32p, C.c_int]),
        "coral_index_select_start_ids": (C.c_int, [vp, C.c_int, C.c_int, i32p]),
        "coral_index_stream": (vp, [vp]),
        "coral_index_get_adjacency": (C.c_int, [vp, i32p]),
        "coral_index_get_start_ids": (C.c_int, [vp, i32p, C.c_int]),
        "coral_index_set_deleted": (C.c_int, [vp, vp]),
        "coral_search_prepare": (C.c_int, [vp, C.c_int, C.c_int, C.c_int]),
        "coral_search_free": (C.c_int, [vp]),
        "coral_search": (C.c_int, [vp, f32p, C.c_int, C.c_int, C.c_int, i32p, f32p, i32p, i64p]),
        "coral_search_async": (C.c_int, [vp, f32p, C.c_int, C.c_int, C.c_int, i32p, f32p, i32p, vp]),
        "coral_search_check": (C.c_int, [vp]),
        "coral_query_order": (C.c_int, [vp, f32p, C.c_int, i32p, vp]),
        "coral_last_kernel_ms": (C.c_float, [vp]),
        "coral_last_total_ms": (C.c_float, [vp]),
        "coral_launch_count": (C.c_int64, [vp]),
        "coral_set_option": (C.c_int, [vp, C.c_char_p, C.c_int]),
        "coral_get_option": (C.c_int, [vp, C.c_char_p, C.POINTER(C.c_int)]),
        "coral_count_hits": (C.c_int, [vp, i32p, i32p, C.c_int, C.c_int, C.c_int, i64p]),
        "coral_exact_knn": (C.c_int, [vp, f32p, C.c_int, C.c_int, i32p, f32p, i64p]),
        "coral_last_dense_ms": (C.c_float, [vp]),
        "coral_last_dense_flops": (C.c_double, [vp]),
        "coral_build_begin": (C.c_int, [vp]),
        "coral_build_nap": (C.c_int, [vp, i32p, C.c_int, C.c_int, C.c_int]),
        "coral_build_connect_enhance": (C.c_int, [vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, i64p]),
        "coral_build_get_graph": (C.c_int, [vp, i32p, f32p, i32p]),
        "coral_build_set_graph": (C.c_int, [vp, i32p, f32p, i32p]),
        "coral_build_end": (C.c_int, [vp]),
        "coral_index_set_live": (C.c_int, [vp, C.c_int64]),
        "coral_build_begin_from_graph": (C.c_int, [vp]),
        "coral_delete": (C.c_int, [vp, i32p, C.c_int, C.c_int]),
        "coral_insert": (C.c_int, [vp, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
        "coral_merge_shards": (C.c_int, [vp, i32p, f32p, C.c_int, C.c_int, C.c_int, i32p, f32p, vp]),
        "coral_map_ids": (C.c_int, [vp, i32p, C.c_int64, i32p, vp]),
        "coral_merge_shards_strided": (C.c_int, [vp, i32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int64, i32p, f32p, vp]),
        "coral_comm_unique_id": (C.c_int, [vp]),
        "coral_comm_create": (C.c_int, [C.POINTER(vp), C.c_int, C.c_int, C.c_int, vp]),
        "coral_comm_create_all": (C.c_int, [C.POINTER(vp), C.POINTER(C.c_int), C.c_int]),
        "coral_comm_set_id_map": (C.c_int, [vp, i32p, C.c_int64]),
        "coral_comm_destroy": (C.c_int, [vp]),
        "coral_comm_world": (C.c_int, [vp]),
        "coral_comm_rank": (C.c_int, [vp]),
        "coral_comm_last_error": (C.c_char_p, [vp]),
        "coral_query_slice": (None, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
        "coral_search_sharded": (C.c_int, [vp, vp, i32p, f32p, C.c_int, C.c_int, C.c_int, i32p, f32p, vp]),
        "coral_last_error": (C.c_char_p, [vp]),
        "coral_search_static": (C.c_int, [C.c_int, vp, f32p, i32p, C.c_int64, C.c_int, C.c_int, C.c_int, i32p, C.c_int,
                                          f32p, C.c_int, C.c_int, C.c_int, i32p, f32p]),
        "coral_search_static_status": (C.c_int, [C.c_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _is_torch(x) -> bool:
    return hasattr(x, "data_ptr") and hasattr(x, "is_cuda")


def _ptr(x, dtype):
    """(pointer, keepalive) of a numpy array or torch tensor of the given numpy dtype."""
    if x is None:
        return None, None
    if _is_torch(x):
        import torch
        want = {np.float32: torch.float32, np.int32: torch.int32, np.uint32: torch.int32}[dtype]
        if x.dtype != want or not x.is_contiguous():
            x = x.to(want).contiguous()
        return C.c_void_p(x.data_ptr()), x
    a = np.ascontiguousarray(x, dtype=dtype)
    return C.c_void_p(a.ctypes.data), a


class Index:
    """Python mirror of the handle: create -> set vectors/graph/start ids -> prepare -> search."""

    def __init__(self, n: int, dim: int, max_degree: int, metric, device: int = 0):
        self._lib = load()
        self._h = C.c_void_p()
        self.n, self.dim, self.max_degree = int(n), int(dim), int(max_degree)
        self.metric = {"l2": L2, "ip": IP, L2: L2, IP: IP}[metric]
        self._keep = []
        rc = self._lib.coral_index_create(C.byref(self._h), device, self.n, self.dim, self.max_degree, self.metric)
        if rc != OK:
            msg = self._lib.coral_last_error(None).decode()
            self._h = C.c_void_p()
            raise CoralError(rc, msg)
        self.device = device

    def _check(self, rc: int):
        if rc != OK:
            raise CoralError(rc, self._lib.coral_last_error(self._h).decode())

    def close(self):
        if getattr(self, "_h", None) is not None and self._h:
            self._lib.coral_index_destroy(self._h)
            self._h = C.c_void_p()
            self._keep.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- index data
    def set_vectors(self, vecs):
        p, k = _ptr(vecs, np.float32)
        assert tuple(k.shape) == (self.n, self.dim)
        self._check(self._lib.coral_index_set_vectors(self._h, p))

    def write_vectors(self, first_row: int, vecs):
        p, k = _ptr(vecs, np.float32)
        assert k.shape[1] == self.dim
        self._check(self._lib.coral_index_write_vectors(self._h, int(first_row), int(k.shape[0]), p))

    def attach_vectors(self, dev_vecs):
        assert _is_torch(dev_vecs) and dev_vecs.is_cuda and dev_vecs.is_contiguous()
        assert tuple(dev_vecs.shape) == (self.n, self.dim)
        self._keep.append(dev_vecs)
        self._check(self._lib.coral_index_attach_vectors(self._h, C.c_void_p(dev_vecs.data_ptr())))

    def set_adjacency(self, adj):
        p, k = _ptr(adj, np.int32)
        assert k.shape[0] == self.n
        self._check(self._lib.coral_index_set_adjacency(self._h, p, int(k.shape[1])))

    def set_slots(self, degs, nbrs):
        """degs: int32 [n]; nbrs: int32 [n, width] (the reference's deg + nbrs[] form)."""
        d = np.ascontiguousarray(degs, dtype=np.int32)
        nb = np.ascontiguousarray(nbrs, dtype=np.int32)
        self._check(self._lib.coral_index_set_slots(self._h, C.c_void_p(d.ctypes.data), 1,
                                                    C.c_void_p(nb.ctypes.data), nb.shape[1]))

    def set_start_ids(self, ids):
        a = np.ascontiguousarray(ids.cpu().numpy() if _is_torch(ids) else ids, dtype=np.int32)
        self._check(self._lib.coral_index_set_start_ids(self._h, C.c_void_p(a.ctypes.data), int(a.size)))

    def select_start_ids(self, first_id, M):
        """Farthest-point sampling of M entry points from `first_id` (the reference's Graph::FPS with a
        caller-chosen first node); installs them and returns them as int32 [M]."""
        out = np.empty(int(M), dtype=np.int32)
        self._check(self._lib.coral_index_select_start_ids(self._h, int(first_id), int(M),
                                                           C.c_void_p(out.ctypes.data)))
        return out

    def get_adjacency(self):
        """The installed adjacency as numpy int32 [n, deg_pad]."""
        adj = np.empty((self.n, self.get_option("deg_pad")), np.int32)
        self._check(self._lib.coral_index_get_adjacency(self._h, C.c_void_p(adj.ctypes.data)))
        return adj

    def get_adjacency_tensor(self, device):
        """The installed adjacency as a CUDA int32 tensor [n, deg_pad] (device-to-device copy)."""
        import torch
        adj = torch.empty((self.n, self.get_option("deg_pad")), dtype=torch.int32, device=device)
        self._check(self._lib.coral_index_get_adjacency(self._h, C.c_void_p(adj.data_ptr())))
        return adj

    def get_start_ids(self):
        m = self._lib.coral_index_get_start_ids(self._h, None, 0)
        out = np.empty(max(m, 0), np.int32)
        self._lib.coral_index_get_start_ids(self._h, C.c_void_p(out.ctypes.data), int(out.size))
        return out

    def set_deleted(self, bits):
        if bits is None:
            self._check(self._lib.coral_index_set_deleted(self._h, None))
            return
        a = np.ascontiguousarray(bits, dtype=np.uint32)
        assert a.size == (self.n + 31) // 32
        self._check(self._lib.coral_index_set_deleted(self._h, C.c_void_p(a.ctypes.data)))

    # ---- options
    def set_option(self, name: str, value: int):
        self._check(self._lib.coral_set_option(self._h, name.encode(), int(value)))

    def get_option(self, name: str) -> int:
        v = C.c_int(0)
        self._check(self._lib.coral_get_option(self._h, name.encode(), C.byref(v)))
        return v.value

    # ---- search
    def prepare(self, max_queries: int, max_L: int, max_k: int):
        self._check(self._lib.coral_search_prepare(self._h, int(max_queries), int(max_L), int(max_k)))

    def search_free(self):
        self._check(self._lib.coral_search_free(self._h))

    def search(self, queries, L: int, k: int, dists: bool = True, stats: bool = False):
        """Host numpy in -> host numpy out; CUDA torch tensor in -> CUDA torch tensors out.

        Returns (ids[Q,k], dists[Q,k] | None, stats[Q,8] | None, total_hops).
        """
        hops = C.c_int64(0)
        if _is_torch(queries) and queries.is_cuda:
            import torch
            q = queries.to(torch.float32).contiguous()
            Q = q.shape[0]
            torch.cuda.current_stream(q.device).synchronize()   # the handle runs on its own stream
            ids = torch.empty((Q, k), dtype=torch.int32, device=q.device)
            dd = torch.empty((Q, k), dtype=torch.float32, device=q.device) if dists else None
            ss = torch.empty((Q, STATS_W), dtype=torch.int32, device=q.device) if stats else None
            rc = self._lib.coral_search(self._h, C.c_void_p(q.data_ptr()), Q, L, k, C.c_void_p(ids.data_ptr()),
                                        C.c_void_p(dd.data_ptr()) if dists else None,
                                        C.c_void_p(ss.data_ptr()) if stats else None, C.byref(hops))
            self._check(rc)
            return ids, dd, ss, int(hops.value)
        q = np.ascontiguousarray(queries, dtype=np.float32)
        Q = q.shape[0]
        ids = np.empty((Q, k), np.int32)
        dd = np.empty((Q, k), np.float32) if dists else None
        ss = np.empty((Q, STATS_W), np.int32) if stats else None
        rc = self._lib.coral_search(self._h, C.c_void_p(q.ctypes.data), Q, L, k, C.c_void_p(ids.ctypes.data),
                                    C.c_void_p(dd.ctypes.data) if dists else None,
                                    C.c_void_p(ss.ctypes.data) if stats else None, C.byref(hops))
        self._check(rc)
        return ids, dd, ss, int(hops.value)

    def search_async(self, d_queries, L, k, d_ids, d_dists=None, d_stats=None, stream=None):
        """Device tensors only; enqueues on `stream` (an int cudaStream_t or None) and returns."""
        rc = self._lib.coral_search_async(
            self._h, C.c_void_p(d_queries.data_ptr()), int(d_queries.shape[0]), L, k, C.c_void_p(d_ids.data_ptr()),
            C.c_void_p(d_dists.data_ptr()) if d_dists is not None else None,
            C.c_void_p(d_stats.data_ptr()) if d_stats is not None else None,
            C.c_void_p(stream) if stream else None)
        self._check(rc)

    def check(self):
        self._check(self._lib.coral_search_check(self._h))

    def query_order(self, d_queries, stream=None):
        """CUDA int32 tensor [Q]: the batch in the locality order (see coral_query_order)."""
        import torch
        order = torch.empty(int(d_queries.shape[0]), dtype=torch.int32, device=d_queries.device)
        self._check(self._lib.coral_query_order(self._h, C.c_void_p(d_queries.data_ptr()), int(d_queries.shape[0]),
                                                C.c_void_p(order.data_ptr()), C.c_void_p(stream) if stream else None))
        return order

    @property
    def last_kernel_ms(self) -> float:
        return float(self._lib.coral_last_kernel_ms(self._h))

    @property
    def last_total_ms(self) -> float:
        return float(self._lib.coral_last_total_ms(self._h))

    @property
    def launch_count(self) -> int:
        return int(self._lib.coral_launch_count(self._h))

    # ---- companions
    def count_hits(self, res, gt, k: int) -> int:
        rp, rk = _ptr(res, np.int32)
        gp, gk = _ptr(gt, np.int32)
        hits = C.c_int64(0)
        self._check(self._lib.coral_count_hits(self._h, rp, gp, int(rk.shape[0]), k, int(gk.shape[1]), C.byref(hits)))
        return int(hits.value)

    def exact_knn(self, queries, k: int, dists: bool = True):
        """Exact k nearest of the handle's vectors.  Host numpy in -> numpy out, CUDA tensor in -> CUDA
        tensors out.  Returns (ids[Q,k], dists[Q,k] | None, number of uncertified queries)."""
        bad = C.c_int64(0)
        if _is_torch(queries) and queries.is_cuda:
            import torch
            q = queries.to(torch.float32).contiguous()
            torch.cuda.current_stream(q.device).synchronize()
            ids = torch.empty((q.shape[0], k), dtype=torch.int32, device=q.device)
            dd = torch.empty((q.shape[0], k), dtype=torch.float32, device=q.device) if dists else None
            self._check(self._lib.coral_exact_knn(self._h, C.c_void_p(q.data_ptr()), int(q.shape[0]), k,
                                                  C.c_void_p(ids.data_ptr()),
                                                  C.c_void_p(dd.data_ptr()) if dists else None, C.byref(bad)))
            return ids, dd, int(bad.value)
        q = np.ascontiguousarray(queries, dtype=np.float32)
        ids = np.empty((q.shape[0], k), np.int32)
        dd = np.empty((q.shape[0], k), np.float32) if dists else None
        self._check(self._lib.coral_exact_knn(self._h, C.c_void_p(q.ctypes.data), int(q.shape[0]), k,
                                              C.c_void_p(ids.ctypes.data),
                                              C.c_void_p(dd.ctypes.data) if dists else None, C.byref(bad)))
        return ids, dd, int(bad.value)

    @property
    def last_dense_tflops(self) -> float:
        ms = float(self._lib.coral_last_dense_ms(self._h))
        return float(self._lib.coral_last_dense_flops(self._h)) / (ms * 1e-3) / 1e12 if ms > 0 else 0.0

    # ---- graph build
    def build_begin(self):
        self._check(self._lib.coral_build_begin(self._h))

    def build_nap(self, lists, batch: int = 0):
        p, k = _ptr(lists, np.int32)
        self._check(self._lib.coral_build_nap(self._h, p, int(k.shape[0]), int(k.shape[1]), int(batch)))

    def build_connect_enhance(self, kb: int, L: int = 0, search_batch: int = 0, nap_batch: int = 0, M: int = 0) -> int:
        n_iso = C.c_int64(0)
        self._check(self._lib.coral_build_connect_enhance(self._h, int(kb), int(L), int(search_batch), int(nap_batch),
                                                          int(M), C.byref(n_iso)))
        return int(n_iso.value)

    def build_get_graph(self):
        """(adj[n, deg_pad] int32, dists[n, deg_pad] float32, deg[n] int32) as numpy arrays."""
        deg_pad = self.get_option("deg_pad")
        adj = np.empty((self.n, deg_pad), np.int32)
        dd = np.empty((self.n, deg_pad), np.float32)
        deg = np.empty(self.n, np.int32)
        self._check(self._lib.coral_build_get_graph(self._h, C.c_void_p(adj.ctypes.data), C.c_void_p(dd.ctypes.data),
                                                    C.c_void_p(deg.ctypes.data)))
        return adj, dd, deg

    def build_set_graph(self, adj, dists, deg):
        a, ka = _ptr(adj, np.int32)
        d, kd = _ptr(dists, np.float32)
        g, kg = _ptr(deg, np.int32)
        self._check(self._lib.coral_build_set_graph(self._h, a, d, g))

    def build_end(self):
        self._check(self._lib.coral_build_end(self._h))

    def set_live(self, live: int):
        self._check(self._lib.coral_index_set_live(self._h, int(live)))

    def update_begin(self):
        self._check(self._lib.coral_build_begin_from_graph(self._h))

    def delete(self, ids, M: int = 0):
        a = np.ascontiguousarray(ids, dtype=np.int32)
        self._check(self._lib.coral_delete(self._h, C.c_void_p(a.ctypes.data), int(a.size), int(M)))

    def insert(self, first_id: int, count: int, kb: int, L: int = 0, batch: int = 0, M: int = 0):
        self._check(self._lib.coral_insert(self._h, int(first_id), int(count), int(kb), int(L), int(batch), int(M)))

    def build(self, train_queries, kb: int = 100, batch: int = 0, ce: bool = True, ce_L: int = 0,
              ce_search_batch: int = 0, ce_nap_batch: int = 0, M: int = 0):
        """The whole build over the handle's vectors, as IndexGPU::BuildGPU runs it
        (src/index_gpu.cpp:308-383): exact k_b nearest base points of every training query, NAP in
        batches, CE of the isolated nodes.  Leaves the graph and CE's entry points installed.
        Returns a dict with the number of isolated nodes and uncertified k-NN rows."""
        knn, _, bad = self.exact_knn(train_queries, kb, dists=False)
        self.build_begin()
        self.build_nap(knn, batch)
        n_iso = self.build_connect_enhance(kb, ce_L, ce_search_batch, ce_nap_batch, M) if ce else 0
        if not ce or n_iso == 0:
            adj, _, deg = self.build_get_graph()
            self.select_start_ids(int(np.nonzero(deg > 0)[0][0]), M or 16)
        self.build_end()
        return {"isolated": n_iso, "uncertified_knn": bad}

    def merge_shards(self, d_ids, d_dists, stream=None):
        """d_ids/d_dists: CUDA tensors [G,Q,k] -> merged CUDA tensors ([Q,k], [Q,k])."""
        import torch
        G, Q, k = d_ids.shape
        oi = torch.empty((Q, k), dtype=torch.int32, device=d_ids.device)
        od = torch.empty((Q, k), dtype=torch.float32, device=d_ids.device)
        self._check(self._lib.coral_merge_shards(self._h, C.c_void_p(d_ids.data_ptr()), C.c_void_p(d_dists.data_ptr()),
                                                 G, Q, k, C.c_void_p(oi.data_ptr()), C.c_void_p(od.data_ptr()),
                                                 C.c_void_p(stream) if stream else None))
        return oi, od

    def map_ids(self, d_ids, d_id_map, stream=None):
        self._check(self._lib.coral_map_ids(self._h, C.c_void_p(d_ids.data_ptr()), int(d_ids.numel()),
                                            C.c_void_p(d_id_map.data_ptr()), C.c_void_p(stream) if stream else None))
