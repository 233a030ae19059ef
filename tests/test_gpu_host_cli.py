"""End to end through the C++ mirror: files in the reference's formats -> efanna2e::IndexGPU
(LoadSearchNeededData, RunPrepare, Search) driven by the test_search_pipeline binary with the
reference's flags -> ids identical to the CPU oracle's."""
import os
import struct
import subprocess

import numpy as np
import pytest

from coral_b200.host import build_host
from oracle import oracle
from tests import cases
from tests.test_host_formats import _literal_block, write_reference_graph_dir

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("metric", ["l2", "ip"])
def test_search_pipeline_driver_matches_oracle(tmp_path, metric):
    import torch
    from coral_b200 import synth
    build_host.build()
    c = cases.structured(metric)
    k = 10
    # for inner product hand the driver un-normalised copies: it must normalise base and queries itself
    scale = np.linspace(0.5, 2.0, c.n, dtype=np.float32)[:, None] if metric == "ip" else 1.0
    qscale = np.float32(3.0) if metric == "ip" else np.float32(1.0)
    (tmp_path / "base.fbin").write_bytes(struct.pack("<ii", c.n, c.dim) + (c.base * scale).astype(np.float32).tobytes())
    (tmp_path / "query.fbin").write_bytes(struct.pack("<ii", len(c.queries), c.dim) + (c.queries * qscale).tobytes())
    gt = synth.exact_knn(torch.from_numpy(c.base), torch.from_numpy(c.queries), 100, metric).numpy()
    (tmp_path / "gt.bin").write_bytes(struct.pack("<ii", gt.shape[0], gt.shape[1]) + gt.astype(np.int32).tobytes())
    degs = (c.adj >= 0).sum(1)
    write_reference_graph_dir(str(tmp_path / "graph"), degs, c.adj, _literal_block)
    (tmp_path / "graph" / "graph.search_start_ids").write_text(
        f"{len(c.start)} " + " ".join(str(int(v)) for v in c.start) + " ")
    (tmp_path / "config.json").write_text('{"dim": %d, "k": 100, "search_start_nodes_num": 16}' % c.dim)
    exe = os.path.join(os.path.dirname(build_host.HOST_LIB), "test_search_pipeline")
    cmd = [exe, "--dataset", "synthetic", "--data_type", "float", "--dist", metric,
           "--base_data_path", str(tmp_path / "base.fbin"), "--query_path", str(tmp_path / "query.fbin"),
           "--gt_path", str(tmp_path / "gt.bin"), "--graph_path", str(tmp_path / "graph"),
           "--config_file", str(tmp_path / "config.json"), "--max_degree", "32", "--k", str(k),
           "--L", "64", "128", "-T", "8", "--csv", str(tmp_path / "out.csv"), "--ids_out", str(tmp_path / "ids.bin")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    rows = [ln.split(",") for ln in (tmp_path / "out.csv").read_text().strip().splitlines()[1:]]
    assert [int(x[0]) for x in rows] == [64, 128]
    ids = np.fromfile(tmp_path / "ids.bin", dtype=np.int32).reshape(len(c.queries), k)     # the last sweep point
    if metric == "ip":
        # the driver normalised scaled copies; normalise the same way before asking the oracle
        b = (c.base * scale).astype(np.float32)
        q = (c.queries * qscale).astype(np.float32)
        for arr in (b, q):                           # reference src/uni.cpp:38-54, float32 throughout
            n2 = np.cumsum(arr * arr, axis=1, dtype=np.float32)[:, -1]      # sequential float32 sum
            inv = (np.float32(1.0) / np.sqrt(n2, dtype=np.float32)).astype(np.float32)
            arr *= inv[:, None]
    else:
        b, q = c.base, c.queries
    ref_ids, _, st = oracle.search(b, c.adj, c.start, q, 128, k, metric)
    assert np.array_equal(ids, ref_ids)
    recall, hops = float(rows[1][3]), float(rows[1][4])
    assert abs(recall - oracle.recall(ref_ids, gt, k)) < 1e-6
    assert abs(hops - st[:, 4].mean()) < 1e-2 * max(1.0, st[:, 4].mean())


def test_driver_reports_errors_instead_of_crashing(tmp_path):
    build_host.build()
    exe = os.path.join(os.path.dirname(build_host.HOST_LIB), "test_search_pipeline")
    r = subprocess.run([exe, "--dataset", "x", "--data_type", "float", "--dist", "l2", "--base_data_path", "/nonexistent",
                        "--query_path", "/nonexistent", "--gt_path", "/nonexistent"], capture_output=True, text=True)
    assert r.returncode != 0 and "cannot" in (r.stdout + r.stderr).lower()
    r = subprocess.run([exe, "--dist", "l2"], capture_output=True, text=True)
    assert r.returncode != 0 and "required" in r.stderr


def test_driver_selects_and_saves_entry_points_when_none_are_stored(tmp_path):
    """A graph directory without graph.search_start_ids: the mirror picks the entry points by
    farthest-point sampling from the lowest-numbered node with an out-edge, saves them in the
    reference's text form, and searches from them."""
    build_host.build()
    c = cases.structured("l2")
    k = 10
    (tmp_path / "base.fbin").write_bytes(struct.pack("<ii", c.n, c.dim) + c.base.tobytes())
    (tmp_path / "query.fbin").write_bytes(struct.pack("<ii", len(c.queries), c.dim) + c.queries.tobytes())
    gt = np.zeros((len(c.queries), 100), np.int32)
    (tmp_path / "gt.bin").write_bytes(struct.pack("<ii", gt.shape[0], gt.shape[1]) + gt.tobytes())
    degs = (c.adj >= 0).sum(1)
    write_reference_graph_dir(str(tmp_path / "graph"), degs, c.adj, _literal_block)
    (tmp_path / "config.json").write_text('{"dim": %d, "k": 100, "search_start_nodes_num": 12}' % c.dim)
    exe = os.path.join(os.path.dirname(build_host.HOST_LIB), "test_search_pipeline")
    cmd = [exe, "--dataset", "synthetic", "--data_type", "float", "--dist", "l2",
           "--base_data_path", str(tmp_path / "base.fbin"), "--query_path", str(tmp_path / "query.fbin"),
           "--gt_path", str(tmp_path / "gt.bin"), "--graph_path", str(tmp_path / "graph"),
           "--config_file", str(tmp_path / "config.json"), "--max_degree", "32", "--k", str(k),
           "--L", "64", "-T", "8", "--ids_out", str(tmp_path / "ids.bin")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    first = int(np.flatnonzero(degs > 0)[0])
    want = oracle.select_start_ids(c.adj, first, 12)
    saved = [int(x) for x in (tmp_path / "graph" / "graph.search_start_ids").read_text().split()]
    assert saved == [12] + want.tolist()
    ids = np.fromfile(tmp_path / "ids.bin", dtype=np.int32).reshape(len(c.queries), k)
    ref_ids, _, _ = oracle.search(c.base, c.adj, want, c.queries, 64, k, "l2")
    assert np.array_equal(ids, ref_ids)


def test_driver_flat_graph_import_deleted_ids_and_device_hit_count(tmp_path):
    """IndexGPU::LoadRoarGraph (flat graph, single entry point), SetDeleted and Search_and_Verify
    through the driver: ids equal the oracle's with the deleted ids skipped, and the hit count
    made on the device equals the recall sum computed from those ids."""
    import ctypes as C
    build_host.build()
    c = cases.structured("l2")
    k, L = 10, 64
    lib = C.CDLL(build_host.HOST_LIB)
    lib.coral_host_flat_graph_roundtrip.argtypes = [C.c_char_p, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_int32,
                                                    C.c_void_p, C.POINTER(C.c_int32)]
    lib.coral_host_flat_graph_roundtrip.restype = C.c_int
    ep = int(c.start[3])
    back = np.empty_like(c.adj)
    ep_back = C.c_int32(-1)
    dp = lib.coral_host_flat_graph_roundtrip(str(tmp_path / "flat.bin").encode(), c.n, c.adj.shape[1], 32,
                                             c.adj.ctypes.data, ep, back.ctypes.data, C.byref(ep_back))
    assert dp == c.adj.shape[1] and ep_back.value == ep
    (tmp_path / "base.fbin").write_bytes(struct.pack("<ii", c.n, c.dim) + c.base.tobytes())
    (tmp_path / "query.fbin").write_bytes(struct.pack("<ii", len(c.queries), c.dim) + c.queries.tobytes())
    # any graph directory satisfies RunPrepare; the flat graph replaces it afterwards
    degs = (c.adj >= 0).sum(1)
    write_reference_graph_dir(str(tmp_path / "graph"), degs, c.adj, _literal_block)
    (tmp_path / "graph" / "graph.search_start_ids").write_text("1 0 ")
    (tmp_path / "config.json").write_text('{"dim": %d, "k": %d}' % (c.dim, k))
    start = np.array([ep], np.int32)
    full_ids, _, _ = oracle.search(c.base, c.adj, start, c.queries, L, L, "l2")
    dead = sorted({int(v) for v in full_ids[:, 0] if v >= 0})      # hide every query's best hit
    (tmp_path / "dead.txt").write_text(" ".join(map(str, dead)))
    want = np.full((len(c.queries), k), -1, np.int32)
    for qi in range(len(c.queries)):
        keep = [v for v in full_ids[qi] if v >= 0 and v not in set(dead)][:k]
        want[qi, :len(keep)] = keep
    gt = want.copy()                                                # ground truth exactly k wide
    gt[:, ::2] = 0                                                  # half of it wrong on purpose
    (tmp_path / "gt.bin").write_bytes(struct.pack("<ii", gt.shape[0], gt.shape[1]) + gt.astype(np.int32).tobytes())
    exe = os.path.join(os.path.dirname(build_host.HOST_LIB), "test_search_pipeline")
    cmd = [exe, "--dataset", "synthetic", "--data_type", "float", "--dist", "l2",
           "--base_data_path", str(tmp_path / "base.fbin"), "--query_path", str(tmp_path / "query.fbin"),
           "--gt_path", str(tmp_path / "gt.bin"), "--graph_path", str(tmp_path / "graph"),
           "--roar_graph", str(tmp_path / "flat.bin"), "--deleted_ids", str(tmp_path / "dead.txt"), "--verify",
           "--config_file", str(tmp_path / "config.json"), "--max_degree", "32", "--k", str(k),
           "--L", str(L), "--ids_out", str(tmp_path / "ids.bin")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    ids = np.fromfile(tmp_path / "ids.bin", dtype=np.int32).reshape(len(c.queries), k)
    assert np.array_equal(ids, want)
    hits = [int(ln.split()[1]) for ln in r.stdout.splitlines() if ln.startswith("hits ")]
    expect = sum(sum(1 for p in gt[qi] if p in ids[qi]) for qi in range(len(c.queries)))
    assert hits == [expect]


def test_driver_shards_builds_per_shard_graphs_and_merges_through_nccl(tmp_path):
    """--shards 1 --seed S --train_path F: the driver partitions the base, builds the shard's graph
    with IndexGPU::BuildGPU (exact lists -> NAP -> CE), writes it in the reference's directory
    layout, searches through coral_search_sharded (a one-rank NCCL communicator), and a second run
    loads the saved graph instead of building -- same ids both times, good recall."""
    import torch
    from coral_b200 import synth
    build_host.build()
    n, dim, k = 8000, 64, 10
    ds = synth.make_l2_mixture(n, 2000, 64, dim=dim, centers=8, seed=21, rot_dims=60, latent_dim=8, latent_jitter=0.5)
    base, train, q = ds.base.numpy(), ds.train.numpy(), ds.test.numpy()
    for name, arr in (("base", base), ("train", train), ("query", q)):
        (tmp_path / f"{name}.fbin").write_bytes(struct.pack("<ii", *arr.shape) + arr.tobytes())
    gt, _ = oracle.exact_knn(base, q, 100, "l2")
    (tmp_path / "gt.bin").write_bytes(struct.pack("<ii", gt.shape[0], gt.shape[1]) + gt.astype(np.int32).tobytes())
    (tmp_path / "config.json").write_text('{"dim": %d, "k": 100, "batch": 256, "enhance_search_batch": 2048, '
                                          '"enhance_nap_batch": 512}' % dim)
    os.makedirs(tmp_path / "graph")
    exe = os.path.join(os.path.dirname(build_host.HOST_LIB), "test_search_pipeline")
    cmd = [exe, "--dataset", "synthetic", "--data_type", "float", "--dist", "l2",
           "--base_data_path", str(tmp_path / "base.fbin"), "--query_path", str(tmp_path / "query.fbin"),
           "--gt_path", str(tmp_path / "gt.bin"), "--graph_path", str(tmp_path / "graph"),
           "--train_path", str(tmp_path / "train.fbin"), "--config_file", str(tmp_path / "config.json"),
           "--max_degree", "32", "--k", str(k), "--L", "64", "--shards", "1", "--seed", "7"]
    outs = []
    for run in range(2):
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout + r.stderr
        assert ("Build shard 0" in r.stdout) == (run == 0)
        row = [ln.split() for ln in r.stdout.splitlines() if ln.startswith("64")][-1]
        outs.append(float(row[3]))
    assert os.path.exists(tmp_path / "graph" / "shard0" / "graph.search_start_ids")
    assert outs[0] == outs[1] and outs[0] >= 0.9


def test_update_driver_slides_the_window_like_the_library_calls(tmp_path):
    """test_update with the reference's flags (tests/test_update.cpp): the index is built over the
    first half of the base, then three rounds of IndexGPU::Delete (oldest third, with repair) +
    IndexGPU::Insert (next third of the second half), verified after each (upd_mode 4).  The graph the
    driver ends with equals the one the same sequence of C-ABI calls gives through the Python
    binding (whose delete and insert are held to the oracle in test_gpu_update.py), and after the last
    round no result is one of the original points.  Recall is only asserted before the first insert:
    with neighbours from the search alone (upd_type 1) a new point enters a full row of a pivot only
    when no closer neighbour occludes it (src/update.cu:150-187), so on a set this small and dense
    most inserted points get no in-edge and recall falls as the window slides -- the CPU restatement
    of the reference kernels shows the same numbers."""
    import ctypes as C
    from coral_b200 import capi, synth
    build_host.build()
    total, dim, deg, k, L, rounds = 6000, 64, 32, 10, 128, 3
    half = total // 2
    ds = synth.make_l2_mixture(total, 1500, 64, dim=dim, centers=8, seed=33, rot_dims=60, latent_dim=8, latent_jitter=0.5)
    base, train, q = ds.base.numpy(), ds.train.numpy(), ds.test.numpy()
    for name, arr in (("base", base), ("train", train), ("query", q)):
        (tmp_path / f"{name}.fbin").write_bytes(struct.pack("<ii", *arr.shape) + arr.tobytes())
    cfg = dict(dim=dim, k=50, batch=256, enhance_search_batch=2048, enhance_nap_batch=512, insert_batch=512,
               test_beam_capacity=128, search_start_nodes_num=16)
    (tmp_path / "config.json").write_text("{" + ", ".join('"%s": %d' % kv for kv in cfg.items()) + "}")
    exe = os.path.join(os.path.dirname(build_host.HOST_LIB), "test_update")
    cmd = [exe, "--dataset", "synthetic", "--data_type", "float", "--dist", "l2", "--upd_mode", "4", "--rounds", str(rounds),
           "--base_data_path", str(tmp_path / "base.fbin"), "--sampled_query_data_path", str(tmp_path / "train.fbin"),
           "--query_path", str(tmp_path / "query.fbin"), "--graph_path", str(tmp_path / "graph"),
           "--config_file", str(tmp_path / "config.json"), "--max_degree", str(deg), "--k", str(k), "--L", str(L),
           "--dump_graph", str(tmp_path / "final"), "--ids_out", str(tmp_path / "ids.bin"), "--csv", str(tmp_path / "eva.csv")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Building initial index..." in r.stdout and "Finished" in r.stdout
    rows = [ln.split(", ") for ln in (tmp_path / "eva.csv").read_text().splitlines()[1:]]
    assert [row[0] for row in rows] == ["0", "1 after delete", "1", "2 after delete", "2", "3 after delete", "3"]
    assert float(rows[0][1]) >= 95.0 and float(rows[1][1]) >= 95.0, rows
    assert all(0.0 <= float(row[1]) <= 100.0 and float(row[4]) > 0 for row in rows), rows
    ids = np.fromfile(tmp_path / "ids.bin", dtype=np.int32).reshape(len(q), k)
    assert ((ids == -1) | ((ids >= half) & (ids < total))).all()       # every original point has been deleted

    # the same sequence through the binding
    step = half // rounds
    with capi.Index(half, dim, deg, "l2") as b:
        b.set_vectors(base[:half])
        b.build(train, kb=cfg["k"], batch=cfg["batch"], ce_L=256, ce_search_batch=cfg["enhance_search_batch"],
                ce_nap_batch=cfg["enhance_nap_batch"], M=16)
        adj0, starts0 = b.get_adjacency(), b.get_start_ids()
    with capi.Index(2 * half, dim, deg, "l2") as ix:
        ix.write_vectors(0, base[:half])
        ix.set_live(half)
        full = np.full((2 * half, adj0.shape[1]), -1, np.int32)
        full[:half] = adj0
        ix.set_adjacency(full)
        ix.set_start_ids(starts0)
        ix.update_begin()
        live = half
        for rd in range(rounds):
            ix.delete(np.arange(rd * step, (rd + 1) * step, dtype=np.int32), M=16)
            ix.write_vectors(live, base[half + rd * step: half + (rd + 1) * step])
            ix.insert(live, step, kb=cfg["k"], L=cfg["test_beam_capacity"], batch=cfg["insert_batch"], M=16)
            live += step
        want_adj, want_starts = ix.get_adjacency()[:live], ix.get_start_ids()
    host = C.CDLL(build_host.HOST_LIB)
    host.coral_host_graph_dir_load.argtypes = [C.c_char_p, C.c_int64, C.c_int, C.c_void_p, C.POINTER(C.c_int)]
    host.coral_host_start_ids_load.argtypes = [C.c_char_p, C.c_void_p, C.c_int]
    got = np.empty((live, 128), np.int32)
    dp = C.c_int(0)
    assert host.coral_host_graph_dir_load(str(tmp_path / "final").encode(), live, deg, got.ctypes.data, C.byref(dp)) == 0
    got = got.reshape(-1)[: live * dp.value].reshape(live, dp.value)
    assert dp.value == want_adj.shape[1] and np.array_equal(got, want_adj)
    st = np.empty(64, np.int32)
    m = host.coral_host_start_ids_load(str(tmp_path / "final" / "graph.search_start_ids").encode(), st.ctypes.data, 64)
    assert m == len(want_starts) and np.array_equal(st[:m], want_starts)


@pytest.mark.parametrize("from_lists", [False, True])
def test_build_driver_writes_the_graph_the_library_builds(tmp_path, from_lists):
    """test_build_pipeline with the reference's flags: IndexGPU::BuildGPU over .fbin files writes a
    graph directory that holds exactly the graph and entry points the same build gives through the
    binding (held to the oracle in test_gpu_build.py), searchable by test_search_pipeline.  With
    --train_gt_file the training queries' lists are read from a file instead of searched."""
    import ctypes as C
    from coral_b200 import capi, synth
    build_host.build()
    n, dim, deg, kb = 5000, 48, 32, 40
    ds = synth.make_ip_cones(n, 1200, 50, dim=dim, clusters=8, seed=5, latent_dim=8, latent_jitter=0.5)
    base, train, q = (np.ascontiguousarray(a.numpy()) for a in (ds.base, ds.train, ds.test))
    for name, arr in (("base", base), ("train", train), ("query", q)):
        (tmp_path / f"{name}.fbin").write_bytes(struct.pack("<ii", *arr.shape) + arr.tobytes())
    # the driver unit-normalises what it loads; take the vectors back through the same loader so that the
    # binding below sees the same bits
    host = C.CDLL(build_host.HOST_LIB)
    host.coral_host_fbin_load.argtypes = [C.c_char_p, C.c_void_p, C.c_int64, C.POINTER(C.c_int64), C.POINTER(C.c_int), C.c_int]
    for name, arr in (("base", base), ("train", train), ("query", q)):
        nn, dd = C.c_int64(0), C.c_int(0)
        assert host.coral_host_fbin_load(str(tmp_path / f"{name}.fbin").encode(), arr.ctypes.data, arr.size, C.byref(nn),
                                         C.byref(dd), 1) == 0 and (nn.value, dd.value) == arr.shape
    gt, _ = oracle.exact_knn(base, q, 10, "ip")
    (tmp_path / "gt.bin").write_bytes(struct.pack("<ii", *gt.shape) + gt.astype(np.int32).tobytes())
    (tmp_path / "config.json").write_text('{"dim": %d, "k": %d, "batch": 256, "enhance_search_batch": 2048, '
                                          '"enhance_nap_batch": 512, "test_beam_capacity": 64}' % (dim, kb))
    lists, _ = oracle.exact_knn(base, train, kb, "ip")
    extra = []
    if from_lists:
        # lists that the exact search would NOT give (each shifted by one rank): the driver must use them
        wide, _ = oracle.exact_knn(base, train, kb + 1, "ip")
        lists = np.ascontiguousarray(wide[:, 1:])
        (tmp_path / "train_gt.bin").write_bytes(struct.pack("<ii", *lists.shape) + lists.astype(np.int32).tobytes())
        extra = ["--train_gt_file", str(tmp_path / "train_gt.bin")]
    exe = os.path.join(os.path.dirname(build_host.HOST_LIB), "test_build_pipeline")
    cmd = [exe, "--data_type", "float", "--dist", "ip", "--dataset", "synthetic", "--base_data_path", str(tmp_path / "base.fbin"),
           "--sampled_query_data_path", str(tmp_path / "train.fbin"), "--M_pjbp", str(deg), "--k", str(kb), "--CE", "1",
           "--graph_path", str(tmp_path / "graph"), "--config_file", str(tmp_path / "config.json"),
           "--query_test_file", str(tmp_path / "query.fbin"), "--gt_test_file", str(tmp_path / "gt.bin"), *extra]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("Search result: recall@10=")][-1]
    assert float(line.split("=")[1].split(",")[0]) >= 0.9, line

    with capi.Index(n, dim, deg, "ip") as ix:
        ix.set_vectors(base)
        ix.build_begin()
        ix.build_nap(lists.astype(np.int32), 256)
        n_iso = ix.build_connect_enhance(kb, 256, 2048, 512, 16)
        assert n_iso > 0
        ix.build_end()
        want_adj, want_starts = ix.get_adjacency(), ix.get_start_ids()
    host.coral_host_graph_dir_load.argtypes = [C.c_char_p, C.c_int64, C.c_int, C.c_void_p, C.POINTER(C.c_int)]
    host.coral_host_start_ids_load.argtypes = [C.c_char_p, C.c_void_p, C.c_int]
    got = np.empty((n, 128), np.int32)
    dp = C.c_int(0)
    assert host.coral_host_graph_dir_load(str(tmp_path / "graph").encode(), n, deg, got.ctypes.data, C.byref(dp)) == 0
    got = got.reshape(-1)[: n * dp.value].reshape(n, dp.value)
    assert dp.value == want_adj.shape[1] and np.array_equal(got, want_adj)
    st = np.empty(64, np.int32)
    m = host.coral_host_start_ids_load(str(tmp_path / "graph" / "graph.search_start_ids").encode(), st.ctypes.data, 64)
    assert m == len(want_starts) and np.array_equal(st[:m], want_starts)


@pytest.mark.parametrize("metric", ["l2", "ip"])
def test_ground_truth_tool_matches_the_brute_force_oracle(tmp_path, metric):
    """comp_gt with the reference's flags (tests/comp_gt.cpp): exact lists in the ground-truth file
    format, equal to the CPU brute force (same distance arithmetic, ties by id)."""
    build_host.build()
    rng = np.random.default_rng(3)
    base = rng.standard_normal((7000, 72), dtype=np.float32)
    q = rng.standard_normal((130, 72), dtype=np.float32)
    for name, arr in (("base", base), ("query", q)):
        (tmp_path / f"{name}.fbin").write_bytes(struct.pack("<ii", *arr.shape) + arr.tobytes())
    exe = os.path.join(os.path.dirname(build_host.HOST_LIB), "comp_gt")
    r = subprocess.run([exe, "--data_type", "float", "--dist", metric, "--base_data_path", str(tmp_path / "base.fbin"),
                        "--query_data_path", str(tmp_path / "query.fbin"), "--gt_save_file", str(tmp_path / "gt.bin"),
                        "--k", "20", "--nq", "100"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = (tmp_path / "gt.bin").read_bytes()
    nq, k = struct.unpack("<ii", raw[:8])
    assert (nq, k) == (100, 20)
    got = np.frombuffer(raw[8:], dtype=np.int32).reshape(nq, k)
    if metric == "ip":
        import ctypes as C
        host = C.CDLL(build_host.HOST_LIB)
        host.coral_host_fbin_load.argtypes = [C.c_char_p, C.c_void_p, C.c_int64, C.POINTER(C.c_int64), C.POINTER(C.c_int), C.c_int]
        for name, arr in (("base", base), ("query", q)):
            nn, dd = C.c_int64(0), C.c_int(0)
            assert host.coral_host_fbin_load(str(tmp_path / f"{name}.fbin").encode(), arr.ctypes.data, arr.size, C.byref(nn),
                                             C.byref(dd), 1) == 0
    want, _ = oracle.exact_knn(base, q[:100], 20, metric)
    assert np.array_equal(got, want)
