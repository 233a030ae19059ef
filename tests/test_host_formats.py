"""The C++ host mirror's file-format readers, exercised without a GPU through the C hooks
of libcoral_host.so: .fbin, graph directory (LZ4 records, .data/.append, isolated nodes),
start ids, flat graph, config.json -- including the malformed inputs the loaders must
refuse instead of crashing."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from coral_b200.host import build_host


@pytest.fixture(scope="module")
def host():
    lib = C.CDLL(build_host.build())
    lib.coral_host_graph_dir_load.argtypes = [C.c_char_p, C.c_int64, C.c_int, C.c_void_p, C.POINTER(C.c_int)]
    lib.coral_host_graph_dir_write.argtypes = [C.c_char_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int]
    lib.coral_host_flat_graph_roundtrip.argtypes = [C.c_char_p, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_int32,
                                                    C.c_void_p, C.POINTER(C.c_int32)]
    lib.coral_host_start_ids_load.argtypes = [C.c_char_p, C.c_void_p, C.c_int]
    lib.coral_host_lz4_decode.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
    lib.coral_host_fbin_load.argtypes = [C.c_char_p, C.c_void_p, C.c_int64, C.POINTER(C.c_int64), C.POINTER(C.c_int), C.c_int]
    lib.coral_host_config_get.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(C.c_double)]
    return lib


def _liblz4():
    for name in ("liblz4.so.1", "liblz4.so"):
        try:
            lib = C.CDLL(name)
            lib.LZ4_compress_default.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_int]
            lib.LZ4_compressBound.argtypes = [C.c_int]
            return lib
        except OSError:
            continue
    return None


def _lz4_compress(lz4, raw: bytes) -> bytes:
    cap = lz4.LZ4_compressBound(len(raw))
    buf = C.create_string_buffer(cap)
    n = lz4.LZ4_compress_default(raw, buf, len(raw), cap)
    assert n > 0
    return buf.raw[:n]


def _literal_block(raw: bytes) -> bytes:
    n = len(raw)
    if n < 15:
        return bytes([n << 4]) + raw
    out, rest = bytearray([0xF0]), n - 15
    while rest >= 255:
        out.append(255)
        rest -= 255
    out.append(rest)
    return bytes(out) + raw


def write_reference_graph_dir(path, degs, nbrs, compress):
    """Writes the layout the reference's DiskPartition produces (src/disk.cpp:382-426)."""
    os.makedirs(path, exist_ok=True)
    data, append, idx = bytearray(), bytearray(), bytearray()
    for i, d in enumerate(degs):
        if d == 0:
            idx += struct.pack("<QIi", 0, 0, 0)
            continue
        raw = struct.pack("<i", d) + np.asarray(nbrs[i][:d], np.int32).tobytes() + np.zeros(d, np.float32).tobytes()
        rec = struct.pack("<ii", i, len(raw)) + compress(raw)
        target, pos = (append, 1) if i % 3 == 0 else (data, 0)      # some records live in the append file
        idx += struct.pack("<QIi", len(target), len(rec), pos)
        target += rec
    open(os.path.join(path, "graph.part0.idx"), "wb").write(idx)
    open(os.path.join(path, "graph.part0.data"), "wb").write(data)
    open(os.path.join(path, "graph.part0.append"), "wb").write(append)


def test_fbin_roundtrip_normalisation_and_truncation(host, tmp_path):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((37, 12)).astype(np.float32)
    x[5] = 0
    p = tmp_path / "base.fbin"
    p.write_bytes(struct.pack("<ii", 37, 12) + x.tobytes())
    out = np.empty_like(x)
    n, dim = C.c_int64(), C.c_int()
    assert host.coral_host_fbin_load(str(p).encode(), out.ctypes.data, out.size, C.byref(n), C.byref(dim), 0) == 0
    assert (n.value, dim.value) == (37, 12) and np.array_equal(out, x)
    assert host.coral_host_fbin_load(str(p).encode(), out.ctypes.data, out.size, C.byref(n), C.byref(dim), 1) == 0
    norms = np.linalg.norm(out, axis=1)
    assert np.allclose(np.delete(norms, 5), 1.0, atol=1e-6) and norms[5] == 0     # zero rows stay zero
    (tmp_path / "short.fbin").write_bytes(struct.pack("<ii", 38, 12) + x.tobytes())
    assert host.coral_host_fbin_load(str(tmp_path / "short.fbin").encode(), None, 0, C.byref(n), C.byref(dim), 0) == -1
    assert host.coral_host_fbin_load(str(tmp_path / "missing.fbin").encode(), None, 0, C.byref(n), C.byref(dim), 0) == -1


@pytest.mark.parametrize("codec", ["lz4", "literals"])
def test_graph_directory_as_the_reference_writes_it(host, tmp_path, codec):
    lz4 = _liblz4()
    if codec == "lz4" and lz4 is None:
        pytest.skip("liblz4 runtime not present")
    compress = (lambda raw: _lz4_compress(lz4, raw)) if codec == "lz4" else _literal_block
    rng = np.random.default_rng(1)
    n, max_degree = 500, 32
    degs = rng.integers(0, 41, n)            # some isolated (0), some above max_degree
    nbrs = [np.sort(rng.integers(0, n, 64)) for _ in range(n)]      # sorted ids compress well
    d = tmp_path / "idx"
    write_reference_graph_dir(str(d), degs, nbrs, compress)
    (d / "graph.search_start_ids").write_text("3 7 8 9 ")
    rows = np.empty((n, 32), np.int32)
    deg_pad = C.c_int()
    assert host.coral_host_graph_dir_load(str(d).encode(), n, max_degree, rows.ctypes.data, C.byref(deg_pad)) == 0
    assert deg_pad.value == 32
    for i in range(n):
        want = list(nbrs[i][:min(degs[i], max_degree)])
        assert list(rows[i][:len(want)]) == want and (rows[i][len(want):] == -1).all()
    ids = np.zeros(8, np.int32)
    assert host.coral_host_start_ids_load(str(d / "graph.search_start_ids").encode(), ids.ctypes.data, 8) == 3
    assert list(ids[:3]) == [7, 8, 9]


def test_graph_directory_written_here_reads_back_and_bad_input_is_refused(host, tmp_path):
    rng = np.random.default_rng(2)
    n = 300
    rows = rng.integers(0, n, (n, 64)).astype(np.int32)
    deg = rng.integers(0, 65, n)
    rows[np.arange(64)[None, :] >= deg[:, None]] = -1
    start = np.array([1, 2, 3, 4], np.int32)
    d = tmp_path / "mine"
    assert host.coral_host_graph_dir_write(str(d).encode(), n, 64, rows.ctypes.data, start.ctypes.data, 4) == 0
    back = np.empty_like(rows)
    dp = C.c_int()
    assert host.coral_host_graph_dir_load(str(d).encode(), n, 64, back.ctypes.data, C.byref(dp)) == 0
    assert dp.value == 64 and np.array_equal(back, rows)
    # index table shorter than n entries
    assert host.coral_host_graph_dir_load(str(d).encode(), n + 50, 64, None, C.byref(dp)) == -1
    # a corrupted LZ4 block (match offset pointing before the start of the output)
    blob = bytearray((d / "graph.part0.data").read_bytes())
    blob[8] = 0x0F            # token: 0 literals, then a match -> offset beyond output
    (d / "graph.part0.data").write_bytes(blob)
    assert host.coral_host_graph_dir_load(str(d).encode(), n, 64, None, C.byref(dp)) == -1
    assert host.coral_host_graph_dir_load(str(tmp_path / "nowhere").encode(), n, 64, None, C.byref(dp)) == -1


def test_lz4_block_decoder_against_liblz4(host):
    lz4 = _liblz4()
    if lz4 is None:
        pytest.skip("liblz4 runtime not present")
    rng = np.random.default_rng(3)
    for size in (1, 13, 200, 5000, 70000):
        raw = bytes(rng.integers(0, 4, size, dtype=np.uint8)) + b"abcabcabcabc" * (size // 10)   # compressible
        comp = _lz4_compress(lz4, raw)
        out = C.create_string_buffer(len(raw))
        assert host.coral_host_lz4_decode(comp, len(comp), out, len(raw)) == len(raw)
        assert out.raw == raw
        assert host.coral_host_lz4_decode(comp, len(comp), out, len(raw) - 1) == -1       # output too small
        if len(comp) > 4:
            assert host.coral_host_lz4_decode(comp, len(comp) - 3, out, len(raw)) != len(raw)   # truncated input


def test_start_ids_truncated_list_is_dropped(host, tmp_path):
    p = tmp_path / "s"
    p.write_text("5 1 2 3")                    # claims 5, holds 3 (reference src/graph.cpp:341-345)
    ids = np.zeros(8, np.int32)
    assert host.coral_host_start_ids_load(str(p).encode(), ids.ctypes.data, 8) == 0
    assert host.coral_host_start_ids_load(str(tmp_path / "none").encode(), ids.ctypes.data, 8) == 0


def test_flat_graph_roundtrip_cuts_at_max_degree(host, tmp_path):
    rng = np.random.default_rng(4)
    n = 200
    rows = rng.integers(0, n, (n, 64)).astype(np.int32)
    deg = rng.integers(0, 65, n)
    rows[np.arange(64)[None, :] >= deg[:, None]] = -1
    out = np.empty((n, 32), np.int32)
    ep = C.c_int32()
    dp = host.coral_host_flat_graph_roundtrip(str(tmp_path / "flat.bin").encode(), n, 64, 32, rows.ctypes.data, 17,
                                              out.ctypes.data, C.byref(ep))
    assert dp == 32 and ep.value == 17
    assert np.array_equal(out, rows[:, :32])


def test_config_json_flat_object(host, tmp_path):
    p = tmp_path / "config.json"
    p.write_text('{\n  "dim": 200,\n  "k": 100,\n\n  "search_start_nodes_num" : 16,\n  "knn_rebuild_thres": 0.1,\n'
                 '  "test_beam_capacity" : 512\n\n}')
    v = C.c_double()
    assert host.coral_host_config_get(str(p).encode(), b"search_start_nodes_num", C.byref(v)) == 0 and v.value == 16
    assert host.coral_host_config_get(str(p).encode(), b"knn_rebuild_thres", C.byref(v)) == 0 and v.value == 0.1
    assert host.coral_host_config_get(str(p).encode(), b"absent", C.byref(v)) == 1
    p.write_text('{"dim": }')
    assert host.coral_host_config_get(str(p).encode(), b"dim", C.byref(v)) == -1


@pytest.mark.parametrize("tool,flag", [("test_search_pipeline", "data_type"), ("test_build_pipeline", "data_type"),
                                       ("test_update", "dataset"), ("comp_gt", "base_data_path")])
def test_drivers_name_a_missing_required_flag(tool, flag):
    """Every driver parses the reference's flags by hand: without its required ones it names the first
    that is missing and returns the reference's -1 before touching a GPU; --help exits 0."""
    import subprocess
    build_host.build()
    exe = os.path.join(os.path.dirname(build_host.HOST_LIB), tool)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert r.returncode == 255 and f"--{flag}' is required" in r.stderr
    r = subprocess.run([exe, "--help"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "flags" in r.stdout
