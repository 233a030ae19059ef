"""The C-ABI library builds for sm_100a, loads without a GPU and exports every symbol the
header declares; without a device it refuses to compute instead of falling back."""
import ctypes
import os
import re

import pytest

from coral_b200 import build as cb
from coral_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "coral_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(coral_[a-z_0-9]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = cb.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/coral_b200.h but not exported"
    assert sorted(capi.EXPORTS) == names
    assert capi.load().coral_compiled_sm() == 100


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(capi.CoralError) as e:
        capi.Index(100, 8, 32, "l2")
    assert e.value.code == capi.ERR_NOGPU
    assert "no CPU fallback" in str(e.value)


def test_product_code_never_touches_the_oracle():
    for base, _, files in os.walk(os.path.join(ROOT, "coral_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                src = open(os.path.join(base, f), errors="ignore").read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"


def test_planner_is_host_arithmetic_and_matches_the_documented_plans():
    lib = capi.load()
    out = (ctypes.c_int * 8)()
    smem = 232448   # opt-in shared memory per CTA on B200
    assert lib.coral_plan(512, 64, smem, out) == capi.OK
    warps, ctas, chunk, n_chunks, stages, smem_bytes, tile, LP = list(out)
    assert chunk * n_chunks == 512 * 4 and chunk == 256 and stages == 1 and LP == 64
    assert warps * ctas == 20 and ctas * (smem_bytes + 1024) <= smem    # 5 CTAs x 4 warps per SM
    assert lib.coral_plan(200, 64, smem, out) == capi.OK                  # 800-byte rows: 400-byte chunks
    assert out[2] == 400 and out[3] == 2 and out[1] >= 5
    assert lib.coral_plan(200, 512, smem, out) == capi.OK                 # only four CTAs fit: 160-byte chunks
    assert out[2] == 160 and out[3] == 5
    assert lib.coral_plan(6, 64, smem, out) == capi.ERR_ARG               # dim % 4
    assert lib.coral_plan(512, 64, 4096, out) == capi.ERR_LIMIT           # nothing fits 4 KB


def test_granted_shared_memory_is_cached_per_device():
    lib = capi.load()
    slot = lib.coral_internal_grant_slot
    seen = set()
    for dev in (0, 1, 7, 63):
        for metric in (0, 1):
            for cluster in (0, 1):
                s = slot(dev, metric, cluster)
                assert s >= 0 and s not in seen, "two (device, metric, variant) triples share a cache slot"
                seen.add(s)
    assert slot(64, 0, 0) == -1 and slot(-1, 0, 0) == -1   # uncached devices always set the attribute
