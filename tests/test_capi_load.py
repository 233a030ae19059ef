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
