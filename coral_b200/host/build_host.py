"""Builds the C++ host mirror: libcoral_host.so (efanna2e::IndexGPU + file-format readers)
and the test_search_pipeline, test_update and test_build_pipeline drivers and the comp_gt tool, all linked against libcoral_b200.so in-tree."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(HERE, "..", "lib")
HOST_LIB = os.path.join(LIB_DIR, "libcoral_host.so")
DRIVER = os.path.join(LIB_DIR, "test_search_pipeline")
UPDATE_DRIVER = os.path.join(LIB_DIR, "test_update")
BUILD_DRIVER = os.path.join(LIB_DIR, "test_build_pipeline")
GT_TOOL = os.path.join(LIB_DIR, "comp_gt")
CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
FLAGS = ["-std=c++17", "-O2", "-fopenmp", "-fPIC", "-Wall"]


def _stale(target: str) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    deps = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cpp", ".h"))]
    deps.append(os.path.join(LIB_DIR, "libcoral_b200.so"))
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force: bool = False) -> str:
    from .. import build as cuda_build
    cuda_build.build()
    if not force and not _stale(HOST_LIB) and not _stale(DRIVER) and not _stale(UPDATE_DRIVER) and not _stale(BUILD_DRIVER) and not _stale(GT_TOOL):
        return HOST_LIB
    link = ["-L" + LIB_DIR, "-lcoral_b200", "-Wl,-rpath,$ORIGIN"]
    src = [os.path.join(HERE, "formats.cpp"), os.path.join(HERE, "index_gpu.cpp")]
    for cmd in ([CXX, *FLAGS, "-shared", "-o", HOST_LIB, *src, *link],
                [CXX, *FLAGS, "-o", DRIVER, os.path.join(HERE, "test_search_pipeline.cpp"), *src, *link],
                [CXX, *FLAGS, "-o", UPDATE_DRIVER, os.path.join(HERE, "test_update.cpp"), *src, *link],
                [CXX, *FLAGS, "-o", BUILD_DRIVER, os.path.join(HERE, "test_build_pipeline.cpp"), *src, *link],
                [CXX, *FLAGS, "-o", GT_TOOL, os.path.join(HERE, "comp_gt.cpp"), *src, *link]):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("host build failed: " + " ".join(cmd[:6]))
    return HOST_LIB


if __name__ == "__main__":
    sys.path.insert(0, os.path.join(HERE, "..", ".."))
    from coral_b200.host import build_host
    print(build_host.build(force=True))
