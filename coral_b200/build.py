"""Builds libcoral_b200.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a only.

A second variant, libcoral_b200_checked.so (-DCORAL_CHECKED), tests every index that addresses
memory inside the search kernel and reports the first bad one instead of faulting; it is what
the environment variable CORAL_B200_CHECKED=1 makes the Python binding load.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libcoral_b200.so")
LIB_CHECKED = os.path.join(LIB_DIR, "libcoral_b200_checked.so")
SOURCES = ["search_kernel.cu", "plan.cu", "dense_topk.cu", "build.cu", "schedule.cu", "capi.cu", "search_static.cu", "start_select.cu", "sharded.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--extended-lambda",
              "-Xcompiler", "-fPIC", "-shared"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(lib: str) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "coral_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> str:
    """Compile the shared library if sources are newer than it; returns its path."""
    lib = LIB_CHECKED if checked else LIB
    if not force and not _stale(lib):
        return lib
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS]
    if checked:
        cmd += ["-DCORAL_CHECKED"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", lib, *[os.path.join(CSRC, s) for s in SOURCES], "-ldl"]
    env = dict(os.environ)
    env.pop("CC", None)   # nvcc should use the system host compiler
    env.pop("CXX", None)
    r = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed building " + os.path.basename(lib))
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build(force="--force" in sys.argv, checked=True))
