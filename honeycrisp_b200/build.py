"""Build libhccuda.so (the C-ABI library) in-tree with nvcc for sm_100a.

`python -m honeycrisp_b200.build [--force] [--verbose]`
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libhccuda.so")
# The same sources with -DHC_DIAGNOSTICS: tile shape, cut of the contraction and thresholds of the
# planner can be forced from the environment.  Only the test-suite loads it.
DIAG_LIB_PATH = os.path.join(PKG_DIR, "libhccuda_diag.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-shared",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libhccuda cannot be built")


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale(path: str = LIB_PATH) -> bool:
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(
        os.path.join(PKG_DIR, "..", "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, diagnostics: bool = False) -> str:
    path = DIAG_LIB_PATH if diagnostics else LIB_PATH
    if not force and not _stale(path):
        return path
    # Several processes may get here at once (one rank per GPU, all finding the library missing):
    # one builds, into a file of its own that replaces the library in one step; the others wait
    # and find it up to date.
    import fcntl
    with open(path + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not _stale(path):
            return path
        tmp = f"{path}.tmp.{os.getpid()}"
        cmd = ([_nvcc()] + NVCC_FLAGS + (["-DHC_DIAGNOSTICS"] if diagnostics else []) +
               (["-Xptxas", "-v"] if verbose else []) + ["-ldl", "-o", tmp] + sources())
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        try:
            subprocess.check_call(cmd)
            os.replace(tmp, path)
        finally:
            if os.path.exists(tmp):
                os.remove(tmp)
    return path


def build_all(force: bool = False, verbose: bool = False):
    return build(force, verbose), build(force, verbose, diagnostics=True)


if __name__ == "__main__":
    print(*build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
