"""Compile ``csrc/*.cu`` into ``lib/libdwconv_b200.so`` with plain ``nvcc`` for sm_100a.

    python depthwise-conv-pytorch_b200/build_dwconv_b200.py [--force] [--verbose]

The shared library has no torch dependency; it is loaded with ``ctypes``
(``dwconv_b200._lib``).  nvcc cross-compiles without a GPU.  This module sits outside
the ``dwconv_b200`` package on purpose: importing the package loads the library, and the
build must be able to run when the library is missing or stale.
"""
import glob
import os
import subprocess
import sys

PKG_ROOT = os.path.dirname(os.path.abspath(__file__))
REPO_ROOT = os.path.dirname(PKG_ROOT)
CSRC = os.path.join(PKG_ROOT, "csrc")
LIB_DIR = os.path.join(PKG_ROOT, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libdwconv_b200.so")
INCLUDE = os.path.join(REPO_ROOT, "include")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps():
    return (_sources() + glob.glob(os.path.join(CSRC, "*.cuh"))
            + glob.glob(os.path.join(INCLUDE, "*.h")))


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(f) > t for f in _deps())


def build_library(force=False, verbose=False):
    """Build the library if a source is newer than it; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = os.environ.get("NVCC") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"),
                                                  "bin", "nvcc")
    os.makedirs(LIB_DIR, exist_ok=True)
    tmp = LIB_PATH + ".tmp"
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [
        "-I", INCLUDE, "-I", CSRC, "-o", tmp] + _sources()
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libdwconv_b200.so")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
