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
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]
OBJ_DIR = os.path.join(PKG_ROOT, "build")


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


def _recorded_deps(dep_file):
    """Project files a translation unit included, from the dependency file nvcc wrote."""
    try:
        with open(dep_file) as f:
            words = f.read().replace("\\\n", " ").split()
    except OSError:
        return None
    roots = (os.path.realpath(CSRC), os.path.realpath(INCLUDE))
    deps = [w for w in words[1:] if os.path.realpath(w).startswith(roots)]
    return deps if all(os.path.exists(d) for d in deps) else None


def _compile_one(nvcc, src, verbose, defines=(), obj_dir=None):
    obj = os.path.join(obj_dir or OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    dep_file = obj[:-2] + ".d"
    deps = _recorded_deps(dep_file) if os.path.exists(obj) else None
    if deps is not None:
        newest = max(os.path.getmtime(f) for f in [src] + deps)
        if os.path.getmtime(obj) >= newest:
            return obj, ""
    cmd = [nvcc] + NVCC_FLAGS + [f"-D{d}" for d in defines] + (["-Xptxas", "-v"] if verbose else []) + [
        "-I", INCLUDE, "-I", CSRC, "-MD", "-MF", dep_file, "-c", "-o", obj, src]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {os.path.basename(src)}:\n{res.stdout}{res.stderr}")
    return obj, res.stdout + res.stderr


def build_library(force=False, verbose=False, defines=(), out=None):
    """Build the library if a source is newer than it; returns its path.

    Each ``.cu`` is compiled to an object in parallel (they are independent translation
    units), then linked into one shared library with the static CUDA runtime.

    ``defines`` / ``out``: a second library with preprocessor symbols set (for instance
    ``DWCONV_B200_TUNING``, which compiles the planner's environment-variable overrides in),
    written to ``out`` with its objects beside it; the shipped library is built without any.
    """
    if out is not None:
        return _build(True, verbose, tuple(defines), os.path.abspath(out))
    if not force and not is_stale():
        return LIB_PATH
    return _build(force, verbose, (), LIB_PATH)


def _build(force, verbose, defines, lib_path):
    from concurrent.futures import ThreadPoolExecutor
    nvcc = os.environ.get("NVCC") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"),
                                                  "bin", "nvcc")
    obj_dir = OBJ_DIR if lib_path == LIB_PATH else lib_path + ".obj"
    os.makedirs(os.path.dirname(lib_path), exist_ok=True)
    os.makedirs(obj_dir, exist_ok=True)
    if force and lib_path == LIB_PATH:
        for f in glob.glob(os.path.join(obj_dir, "*.o")):
            os.remove(f)
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(lambda src: _compile_one(nvcc, src, verbose, defines, obj_dir),
                                _sources()))
    if verbose:
        sys.stderr.write("".join(log for _, log in results))
    tmp = lib_path + ".tmp"
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
           "-o", tmp] + [obj for obj, _ in results]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed linking libdwconv_b200.so")
    os.replace(tmp, lib_path)
    return lib_path


BINDING_NAME = "_dwconv_b200_torch"
BINDING_SRC = os.path.join(CSRC, "torch_binding.cpp")
BINDING_PATH = os.path.join(LIB_DIR, BINDING_NAME + ".so")


def binding_is_stale():
    if not os.path.exists(BINDING_PATH):
        return True
    t = os.path.getmtime(BINDING_PATH)
    return any(os.path.getmtime(f) > t
               for f in [BINDING_SRC] + glob.glob(os.path.join(INCLUDE, "*.h")))


def build_binding(force=False):
    """Compile ``csrc/torch_binding.cpp`` (the tensor-level pybind11 module, host code only)
    into ``lib/_dwconv_b200_torch.so`` with the C++ compiler, against this interpreter's
    torch headers, linked to ``libdwconv_b200.so`` beside it.  Returns its path.

    The module is an accelerator for the Python call path: ``dwconv_b200._C`` runs over
    ctypes without it.
    """
    if not force and not binding_is_stale():
        return BINDING_PATH
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    build_library()
    # the system compiler by name: the module must share the process's libstdc++.so with torch
    # (a toolchain that links its own static copy yields a module that crashes in iostreams)
    cxx = os.environ.get("DWCONV_B200_CXX", "g++")
    flags = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
             f"-DTORCH_EXTENSION_NAME={BINDING_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    get_abi = getattr(ce, "_get_pybind11_abi_build_flags", None)
    if get_abi is not None:
        flags += get_abi()
    includes = [INCLUDE, sysconfig.get_path("include")] + ce.include_paths("cuda")
    lib_dirs = ce.library_paths("cuda")
    tmp = BINDING_PATH + ".tmp"
    cmd = ([cxx] + flags + [f"-I{i}" for i in includes] + ["-o", tmp, BINDING_SRC]
           + [f"-L{d}" for d in lib_dirs + [LIB_DIR]]
           + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
              "-ldwconv_b200", "-Wl,-rpath,$ORIGIN"])
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"{cxx} failed on torch_binding.cpp:\n{res.stdout}{res.stderr}")
    nm = subprocess.run(["nm", "-D", "--defined-only", tmp], capture_output=True, text=True)
    if nm.returncode == 0 and "_ZNSt8ios_base4InitC1Ev" in nm.stdout:
        os.remove(tmp)
        raise RuntimeError(f"{cxx} linked a static copy of libstdc++ into the module; build it with "
                           "a compiler that links libstdc++.so (set DWCONV_B200_CXX)")
    os.replace(tmp, BINDING_PATH)
    return BINDING_PATH


if __name__ == "__main__":
    _defs = [a[2:] for a in sys.argv[1:] if a.startswith("-D")]
    _out = next((a[6:] for a in sys.argv[1:] if a.startswith("--out=")), None)
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                        defines=_defs, out=_out))
    if _out is None and "--no-binding" not in sys.argv:
        print(build_binding(force="--force" in sys.argv))
