"""Compile the UNMODIFIED reference extension into ``oracle/_ref/`` (git-ignored).

Test infrastructure.  The reference (rosinality/depthwise-conv-pytorch) is a
PyTorch CUDA extension of two source files, ``torch_dwconv/dwconv.cpp`` and
``torch_dwconv/dwconv_kernel.cu``.  This recipe does not run the reference's
own ``setup.py``: it calls ``nvcc`` (through ``torch.utils.cpp_extension.load``)
on those two files.

One obstacle, handled without touching the sources: ``dwconv_kernel.cu:11``
includes ``"cub/cub.cuh"``, which a quoted include resolves to the CUB 1.8 copy
vendored beside it, and that copy collides with the toolkit's CUB that the ATen
headers pull in.  The two files (and the package's two ``.py`` files) are
therefore staged in a temporary directory WITHOUT the vendored ``cub/`` folder,
so the include resolves to the toolkit's CUB.  Nothing is copied into the
tracked tree; the only outputs are ``oracle/_ref/torch_dwconv/{_C.so,*.py}`` and a copy of
the reference's two test files in ``oracle/_ref/test/`` (git-ignored like the rest of
``oracle/_ref``; ``tests/test_reference_suite_gpu.py`` runs them unchanged).

Usage:  python oracle/build_ref.py [/path/to/reference]
        (default: the directory named by the environment variable DWCONV_REFERENCE_DIR,
        else a sibling checkout ``reference/`` beside this repository)
"""
import glob
import os
import shutil
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "torch_dwconv")


def default_reference_dir():
    """Where the reference checkout is looked for when no path is given."""
    return os.environ.get("DWCONV_REFERENCE_DIR") or os.path.join(
        os.path.dirname(os.path.dirname(HERE)), "reference")


def build_ref(ref_root=None, verbose=False):
    src = os.path.join(ref_root or default_reference_dir(), "torch_dwconv")
    if not os.path.isdir(src):
        return None
    so = os.path.join(OUT, "_C.so")
    # the reference's own test files, to be run unchanged against this library and against the
    # reference build (they import ``torch_dwconv``; which package that is, the runner decides)
    tdir = os.path.join(os.path.dirname(OUT), "test")
    tsrc = os.path.join(os.path.dirname(src), "test")
    if os.path.isdir(tsrc):
        os.makedirs(tdir, exist_ok=True)
        for f in ("test_forward.py", "test_grad.py"):
            if os.path.exists(os.path.join(tsrc, f)):
                shutil.copy(os.path.join(tsrc, f), tdir)
    newest = max(os.path.getmtime(os.path.join(src, f))
                 for f in ("dwconv.cpp", "dwconv_kernel.cu", "dwconv.py"))
    if os.path.exists(so) and os.path.getmtime(so) >= newest:
        return so
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    from torch.utils.cpp_extension import load

    os.makedirs(OUT, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="dwconv_ref_") as tmp:
        for f in ("dwconv.cpp", "dwconv_kernel.cu"):
            shutil.copy(os.path.join(src, f), tmp)
        bdir = os.path.join(tmp, "build")
        os.makedirs(bdir)
        load(name="_C", sources=[os.path.join(tmp, "dwconv.cpp"),
                                 os.path.join(tmp, "dwconv_kernel.cu")],
             build_directory=bdir, is_python_module=False, verbose=verbose,
             extra_cuda_cflags=["-O3", "-w"], extra_cflags=["-O3", "-w"])
        built = glob.glob(os.path.join(bdir, "_C*.so"))
        if not built:
            raise RuntimeError("reference extension did not build")
        shutil.copy(built[0], so)
    for f in ("__init__.py", "dwconv.py"):
        shutil.copy(os.path.join(src, f), OUT)
    return so


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else None
    print(build_ref(root, verbose=True))
