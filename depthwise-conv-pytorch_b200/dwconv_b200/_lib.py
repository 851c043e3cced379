"""ctypes binding of ``libdwconv_b200.so`` (declarations: ``include/dwconv_b200.h``).

There is no fallback: if the library is missing, importing this module raises.
"""
import ctypes
import os

LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib",
                        "libdwconv_b200.so")
_BUILD_HINT = "python depthwise-conv-pytorch_b200/build_dwconv_b200.py"

F32, F16, F64, BF16 = 0, 1, 2, 3
PATH_AUTO, PATH_DIRECT, PATH_ROWS, PATH_TILES = 0, 1, 2, 3
OK = 0


ACT_NONE, ACT_RELU, ACT_RELU6, ACT_SILU, ACT_HARDSWISH = 0, 1, 2, 3, 4


class Epilogue(ctypes.Structure):
    """Mirror of ``dwconv_b200_epilogue``."""
    _fields_ = [("scale", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("activation", ctypes.c_int)]


class Shape(ctypes.Structure):
    """Mirror of ``dwconv_b200_shape``."""
    _fields_ = [(n, ctypes.c_int) for n in
                ("N", "C", "H", "W", "kh", "kw", "sh", "sw", "ph", "pw", "Ho", "Wo")]


def _load():
    path = os.environ.get("DWCONV_B200_LIB", LIB_PATH)
    if not os.path.exists(path):
        raise RuntimeError(
            f"dwconv_b200: {path} not found. Build it with `{_BUILD_HINT}` "
            "(needs nvcc); there is no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(path)
    vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    sp = ctypes.POINTER(Shape)
    sig = {
        "dwconv_b200_version": (ci, []),
        "dwconv_b200_status_string": (ctypes.c_char_p, [ci]),
        "dwconv_b200_last_cuda_error": (ci, []),
        "dwconv_b200_set_path": (ci, [ci]),
        "dwconv_b200_last_path": (ci, []),
        "dwconv_b200_device_status": (ci, []),
        "dwconv_b200_debug_plan": (ci, [ci, ci, sp, ci, ctypes.POINTER(ci)]),
        "dwconv_b200_out_size": (ci, [ci] * 6),
        "dwconv_b200_forward": (ci, [vp, vp, vp, ci, sp, vp]),
        "dwconv_b200_forward_epilogue": (ci, [vp, vp, vp, ci, sp, ctypes.POINTER(Epilogue), vp]),
        "dwconv_b200_backward_input": (ci, [vp, vp, vp, ci, sp, vp]),
        "dwconv_b200_forward_nhwc": (ci, [vp, vp, vp, ci, sp, ctypes.POINTER(Epilogue), vp]),
        "dwconv_b200_backward_input_nhwc": (ci, [vp, vp, vp, ci, sp, vp]),
        "dwconv_b200_backward_filter_nhwc": (ci, [vp, vp, vp, vp, sz, ci, sp, vp]),
        "dwconv_b200_backward_nhwc": (ci, [vp, vp, vp, vp, vp, vp, sz, ci, sp, vp]),
        "dwconv_b200_backward_filter_workspace_bytes": (sz, [ci, sp]),
        "dwconv_b200_backward_filter": (ci, [vp, vp, vp, vp, sz, ci, sp, vp]),
        "dwconv_b200_backward": (ci, [vp, vp, vp, vp, vp, vp, sz, ci, sp, vp]),
        "dwconv_b200_backward_accumulate": (ci, [vp, vp, vp, vp, vp, ci, vp, sz, ci, sp, vp]),
        "dwconv_b200_use_dwconv2d_small": (ci, [ci] * 10),
        "dwconv_b200_dwconv2d": (ci, [vp, vp, vp, ci] + [ci] * 15 + [vp]),
        "dwconv_b200_dwconv2d_small": (ci, [vp, vp, vp, ci] + [ci] * 13 + [vp]),
        "dwconv_b200_dwconv2d_backward_kernel": (ci, [vp, vp, vp, vp, sz, ci] + [ci] * 14 + [vp]),
        "dwconv_b200_static_scratch_bytes": (sz, []),
        "dwconv_b200_backward_filter_static": (ci, [vp, vp, vp, ci, sp, vp]),
        "dwconv_b200_copy_async": (ci, [vp, vp, sz, vp]),
        "dwconv_b200_exchange_bytes": (sz, [ci] * 5),
        "dwconv_b200_exchange_create": (ci, [ci] * 6 + [ctypes.POINTER(vp), ctypes.c_char_p]),
        "dwconv_b200_exchange_connect": (ci, [vp, ctypes.c_char_p]),
        "dwconv_b200_exchange_destroy": (ci, [vp]),
        "dwconv_b200_exchange_finish": (ci, [vp, vp, vp]),
        "dwconv_b200_backward_filter_exchange": (ci, [vp, vp, vp, vp, sz, ci, sp, vp, vp]),
        "dwconv_b200_backward_exchange": (ci, [vp, vp, vp, vp, vp, vp, sz, ci, sp, vp, vp]),
        "dwconv_b200_backward_filter_allreduce": (ci, [vp, vp, vp, vp, sz, ci, sp, vp, vp]),
        "dwconv_b200_backward_allreduce": (ci, [vp, vp, vp, vp, vp, vp, sz, ci, sp, vp, vp]),
    }
    for name, (res, args) in sig.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise RuntimeError(f"dwconv_b200: {path} is stale (no symbol {name}); rebuild it with "
                               f"`{_BUILD_HINT}`") from None
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()

NATIVE_PATH = os.path.join(os.path.dirname(LIB_PATH), "_dwconv_b200_torch.so")


def _load_native():
    """The compiled tensor-level module (``csrc/torch_binding.cpp``), or None.

    It is an accelerator for the Python call path, not a second implementation: it calls the
    same ``libdwconv_b200.so`` (linked by a relative run path, so the dynamic loader hands it
    the image ``ctypes`` loaded above).  Not used when ``DWCONV_B200_LIB`` points at another
    library, when ``DWCONV_B200_NO_NATIVE`` is set, or when it was built against another
    library version.
    """
    if (os.environ.get("DWCONV_B200_NO_NATIVE", "0") not in ("", "0")
            or "DWCONV_B200_LIB" in os.environ or not os.path.exists(NATIVE_PATH)):
        return None
    import importlib.machinery
    import importlib.util
    import torch  # noqa: F401  (the module's torch symbols must be loaded first)
    name = "_dwconv_b200_torch"
    try:
        loader = importlib.machinery.ExtensionFileLoader(name, NATIVE_PATH)
        spec = importlib.util.spec_from_file_location(name, NATIVE_PATH, loader=loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
    except ImportError as e:  # built against another torch: say so once, run over ctypes
        import warnings
        warnings.warn(f"dwconv_b200: {NATIVE_PATH} does not load ({e}); using the ctypes path. "
                      f"Rebuild it with `{_BUILD_HINT}`.")
        return None
    if mod.library_version() != lib.dwconv_b200_version():
        return None
    return mod


native = _load_native()

EXPORTS = (
    "dwconv_b200_version", "dwconv_b200_status_string", "dwconv_b200_last_cuda_error",
    "dwconv_b200_set_path", "dwconv_b200_last_path", "dwconv_b200_device_status",
    "dwconv_b200_debug_plan", "dwconv_b200_out_size",
    "dwconv_b200_forward", "dwconv_b200_forward_epilogue", "dwconv_b200_backward_input",
    "dwconv_b200_backward_filter_workspace_bytes", "dwconv_b200_backward_filter",
    "dwconv_b200_forward_nhwc", "dwconv_b200_backward_input_nhwc", "dwconv_b200_backward_filter_nhwc",
    "dwconv_b200_backward_nhwc",
    "dwconv_b200_backward", "dwconv_b200_backward_accumulate", "dwconv_b200_backward_exchange",
    "dwconv_b200_backward_filter_allreduce", "dwconv_b200_backward_allreduce",
    "dwconv_b200_use_dwconv2d_small", "dwconv_b200_dwconv2d", "dwconv_b200_dwconv2d_small",
    "dwconv_b200_dwconv2d_backward_kernel", "dwconv_b200_static_scratch_bytes",
    "dwconv_b200_backward_filter_static",
    "dwconv_b200_copy_async",
    "dwconv_b200_exchange_bytes", "dwconv_b200_exchange_create", "dwconv_b200_exchange_connect",
    "dwconv_b200_exchange_destroy", "dwconv_b200_exchange_finish",
    "dwconv_b200_backward_filter_exchange",
)


def status_string(code):
    return lib.dwconv_b200_status_string(int(code)).decode()


def device_status():
    """Synchronises the current device and returns (and clears) the flags its kernels raised
    when one of their bounded waits ran out: 0 = none, bit 0 forward / backward-input, bit 1
    backward-filter, bit 2 the exchange between GPUs, -1 = the device reported an error."""
    return int(lib.dwconv_b200_device_status())


def check_device_status(what):
    """Raises if a kernel gave up waiting since the last check (its output is then incomplete)."""
    v = device_status()
    if v != 0:
        names = [n for bit, n in ((1, "forward/backward-input"), (2, "backward-filter"),
                                  (4, "exchange between GPUs")) if v > 0 and v & bit]
        raise RuntimeError(f"dwconv_b200.{what}: a kernel's bounded wait expired "
                           f"(device status {v}: {', '.join(names) or 'CUDA error'}); "
                           "the results of the calls since the last check are incomplete")


# DWCONV_B200_CHECK_STATUS=1: the autograd function synchronises and checks the device flags
# after every backward (debugging aid: costs a device synchronisation per call).
CHECK_STATUS = os.environ.get("DWCONV_B200_CHECK_STATUS", "0") not in ("", "0")


def check(code, what):
    """Turn a non-zero status into the RuntimeError a torch extension would raise."""
    if code != OK:
        detail = status_string(code)
        if code == 5:
            detail += f" [cudaError {lib.dwconv_b200_last_cuda_error()}]"
        raise RuntimeError(f"dwconv_b200.{what}: {detail}")
