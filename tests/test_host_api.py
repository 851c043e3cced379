"""Host-side behaviour that needs no GPU: the library loads and exports what the header
declares, argument validation, and the Python API's error behaviour (same texts as the
reference, fixtures from tests/golden/make_golden.py)."""
import ctypes
import glob
import os
import re

import pytest
import torch

from conftest import ROOT, golden


def _declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        src = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names.update(re.findall(r"\b(dwconv_b200_\w+)\s*\(", src))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    from dwconv_b200 import _lib
    declared = _declared_symbols()
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(_lib.lib, name), f"{name} declared in include/ but not exported"
    assert _lib.lib.dwconv_b200_version() >= 100
    assert set(_lib.EXPORTS) <= set(declared)


def test_status_strings():
    from dwconv_b200 import _lib
    seen = {_lib.status_string(i) for i in range(8)}
    assert len(seen) == 8 and "ok" in seen
    assert _lib.status_string(99) == "unknown status"


def test_out_size_and_small_test_match_reference_table():
    from dwconv_b200 import _lib
    for H, W, kh, kw, sh, sw, ph, pw, want in golden().meta["use_small_table"]:
        got = _lib.lib.dwconv_b200_use_dwconv2d_small(H, W, kh, kw, 1, 1, sh, sw, ph, pw)
        assert got == want, (H, W, kh, kw, sh, sw, ph, pw)
    for m in golden().meta["cases"]:
        t = golden().tensors(m["name"])
        for ax, (n_in, k) in enumerate(((m["H"], m["kh"]), (m["W"], m["kw"]))):
            got = _lib.lib.dwconv_b200_out_size(n_in, 1, m["padding"][ax], m["padding"][ax], k,
                                                m["stride"][ax])
            assert got == t["y"].shape[2 + ax]


def test_argument_validation_returns_status_before_any_launch():
    from dwconv_b200 import _lib
    L = _lib.lib
    s = _lib.Shape(1, 1, 8, 8, 3, 3, 1, 1, 1, 1, 8, 8)
    fake = ctypes.c_void_p(0x1000)  # never dereferenced: validation fails first
    assert L.dwconv_b200_forward(None, fake, fake, _lib.F32, s, None) == 1
    assert L.dwconv_b200_forward(fake, fake, fake, 9, s, None) == 2
    assert L.dwconv_b200_forward(ctypes.c_void_p(0x1002), fake, fake, _lib.F32, s, None) == 3
    assert L.dwconv_b200_forward(fake, fake, fake, _lib.F32, None, None) == 1
    bad = _lib.Shape(1, 1, 8, 8, 3, 3, 0, 1, 1, 1, 8, 8)
    assert L.dwconv_b200_backward_input(fake, fake, fake, _lib.F32, bad, None) == 1
    neg = _lib.Shape(1, 1, 8, 8, 3, 3, 1, 1, -1, 1, 8, 8)
    assert L.dwconv_b200_forward(fake, fake, fake, _lib.F32, neg, None) == 1
    huge = _lib.Shape(1, 1, 1 << 16, 1 << 16, 3, 3, 1, 1, 1, 1, 1 << 16, 1 << 16)
    assert L.dwconv_b200_forward(fake, fake, fake, _lib.F32, huge, None) == 7
    # backward-filter: workspace checks
    need = L.dwconv_b200_backward_filter_workspace_bytes(_lib.F32, s)
    assert need >= 16 and need % 16 == 0
    assert L.dwconv_b200_backward_filter(fake, fake, fake, None, need, _lib.F32, s, None) == 1
    assert L.dwconv_b200_backward_filter(fake, fake, fake, ctypes.c_void_p(0x1008), need,
                                         _lib.F32, s, None) == 3
    assert L.dwconv_b200_backward_filter(fake, fake, fake, fake, need - 1, _lib.F32, s, None) == 4
    assert L.dwconv_b200_backward_filter_workspace_bytes(9, s) == 0
    assert L.dwconv_b200_backward_filter_workspace_bytes(_lib.F32, bad) == 0
    # operator form: the two directions it serves, and the ones it refuses
    assert L.dwconv_b200_dwconv2d(fake, fake, fake, _lib.F32, 1, 1, 8, 8, 3, 3, 2, 2, 2, 2,
                                  1, 1, 1, 1, 1, None) == 6
    assert L.dwconv_b200_dwconv2d(fake, fake, fake, _lib.F32, 1, 1, 8, 8, 3, 3, 1, 1, 0, 1,
                                  1, 1, 1, 1, 1, None) == 1
    assert L.dwconv_b200_set_path(7) == -1
    assert L.dwconv_b200_set_path(_lib.PATH_AUTO) == _lib.PATH_AUTO


def test_workspace_covers_every_kernel_family():
    from dwconv_b200 import _lib
    for m in golden().meta["cases"]:
        t = golden().tensors(m["name"])
        s = _lib.Shape(m["N"], m["C"], m["H"], m["W"], m["kh"], m["kw"], *m["stride"],
                       *m["padding"], t["y"].shape[2], t["y"].shape[3])
        for code, acc in ((_lib.F32, 4), (_lib.F16, 4), (_lib.F64, 8)):
            b = _lib.lib.dwconv_b200_backward_filter_workspace_bytes(code, s)
            assert b >= m["C"] * m["kh"] * m["kw"] * acc


def test_python_api_error_texts_match_reference():
    import dwconv_b200 as d
    err = golden().meta["errors"]

    def expect(key, fn):
        kind, text = err[key]
        with pytest.raises({"ValueError": ValueError, "RuntimeError": RuntimeError}[kind]) as ei:
            fn()
        assert str(ei.value) == text

    expect("dilation", lambda: d.check_options(4, 4, 2, None, None))
    expect("groups", lambda: d.check_options(4, 4, 1, 2, None))
    expect("channels", lambda: d.check_options(4, 8, 1, None, None))
    expect("bias", lambda: d.check_options(4, 4, 1, None, True))
    expect("padding_mode", lambda: d.check_options(4, 4, 1, None, None, "reflect"))
    expect("tuple_len", lambda: d.make_tuple((1, 2, 3), 2))
    expect("cpu_tensor", lambda: d.depthwise_conv2d(torch.zeros(1, 2, 40, 40),
                                                    torch.zeros(2, 1, 3, 3)))
    mt = err["make_tuple"]
    assert list(d.make_tuple(3, 2)) == mt["int"]
    assert list(d.make_tuple([3], 2)) == mt["list1"]
    assert list(d.make_tuple((1, 2), 2)) == mt["tuple2"]
    # same validation through the public function and the module constructor
    x, w = torch.zeros(1, 4, 8, 8), torch.zeros(4, 1, 3, 3)
    with pytest.raises(ValueError, match="dilations"):
        d.depthwise_conv2d(x, w, dilation=2)
    with pytest.raises(ValueError, match="groups"):
        d.depthwise_conv2d(x, w, groups=2)
    with pytest.raises(ValueError, match="bias"):
        d.depthwise_conv2d(x, w, torch.ones(1))
    with pytest.raises(ValueError, match="in_channels != out_channels"):
        d.depthwise_conv2d(x, torch.zeros(8, 1, 3, 3))
    with pytest.raises(ValueError, match="non-zero paddings"):
        d.DepthwiseConv2d(4, 4, 3, padding_mode="circular")


def test_cpu_tensors_never_fall_back():
    """The reference lets small maps it cannot serve fall through to F.conv2d, which also
    runs on CPU; this library has no such route."""
    import dwconv_b200 as d
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        d.depthwise_conv2d(torch.zeros(1, 2, 28, 28), torch.zeros(2, 1, 3, 3), stride=2, padding=1)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        d._C.dwconv2d(torch.zeros(1, 2, 40, 40), torch.zeros(2, 1, 3, 3), 1, 1, 1, 1, 1, 1, 1, 1, True)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        d._C.dwconv2d_backward_kernel(torch.zeros(1, 2, 8, 8), torch.zeros(1, 2, 8, 8),
                                      torch.zeros(2, 1, 3, 3), 1, 1, 1, 1, 1, 1)


def test_compiled_binding_loads_and_mirrors_the_ctypes_forms():
    """The pybind11 module is built, loads without a GPU, reports the library's version, has the
    reference module's four names plus forward / backward, and refuses bad arguments with the
    same texts as the ctypes forms it replaces."""
    import dwconv_b200 as d
    from dwconv_b200 import _lib
    nat = _lib.native
    assert nat is not None, "lib/_dwconv_b200_torch.so missing: run build_dwconv_b200.py"
    assert nat.library_version() == _lib.lib.dwconv_b200_version()
    for fn in ("use_dwconv2d_small", "dwconv2d", "dwconv2d_small", "dwconv2d_backward_kernel",
               "forward", "backward"):
        assert callable(getattr(nat, fn))
    assert d._C.dwconv2d is nat.dwconv2d
    x, w = torch.zeros(1, 2, 8, 8), torch.zeros(2, 1, 3, 3)
    bad = [
        ("dwconv2d", (x, w, 1, 1, 1, 1, 1, 1, 1, 1, True)),
        ("dwconv2d", (x.cuda() if torch.cuda.is_available() else x, w, 1, 1, 1, 1, 1, 1, 1, 1, True)),
        ("dwconv2d_small", (x, w, 1, 1, 1, 1, 1, 1, True)),
        ("dwconv2d_backward_kernel", (x, x, w, 1, 1, 1, 1, 1, 1)),
    ]
    for name, args in bad:
        texts = []
        for fn in (d._C.CTYPES_FORMS[name], getattr(nat, name)):
            with pytest.raises(RuntimeError) as ei:
                fn(*args)
            texts.append(str(ei.value).splitlines()[0])
        assert texts[0] == texts[1], name
    for small in ((14, 14, 3, 1, 1), (40, 40, 3, 1, 1), (14, 14, 5, 2, 2), (7, 7, 3, 1, 0)):
        H, W, k, s, p = small
        xs, ws = torch.zeros(1, 1, H, W), torch.zeros(1, 1, k, k)
        assert nat.use_dwconv2d_small(xs, ws, 1, 1, s, s, p, p) == \
            d._C.use_dwconv2d_small(xs, ws, 1, 1, s, s, p, p)


def test_module_surface_and_state_dict():
    import dwconv_b200 as d
    m = d.DepthwiseConv2d(6, 6, 5, stride=2, padding=2)
    assert list(m.state_dict().keys()) == ["weight"]
    assert tuple(m.weight.shape) == (6, 1, 5, 5)
    assert (m.stride, m.padding, m.in_channel, m.kernel_size, m.custom) == (2, 2, 6, 5, True)
    ref = torch.nn.Conv2d(6, 6, 5, stride=2, padding=2, groups=6, bias=False)
    m.load_state_dict(ref.state_dict())  # same key and shape as nn.Conv2d(groups=C, bias=False)
    x = torch.randn(2, 6, 9, 9)
    plain = d.DepthwiseConv2d(6, 6, 5, stride=2, padding=2, custom=False)
    plain.load_state_dict(ref.state_dict())
    assert torch.equal(plain(x), ref(x))  # custom=False is PyTorch's own operator


def test_compat_import_name():
    import torch_dwconv
    import dwconv_b200
    assert torch_dwconv.depthwise_conv2d is dwconv_b200.depthwise_conv2d
    assert torch_dwconv.DepthwiseConv2d is dwconv_b200.DepthwiseConv2d
    for fn in ("use_dwconv2d_small", "dwconv2d", "dwconv2d_small", "dwconv2d_backward_kernel"):
        assert callable(getattr(torch_dwconv._C, fn))


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    import importlib
    import subprocess
    import sys
    code = ("import os,sys; os.environ['DWCONV_B200_LIB']=r'%s'; sys.path.insert(0, r'%s');"
            "import dwconv_b200") % (str(tmp_path / "nope.so"),
                                     os.path.join(ROOT, "depthwise-conv-pytorch_b200"))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert r.returncode != 0 and "no CPU or PyTorch fallback" in r.stderr


def test_chunk_bounds_cover_the_batch_once():
    from dwconv_b200.host import chunk_bounds
    for n, image_bytes, chunk in ((128, 451584, None), (1, 100, None), (2, 1 << 20, None),
                                  (128, 1605632, None), (7, 1 << 30, None), (1000, 1000, None),
                                  (13, 5000, 4), (5, 5000, 99)):
        b = chunk_bounds(n, image_bytes, chunk)
        assert b[0][0] == 0 and b[-1][1] == n
        assert all(b[i][1] == b[i + 1][0] for i in range(len(b) - 1))
        assert all(hi > lo for lo, hi in b)
    assert len(chunk_bounds(128, 451584)) == 8            # eight chunks of 16 images
    assert len(chunk_bounds(1000, 1000)) == 1             # too small to be worth cutting
    assert [hi - lo for lo, hi in chunk_bounds(13, 5000, 4)] == [4, 4, 4, 1]
    assert chunk_bounds(10, 5000, [2, 5, 3]) == [(0, 2), (2, 7), (7, 10)]
    with pytest.raises(ValueError):
        chunk_bounds(10, 5000, [2, 5])


def test_conv2d_interchange_round_trip():
    import dwconv_b200
    conv = torch.nn.Conv2d(6, 6, 5, stride=2, padding=2, groups=6, bias=False)
    m = dwconv_b200.from_conv2d(conv)
    assert isinstance(m, dwconv_b200.DepthwiseConv2d)
    assert torch.equal(m.weight, conv.weight) and m.weight.data_ptr() != conv.weight.data_ptr()
    assert dwconv_b200.make_tuple(m.stride, 2) == (2, 2) and m.kernel_size == 5
    back = dwconv_b200.to_conv2d(m)
    assert back.groups == 6 and back.bias is None and torch.equal(back.weight, conv.weight)
    x = torch.randn(2, 6, 9, 9)
    assert torch.equal(back(x), conv(x))
    # state_dict keys and shapes are interchangeable as they are
    conv.load_state_dict(m.state_dict())
    for bad in (torch.nn.Conv2d(6, 6, 3, groups=6, bias=True), torch.nn.Conv2d(6, 6, 3, groups=3, bias=False),
                torch.nn.Conv2d(6, 6, 3, groups=6, dilation=2, bias=False),
                torch.nn.Conv2d(6, 12, 3, groups=6, bias=False)):
        with pytest.raises(ValueError):
            dwconv_b200.from_conv2d(bad)


def test_depthwise_stack_layout():
    import dwconv_b200
    stack = dwconv_b200.DepthwiseStack()
    assert len(stack.layers) == 7
    assert stack.input_shapes(128)[0] == (128, 32, 112, 112) and stack.input_shapes(2)[-1] == (2, 1152, 7, 7)
    assert [tuple(l.weight.shape) for l in stack.layers][2] == (144, 1, 5, 5)
    assert sorted(stack.state_dict()) == [f"layers.{i}.weight" for i in range(7)]
    with pytest.raises(ValueError):
        stack([torch.zeros(1)])
