"""The allocation-free filter-gradient entry point, dwconv_b200_backward_filter_static.

Some hosts of this library cannot allocate device memory where they need dW: an inference
or training engine that hands out a fixed device budget at start-up, a real-time loop that
must not block on the allocator, a plugin whose host owns every byte of device memory.  For
them the library keeps the reduction scratch in a fixed array of its own device image.  This
test calls that entry point through the C ABI, twice in a row on different problems (the
array is shared and keeps the previous call's contents), and checks each result against the
ordinary entry point, which takes a caller-allocated workspace.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import pytest
import torch

import oracle
from conftest import assert_dw_close
from dwconv_b200 import _lib
from gpu_util import CODE, c_backward_filter, make_shape, seeded

pytestmark = pytest.mark.gpu


def _static(x, dy, k_hw, stride, padding):
    s = make_shape(x.shape, k_hw, stride, padding)
    dw = torch.full((s.C, 1, k_hw[0], k_hw[1]), float("nan"), dtype=x.dtype, device=x.device)
    st = _lib.lib.dwconv_b200_backward_filter_static(
        x.data_ptr(), dy.data_ptr(), dw.data_ptr(), CODE[x.dtype], s,
        torch.cuda.current_stream().cuda_stream)
    return st, dw


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    assert _lib.lib.dwconv_b200_static_scratch_bytes() == 4 << 20
    problems = [
        # a larger problem first, so the second call finds the array full of stale partials
        ((16, 48, 28, 28), (5, 5), 2, 2, torch.float32),
        ((6, 10, 14, 14), (3, 3), 1, 1, torch.float32),
        ((4, 6, 20, 24), (7, 7), 1, 3, torch.float16),
        ((3, 4, 9, 11), (3, 3), 1, 1, torch.float64),
    ]
    for i, (shape, k, s, p, dt) in enumerate(problems):
        x, w, dy = seeded(shape, k, s, p, dt, seed=40 + i)
        st, got = _static(x, dy, k, s, p)
        assert st == 0, _lib.status_string(st)
        st, want = c_backward_filter(x, dy, k, s, p)
        assert st == 0
        torch.cuda.synchronize()
        assert not torch.isnan(got).any()
        # same tolerance as every other filter-gradient check in this suite
        assert_dw_close(got, want, dt, f"static vs workspace [{i}]")
        assert_dw_close(got, oracle.backward_filter(x, dy, k, s, p), dt, f"static vs oracle [{i}]")
    # same problem again, back to back on one stream: results repeat bit for bit
    x, w, dy = seeded(problems[0][0], problems[0][1], 2, 2, torch.float32, seed=40)
    a = _static(x, dy, (5, 5), 2, 2)[1]
    b = _static(x, dy, (5, 5), 2, 2)[1]
    torch.cuda.synchronize()
    assert torch.equal(a, b)


def test_static_scratch_rejects_what_does_not_fit():
    L = _lib.lib
    big = _lib.Shape(2, 4096, 40, 40, 31, 31, 1, 1, 15, 15, 40, 40)  # 4096*961*4 B > 4 MiB
    x = torch.zeros(8, device="cuda")
    st = L.dwconv_b200_backward_filter_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), _lib.F32,
                                              big, None)
    assert st == 7 and "exceeds" in _lib.status_string(st)
    ok = _lib.Shape(1, 1, 4, 4, 3, 3, 1, 1, 1, 1, 4, 4)
    assert L.dwconv_b200_backward_filter_static(None, x.data_ptr(), x.data_ptr(), _lib.F32, ok,
                                                None) == 1
    assert L.dwconv_b200_backward_filter_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), 9, ok,
                                                None) == 2
