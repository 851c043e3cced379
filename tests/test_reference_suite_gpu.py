"""The reference's own test files, unchanged, against this library.

``oracle/build_ref.py`` leaves a copy of the reference's ``test/test_forward.py`` and
``test/test_grad.py`` in ``oracle/_ref/test/`` (not tracked; made where a reference checkout is
present).  They ``import torch_dwconv``: run once with the compatibility package of this
library first on the path, and once with the reference's own build, each in a child process.
Every case the reference passes on this GPU must pass here too.  (Its forward cases demand
``max|F.conv2d - custom| < 1e-8`` in fp32 against PyTorch's CUDA convolution; whether that holds
depends on the summation order of the cuDNN kernel PyTorch picks on the machine, for the
reference exactly as for this library, whose results equal the reference's bit for bit.)
"""
import os
import re
import subprocess
import sys

import pytest

from conftest import PKG, ROOT

pytestmark = pytest.mark.gpu

REF = os.path.join(ROOT, "oracle", "_ref")
TESTS = os.path.join(REF, "test")


def _run(first_on_path, files):
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join(first_on_path + [env.get("PYTHONPATH", "")])
    cmd = [sys.executable, "-m", "pytest", "-q", "-rA", "-p", "no:cacheprovider", "--rootdir", TESTS] + files
    res = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=TESTS, timeout=1500)
    outcome = {}
    for line in res.stdout.splitlines():
        m = re.match(r"(PASSED|FAILED|ERROR)\s+(\S+)", line)
        if m:
            outcome[m.group(2).split(" ")[0]] = m.group(1)
    return outcome, res.stdout[-1500:] + res.stderr[-500:]


def test_reference_test_files_unchanged():
    files = [f for f in ("test_forward.py", "test_grad.py") if os.path.exists(os.path.join(TESTS, f))]
    if not files:
        pytest.skip("no copy of the reference's test files (oracle/build_ref.py makes one)")
    mine, log = _run([os.path.join(PKG, "compat"), PKG], files)
    assert len(mine) >= 40, f"the reference's cases did not run:\n{log}"
    # gradients: all 28 gradcheck cases, whatever the reference does
    grad_failed = [k for k, v in mine.items() if "test_grad" in k and v != "PASSED"]
    assert not grad_failed, f"{grad_failed}\n{log}"
    if not os.path.exists(os.path.join(REF, "torch_dwconv", "_C.so")):
        pytest.skip("reference build absent: forward cases not compared")
    theirs, log2 = _run([REF], ["test_forward.py"])
    assert theirs, f"the reference's own run produced nothing:\n{log2}"
    worse = [k for k, v in theirs.items() if v == "PASSED" and mine.get(k) != "PASSED"]
    assert not worse, f"passes with the reference's kernels but not here: {worse}\n{log}"
