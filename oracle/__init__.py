"""CPU oracle for the depthwise-conv2d path: test infrastructure, never shipped.

Only the test-suite, ``__graft_entry__.smoke`` and the CPU-baseline legs of
``bench.py`` may import this package.  See ``oracle.py``.
"""
from .oracle import *  # noqa: F401,F403
