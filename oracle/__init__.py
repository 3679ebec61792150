"""CPU oracle for the FastNN matmul path.  TEST INFRASTRUCTURE ONLY.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``
may import this package; the product path (``fastnn_b200``) never does.
"""
from .oracle import *  # noqa: F401,F403
