"""chromofold_b200 — sealed-KV decode attention for B200 (sm_100a).

The product is the shared library built from csrc/ and declared under include/chromofold_b200/; the Python modules
here are the host-side mirror used by the tests and the benchmark.
"""
from . import _native  # noqa: F401
