"""ironmill_b200: B200 (sm_100a) decode backend for ironmill behind a C ABI.

The product is ``libironmill_cuda.so`` (sources in ``csrc/``, declarations in
``include/ironmill_cuda.h``).  The Python modules are a thin ctypes mirror of the
reference's host-side interface for this path, used by the tests and the benchmark.
"""
from ._lib import CudaSysError, lib, check, last_error  # noqa: F401

__all__ = ["CudaSysError", "lib", "check", "last_error"]
