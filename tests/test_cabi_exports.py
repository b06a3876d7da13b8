"""The C-ABI library loads on a CPU-only machine and exports every function that
include/ironmill_cuda.h declares (no compute call is made here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ironmill_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(im_cuda_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def cdll():
    from ironmill_b200 import build
    path = build.build()
    return ctypes.CDLL(path)


def test_header_declares_something():
    names = declared_functions()
    assert "im_cuda_matvec_affine" in names and "im_cuda_quantize_affine" in names and len(names) > 20


def test_every_declared_symbol_is_exported(cdll):
    missing = [n for n in declared_functions() if not hasattr(cdll, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_error_plumbing_without_gpu(cdll):
    cdll.im_cuda_last_error.restype = ctypes.c_char_p
    assert cdll.im_cuda_abi_version() >= 1
    # freeing NULL handles is a no-op
    cdll.im_cuda_device_free(None)
    cdll.im_cuda_buffer_free(None)
    cdll.im_cuda_affine_weight_free(None)
    # invalid arguments are reported through the status + thread-local message
    rc = cdll.im_cuda_quantize_affine(None, None, ctypes.c_size_t(4), ctypes.c_size_t(4), 4, 3, None, None, None, None)
    assert rc == -1 and b"bit_width" in cdll.im_cuda_last_error()


def test_product_package_never_touches_the_oracle():
    """The shipped package must not import, load or execute anything under oracle/."""
    pkg = os.path.join(ROOT, "ironmill_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                src = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"
