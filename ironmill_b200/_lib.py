"""ctypes binding of libironmill_cuda.so (the C ABI declared in include/ironmill_cuda.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libironmill_cuda.so")

IM_OK = 0
IM_DTYPE_F16 = 0
IM_DTYPE_F32 = 1

STATUS_NAMES = {
    0: "IM_OK", -1: "IM_ERR_INVALID", -2: "IM_ERR_CUDA", -3: "IM_ERR_ALLOC", -4: "IM_ERR_BOUNDS",
    -5: "IM_ERR_TIMEOUT", -6: "IM_ERR_NCCL", -7: "IM_ERR_STATE", -8: "IM_ERR_NO_DEVICE",
}


class CudaSysError(RuntimeError):
    """Counterpart of MetalSysError (crates/ironmill-metal-sys/src/error.rs:5-41)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code
        self.message = message


_lib = None

_VOIDP_RESTYPE = ("im_cuda_buffer_ptr",)
_SIZE_RESTYPE = ("im_cuda_device_allocated_bytes", "im_cuda_buffer_length", "im_cuda_affine_weight_bytes",
                 "im_cuda_model_memory_bytes", "im_cuda_model_step_bytes", "im_cuda_tq_scratch_bytes",
                 "im_cuda_sdpa_f16_scratch_bytes", "im_cuda_tq_prefill_scratch_bytes")
_VOID_RESTYPE = ("im_cuda_device_free", "im_cuda_buffer_free", "im_cuda_affine_weight_free", "im_cuda_model_free",
                 "im_cuda_tq_free", "im_cuda_tp_free")


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise CudaSysError(-8, f"{LIB_PATH} not built: run `python -m ironmill_b200.build`")
        _lib = C.CDLL(LIB_PATH)
        _lib.im_cuda_last_error.restype = C.c_char_p
        for name in _VOIDP_RESTYPE:
            if hasattr(_lib, name):
                getattr(_lib, name).restype = C.c_void_p
        for name in _SIZE_RESTYPE:
            if hasattr(_lib, name):
                getattr(_lib, name).restype = C.c_size_t
        for name in _VOID_RESTYPE:
            if hasattr(_lib, name):
                getattr(_lib, name).restype = None
    return _lib


def last_error() -> str:
    return lib().im_cuda_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    if rc != IM_OK:
        raise CudaSysError(rc, last_error())


def vp(x) -> C.c_void_p:
    """Device or host pointer argument from an int address, a torch tensor or a numpy array."""
    if x is None:
        return C.c_void_p(None)
    if isinstance(x, int):
        return C.c_void_p(x)
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    if hasattr(x, "ctypes"):
        return C.c_void_p(x.ctypes.data)
    raise TypeError(type(x))
