"""ctypes binding of libsimplicial_attn_b200.so (declarations: include/simplicial_attn_b200.h).

This is the only place the Python layer touches native code.  There is no fallback: if the
library has not been built, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

SA_OK = 0
SA_ERR_DEVICE_TIMEOUT = 7
SA_BF16, SA_F16, SA_F32 = 0, 1, 2
SA_ALGO_AUTO, SA_ALGO_GENERAL, SA_ALGO_TCGEN05 = 0, 1, 2

EXPORTS = ("sa_forward", "sa_backward", "sa_forward_workspace_size", "sa_backward_workspace_size", "sa_read_status",
           "sa_resolve_algo", "sa_strerror", "sa_version", "sa_kernel_launches", "sa_backward_static",
           "sa_backward_static_capacity", "sa_read_status_static", "sa_read_status_ex", "sa_set_wait_limit_ns",
           "sa_selftest_wait_timeout", "sa_copy_rows_async")


class Strides(ctypes.Structure):
    _fields_ = [("b", ctypes.c_int64), ("n", ctypes.c_int64), ("h", ctypes.c_int64)]


class Params(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_int32) for n in ("B", "N", "H", "Hkv", "D", "w1", "w2", "halo1", "halo2", "dtype", "algo")]
                + [(n, ctypes.c_float) for n in ("scale", "k2_bias", "v2_bias")]
                + [(n, Strides) for n in ("q", "k1", "k2", "v1", "v2", "o", "d_o", "dq", "dk1", "dk2", "dv1", "dv2")])


class SimplicialAttnError(RuntimeError):
    def __init__(self, fn: str, status: int):
        self.status = status
        super().__init__(f"{fn} failed with status {status}: {strerror(status)}")


_lib = None


def lib_path() -> str:
    return _build.LIB


def load():
    """Loads the shared library (building it first when a compiler is present and it is stale)."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    if _build.have_compiler():
        path = _build.build()              # returns at once unless the library was built from other sources
    elif not os.path.exists(path):
        raise OSError(f"{path} is missing and there is no nvcc to build it")
    lib = ctypes.CDLL(path)
    vp, sz = ctypes.c_void_p, ctypes.c_size_t
    pp = ctypes.POINTER(Params)
    lib.sa_forward.argtypes = [pp] + [vp] * 8 + [sz, vp]
    lib.sa_forward.restype = ctypes.c_int
    lib.sa_backward.argtypes = [pp] + [vp] * 14 + [sz, vp]
    lib.sa_backward.restype = ctypes.c_int
    lib.sa_backward_static.argtypes = [pp] + [vp] * 14
    lib.sa_backward_static.restype = ctypes.c_int
    lib.sa_backward_static_capacity.restype = sz
    lib.sa_forward_workspace_size.argtypes = [pp]
    lib.sa_forward_workspace_size.restype = sz
    lib.sa_backward_workspace_size.argtypes = [pp]
    lib.sa_backward_workspace_size.restype = sz
    lib.sa_read_status.argtypes = [vp, vp]
    lib.sa_read_status.restype = ctypes.c_int
    lib.sa_read_status_ex.argtypes = [vp, vp, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    lib.sa_read_status_ex.restype = ctypes.c_int
    lib.sa_status_relay.argtypes = [vp] * 7
    lib.sa_status_relay.restype = ctypes.c_int
    lib.sa_read_status_static.argtypes = [vp]
    lib.sa_read_status_static.restype = ctypes.c_int
    lib.sa_set_wait_limit_ns.argtypes = [ctypes.c_uint64]
    lib.sa_set_wait_limit_ns.restype = None
    lib.sa_selftest_wait_timeout.argtypes = [vp, ctypes.c_uint64, vp]
    lib.sa_selftest_wait_timeout.restype = ctypes.c_int
    lib.sa_copy_rows_async.argtypes = [vp, sz, vp, sz, sz, sz, vp]
    lib.sa_copy_rows_async.restype = ctypes.c_int
    lib.sa_resolve_algo.argtypes = [pp]
    lib.sa_resolve_algo.restype = ctypes.c_int
    lib.sa_strerror.argtypes = [ctypes.c_int]
    lib.sa_strerror.restype = ctypes.c_char_p
    lib.sa_version.restype = ctypes.c_int
    lib.sa_kernel_launches.restype = ctypes.c_uint64
    _lib = lib
    return lib


def strerror(status: int) -> str:
    return load().sa_strerror(int(status)).decode()


def check(fn: str, status: int) -> None:
    if status != SA_OK:
        raise SimplicialAttnError(fn, status)
