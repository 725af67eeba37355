"""ctypes binding of the C loop oracle (`oracle/simplicial_oracle.c`).  TEST INFRASTRUCTURE ONLY.

The C file restates `simplicial/reference.py:8-76` of the reference; this module only loads the
shared object that `oracle/Makefile` builds and marshals contiguous fp32 torch/numpy buffers.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libsimplicial_oracle.so")


class _Dims(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int), ("N", ctypes.c_int), ("H", ctypes.c_int), ("Hkv", ctypes.c_int),
                ("D", ctypes.c_int), ("w1", ctypes.c_int), ("w2", ctypes.c_int), ("halo1", ctypes.c_int),
                ("halo2", ctypes.c_int), ("scale", ctypes.c_float), ("k2_bias", ctypes.c_float),
                ("v2_bias", ctypes.c_float)]


def build(force: bool = False) -> str:
    """Compile the oracle with gcc if the shared object is missing or older than its source."""
    src = os.path.join(_HERE, "simplicial_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.sa_oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().sa_oracle_num_threads())


def set_threads(n: int) -> int:
    """Use `n` OpenMP threads from now on (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    lib().sa_oracle_set_threads(ctypes.c_int(int(n)))
    return num_threads()


def _f32(t):
    t = t.detach().to(torch.float32).contiguous()
    return t, ctypes.c_void_p(t.data_ptr())


def _dims(q, k1, k2, w1, w2, scale, k2_bias, v2_bias):
    B, N, H, D = q.shape
    d = _Dims(B, N, H, k1.shape[2], D, min(w1, k1.shape[1]), min(w2, k2.shape[1]),
              k1.shape[1] - N, k2.shape[1] - N, float(scale), float(k2_bias), float(v2_bias))
    return d


def forward(q, k1, k2, v1, v2, w1, w2, scale, k2_bias=0.0, v2_bias=0.0, row_begin=0, row_end=None):
    """Rows [row_begin,row_end) of O [B,N,H,D] and LSE [B,H,N]; other rows are zero."""
    d = _dims(q, k1, k2, w1, w2, scale, k2_bias, v2_bias)
    row_end = d.N if row_end is None else row_end
    keep = [_f32(t) for t in (q, k1, k2, v1, v2)]
    o = torch.zeros(q.shape, dtype=torch.float32)
    lse = torch.zeros(d.B, d.H, d.N, dtype=torch.float32)
    rc = lib().sa_oracle_forward(ctypes.byref(d), *[p for _, p in keep], ctypes.c_void_p(o.data_ptr()),
                                 ctypes.c_void_p(lse.data_ptr()), ctypes.c_int(row_begin), ctypes.c_int(row_end))
    if rc != 0:
        raise ValueError("sa_oracle_forward rejected its arguments")
    return o, lse


def backward(q, k1, k2, v1, v2, do, w1, w2, scale, k2_bias=0.0, v2_bias=0.0, row_begin=0, row_end=None):
    """Gradient share of query rows [row_begin,row_end): (dq, dk1, dk2, dv1, dv2), fp32."""
    d = _dims(q, k1, k2, w1, w2, scale, k2_bias, v2_bias)
    row_end = d.N if row_end is None else row_end
    keep = [_f32(t) for t in (q, k1, k2, v1, v2, do)]
    outs = [torch.zeros(t.shape, dtype=torch.float32) for t in (q, k1, k2, v1, v2)]
    rc = lib().sa_oracle_backward(ctypes.byref(d), *[p for _, p in keep],
                                  *[ctypes.c_void_p(t.data_ptr()) for t in outs],
                                  ctypes.c_int(row_begin), ctypes.c_int(row_end))
    if rc != 0:
        raise ValueError("sa_oracle_backward rejected its arguments")
    return tuple(outs)
