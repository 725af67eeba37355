"""The bounded device-side waits: a wait that runs out must leave SA_ERR_DEVICE_TIMEOUT in the status
word, the kernel must return by itself, and the context must stay usable.

The failure is made without faulting anything: the library's self-test kernel waits, with a limit of
a few milliseconds, on a barrier that nothing ever arrives on (`sa_selftest_wait_timeout`).  It goes
through the same `mbar_wait` as every wait inside the attention kernels.
"""
import ctypes
import math
import time

import pytest
import torch

import simplical_attn_b200 as sab
from oracle import simplicial_oracle as so
from simplical_attn_b200 import _abi
from simplical_attn_b200 import simplicial_attn as host

pytestmark = pytest.mark.gpu


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_wait_runs_out_and_context_survives():
    lib = _abi.load()
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    ptr = ctypes.c_void_p(ws.data_ptr())
    assert lib.sa_read_status(ptr, _stream()) == _abi.SA_OK
    t0 = time.perf_counter()
    assert lib.sa_selftest_wait_timeout(ptr, 3_000_000, _stream()) == _abi.SA_OK          # 3 ms limit
    where, block = ctypes.c_int(-1), ctypes.c_int(-1)
    rc = lib.sa_read_status_ex(ptr, _stream(), ctypes.byref(where), ctypes.byref(block))
    elapsed = time.perf_counter() - t0
    assert rc == _abi.SA_ERR_DEVICE_TIMEOUT and "wait" in _abi.strerror(rc)
    assert where.value == 90 and block.value == 0                                         # the first wait of the probe, block 0
    assert 0.002 <= elapsed < 1.0                                                         # it waited for the limit, then returned
    assert lib.sa_read_status(ptr, _stream()) == _abi.SA_OK                               # reading cleared the word
    # limits outside (0, 0.1 s] are refused: the self-test never occupies the GPU for long
    assert lib.sa_selftest_wait_timeout(ptr, 0, _stream()) == 4
    assert lib.sa_selftest_wait_timeout(ptr, 10**9, _stream()) == 4
    # the context is intact: a normal call right afterwards gives the right answer
    q, k1, k2, v1, v2, do = so.make_inputs(1, 96, 2, 2, 128, seed=5, seed_do=6)
    dev = [t.cuda().to(torch.bfloat16) for t in (q, k1, k2, v1, v2)]
    scale = 1.0 / math.sqrt(128)
    o, lse = sab.two_simplicial_attn_fwd_kernel(*dev, 32, 16, scale, algo="tcgen05")
    ref = so.forward(q, k1, k2, v1, v2, 32, 16, scale)
    assert float((o.float().cpu() - ref[0]).abs().max()) <= 2e-2
    sab.check_device_status()


def test_python_layer_reports_a_timeout_left_by_an_earlier_call():
    """The status watch of the Python layer: a status word that a kernel of an earlier call left
    non-zero is raised by `check_device_status()` (and by the next call once that kernel has finished)."""
    lib = _abi.load()
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    assert lib.sa_selftest_wait_timeout(ctypes.c_void_p(ws.data_ptr()), 2_000_000, _stream()) == _abi.SA_OK
    host._status_watch.watch(ws, "selftest")
    with pytest.raises(_abi.SimplicialAttnError) as e:
        sab.check_device_status()
    assert e.value.status == _abi.SA_ERR_DEVICE_TIMEOUT and "wait site 90" in str(e.value)
    sab.check_device_status()                                                             # reported once


def test_wait_limit_setter_keeps_results():
    """A shorter (still generous) limit for the real kernels changes nothing about their results."""
    lib = _abi.load()
    q, k1, k2, v1, v2, do = so.make_inputs(1, 200, 2, 1, 128, seed=8, seed_do=9)
    dev = [t.cuda().to(torch.bfloat16) for t in (q, k1, k2, v1, v2, do)]
    scale = 1.0 / math.sqrt(128)
    o0, lse0 = sab.two_simplicial_attn_fwd_kernel(*dev[:5], 64, 32, scale, algo="tcgen05")
    g0 = sab.two_simplicial_attn_bwd(*dev[:5], o0, lse0, dev[5], 64, 32, scale, algo="tcgen05")
    lib.sa_set_wait_limit_ns(200_000_000)
    try:
        o1, lse1 = sab.two_simplicial_attn_fwd_kernel(*dev[:5], 64, 32, scale, algo="tcgen05")
        g1 = sab.two_simplicial_attn_bwd(*dev[:5], o1, lse1, dev[5], 64, 32, scale, algo="tcgen05")
    finally:
        lib.sa_set_wait_limit_ns(0)
    sab.check_device_status()
    assert torch.equal(o0, o1) and all(torch.equal(a, b) for a, b in zip(g0, g1))
