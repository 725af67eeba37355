"""The allocation-free backward entry point, sa_backward_static.

Some callers of this library cannot get a device workspace at the moment they need gradients: a
plugin that runs inside the host framework's allocator callback (asking the allocator again would
re-enter it), a worker in a process whose device memory has been handed out completely to a pool it
does not own (a cudaMalloc simply fails), a loop that must not take the allocation lock.  For them
the library carries a fixed 32 MiB scratch array in its own image, and sa_backward_static uses it in
place of a caller workspace.

This file is collected last on purpose: it checks the entry point against the regular sa_backward
(same inputs, same outputs expected) on two consecutive calls -- the second call finds the scratch
as the first one left it -- and it passes both on its own in a fresh process and after every other
GPU test has run in the same process.
"""
import ctypes
import math

import pytest
import torch

import simplical_attn_b200 as sab
from oracle import simplicial_oracle as so
from simplical_attn_b200 import _abi
from simplical_attn_b200 import simplicial_attn as host

pytestmark = pytest.mark.gpu


def _problem(seed, B, N, H, Hkv, D, w1, w2):
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=seed, seed_do=seed + 1)
    dev = [t.cuda().to(torch.bfloat16) for t in (q, k1, k2, v1, v2, do)]
    scale = 1.0 / math.sqrt(D)
    o, lse = sab.two_simplicial_attn_fwd_kernel(*dev[:5], w1, w2, scale)
    ref = sab.two_simplicial_attn_bwd(*dev[:5], o, lse, dev[5], w1, w2, scale)     # caller-workspace entry point
    return dev, o, lse, scale, ref


def _call_static(dev, o, lse, scale, w1, w2, grads=None):
    lib = _abi.load()
    q, k1, k2, v1, v2, do = dev
    if grads is None:
        grads = [torch.empty_like(t) for t in (q, k1, k2, v1, v2)]
    p = host._make_params(q, k1, k2, v1, v2, o, w1, w2, scale, 0.0, 0.0, 0, 0, "auto")
    p.d_o = host._strides(do)
    p.dq, p.dk1, p.dk2, p.dv1, p.dv2 = (host._strides(g) for g in grads)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.sa_backward_static(ctypes.byref(p), ptr(q), ptr(k1), ptr(k2), ptr(v1), ptr(v2), ptr(o), ptr(lse), ptr(do),
                                *[ptr(g) for g in grads], ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, grads


def _free_bytes():
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def test_static_backward_matches_workspace_backward_twice():
    # two different problems back to back: the second call reuses the scratch the first one filled
    for seed, shape in ((21, (1, 384, 4, 2, 128, 160, 32)), (33, (2, 200, 2, 2, 64, 48, 16))):
        B, N, H, Hkv, D, w1, w2 = shape
        dev, o, lse, scale, ref = _problem(seed, B, N, H, Hkv, D, w1, w2)
        _call_static(dev, o, lse, scale, w1, w2)          # first use on this device resolves the scratch address
        grads = [torch.empty_like(t) for t in dev[:5]]
        free_before = _free_bytes()
        rc, grads = _call_static(dev, o, lse, scale, w1, w2, grads)
        assert rc == _abi.SA_OK, _abi.strerror(rc)
        assert _free_bytes() == free_before, "the call changed the amount of free device memory"
        # the scratch's own status word: nothing timed out, and it is read through its own reader
        assert _abi.load().sa_read_status_static(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == _abi.SA_OK
        for name, g, r in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, ref):
            assert so.rel_l2(g.float().cpu(), r.float().cpu()) <= 1e-2, name      # the gradient tolerance of the parity tests
            assert torch.equal(g, r), name                                          # same kernels, same order: same bits


def test_static_backward_rejects_oversized_problem():
    lib = _abi.load()
    cap = lib.sa_backward_static_capacity()
    assert cap == 32 << 20
    B, N, H, D = 4, 8192, 16, 128                      # needs far more than 32 MiB of partial-sum buffers
    x = torch.empty(1, device="cuda", dtype=torch.bfloat16)
    p = _abi.Params()
    p.B, p.N, p.H, p.Hkv, p.D, p.w1, p.w2 = B, N, H, H, D, 512, 32
    p.dtype, p.algo, p.scale = _abi.SA_BF16, _abi.SA_ALGO_AUTO, 0.1
    for nm in ("q", "k1", "k2", "v1", "v2", "o", "d_o", "dq", "dk1", "dk2", "dv1", "dv2"):
        setattr(p, nm, _abi.Strides(N * H * D, H * D, D))
    assert lib.sa_backward_workspace_size(ctypes.byref(p)) > cap
    ptr = ctypes.c_void_p(x.data_ptr())
    rc = lib.sa_backward_static(ctypes.byref(p), *([ptr] * 14), ctypes.c_void_p(0))
    assert rc == 5 and "workspace" in _abi.strerror(rc)
