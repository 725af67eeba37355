"""Host-side mirror of the reference's operator interface for 2-simplicial attention.

Same names, argument meaning and return values as the reference's
`simplicial/triton_impl.py` (`TwoSimplicialAttentionFunction`, :15-158; `TwoSimplicialAttention`,
:161-186); the Triton launches are replaced by calls through the C ABI of
libsimplicial_attn_b200.so.  torch supplies device memory and the current stream, nothing else.

Additions that keep the reference call signature valid:
  * K/V may have fewer heads than Q (`H % Hkv == 0`); query head h reads KV head h // (H // Hkv).
  * `two_simplicial_attention(..., halo1=, halo2=)` accepts K/V with leading halo rows (used by the
    sequence-sharded path in `simplical_attn_b200.sharded`).
Windows follow the reference's kernels: j in (i-w1, i], k in (i-w2, i]
(`simplicial/kernels.py:133-136`).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import _abi

_DTYPES = {torch.bfloat16: _abi.SA_BF16, torch.float16: _abi.SA_F16, torch.float32: _abi.SA_F32}
_ALGOS = {"auto": _abi.SA_ALGO_AUTO, "general": _abi.SA_ALGO_GENERAL, "tcgen05": _abi.SA_ALGO_TCGEN05}

# Kernel family used by the autograd function; tests switch it to cross-check the two families.
default_algo = "auto"


def _strides(t: Optional[torch.Tensor]) -> _abi.Strides:
    if t is None:
        return _abi.Strides(0, 0, 0)
    return _abi.Strides(t.stride(0), t.stride(1), t.stride(2))


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _check_inputs(q, k1, k2, v1, v2, halo1, halo2):
    if not q.is_cuda:
        raise RuntimeError("simplical_attn_b200 runs on CUDA tensors only; there is no CPU path")
    if q.dim() != 4:
        raise ValueError("q must be [batch, seq_len, num_heads, head_dim]")
    B, N, H, D = q.shape
    if q.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {q.dtype}")
    for name, t, halo in (("k1", k1, halo1), ("v1", v1, halo1), ("k2", k2, halo2), ("v2", v2, halo2)):
        if t.dtype != q.dtype or t.device != q.device:
            raise TypeError(f"{name} must match q's dtype and device")
        if t.dim() != 4 or t.shape[0] != B or t.shape[1] != N + halo or t.shape[3] != D:
            raise ValueError(f"{name} must be [batch, seq_len + halo, kv_heads, head_dim], got {tuple(t.shape)}")
        if t.shape[2] != k1.shape[2] or H % t.shape[2] != 0:
            raise ValueError("K/V tensors must share a head count that divides the query head count")
    return B, N, H, k1.shape[2], D


def _unit_inner(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def _make_params(q, k1, k2, v1, v2, o, w1, w2, scale, k2_bias, v2_bias, halo1, halo2, algo):
    B, N, H, D = q.shape
    p = _abi.Params()
    p.B, p.N, p.H, p.Hkv, p.D = B, N, H, k1.shape[2], D
    p.w1, p.w2, p.halo1, p.halo2 = int(w1), int(w2), int(halo1), int(halo2)
    p.dtype = _DTYPES[q.dtype]
    p.algo = _ALGOS[algo]
    p.scale, p.k2_bias, p.v2_bias = float(scale), float(k2_bias), float(v2_bias)
    p.q, p.k1, p.k2, p.v1, p.v2, p.o = (_strides(t) for t in (q, k1, k2, v1, v2, o))
    return p


def _workspace(nbytes: int, device) -> torch.Tensor:
    ws = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
    ws[:256].zero_()          # the device status word must start at zero
    return ws


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class _StatusWatch:
    """Surfaces device-side timeouts without a synchronisation per call.

    After every launch the status word of the call's workspace is copied, stream-ordered, into a
    pinned host slot and an event is recorded.  The next call on the same device looks at the slots
    whose event has already completed (a non-blocking query) and raises if one of them holds an
    error.  `flush()` synchronises and checks everything that is still pending."""

    SLOTS = 32                      # pinned status slots per device, reused

    def __init__(self):
        self._dev = {}              # device index -> (view of the pinned [SLOTS, 4] int32 slots, free slots, pending, stream, ...)

    def _state(self, index: int):
        st = self._dev.get(index)
        if st is None:
            dev = torch.device("cuda", index)
            side = torch.cuda.Stream(dev)
            host = torch.zeros(self.SLOTS, 4, dtype=torch.int32).pin_memory()
            small = torch.empty(self.SLOTS, 4, dtype=torch.int32, device=dev)
            events = []
            for _ in range(self.SLOTS):                # created once, reused: (workspace copy done, host copy done)
                pair = (torch.cuda.Event(), torch.cuda.Event())
                for ev in pair:
                    ev.record(side)                    # a torch event gets its CUDA handle at its first record
                events.append(pair)
            st = (host.numpy(), list(range(self.SLOTS)), [], side, small, events, host.data_ptr(), small.data_ptr(),
                  side.cuda_stream, host)
            self._dev[index] = st
        return st

    def watch(self, ws: torch.Tensor, label: str, stream_handle=None) -> None:
        _, free, pending, side, small, events, host_ptr, small_ptr, side_handle, _ = self._state(ws.device.index)
        if not free:
            self.poll(ws.device, wait_oldest=True)
        i = free.pop()
        # The status word first goes to a small device slot, on the caller's stream (16 bytes, device to device),
        # so that the workspace itself is not held any longer than the kernels need it.  The device-to-host copy
        # then runs on a stream of its own: on the caller's stream it would queue behind whatever large transfers
        # keep the copy engines busy and hold the caller's next kernels back.  One library call does all of it
        # (a handful of Python-level stream and event operations would cost more than a small problem's kernels).
        if stream_handle is None:
            stream_handle = torch.cuda.current_stream(ws.device).cuda_stream
        ready, done = events[i]
        rc = _abi.load().sa_status_relay(ws.data_ptr(), small_ptr + 16 * i, host_ptr + 16 * i, stream_handle, side_handle,
                                         ready.cuda_event, done.cuda_event)
        _abi.check("sa_status_relay", rc)
        pending.append((done, i, label))

    def poll(self, device: torch.device, wait: bool = False, wait_oldest: bool = False) -> None:
        if device.index not in self._dev:
            return
        host, free, pending = self._state(device.index)[:3]
        bad = None
        keep = []
        for n, (ev, i, label) in enumerate(pending):
            if wait or (wait_oldest and n == 0):
                ev.synchronize()
            if ev.query():
                if host[i, 0] != 0 and bad is None:          # (a numpy view of the pinned slots: cheap to read)
                    bad = (label, int(host[i, 0]), int(host[i, 1]), int(host[i, 2]))
                free.append(i)
            else:
                keep.append((ev, i, label))
        pending[:] = keep
        if bad is not None:
            raise _abi.SimplicialAttnError(f"{bad[0]} (device side: wait site {bad[2]}, block {bad[3]})", bad[1])

    def flush(self, device=None) -> None:
        if device is None:
            indices = list(self._dev)
        else:
            d = torch.device(device)
            indices = [d.index if d.index is not None else torch.cuda.current_device()]
        for index in indices:
            self.poll(torch.device("cuda", index), wait=True)


_status_watch = _StatusWatch()


def check_device_status(device=None) -> None:
    """Synchronises and raises `SimplicialAttnError` if a kernel of an earlier call on `device`
    (default: every device used so far) gave up on a bounded wait.  Earlier calls are also checked,
    without synchronising, at the start of every later call."""
    _status_watch.flush(device)


def two_simplicial_attn_fwd_kernel(q, k1, k2, v1, v2, w1, w2, scale, k2_bias=0.0, v2_bias=0.0, halo1=0, halo2=0,
                                   algo=None):
    """Forward launch (the reference's kernel of the same name, `simplicial/kernels.py:11-171`).
    Returns (O, LSE) with LSE = log sum exp of the logits, fp32 [B, H, N] (the reference's `M`)."""
    lib = _abi.load()
    q, k1, k2, v1, v2 = (_unit_inner(t) for t in (q, k1, k2, v1, v2))
    B, N, H, Hkv, D = _check_inputs(q, k1, k2, v1, v2, halo1, halo2)
    _status_watch.poll(q.device)
    o = torch.empty_like(q)                                   # triton_impl.py:23
    lse = torch.empty((B, H, N), device=q.device, dtype=torch.float32)
    p = _make_params(q, k1, k2, v1, v2, o, w1, w2, scale, k2_bias, v2_bias, halo1, halo2, algo or default_algo)
    ws = _workspace(lib.sa_forward_workspace_size(ctypes.byref(p)), q.device)
    sh = torch.cuda.current_stream().cuda_stream
    rc = lib.sa_forward(ctypes.byref(p), _ptr(q), _ptr(k1), _ptr(k2), _ptr(v1), _ptr(v2), _ptr(o), _ptr(lse), _ptr(ws),
                        ws.numel(), ctypes.c_void_p(sh))
    _abi.check("sa_forward", rc)
    if debug_device_status:
        _abi.check("sa_forward (device)", lib.sa_read_status(_ptr(ws), ctypes.c_void_p(sh)))
    else:
        _status_watch.watch(ws, "sa_forward", sh)
    return o, lse


def two_simplicial_attn_bwd(q, k1, k2, v1, v2, o, lse, d_o, w1, w2, scale, k2_bias=0.0, v2_bias=0.0, halo1=0, halo2=0,
                            need=(True, True, True, True, True), algo=None):
    """Backward launches (the reference's compute_D_kernel + two_simplicial_attn_bwd_kv1_kernel +
    two_simplicial_attn_bwd_kv2_kernel, `simplicial/kernels.py:175-571`).  Returns
    (dq, dk1, dk2, dv1, dv2), `None` where `need[i]` is false."""
    lib = _abi.load()
    q, k1, k2, v1, v2, o, d_o = (_unit_inner(t) for t in (q, k1, k2, v1, v2, o, d_o))
    _check_inputs(q, k1, k2, v1, v2, halo1, halo2)
    _status_watch.poll(q.device)
    grads = [torch.empty_like(t) if n else None for t, n in zip((q, k1, k2, v1, v2), need)]
    p = _make_params(q, k1, k2, v1, v2, o, w1, w2, scale, k2_bias, v2_bias, halo1, halo2, algo or default_algo)
    p.d_o = _strides(d_o)
    p.dq, p.dk1, p.dk2, p.dv1, p.dv2 = (_strides(g) for g in grads)
    ws = _workspace(lib.sa_backward_workspace_size(ctypes.byref(p)), q.device)
    sh = torch.cuda.current_stream().cuda_stream
    rc = lib.sa_backward(ctypes.byref(p), _ptr(q), _ptr(k1), _ptr(k2), _ptr(v1), _ptr(v2), _ptr(o), _ptr(lse), _ptr(d_o),
                         *[_ptr(g) for g in grads], _ptr(ws), ws.numel(), ctypes.c_void_p(sh))
    _abi.check("sa_backward", rc)
    if debug_device_status:
        _abi.check("sa_backward (device)", lib.sa_read_status(_ptr(ws), ctypes.c_void_p(sh)))
    else:
        _status_watch.watch(ws, "sa_backward", sh)
    return tuple(grads)


# When true every call synchronises and raises at once if a device-side bounded wait gave up; otherwise
# such a timeout is raised by the next call after the kernels have finished, or by check_device_status().
debug_device_status = False


def two_simplicial_attn_bwd_kv1_kernel(q, k1, k2, v1, v2, o, lse, d_o, w1, w2, scale, k2_bias=0.0, v2_bias=0.0, **kw):
    """dQ, dK1, dV1 (the outputs of the reference kernel of this name, `simplicial/kernels.py:175-382`)."""
    g = two_simplicial_attn_bwd(q, k1, k2, v1, v2, o, lse, d_o, w1, w2, scale, k2_bias, v2_bias,
                                need=(True, True, False, True, False), **kw)
    return g[0], g[1], g[3]


def two_simplicial_attn_bwd_kv2_kernel(q, k1, k2, v1, v2, o, lse, d_o, w1, w2, scale, k2_bias=0.0, v2_bias=0.0, **kw):
    """dK2, dV2 (the outputs of the reference kernel of this name, `simplicial/kernels.py:386-566`)."""
    g = two_simplicial_attn_bwd(q, k1, k2, v1, v2, o, lse, d_o, w1, w2, scale, k2_bias, v2_bias,
                                need=(False, False, True, False, True), **kw)
    return g[2], g[4]


def compute_D_kernel(grad_output, output):
    """Delta_i = sum_d dO*O, fp32 [B, H, N].  The reference's helper (`simplicial/kernels.py:569-571`)
    returns it in the input dtype laid out [B, N, H]; the backward kernels here compute Delta
    themselves, so this is kept for callers that want the value."""
    return (grad_output.float() * output.float()).sum(-1).permute(0, 2, 1).contiguous()


class TwoSimplicialAttentionFunction(torch.autograd.Function):
    """Autograd function with the reference's signature (`simplicial/triton_impl.py:15-158`)."""

    @staticmethod
    def forward(ctx, q, k1, k2, v1, v2, w1, w2, scale, k2_bias, v2_bias, halo1=0, halo2=0):
        o, lse = two_simplicial_attn_fwd_kernel(q, k1, k2, v1, v2, w1, w2, scale, k2_bias, v2_bias, halo1, halo2)
        ctx.save_for_backward(q, k1, k2, v1, v2, o, lse)          # triton_impl.py:54
        ctx.cfg = (w1, w2, scale, k2_bias, v2_bias, halo1, halo2)
        return o

    @staticmethod
    def backward(ctx, grad_output):
        q, k1, k2, v1, v2, o, lse = ctx.saved_tensors
        w1, w2, scale, k2_bias, v2_bias, halo1, halo2 = ctx.cfg
        need = tuple(bool(n) for n in ctx.needs_input_grad[:5])   # triton_impl.py:73-77
        grads = two_simplicial_attn_bwd(q, k1, k2, v1, v2, o, lse, grad_output, w1, w2, scale, k2_bias, v2_bias,
                                        halo1, halo2, need)
        return grads + (None,) * 7


def two_simplicial_attention(q, k1, k2, v1, v2, w1, w2, scale=None, k2_bias=0.0, v2_bias=0.0, halo1=0, halo2=0):
    """Functional form; `scale` defaults to 1/sqrt(head_dim) (`simplicial/triton_impl.py:169`)."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return TwoSimplicialAttentionFunction.apply(q, k1, k2, v1, v2, w1, w2, scale, k2_bias, v2_bias, halo1, halo2)


class TwoSimplicialAttention(torch.nn.Module):
    """Module with the reference's constructor and call (`simplicial/triton_impl.py:161-186`); it
    has no parameters or buffers, so its state_dict is empty like the reference's."""

    def __init__(self, head_dim, w1=64, w2=64, scale=None, k2_bias=0.0, v2_bias=0.0):
        super().__init__()
        self.head_dim = head_dim
        self.w1 = w1
        self.w2 = w2
        self.scale = scale if scale is not None else (1.0 / math.sqrt(head_dim))
        self.k2_bias = k2_bias
        self.v2_bias = v2_bias

    def forward(self, q, k1, k2, v1, v2):
        return TwoSimplicialAttentionFunction.apply(q, k1, k2, v1, v2, self.w1, self.w2, self.scale, self.k2_bias,
                                                    self.v2_bias)
