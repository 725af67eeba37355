"""Forward + backward for tensors that live in pinned HOST memory.

The operator itself works on device tensors (`simplicial_attn.py`).  When inputs and results live on
the host -- the situation of the reference's CPU-side callers, and of this repository's end-to-end
benchmark -- copying everything over, computing, and copying everything back leaves the GPU idle
during the copies.  `HostPipeline` splits the batch into chunks and runs three CUDA streams: chunk
c+1 is uploaded while chunk c is computed and chunk c-1 is downloaded (PCIe is full duplex).  The
sequences of a batch are independent, so the results are exactly those of one big call.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from . import simplicial_attn as _op


class HostPipeline:
    """Reusable buffers and streams for repeated host-to-host forward+backward calls of one shape."""

    def __init__(self, device, chunk: int = 1):
        # chunk = sequences per pipeline stage.  The first upload and the last download are not hidden
        # by compute, so small chunks win as long as one chunk fills the GPU: at B16 H16 N8192 D128
        # one sequence per chunk measured 129.5 ms per call, two 135.8 ms, four 148.7 ms.
        self.device = torch.device(device)
        self.chunk = int(chunk)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_comp = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._bufs = None

    def _buffers(self, host_inputs: Sequence[torch.Tensor]):
        key = tuple((tuple(t.shape[1:]), t.dtype) for t in host_inputs)
        if self._bufs is None or self._bufs[0] != key:
            slots = [[torch.empty((self.chunk,) + tuple(t.shape[1:]), dtype=t.dtype, device=self.device)
                      for t in host_inputs] for _ in range(2)]
            self._bufs = (key, slots)
        return self._bufs[1]

    def forward_backward(self, q, k1, k2, v1, v2, d_o, w1: int, w2: int, scale: Optional[float] = None,
                         k2_bias: float = 0.0, v2_bias: float = 0.0, out: Optional[Sequence[torch.Tensor]] = None):
        """All six arguments are pinned host tensors [B, N, H(kv), D]; returns pinned host tensors
        (o, dq, dk1, dk2, dv1, dv2) (`out` reuses given ones).  Synchronises before returning."""
        host_in = (q, k1, k2, v1, v2, d_o)
        if any(t.is_cuda for t in host_in):
            raise ValueError("HostPipeline takes host tensors; use TwoSimplicialAttention for device tensors")
        if scale is None:
            scale = 1.0 / math.sqrt(q.shape[-1])
        B = q.shape[0]
        if out is None:
            out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (q, q, k1, k2, v1, v2)]
        slots = self._buffers(host_in)
        free = [torch.cuda.Event(), torch.cuda.Event()]          # buffer slot no longer read by the compute stream
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        nchunks = (B + self.chunk - 1) // self.chunk
        for c in range(nchunks):
            b0, b1 = c * self.chunk, min(B, (c + 1) * self.chunk)
            n = b1 - b0
            slot = slots[c % 2]
            ready = torch.cuda.Event()
            with torch.cuda.stream(self.s_in):
                if c >= 2:
                    self.s_in.wait_event(free[c % 2])
                for dst, src in zip(slot, host_in):
                    dst[:n].copy_(src[b0:b1], non_blocking=True)
                ready.record(self.s_in)
            done = torch.cuda.Event()
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(ready)
                dq_, dk1_, dk2_, dv1_, dv2_, ddo = (t[:n] for t in slot)
                o, lse = _op.two_simplicial_attn_fwd_kernel(dq_, dk1_, dk2_, dv1_, dv2_, w1, w2, scale, k2_bias, v2_bias)
                grads = _op.two_simplicial_attn_bwd(dq_, dk1_, dk2_, dv1_, dv2_, o, lse, ddo, w1, w2, scale, k2_bias, v2_bias)
                free[c % 2] = torch.cuda.Event()
                free[c % 2].record(self.s_comp)
                done.record(self.s_comp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for dst, src in zip(out, (o,) + tuple(grads)):
                    src.record_stream(self.s_out)
                    dst[b0:b1].copy_(src, non_blocking=True)
        for s in (self.s_in, self.s_comp, self.s_out):
            cur.wait_stream(s)
        torch.cuda.synchronize(self.device)
        return tuple(out)
