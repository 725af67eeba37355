"""Forward + backward for tensors that live in pinned HOST memory.

The operator itself works on device tensors (`simplicial_attn.py`).  When inputs and results live on
the host -- the situation of the reference's CPU-side callers, and of this repository's end-to-end
benchmark -- copying everything over, computing, and copying everything back leaves the GPU idle
during the copies.  `HostPipeline` cuts the work into chunks and runs three CUDA streams: chunk c+1
is uploaded while chunk c is computed and chunk c-1 is downloaded (PCIe is full duplex).

A chunk is one sequence, or one group of heads of one sequence: sequences are independent and so are
KV-head groups, so the results are exactly those of one call per chunk.  The first upload and the
last download cannot be hidden behind compute, which is why the first and the last chunk are small
(a quarter of a sequence's heads) while the chunks in between are whole sequences, large enough to
fill every multiprocessor several times over.  A head group of a `[B, N, H, D]` host tensor is
strided (pieces of `heads * D` elements, `H * D` apart); it moves with one strided copy per tensor
(`sa_copy_rows_async`), no staging.
"""
from __future__ import annotations

import contextlib
import ctypes
import math
import os
from typing import List, Optional, Sequence, Tuple

import torch

from . import _abi
from . import simplicial_attn as _op


def _cpu_list(text: str) -> set:
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def local_cpus(device) -> Optional[set]:
    """CPUs on the NUMA node the GPU's PCIe slot hangs off (from sysfs), or None where the system does
    not say (a container without that part of sysfs, a single-node host)."""
    try:
        pr = torch.cuda.get_device_properties(torch.device(device))
        path = "/sys/bus/pci/devices/%04x:%02x:%02x.0/local_cpulist" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        with open(path) as f:
            cpus = _cpu_list(f.read())
        return cpus or None
    except (OSError, AttributeError, ValueError, RuntimeError, AssertionError):
        return None


@contextlib.contextmanager
def near(device):
    """Host memory allocated inside this block (pinned buffers in particular) comes from the NUMA node of
    the GPU: the calling thread is confined to that node's CPUs for the duration, and pages are placed
    where the thread that first touches them runs.  With one process per GPU on a two-socket host this
    keeps every process's transfers off the socket interconnect.  Does nothing where the node is unknown
    or none of its CPUs is available to the process; yields whether it took effect."""
    cpus = local_cpus(device)
    try:
        before = os.sched_getaffinity(0)
    except (AttributeError, OSError):
        before = None
    use = (cpus & before) if (cpus and before) else None
    if use and use != before:
        os.sched_setaffinity(0, use)
        try:
            yield True
        finally:
            os.sched_setaffinity(0, before)
    else:
        yield False


def plan_chunks(batch: int, kv_heads: int, edge_fraction: float = 0.25) -> List[Tuple[int, int, int]]:
    """Chunks `(sequence, first KV head, end KV head)` in processing order: whole sequences, except
    that the first sequence starts and the last one ends with a small head group."""
    edge = max(1, int(round(kv_heads * edge_fraction)))
    if edge >= kv_heads:
        return [(b, 0, kv_heads) for b in range(batch)]
    chunks: List[Tuple[int, int, int]] = []
    for b in range(batch):
        cuts = [0, kv_heads]
        if b == 0:
            cuts.insert(1, edge)
        if b == batch - 1 and kv_heads - edge > cuts[-2]:
            cuts.insert(len(cuts) - 1, kv_heads - edge)
        chunks += [(b, cuts[i], cuts[i + 1]) for i in range(len(cuts) - 1)]
    return chunks


class HostPipeline:
    """Reusable buffers and streams for repeated host-to-host forward+backward calls of one shape."""

    def __init__(self, device, edge_fraction: float = 0.25):
        self.device = torch.device(device)
        self.edge_fraction = float(edge_fraction)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_comp = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._bufs = None

    def _buffers(self, host_inputs: Sequence[torch.Tensor]):
        key = tuple((tuple(t.shape[1:]), t.dtype) for t in host_inputs)
        if self._bufs is None or self._bufs[0] != key:
            # two slots of one full sequence each; a head-group chunk uses the leading part of a slot
            slots = [[torch.empty(t.shape[1:].numel(), dtype=t.dtype, device=self.device) for t in host_inputs]
                     for _ in range(2)]
            self._bufs = (key, slots)
        return self._bufs[1]

    @staticmethod
    def _copy_heads(lib, dst: torch.Tensor, src: torch.Tensor, stream) -> None:
        """dst, src: [N, heads, D] views of equal shape, each row-strided with contiguous (heads, D)."""
        n, heads, d = src.shape
        es = src.element_size()
        if src.stride(1) != d or dst.stride(1) != d or src.stride(2) != 1 or dst.stride(2) != 1:
            raise ValueError("HostPipeline needs tensors whose (head, dim) block is contiguous")
        rc = lib.sa_copy_rows_async(ctypes.c_void_p(dst.data_ptr()), dst.stride(0) * es, ctypes.c_void_p(src.data_ptr()),
                                    src.stride(0) * es, heads * d * es, n, ctypes.c_void_p(stream.cuda_stream))
        _abi.check("sa_copy_rows_async", rc)

    def forward_backward(self, q, k1, k2, v1, v2, d_o, w1: int, w2: int, scale: Optional[float] = None,
                         k2_bias: float = 0.0, v2_bias: float = 0.0, out: Optional[Sequence[torch.Tensor]] = None):
        """All six arguments are pinned host tensors [B, N, H(kv), D]; returns pinned host tensors
        (o, dq, dk1, dk2, dv1, dv2) (`out` reuses given ones).  Synchronises before returning."""
        host_in = (q, k1, k2, v1, v2, d_o)
        if any(t.is_cuda for t in host_in):
            raise ValueError("HostPipeline takes host tensors; use TwoSimplicialAttention for device tensors")
        if scale is None:
            scale = 1.0 / math.sqrt(q.shape[-1])
        lib = _abi.load()
        B, N, H, D = q.shape
        Hkv = k1.shape[2]
        G = H // Hkv
        if out is None:
            out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (q, q, k1, k2, v1, v2)]
        slots = self._buffers(host_in)
        free = [torch.cuda.Event(), torch.cuda.Event()]          # buffer slot no longer read by the compute stream
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        is_q = (True, False, False, False, False, True)          # which inputs carry query heads
        out_is_q = (True, True, False, False, False, False)      # o, dq | dk1, dk2, dv1, dv2
        for c, (b, hk0, hk1) in enumerate(plan_chunks(B, Hkv, self.edge_fraction)):
            slot = slots[c % 2]
            ready = torch.cuda.Event()
            views = []
            with torch.cuda.stream(self.s_in):
                if c >= 2:
                    self.s_in.wait_event(free[c % 2])
                for buf, src, qh in zip(slot, host_in, is_q):
                    h0, h1 = (hk0 * G, hk1 * G) if qh else (hk0, hk1)
                    dst = buf[:N * (h1 - h0) * D].view(1, N, h1 - h0, D)
                    self._copy_heads(lib, dst[0], src[b, :, h0:h1], self.s_in)
                    views.append(dst)
                ready.record(self.s_in)
            done = torch.cuda.Event()
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(ready)
                dq_, dk1_, dk2_, dv1_, dv2_, ddo = views
                o, lse = _op.two_simplicial_attn_fwd_kernel(dq_, dk1_, dk2_, dv1_, dv2_, w1, w2, scale, k2_bias, v2_bias)
                grads = _op.two_simplicial_attn_bwd(dq_, dk1_, dk2_, dv1_, dv2_, o, lse, ddo, w1, w2, scale, k2_bias, v2_bias)
                free[c % 2] = torch.cuda.Event()
                free[c % 2].record(self.s_comp)
                done.record(self.s_comp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for dst, src, qh in zip(out, (o,) + tuple(grads), out_is_q):
                    h0, h1 = (hk0 * G, hk1 * G) if qh else (hk0, hk1)
                    src.record_stream(self.s_out)
                    self._copy_heads(lib, dst[b, :, h0:h1], src[0], self.s_out)
        for s in (self.s_in, self.s_comp, self.s_out):
            cur.wait_stream(s)
        torch.cuda.synchronize(self.device)
        _op.check_device_status(self.device)
        return tuple(out)
