"""Sequence-sharded 2-simplicial attention: each rank owns a contiguous block of N/P query rows.

The reference has no multi-GPU path; this is the long-sequence configuration of the target
(N split over the GPUs of one box).  Because the windows are causal and local, rank r needs from
rank r-1 only the last w1-1 rows of K1/V1 and the last w2-1 rows of K2/V2 (its "halo"); in the
backward it returns the gradient of those halo rows to rank r-1, which adds them to its own.

All four tensors travel in ONE batched point-to-point exchange per direction (NCCL over NVLink on
GPUs, gloo in the CPU tests).  The halo is received straight into the head of a `[halo | shard]`
buffer that the kernels then read with a row offset (`halo1`, `halo2`); on GPUs the exchange runs on
a side stream while the main stream copies the local rows into the tail of that buffer.  The kernels
only ever read local memory.  A caller that lets its K/V projections write directly into the tail of
such a buffer (`kv_buffer(...)` / `local_rows(...)`) skips that copy as well.

Requires every shard to hold at least max(w1, w2) - 1 rows, so that a halo comes from the immediate
predecessor only.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n_total: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows [start, end) of the sequence owned by `rank`: equal blocks, the remainder spread over
    the first ranks."""
    base, rem = divmod(n_total, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def halo_rows(window: int, shard_start: int) -> int:
    """Rows a shard starting at global row `shard_start` needs from its predecessor."""
    return max(0, min(window - 1, shard_start))


def check_partition(n_total: int, world: int, w1: int, w2: int) -> None:
    """Every shard but the last must hold the rows its successor needs as halo."""
    for r in range(world - 1):
        s, e = shard_bounds(n_total, world, r)
        need = halo_rows(max(w1, w2), e)
        if e - s < need:
            raise ValueError(f"shard {r} has {e - s} rows but its successor needs a halo of {need} rows; "
                             f"use fewer ranks or smaller windows")


def kv_buffer(batch: int, n_local: int, heads: int, head_dim: int, halo: int, dtype, device) -> torch.Tensor:
    """A `[batch, halo + n_local, heads, head_dim]` buffer.  Write this rank's K (or V) rows into
    `local_rows(buf, halo)` and pass that view to `two_simplicial_attention_sharded`: the halo is then
    received into the head of the same buffer and nothing is copied."""
    return torch.empty((batch, halo + n_local, heads, head_dim), dtype=dtype, device=device)


def local_rows(buf: torch.Tensor, halo: int) -> torch.Tensor:
    return buf[:, halo:]


def _global_rank(group, group_rank: int) -> int:
    return dist.get_global_rank(group, group_rank) if group is not None else group_rank


_side_streams = {}


def _side_stream(device: torch.device):
    s = _side_streams.get(device.index)
    if s is None:
        s = torch.cuda.Stream(device)
        _side_streams[device.index] = s
    return s


def _extended(x: torch.Tensor, halo: int) -> Tuple[torch.Tensor, bool]:
    """The `[halo | shard]` buffer of a local tensor.  If `x` already is the tail of such a buffer
    (see `kv_buffer`) that buffer is used as it is; otherwise a new one is made and the second value
    says that the local rows still have to be copied into it."""
    base = x._base
    if (halo > 0 and base is not None and base.dim() == 4 and base.is_contiguous() and base.shape[1] == halo + x.shape[1]
            and base.shape[0] == x.shape[0] and base.shape[2:] == x.shape[2:] and x.stride() == base.stride()
            and x.data_ptr() == base[:, halo:].data_ptr()):
        return base.detach(), False
    if halo == 0:
        return x.detach(), False                       # nothing to put in front: the local tensor is the buffer
    ext = x.new_empty((x.shape[0], halo + x.shape[1]) + tuple(x.shape[2:]))
    return ext, True


def _exchange(recv: Sequence[Optional[torch.Tensor]], send: Sequence[Optional[torch.Tensor]], recv_from: int, send_to: int,
              group, tag: int) -> None:
    """One batched exchange: every tensor of `recv` (from `recv_from`) and of `send` (to `send_to`);
    entries that are None are skipped.  Blocks the current stream (or thread) until it is complete."""
    ops = []
    for i, t in enumerate(recv):
        if t is not None:
            ops.append(dist.P2POp(dist.irecv, t, _global_rank(group, recv_from), group=group, tag=tag + i))
    for i, t in enumerate(send):
        if t is not None:
            ops.append(dist.P2POp(dist.isend, t, _global_rank(group, send_to), group=group, tag=tag + i))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()


class _HaloExchange(torch.autograd.Function):
    """forward: four local tensors `[B, n, H, D]` -> four `[B, halo + n, H, D]` buffers whose first
    `halo` rows come from rank-1 (and whose last `send` rows went to rank+1), all in one batched
    exchange.  backward: the gradients of the four halos go back to rank-1 in one batched exchange and
    the gradients received from rank+1 are added to the last `send` rows."""

    @staticmethod
    def forward(ctx, k1, k2, v1, v2, h1: int, h2: int, s1: int, s2: int, group):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        xs, halos, sends = (k1, k2, v1, v2), (h1, h2, h1, h2), (s1, s2, s1, s2)
        ctx.cfg = (h1, h2, s1, s2, group)
        has_pred, has_succ = rank > 0, rank < world - 1
        exts, need_copy = zip(*[_extended(x, h if has_pred else 0) for x, h in zip(xs, halos)])
        cuda = k1.is_cuda
        cur = torch.cuda.current_stream(k1.device) if cuda else None
        side = _side_stream(k1.device) if cuda else None

        def do_exchange():
            recv, stage, send = [], [], []
            for x, ext, h, s in zip(xs, exts, halos, sends):
                r = None
                if has_pred and h > 0:
                    head = ext[:, :h]
                    r = head if head.is_contiguous() else x.new_empty(head.shape)      # B > 1: through a small staging buffer
                recv.append(r)
                stage.append(r)
                send.append(x[:, x.shape[1] - s:].contiguous() if (has_succ and s > 0) else None)
            _exchange(recv, send, rank - 1, rank + 1, group, 100)
            for ext, h, r in zip(exts, halos, stage):
                if r is not None and r.data_ptr() != ext.data_ptr():
                    ext[:, :h].copy_(r)

        if cuda:
            side.wait_stream(cur)                      # the rows to send were produced on the current stream
            with torch.cuda.stream(side):
                do_exchange()
            for ext in exts:
                ext.record_stream(side)
        else:
            do_exchange()
        for x, ext, h, cp in zip(xs, exts, halos, need_copy):      # meanwhile: local rows into the tail
            if cp:
                ext[:, (h if has_pred else 0):].copy_(x)
        if cuda:
            cur.wait_stream(side)
        return exts

    @staticmethod
    def backward(ctx, g1, g2, g3, g4):
        h1, h2, s1, s2, group = ctx.cfg
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        has_pred, has_succ = rank > 0, rank < world - 1
        gs, halos, sends = (g1, g2, g3, g4), (h1, h2, h1, h2), (s1, s2, s1, s2)
        back = [g[:, :h].contiguous() if (has_pred and h > 0) else None for g, h in zip(gs, halos)]
        incoming = [g.new_empty((g.shape[0], s) + tuple(g.shape[2:])) if (has_succ and s > 0) else None
                    for g, s in zip(gs, sends)]
        # gradient halos travel against the forward direction: to rank-1, from rank+1
        _exchange(incoming, back, rank + 1, rank - 1, group, 200)
        out: List[torch.Tensor] = []
        for g, h, inc in zip(gs, halos, incoming):
            loc = g[:, h:] if (has_pred and h > 0) else g
            if inc is not None:
                loc = loc.clone()
                n = loc.shape[1]
                loc[:, n - inc.shape[1]:] += inc          # fixed order: own share first, then the successor's
            out.append(loc)
        return (*out, None, None, None, None, None)


def two_simplicial_attention_sharded(q, k1, k2, v1, v2, w1: int, w2: int, n_total: int, scale: Optional[float] = None,
                                     k2_bias: float = 0.0, v2_bias: float = 0.0, group=None,
                                     attn_fn: Optional[Callable] = None):
    """Attention over this rank's shard.  q, k1, k2, v1, v2 are the LOCAL rows [B, n_local, H(kv), D]
    of a sequence of `n_total` rows split by `shard_bounds`.  `attn_fn(q, k1, k2, v1, v2, w1, w2,
    scale, k2_bias, v2_bias, halo1, halo2)` is the single-device operator (default: this library's
    CUDA kernels); it must accept K/V with leading halo rows."""
    if attn_fn is None:
        from .simplicial_attn import two_simplicial_attention as attn_fn
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    check_partition(n_total, world, w1, w2)
    start, end = shard_bounds(n_total, world, rank)
    if q.shape[1] != end - start:
        raise ValueError(f"rank {rank} must hold rows [{start}, {end}) but got {q.shape[1]} rows")
    h1, h2 = halo_rows(w1, start), halo_rows(w2, start)
    # rows the successor needs from this rank
    s1 = halo_rows(w1, end) if rank < world - 1 else 0
    s2 = halo_rows(w2, end) if rank < world - 1 else 0
    k1e, k2e, v1e, v2e = _HaloExchange.apply(k1, k2, v1, v2, h1, h2, s1, s2, group)
    return attn_fn(q, k1e, k2e, v1e, v2e, w1, w2, scale, k2_bias, v2_bias, h1, h2)
