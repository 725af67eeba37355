"""Sequence-sharded 2-simplicial attention: each rank owns a contiguous block of N/P query rows.

The reference has no multi-GPU path; this is the long-sequence configuration of the target
(N split over the GPUs of one box).  Because the windows are causal and local, rank r needs from
rank r-1 only the last w1-1 rows of K1/V1 and the last w2-1 rows of K2/V2 (its "halo"); in the
backward it returns the gradient of those halo rows to rank r-1, which adds them to its own.  The
exchange is one point-to-point message per tensor and direction (NCCL over NVLink on GPUs, gloo in
the CPU tests); the halo lands in local memory first and the kernels only ever read local memory.

Requires every shard to hold at least max(w1, w2) - 1 rows, so that a halo comes from the immediate
predecessor only.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

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


class _HaloExchange(torch.autograd.Function):
    """forward: [B, n, H, D] -> [B, halo + n, H, D] with `halo` rows received from rank-1 in front
    (and the last `send` rows of x sent to rank+1).  backward: the gradient of the halo rows goes
    back to rank-1 and the gradient received from rank+1 is added to the last `send` rows."""

    @staticmethod
    def forward(ctx, x, recv_rows: int, send_rows: int, group, tag: int):
        rank = dist.get_rank(group)
        world = dist.get_world_size(group)
        ctx.cfg = (recv_rows, send_rows, group, tag)
        ops = []
        halo = None
        if recv_rows > 0 and rank > 0:
            halo = x.new_empty((x.shape[0], recv_rows) + tuple(x.shape[2:]))
            ops.append(dist.P2POp(dist.irecv, halo, _global_rank(group, rank - 1), group=group, tag=tag))
        send_buf = None
        if send_rows > 0 and rank < world - 1:
            send_buf = x[:, x.shape[1] - send_rows:].contiguous()
            ops.append(dist.P2POp(dist.isend, send_buf, _global_rank(group, rank + 1), group=group, tag=tag))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return x if halo is None else torch.cat([halo, x], dim=1)

    @staticmethod
    def backward(ctx, grad_ext):
        recv_rows, send_rows, group, tag = ctx.cfg
        rank = dist.get_rank(group)
        world = dist.get_world_size(group)
        has_halo = recv_rows > 0 and rank > 0
        ops = []
        back = None
        if has_halo:
            back = grad_ext[:, :recv_rows].contiguous()
            ops.append(dist.P2POp(dist.isend, back, _global_rank(group, rank - 1), group=group, tag=tag + 1))
        incoming = None
        if send_rows > 0 and rank < world - 1:
            incoming = grad_ext.new_empty((grad_ext.shape[0], send_rows) + tuple(grad_ext.shape[2:]))
            ops.append(dist.P2POp(dist.irecv, incoming, _global_rank(group, rank + 1), group=group, tag=tag + 1))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        grad = grad_ext[:, recv_rows:] if has_halo else grad_ext
        if incoming is not None:
            grad = grad.clone()
            n = grad.shape[1]
            grad[:, n - send_rows:] += incoming        # fixed order: own share first, then the successor's
        return grad, None, None, None, None


def _global_rank(group, group_rank: int) -> int:
    return dist.get_global_rank(group, group_rank) if group is not None else group_rank


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
    k1e = _HaloExchange.apply(k1, h1, s1, group, 10)
    v1e = _HaloExchange.apply(v1, h1, s1, group, 20)
    k2e = _HaloExchange.apply(k2, h2, s2, group, 30)
    v2e = _HaloExchange.apply(v2, h2, s2, group, 40)
    return attn_fn(q, k1e, k2e, v1e, v2e, w1, w2, scale, k2_bias, v2_bias, h1, h2)
