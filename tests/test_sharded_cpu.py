"""Sequence sharding with halo exchange, exercised on CPU ranks over gloo (world size 2 and 3).

The single-device operator is stood in for by the CPU oracle (the torch restatement pinned to the
reference's outputs), so these tests cover the partition arithmetic, the forward halo exchange and
the reverse exchange of halo gradients: the sharded result must equal the unsharded one.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import simplicial_oracle as so
from simplical_attn_b200 import sharded


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_attn(q, k1, k2, v1, v2, w1, w2, scale, k2_bias, v2_bias, halo1, halo2):
    return so.forward(q, k1, k2, v1, v2, w1, w2, scale, k2_bias, v2_bias, halo1, halo2)[0]


def _worker(rank, world, port, cfg, out_dir, use_buffers=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, N, H, Hkv, D, w1, w2 = cfg
        q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=7, seed_do=8)
        s, e = sharded.shard_bounds(N, world, rank)
        loc = [t[:, s:e].clone().requires_grad_(True) for t in (q, k1, k2, v1, v2)]
        args = list(loc)
        if use_buffers:
            # the caller writes its K/V rows straight into the tail of a [halo | shard] buffer: no copy inside
            for i, w in ((1, w1), (2, w2), (3, w1), (4, w2)):
                h = sharded.halo_rows(w, s)
                buf = sharded.kv_buffer(B, e - s, Hkv, D, h, loc[i].dtype, loc[i].device)
                view = sharded.local_rows(buf, h)
                view.copy_(loc[i])
                args[i] = view
        o = sharded.two_simplicial_attention_sharded(*args, w1, w2, N, scale=0.2, attn_fn=_oracle_attn)
        o.backward(do[:, s:e])
        torch.save({"o": o.detach(), "grads": [t.grad for t in loc], "range": (s, e)}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,cfg,use_buffers", [
    (2, (1, 48, 2, 1, 16, 12, 5), False),
    (3, (2, 50, 2, 2, 16, 9, 9), False),          # uneven shards 17/17/16, batch 2 (halo through a staging buffer)
    (2, (1, 40, 2, 2, 16, 21, 3), False),         # halo as long as a shard allows
    (3, (1, 45, 2, 1, 16, 11, 4), True),          # K/V written by the caller into [halo | shard] buffers
    (2, (2, 36, 2, 2, 16, 8, 8), True),
])
def test_sharded_equals_unsharded(world, cfg, use_buffers, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, cfg, str(tmp_path), use_buffers), nprocs=world, join=True)
    B, N, H, Hkv, D, w1, w2 = cfg
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=7, seed_do=8)
    ref = so.forward_backward(q, k1, k2, v1, v2, do, w1, w2, 0.2)
    for r in range(world):
        got = torch.load(os.path.join(str(tmp_path), f"r{r}.pt"))
        s, e = got["range"]
        assert float((got["o"] - ref[0][:, s:e]).abs().max()) <= 1e-5
        for g, full in zip(got["grads"], ref[2:]):
            assert float((g - full[:, s:e]).abs().max()) <= 1e-4


def test_partition_arithmetic():
    assert [sharded.shard_bounds(50, 3, r) for r in range(3)] == [(0, 17), (17, 34), (34, 50)]
    assert sharded.halo_rows(1024, 8192) == 1023 and sharded.halo_rows(64, 0) == 0 and sharded.halo_rows(64, 10) == 10
    sharded.check_partition(65536, 8, 1024, 64)
    with pytest.raises(ValueError):
        sharded.check_partition(64, 8, 32, 4)       # 8-row shards cannot supply a 31-row halo
