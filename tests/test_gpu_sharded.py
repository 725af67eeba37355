"""Sequence sharding on real GPUs (NCCL point-to-point halo exchange, one process per GPU).

Skipped unless two CUDA devices are visible.  Each rank runs this library's CUDA kernels on its
shard; the gathered result must match the single-GPU run of the same kernels on the whole sequence
(O bit for bit: halo rows are inputs; gradients within the bf16 tolerance: halo-row gradients are
summed in a different order).  NVLS is switched off for the child processes.
"""
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(cfg):
    from oracle import simplicial_oracle as so
    B, N, H, Hkv, D, w1, w2 = cfg
    return [t.to(torch.bfloat16) for t in so.make_inputs(B, N, H, Hkv, D, seed=17, seed_do=18)]


def _worker(rank, world, port, cfg, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from simplical_attn_b200 import sharded
        B, N, H, Hkv, D, w1, w2 = cfg
        q, k1, k2, v1, v2, do = _inputs(cfg)
        s, e = sharded.shard_bounds(N, world, rank)
        loc = [t[:, s:e].cuda().contiguous().requires_grad_(True) for t in (q, k1, k2, v1, v2)]
        o = sharded.two_simplicial_attention_sharded(*loc, w1, w2, N)
        o.backward(do[:, s:e].cuda())
        torch.cuda.synchronize()
        torch.save({"o": o.detach().cpu(), "grads": [t.grad.cpu() for t in loc], "range": (s, e)},
                   os.path.join(out_dir, f"r{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_sharded_matches_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import simplical_attn_b200 as sab
    from oracle import simplicial_oracle as so
    cfg = (1, 4096, 4, 2, 128, 1024, 64)       # the long-sequence configuration's windows
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), cfg, str(tmp_path)), nprocs=world, join=True)
    B, N, H, Hkv, D, w1, w2 = cfg
    q, k1, k2, v1, v2, do = _inputs(cfg)
    full = [t.cuda().requires_grad_(True) for t in (q, k1, k2, v1, v2)]
    o = sab.two_simplicial_attention(*full, w1, w2, 1.0 / math.sqrt(D))
    o.backward(do.cuda())
    for r in range(world):
        got = torch.load(os.path.join(str(tmp_path), f"r{r}.pt"))
        s, e = got["range"]
        assert torch.equal(got["o"], o.detach().cpu()[:, s:e])
        for g, f in zip(got["grads"], full):
            assert so.rel_l2(g.float(), f.grad.cpu()[:, s:e].float()) <= 1e-2
