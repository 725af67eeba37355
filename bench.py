#!/usr/bin/env python3
"""Benchmark of the 2-simplicial attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: the batch x head-parallel point the headline metric is quoted on -- B=16, H=Hkv=16,
N=8192, D=128, w1=512, w2=32, bf16, forward + backward; with N GPUs each rank takes B/N sequences
(no data-path collective; strong scaling).  Inputs are seeded N(0,1) synthetic tensors.

One step = one forward and one backward over the rank's batch.  `value` is whole-job TFLOP/s with
inputs resident in HBM, counting 16*B*H*N*w1*w2*D FLOPs per step (2 contractions forward, 6
backward, 2*B*H*N*w1*w2*D each).  `e2e` is the same metric through the library's host-tensor call
(`HostPipeline.forward_backward`: pinned host buffers in and out): host->device copies of the six
inputs and device->host copies of O and the five gradients inside the timed region, overlapped with
the kernels by batch chunks.  `roofline` describes the dominant kernel; `cpu_baseline`
times the C loop oracle on the host cores on a bounded sample of the same workload.

`--impl reference` times the reference's algorithm on the host cores (the C restatement of its
loop; the reference itself is a Python triple loop that does not reach these sizes), with every
core the process may use.

With two or more ranks the line also carries `c4_sharded`: the long-sequence configuration (B1 H16
N65536 D128 w1=1024 w2=64) split along N over the ranks, halo exchange inside the timed region, with
the rows at a rank boundary checked against the CPU oracle.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(B=16, H=16, Hkv=16, N=8192, D=128, w1=512, w2=32)
LONG_SEQUENCE = dict(B=1, H=16, Hkv=16, N=65536, D=128, w1=1024, w2=64)     # split along N over the ranks
# DRAM bytes per launch of each big kernel for ONE batch element of WORKLOAD (dram__bytes_read.sum +
# dram__bytes_write.sum of the ncu captures summarised under profiles/), and the library version those
# captures were taken with: the figures are only reported while the library still has that version.
TRAFFIC = dict(lib_version=200, fwd_tc_kernel=193.6e6, bwd_col_kernel=249.1e6, bwd_row_kernel=396.3e6)
FALLBACK_PEAKS = dict(bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, hbm_gbs=6650.0)


def flops_unit(B, H, N, D, w1, w2):
    """One trilinear contraction over nominal (full) windows: 2*B*H*N*w1*w2*D."""
    return 2.0 * B * H * N * w1 * w2 * D


def flops_unit_exact(B, H, N, D, w1, w2):
    """The same over the (j, k) pairs that exist: the first rows of a sequence have shorter windows."""
    triples = sum(min(i + 1, w1) * min(i + 1, w2) for i in range(min(N, max(w1, w2)))) + max(0, N - max(w1, w2)) * w1 * w2
    return 2.0 * B * H * D * triples


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [x for x in sm if x > 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def make_inputs(Bl, cfg, device, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    shape_q = (Bl, cfg["N"], cfg["H"], cfg["D"])
    shape_kv = (Bl, cfg["N"], cfg["Hkv"], cfg["D"])
    host = [torch.randn(shape_q, generator=g).to(torch.bfloat16)]
    host += [torch.randn(shape_kv, generator=g).to(torch.bfloat16) for _ in range(4)]
    g1 = torch.Generator(device="cpu").manual_seed(seed + 1)
    host.append(torch.randn(shape_q, generator=g1).to(torch.bfloat16))
    host = [t.pin_memory() for t in host]
    return host


def cpu_oracle_rate(cfg, target_s=12.0, threads=None):
    """TFLOP/s (same FLOP convention) of the C loop oracle on a bounded sample: one (batch, head)
    slice of R query rows with full windows (halo rows in front), forward + backward."""
    from oracle import c_oracle, simplicial_oracle as so
    D, w1, w2 = cfg["D"], cfg["w1"], cfg["w2"]
    scale = 1.0 / math.sqrt(D)
    # every core this process may run on, whatever OMP_NUM_THREADS a launcher exported
    cores = c_oracle.set_threads(threads or host_threads())

    def run(R):
        q, k1, k2, v1, v2, do = so.make_inputs(1, R, 1, 1, D, seed=5, seed_do=6, halo1=w1 - 1, halo2=w2 - 1)
        t0 = time.perf_counter()
        c_oracle.forward(q, k1, k2, v1, v2, w1, w2, scale)
        c_oracle.backward(q, k1, k2, v1, v2, do, w1, w2, scale)
        return time.perf_counter() - t0

    r0 = 32 * cores
    t_probe = run(r0)
    R = int(max(r0, min(64 * r0, r0 * target_s / max(t_probe, 1e-3))))
    R = (R // (32 * cores)) * 32 * cores
    t = run(R)
    fl = 8.0 * flops_unit(1, 1, R, D, w1, w2)
    return fl / t / 1e12, cores, R, t


def cpu_oracle_c1():
    """Seconds the C loop oracle takes for the reference's own CPU-runnable case in full (B1 H2 N256
    D64 w1=64 w2=16): forward, and forward + backward."""
    from oracle import c_oracle, simplicial_oracle as so
    q, k1, k2, v1, v2, do = so.make_inputs(1, 256, 2, 2, 64, seed=0, seed_do=1, bf16_round=False)
    scale = 1.0 / math.sqrt(64)
    t0 = time.perf_counter()
    c_oracle.forward(q, k1, k2, v1, v2, 64, 16, scale)
    t1 = time.perf_counter()
    c_oracle.backward(q, k1, k2, v1, v2, do, 64, 16, scale)
    t2 = time.perf_counter()
    return {"config": "B1 H2 N256 D64 w1=64 w2=16 fp32", "forward_s": t1 - t0, "forward_backward_s": t2 - t0,
            "note": "C restatement of the loop; the reference's own Python loop is unavailable on this box "
                    "(the reference checkout does not travel)"}


def run_reference_arm(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step = []
    rows = 0
    cores = 0
    for it in range(args.warmup + args.steps):
        rate, cores, rows, t = cpu_oracle_rate(cfg, target_s=4.0)
        if it >= args.warmup:
            per_step.append((rate, t))
    value = statistics.mean(r for r, _ in per_step)
    ms = statistics.mean(t for _, t in per_step) * 1e3
    sample = (f"forward+backward of {rows} query rows of one (batch, head), full windows, per step; the rate is "
              f"extrapolated to the workload, ms_per_step is the sample's time")
    line = {
        "impl": "reference", "metric": "fwd+bwd TFLOP/s (N=8192,D=128,w1=512,w2=32)", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(cfg), **cfg},
        "parallelism": f"{cores} host threads (OpenMP)",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample,
                         "extrapolated": True, "c1_full": cpu_oracle_c1()},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(cfg):
    return (f"batch x head-parallel fwd+bwd B{cfg['B']} H{cfg['H']} Hkv{cfg['Hkv']} N{cfg['N']} D{cfg['D']} "
            f"w1={cfg['w1']} w2={cfg['w2']}")


def run_shape_sweeps(sab, device, timed):
    """The reference's own sweeps (simplicial/test_performance.py:409-482: sequence length, batch,
    heads, head dim and window at its small base shape B2 H4 N512 D64 w 32/32), forward and
    forward + backward, bf16.  Head dims outside the tensor-core kernels run on the general kernels."""
    base = dict(B=2, N=512, H=4, D=64, w=32)
    grids = {"N": [64, 128, 256, 512, 1024, 2048], "B": [1, 2, 4, 8, 16, 32], "H": [1, 2, 4, 8, 16, 32],
             "D": [32, 64, 128, 256, 512], "w": [8, 16, 32, 64, 128, 256]}
    out = []
    for axis, values in grids.items():
        for v in values:
            c = dict(base)
            c[axis] = v
            pt = {"axis": axis, **c}
            if c["D"] > 256:
                pt["unsupported"] = "head dim above 256"
                out.append(pt)
                continue
            g = torch.Generator(device="cpu").manual_seed(1)
            ts = [torch.randn(c["B"], c["N"], c["H"], c["D"], generator=g).to(torch.bfloat16).to(device) for _ in range(6)]
            scale = 1.0 / math.sqrt(c["D"])
            fwd = lambda: sab.two_simplicial_attn_fwd_kernel(*ts[:5], c["w"], c["w"], scale)
            o_, lse_ = fwd()
            both = lambda: sab.two_simplicial_attn_bwd(*ts[:5], *sab.two_simplicial_attn_fwd_kernel(*ts[:5], c["w"], c["w"], scale),
                                                       ts[5], c["w"], c["w"], scale)
            pt["fwd_ms"] = timed(fwd, 5, 2)
            pt["fwd_bwd_ms"] = timed(both, 5, 2)
            u = flops_unit(c["B"], c["H"], c["N"], c["D"], min(c["w"], c["N"]), min(c["w"], c["N"]))
            pt["fwd_bwd_tflops"] = 8.0 * u / (pt["fwd_bwd_ms"] * 1e-3) / 1e12
            out.append(pt)
    return out


def run_long_sequence_sharded(dist, device, rank, world, args, barrier):
    """The long-sequence configuration split along N: every rank owns N/world query rows and receives
    the (w1-1)-row K1/V1 and (w2-1)-row K2/V2 halos from its predecessor (one batched NCCL exchange per
    direction, inside the timed region).  Rows at the boundary between ranks 0 and 1 are checked
    against the C loop oracle."""
    from simplical_attn_b200 import sharded
    cfg = dict(LONG_SEQUENCE)
    B, H, Hkv, N, D, w1, w2 = (cfg[k] for k in ("B", "H", "Hkv", "N", "D", "w1", "w2"))
    scale = 1.0 / math.sqrt(D)
    s0, s1 = sharded.shard_bounds(N, world, rank)
    n = s1 - s0
    g = torch.Generator(device="cpu").manual_seed(4000 + rank)
    loc = [torch.randn(B, n, H if i == 0 else Hkv, D, generator=g).to(torch.bfloat16).to(device) for i in range(5)]
    do = torch.randn(B, n, H, D, generator=g).to(torch.bfloat16).to(device)
    leaves = [t.requires_grad_(True) for t in loc]

    def step():
        for t in leaves:
            t.grad = None
        o = sharded.two_simplicial_attention_sharded(*leaves, w1, w2, N, scale)
        o.backward(do)
        return o

    def timed_max(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1) / steps], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    steps = max(2, min(args.steps, 5))
    ms = timed_max(step, steps, 2)
    h1, h2 = sharded.halo_rows(w1, s0), sharded.halo_rows(w2, s0)
    e1 = sharded.halo_rows(w1, s1) if rank < world - 1 else 0
    e2 = sharded.halo_rows(w2, s1) if rank < world - 1 else 0
    with torch.no_grad():
        halo_ms = timed_max(lambda: sharded._HaloExchange.apply(*[t.detach() for t in leaves[1:]], h1, h2, e1, e2, None), 5, 2)

    # boundary rows: the first rows of rank 1 see the halo over their whole windows
    check_rows = 8
    with torch.no_grad():
        o = sharded.two_simplicial_attention_sharded(*[t.detach() for t in leaves], w1, w2, N, scale)
    err = None
    tail = w1 - 1 + 64
    if rank == 1:
        pack = [o[:, :check_rows].contiguous()] + [t.detach()[:, :check_rows].contiguous() for t in leaves]
        for req in dist.batch_isend_irecv([dist.P2POp(dist.isend, t, 0) for t in pack]):
            req.wait()
    if rank == 0:
        got = [torch.empty(B, check_rows, H if i in (0, 1) else Hkv, D, dtype=torch.bfloat16, device=device) for i in range(6)]
        for req in dist.batch_isend_irecv([dist.P2POp(dist.irecv, t, 1) for t in got]):
            req.wait()
        torch.cuda.synchronize()
        from oracle import c_oracle
        c_oracle.set_threads(host_threads())
        parts = [torch.cat([a.detach()[:, n - tail:], b], dim=1).float().cpu() for a, b in zip(leaves, got[1:])]
        ro, _ = c_oracle.forward(*parts, w1, w2, scale, row_begin=tail, row_end=tail + check_rows)
        err = float((got[0].float().cpu() - ro[:, tail:tail + check_rows]).abs().max())
    barrier()
    u = flops_unit(B, H, N, D, w1, w2)
    tf = 8.0 * u / (ms * 1e-3) / 1e12
    return {"workload": f"fwd+bwd B{B} H{H} N{N} D{D} w1={w1} w2={w2} split along N over {world} ranks ({n} rows each)",
            "tflops": tf, "tflops_per_gpu": tf / world, "ms_per_step": ms, "halo_ms": halo_ms, "steps": steps,
            "halo_bytes_per_rank_each_way": 2 * ((w1 - 1) + (w2 - 1)) * Hkv * D * 2,
            "frac_of_nominal_2250": tf / world / 2250.0,
            "boundary_rows_checked": f"rows {s1 if rank == 0 else ''}..+{check_rows} (first rows of rank 1) against the C loop oracle",
            "boundary_max_abs_err": err}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="override the global batch (profiling on a small case)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--sweep", action="store_true",
                    help="also time the window sweep w1 in {128,256,512,1024} x w2 in {16,32,64} (adds a 'sweep' key)")
    ap.add_argument("--shape-sweeps", action="store_true",
                    help="also time the reference's own sweeps over N, B, H, D and w (adds a 'shape_sweeps' key)")
    ap.add_argument("--no-sharded", action="store_true", help="skip the sequence-sharded configuration at 2+ ranks")
    args = ap.parse_args()
    cfg = dict(WORKLOAD)
    if args.batch is not None:
        cfg["B"] = args.batch
    if args.impl == "reference":
        run_reference_arm(args, cfg)
        return

    import simplical_attn_b200 as sab
    from simplical_attn_b200 import _abi
    import ctypes

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    if cfg["B"] % world != 0:
        raise SystemExit(f"global batch {cfg['B']} is not divisible by {world} ranks")
    Bl = cfg["B"] // world
    D, w1, w2 = cfg["D"], cfg["w1"], cfg["w2"]
    scale = 1.0 / math.sqrt(D)
    _abi.load()

    from simplical_attn_b200.host_pipeline import HostPipeline, near
    with near(device) as numa_local:          # pinned host buffers on the GPU's NUMA node, where the system tells it
        host = make_inputs(Bl, cfg, device, seed=100 * rank)
        host_out = [torch.empty_like(h).pin_memory() for h in (host[0], host[0], host[1], host[2], host[3], host[4])]
    dev = [t.to(device, non_blocking=True) for t in host]
    torch.cuda.synchronize()
    q, k1, k2, v1, v2, do = dev

    def step_resident():
        o, lse = sab.two_simplicial_attn_fwd_kernel(q, k1, k2, v1, v2, w1, w2, scale)
        grads = sab.two_simplicial_attn_bwd(q, k1, k2, v1, v2, o, lse, do, w1, w2, scale)
        return o, grads

    pipe = HostPipeline(device)

    def step_e2e():
        # the library's host-tensor entry point: pinned host inputs in, pinned host results out; the
        # uploads, kernels and downloads of successive batch chunks overlap on three streams
        pipe.forward_backward(*host, w1, w2, scale, out=host_out)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if dist is not None:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    # per-kernel timing for the roofline (CUDA events on the launching stream, after warm-up)
    def time_phase(fn, reps):
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(reps):
            fn()
        ev1.record()
        torch.cuda.synchronize()
        return ev0.elapsed_time(ev1) / reps

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    lib = _abi.load()
    for _ in range(args.warmup):
        step_resident()
    n0 = lib.sa_kernel_launches()
    ms_step = timed(step_resident, args.steps, 0)
    launches = int(lib.sa_kernel_launches() - n0)
    clocks = sampler.stop() if sampler else None

    o, lse = sab.two_simplicial_attn_fwd_kernel(q, k1, k2, v1, v2, w1, w2, scale)
    reps = max(2, args.steps)
    ms_fwd = time_phase(lambda: sab.two_simplicial_attn_fwd_kernel(q, k1, k2, v1, v2, w1, w2, scale), reps)
    ms_bwd = time_phase(lambda: sab.two_simplicial_attn_bwd(q, k1, k2, v1, v2, o, lse, do, w1, w2, scale), reps)
    # the two big backward kernels on their own (each call also runs the tiny Delta/LSE2 pre-pass,
    # the second one the dK2/dV2 reduction: together < 1 % of the time)
    ms_col = time_phase(lambda: sab.two_simplicial_attn_bwd(q, k1, k2, v1, v2, o, lse, do, w1, w2, scale,
                                                            need=(False, True, False, True, False)), reps)
    ms_row = time_phase(lambda: sab.two_simplicial_attn_bwd(q, k1, k2, v1, v2, o, lse, do, w1, w2, scale,
                                                            need=(True, False, True, False, True)), reps)
    del o, lse

    sweep = None
    if args.sweep:
        sweep = []
        for sw1 in (128, 256, 512, 1024):
            for sw2 in (16, 32, 64):
                def one():
                    o_, lse_ = sab.two_simplicial_attn_fwd_kernel(q, k1, k2, v1, v2, sw1, sw2, scale)
                    sab.two_simplicial_attn_bwd(q, k1, k2, v1, v2, o_, lse_, do, sw1, sw2, scale)
                ms = timed(one, 2, 1)
                u = flops_unit(cfg["B"], cfg["H"], cfg["N"], D, sw1, sw2)
                sweep.append({"w1": sw1, "w2": sw2, "ms_per_step": ms, "tflops": 8.0 * u / (ms * 1e-3) / 1e12})

    ms_e2e = None
    if not args.no_e2e:
        ms_e2e = timed(step_e2e, args.steps, args.warmup)

    shape_sweeps = run_shape_sweeps(sab, device, timed) if args.shape_sweeps else None

    c4 = None
    if world > 1 and not args.no_sharded:
        c4 = run_long_sequence_sharded(dist, device, rank, world, args, barrier)

    unit_total = flops_unit(cfg["B"], cfg["H"], cfg["N"], D, w1, w2)
    unit_exact = flops_unit_exact(cfg["B"], cfg["H"], cfg["N"], D, w1, w2)
    unit_rank = unit_total / world
    value = 8.0 * unit_total / (ms_step * 1e-3) / 1e12

    if rank == 0:
        peaks, peak_kind = load_peaks()
        peak = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
        p = _abi.Params()
        p.B, p.N, p.H, p.Hkv, p.D, p.w1, p.w2 = Bl, cfg["N"], cfg["H"], cfg["Hkv"], D, w1, w2
        p.dtype, p.algo, p.scale = _abi.SA_BF16, _abi.SA_ALGO_AUTO, scale
        for nm, t in zip(("q", "k1", "k2", "v1", "v2", "o", "d_o", "dq", "dk1", "dk2", "dv1", "dv2"),
                         (q, k1, k2, v1, v2, q, do, q, k1, k2, v1, v2)):
            setattr(p, nm, _abi.Strides(t.stride(0), t.stride(1), t.stride(2)))
        algo = _abi.load().sa_resolve_algo(ctypes.byref(p))
        family = {1: "general (CUDA cores)", 2: "tcgen05"}.get(algo, str(algo))
        # Per-kernel roofline.  Credited FLOPs (minimum contraction count, 8 units per step): forward 2
        # (S, P.V1); column kernel 3 (dV1, dK1 and half of the shared S/dP recomputation); row kernel 3
        # (G, U and the other half).  DRAM traffic per launch comes from the ncu capture of a one-batch
        # case (profiles/), scaled by the rank's batch: traffic grows in proportion to the batch.
        lib_version = int(_abi.load().sa_version())
        traffic_ok = algo == 2 and lib_version == TRAFFIC["lib_version"]
        kernels = {
            "fwd_tc_kernel": (ms_fwd, 2.0 * unit_rank, TRAFFIC["fwd_tc_kernel"] * Bl),
            "bwd_col_kernel": (ms_col, 3.0 * unit_rank, TRAFFIC["bwd_col_kernel"] * Bl),
            "bwd_row_kernel": (ms_row, 3.0 * unit_rank, TRAFFIC["bwd_row_kernel"] * Bl),
        }
        # the row kernel has two variants; the library picks the one with separate operand / epilogue warpgroups for
        # 9..64 K2 positions per query (the bench workload)
        symbols = {"fwd_tc_kernel": "fwd_tc_kernel", "bwd_col_kernel": "bwd_col_kernel",
                   "bwd_row_kernel": "bwd_row2_kernel" if 9 <= cfg["w2"] <= 64 else "bwd_row_kernel"}
        dom = max(kernels, key=lambda k: kernels[k][0])
        dom_ms, dom_fl, dom_traffic = kernels[dom]
        achieved = dom_fl / (dom_ms * 1e-3) / 1e12
        roof = {"bound": "tensor", "kernel": f"{symbols[dom]} ({family})", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "peak_source": f"{peak_kind} bf16 sustained (cuBLAS)",
                "traffic": dom_traffic if traffic_ok else None,
                "traffic_unit": f"bytes per launch (ncu capture of one batch element with library version "
                                f"{TRAFFIC['lib_version']}, scaled by the rank's batch; null when the library differs)",
                "frac_of_nominal_2250": achieved / 2250.0,
                "per_kernel": {k: {"symbol": symbols[k], "ms": v[0], "tflops": v[1] / (v[0] * 1e-3) / 1e12,
                                   "frac": v[1] / (v[0] * 1e-3) / 1e12 / peak} for k, v in kernels.items()},
                "forward": {"ms": ms_fwd, "tflops": 2.0 * unit_rank / (ms_fwd * 1e-3) / 1e12},
                "backward": {"ms": ms_bwd, "tflops": 6.0 * unit_rank / (ms_bwd * 1e-3) / 1e12}}
        line = {
            "metric": "fwd+bwd TFLOP/s (N=8192,D=128,w1=512,w2=32)", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(cfg), **cfg},
            "parallelism": f"batch split over {world} GPU(s)",
            "l2": "inputs (6 x %.0f MB per rank) exceed the 126 MB L2" % (q.numel() * 2 / 1e6),
            "kernels": family, "library_version": lib_version,
            "flops": {"per_step_nominal_8U": 8.0 * unit_total, "per_step_exact_triples": 8.0 * unit_exact,
                      "exact_over_nominal": unit_exact / unit_total,
                      "value_exact_triples": 8.0 * unit_exact / (ms_step * 1e-3) / 1e12,
                      "note": "value counts nominal full windows (2*B*H*N*w1*w2*D per contraction, 8 per step); the exact "
                              "figure counts the (j,k) pairs that exist (the first rows of a sequence have shorter windows)"},
            "frac_of_peak": {"measured_sustained": value / world / peak, "nominal_2250": value / world / 2250.0},
            "clocks": clocks, "gpu_launches": launches, "roofline": roof,
        }
        if shape_sweeps is not None:
            line["shape_sweeps"] = shape_sweeps
        if c4 is not None:
            line["c4_sharded"] = c4
        if sweep is not None:
            for pt in sweep:
                pt["frac_of_measured_peak"] = pt["tflops"] / world / peak
                pt["frac_of_nominal_2250"] = pt["tflops"] / world / 2250.0
            line["sweep"] = sweep
        if ms_e2e is not None:
            h2d = sum(t.numel() * t.element_size() for t in host)
            d2h = sum(t.numel() * t.element_size() for t in host_out)
            line["e2e"] = {"value": 8.0 * unit_total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "host_buffers": "pinned, on the GPU's NUMA node" if numa_local else "pinned, default placement"}
        if world == 1 and not args.no_cpu_baseline:
            rate, cores, rows, t = cpu_oracle_rate(cfg)
            line["cpu_baseline"] = {"value": rate, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": f"C loop oracle, forward+backward of {rows} query rows of one "
                                              f"(batch, head) with full windows, {t:.1f} s",
                                    "extrapolated": True, "c1_full": cpu_oracle_c1()}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
