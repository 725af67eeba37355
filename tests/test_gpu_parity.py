"""GPU parity: the CUDA kernels, called through the C ABI, against the reference's golden vectors
and against the CPU oracle (which tests/test_oracle.py pins to those vectors).

Tolerances (stated by the target for bf16 kernels vs the fp32 reference on bf16-rounded inputs):
max-abs <= 2e-2 on O, relative L2 <= 1e-2 on each gradient.  fp32 tensors through the general
kernels are held to 1e-4.
"""
import math

import pytest
import torch

import simplical_attn_b200 as sab
from oracle import c_oracle, simplicial_oracle as so
from simplical_attn_b200 import simplicial_attn as host
from tests import golden_util as gu

pytestmark = pytest.mark.gpu

TOL_O_BF16 = 2e-2
TOL_G_BF16 = 1e-2
TOL_F32 = 1e-4
DEV = "cuda"
TC_BWD_READY = True


def _grad_err(a, b):
    """Relative L2 against the reference gradient.  Where the reference gradient is zero (one
    (j,k) pair per query: softmax weight 1, no logit gradient) the error is absolute and scaled by
    0.1: a bf16 kernel then returns scale * (dO.(V1*V2) - dO.O) * K, which is the rounding of the
    stored O (2^-9 relative) times values of order 10, not zero."""
    if float(b.abs().max()) < 1e-5:
        return 0.1 * float((a.float().cpu() - b).abs().max())
    return so.rel_l2(a.float().cpu(), b)


def _run(ins, cfg, algo, dtype=torch.bfloat16, need=(True,) * 5, halo1=0, halo2=0):
    t = {k: v.to(DEV).to(dtype) for k, v in ins.items()}
    o, lse = sab.two_simplicial_attn_fwd_kernel(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], cfg["w1"], cfg["w2"],
                                                cfg["scale"], cfg["k2_bias"], cfg["v2_bias"], halo1, halo2, algo=algo)
    grads = sab.two_simplicial_attn_bwd(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], o, lse, t["do"], cfg["w1"], cfg["w2"],
                                        cfg["scale"], cfg["k2_bias"], cfg["v2_bias"], halo1, halo2, need,
                                        algo=algo if (algo != "tcgen05" or TC_BWD_READY) else "auto")
    torch.cuda.synchronize()
    return o, lse, grads


def _tc_supported(cfg):
    return cfg["D"] in (64, 128) and min(cfg["w2"], cfg["N"]) <= 1024


@pytest.mark.parametrize("name", gu.names())
def test_general_bf16_vs_reference_golden(name):
    cfg, ins, outs = gu.load(name)
    o, _, grads = _run(ins, cfg, "general")
    assert float((o.float().cpu() - outs["o"]).abs().max()) <= TOL_O_BF16
    for nm, g in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads):
        assert _grad_err(g, outs[nm]) <= TOL_G_BF16, nm


@pytest.mark.parametrize("name", gu.names())
def test_general_fp32_vs_reference_golden(name):
    cfg, ins, outs = gu.load(name)
    o, _, grads = _run(ins, cfg, "general", dtype=torch.float32)
    assert float((o.cpu() - outs["o"]).abs().max()) <= TOL_F32
    for nm, g in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads):
        assert _grad_err(g, outs[nm]) <= TOL_F32, nm


@pytest.mark.parametrize("name", [n for n in gu.names() if _tc_supported(gu.load(n)[0])])
def test_tensor_core_vs_reference_golden(name):
    cfg, ins, outs = gu.load(name)
    o, _, grads = _run(ins, cfg, "tcgen05")
    assert float((o.float().cpu() - outs["o"]).abs().max()) <= TOL_O_BF16
    for nm, g in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads):
        assert _grad_err(g, outs[nm]) <= TOL_G_BF16, nm


# B, N, H, Hkv, D, w1, w2, k2_bias, v2_bias, halo1, halo2
ORACLE_CASES = [
    (1, 300, 2, 1, 128, 100, 32, 0.0, 0.0, 0, 0),      # grouped heads, ragged N
    (2, 200, 2, 2, 128, 512, 32, 0.0, 0.0, 0, 0),      # w1 > N
    (1, 260, 2, 2, 128, 130, 16, 0.0, 0.0, 0, 0),      # two column tiles, 16 delta slots
    (1, 150, 1, 1, 128, 40, 64, 0.0, 0.0, 0, 0),       # 64 delta slots: a query spans two warps
    (1, 140, 2, 2, 64, 33, 5, 0.1, -0.2, 0, 0),        # odd windows, biases
    (1, 96, 2, 1, 128, 48, 12, 0.0, 0.0, 47, 11),      # a sequence shard with halo rows
    (1, 520, 1, 1, 64, 24, 1, 0.0, 0.0, 0, 0),         # w2 = 1: 128 queries per row tile
    (1, 130, 2, 2, 128, 300, 128, 0.0, 0.0, 0, 0),     # widest K2 window: one query per row tile
    (1, 210, 2, 1, 64, 70, 14, 0.05, 0.0, 0, 0),       # D = 64 with 16 delta slots, two of them masked
    (1, 300, 2, 2, 64, 90, 50, 0.0, 0.1, 0, 0),        # D = 64 with 64 delta slots
    (1, 333, 4, 2, 64, 100, 32, 0.0, 0.0, 0, 0),       # D = 64 with 32 delta slots, grouped heads
    (1, 200, 2, 2, 64, 70, 24, 0.1, 0.0, 69, 23),      # D = 64, 32 delta slots (8 masked), bias, halo rows
]


@pytest.mark.parametrize("case", ORACLE_CASES)
@pytest.mark.parametrize("algo", ["general", "tcgen05"])
def test_vs_cpu_oracle(case, algo):
    B, N, H, Hkv, D, w1, w2, kb, vb, h1, h2 = case
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=3, seed_do=4, halo1=h1, halo2=h2)
    scale = 1.0 / math.sqrt(D)
    cfg = dict(w1=w1, w2=w2, scale=scale, k2_bias=kb, v2_bias=vb)
    ins = dict(q=q, k1=k1, k2=k2, v1=v1, v2=v2, do=do)
    o, lse, grads = _run(ins, cfg, algo, halo1=h1, halo2=h2)
    ref = so.forward_backward(q, k1, k2, v1, v2, do, w1, w2, scale, kb, vb, h1, h2)
    assert float((o.float().cpu() - ref[0]).abs().max()) <= TOL_O_BF16
    assert float((lse.cpu() - ref[1]).abs().max()) <= 2e-2
    for nm, g, r in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, ref[2:]):
        assert _grad_err(g, r) <= TOL_G_BF16, nm


# K2 windows wider than one pass of the tensor-core kernels (128 positions): the library chains passes over
# 128-position chunks of the window.  B, N, H, Hkv, D, w1, w2, k2_bias, v2_bias, halo1, halo2
WIDE_K2_CASES = [
    (1, 400, 2, 1, 128, 64, 256, 0.0, 0.0, 0, 0),      # two full chunks, grouped heads
    (1, 330, 2, 2, 128, 40, 160, 0.0, 0.0, 0, 0),      # a full chunk and a 32-position one
    (1, 300, 1, 1, 64, 48, 300, 0.1, -0.1, 0, 0),      # window wider than the sequence is long, D = 64, biases, three chunks
    (1, 200, 2, 2, 128, 30, 200, 0.0, 0.0, 29, 199),   # a sequence shard with halo rows in front
]


@pytest.mark.parametrize("case", WIDE_K2_CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_wide_k2_window_vs_cpu_oracle(case, dtype):
    B, N, H, Hkv, D, w1, w2, kb, vb, h1, h2 = case
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=5, seed_do=6, halo1=h1, halo2=h2)
    scale = 1.0 / math.sqrt(D)
    cfg = dict(w1=w1, w2=w2, scale=scale, k2_bias=kb, v2_bias=vb)
    ins = dict(q=q, k1=k1, k2=k2, v1=v1, v2=v2, do=do)
    o, lse, grads = _run(ins, cfg, "tcgen05", dtype=dtype, halo1=h1, halo2=h2)
    if dtype == torch.float16:
        q, k1, k2, v1, v2, do = (t.to(torch.float16).float() for t in (q, k1, k2, v1, v2, do))
    ref = so.forward_backward(q, k1, k2, v1, v2, do, w1, w2, scale, kb, vb, h1, h2)
    assert float((o.float().cpu() - ref[0]).abs().max()) <= TOL_O_BF16
    assert float((lse.cpu() - ref[1]).abs().max()) <= 2e-2
    for nm, g, r in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, ref[2:]):
        assert _grad_err(g, r) <= TOL_G_BF16, nm


@pytest.mark.parametrize("shape", [(260, 128, 130, 16), (300, 128, 100, 32), (150, 128, 40, 64), (210, 64, 70, 14), (333, 64, 100, 32),
                                   (130, 128, 300, 128), (330, 128, 40, 160)])
@pytest.mark.parametrize("algo", ["tcgen05", "general"])
def test_nothing_behind_the_tensors_is_read_into_the_results(shape, algo):
    """The last 128-row tile of a sequence has rows for queries past the end; their K2 / V2 window rows lie
    past the end of K2 / V2.  Whatever is in memory there (here: NaN, the tensors are views of larger buffers)
    must not reach any result."""
    N, D, w1, w2 = shape
    B, H, Hkv = 1, 2, 2
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=21, seed_do=22)
    scale = 1.0 / math.sqrt(D)

    def padded(t):
        big = torch.full((B, N + 192, t.shape[2], D), float("nan"), dtype=torch.bfloat16, device=DEV)
        big[:, :N] = t.to(DEV).to(torch.bfloat16)
        return big[:, :N]

    clean = [t.to(DEV).to(torch.bfloat16) for t in (q, k1, k2, v1, v2, do)]
    dirty = [padded(t) for t in (q, k1, k2, v1, v2, do)]
    outs = []
    for ts in (clean, dirty):
        o, lse = sab.two_simplicial_attn_fwd_kernel(*ts[:5], w1, w2, scale, algo=algo)
        grads = sab.two_simplicial_attn_bwd(*ts[:5], o, lse, ts[5], w1, w2, scale, algo=algo)
        outs.append((o, lse) + tuple(grads))
    torch.cuda.synchronize()
    for nm, a, b in zip(("o", "lse", "dq", "dk1", "dk2", "dv1", "dv2"), *outs):
        assert bool(torch.isfinite(b.float()).all()), nm
        assert torch.equal(a, b), nm


@pytest.mark.parametrize("shape", [(1, 700, 4, 2, 128, 200, 32, 0, 0), (2, 260, 2, 2, 128, 130, 16, 0, 0), (1, 150, 2, 1, 128, 40, 64, 0, 0),
                                   (1, 130, 2, 2, 128, 300, 128, 0, 0), (1, 330, 2, 2, 128, 40, 160, 0, 0), (1, 333, 4, 2, 64, 100, 32, 0, 0),
                                   (1, 96, 2, 1, 128, 48, 12, 47, 11)])
def test_workspace_contents_do_not_matter(shape, monkeypatch):
    """The kernels write every partial sum of the workspace before they read it: a workspace full of NaN
    bit patterns (behind the status word, which must start at zero) gives the same results, bit for bit."""
    B, N, H, Hkv, D, w1, w2, h1, h2 = shape
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=31, seed_do=32, halo1=h1, halo2=h2)
    cfg = dict(w1=w1, w2=w2, scale=1.0 / math.sqrt(D), k2_bias=0.0, v2_bias=0.0)
    ins = dict(q=q, k1=k1, k2=k2, v1=v1, v2=v2, do=do)
    clean = _run(ins, cfg, "tcgen05", halo1=h1, halo2=h2)

    def nan_workspace(nbytes, device):
        ws = torch.full((max(int(nbytes), 256),), 0xFF, dtype=torch.uint8, device=device)
        ws[:256].zero_()
        return ws

    monkeypatch.setattr(host, "_workspace", nan_workspace)
    dirty = _run(ins, cfg, "tcgen05", halo1=h1, halo2=h2)
    for nm, a, b in zip(("o", "lse"), clean[:2], dirty[:2]):
        assert torch.equal(a, b), nm
    for nm, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), clean[2], dirty[2]):
        assert bool(torch.isfinite(b.float()).all()) and torch.equal(a, b), nm


def test_tensor_core_vs_general_medium():
    """Same bf16 inputs through both kernel families at a size the CPU oracle would take minutes for."""
    B, N, H, Hkv, D, w1, w2 = 1, 2048, 4, 2, 128, 512, 32
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D)
    cfg = dict(w1=w1, w2=w2, scale=1.0 / math.sqrt(D), k2_bias=0.0, v2_bias=0.0)
    ins = dict(q=q, k1=k1, k2=k2, v1=v1, v2=v2, do=do)
    o_t, lse_t, g_t = _run(ins, cfg, "tcgen05")
    o_g, lse_g, g_g = _run(ins, cfg, "general")
    assert float((o_t.float() - o_g.float()).abs().max()) <= 3e-2      # two bf16-rounded results
    assert float((lse_t - lse_g).abs().max()) <= 1e-2
    for nm, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), g_t, g_g):
        assert so.rel_l2(a.float().cpu(), b.float().cpu()) <= TOL_G_BF16, nm


def test_full_size_forward_row_slices_vs_oracle():
    """The forward configuration quoted for one GPU (B2 H8 N8192 D128 w 512/32, storage [B,H,N,D]):
    row slices at the start, across a window boundary, in the middle and at the end are compared
    with the C loop oracle; the whole output is checked finite and against the general kernels on
    one (batch, head)."""
    B, N, H, D, w1, w2 = 2, 8192, 8, 128, 512, 32
    scale = 1.0 / math.sqrt(D)
    q, k1, k2, v1, v2, _ = so.make_inputs(B, N, H, H, D)
    dev = [t.to(DEV).to(torch.bfloat16).permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3) for t in (q, k1, k2, v1, v2)]
    assert dev[0].stride(2) == N * D                                    # [B,H,N,D] storage
    o, lse = sab.two_simplicial_attn_fwd_kernel(*dev, w1, w2, scale, algo="tcgen05")
    torch.cuda.synchronize()
    assert bool(torch.isfinite(o.float()).all()) and bool(torch.isfinite(lse).all())
    for lo, hi in ((0, 40), (500, 530), (4090, 4100), (8180, 8192)):
        ro, rl = c_oracle.forward(q, k1, k2, v1, v2, w1, w2, scale, row_begin=lo, row_end=hi)
        assert float((o[:, lo:hi].float().cpu() - ro[:, lo:hi]).abs().max()) <= TOL_O_BF16
        assert float((lse[:, :, lo:hi].cpu() - rl[:, :, lo:hi]).abs().max()) <= 2e-2
    sl = [t[1:2, :, 3:4].contiguous() for t in dev]
    og, lg = sab.two_simplicial_attn_fwd_kernel(*sl, w1, w2, scale, algo="general")
    assert float((o[1:2, :, 3:4].float() - og.float()).abs().max()) <= 3e-2
    assert float((lse[1:2, 3:4] - lg).abs().max()) <= 1e-2


def _module_inputs(B=1, N=96, H=2, D=64, dtype=torch.bfloat16, seed=11, scale_in=1.0):
    g = torch.Generator().manual_seed(seed)
    return [(scale_in * torch.randn(B, N, H, D, generator=g)).to(DEV).to(dtype).requires_grad_(True) for _ in range(5)]


def test_module_autograd_and_accumulation():
    """Public call: gradients exist for every input, None-gating follows requires_grad, and a second
    backward doubles .grad (the reference's test_gradient_accumulation, test_correctness.py:290-318)."""
    ins = _module_inputs()
    attn = sab.TwoSimplicialAttention(64, w1=16, w2=8)
    attn(*ins).sum().backward()
    first = [t.grad.clone() for t in ins]
    assert all(bool(torch.isfinite(g.float()).all()) and float(g.float().abs().sum()) > 0 for g in first)
    attn(*ins).sum().backward()
    for t, g in zip(ins, first):
        assert torch.allclose(t.grad.float(), 2 * g.float(), atol=1e-2, rtol=1e-2)
    ins2 = _module_inputs()
    ins2[1].requires_grad_(False)
    ins2[4].requires_grad_(False)
    attn(*ins2).sum().backward()
    assert ins2[1].grad is None and ins2[4].grad is None and ins2[0].grad is not None


@pytest.mark.parametrize("algo", ["general", "tcgen05"])
def test_deterministic(algo):
    host.default_algo = algo
    try:
        outs = []
        for _ in range(2):
            ins = _module_inputs(N=200, D=128)
            o = sab.TwoSimplicialAttention(128, w1=64, w2=16)(*ins)
            o.backward(torch.ones_like(o))
            outs.append([o.detach().clone()] + [t.grad.clone() for t in ins])
        for a, b in zip(*outs):
            assert torch.equal(a, b)
    finally:
        host.default_algo = "auto"


@pytest.mark.parametrize("algo", ["general", "tcgen05"])
def test_edge_cases_finite(algo):
    """The reference's TestEdgeCases (test_correctness.py:321-396): w=1, w > N, zeros, large inputs."""
    host.default_algo = algo
    try:
        for (N, w1, w2, fill) in ((32, 1, 1, None), (32, 100, 100, None), (32, 8, 8, 0.0), (32, 8, 8, 10.0)):
            ins = _module_inputs(N=N, D=64)
            if fill is not None:
                ins = [torch.full_like(t, fill).requires_grad_(True) for t in ins]
            o = sab.TwoSimplicialAttention(64, w1=w1, w2=w2)(*ins)
            o.sum().backward()
            assert o.shape == ins[0].shape and bool(torch.isfinite(o.float()).all())
            assert all(bool(torch.isfinite(t.grad.float()).all()) for t in ins)
            if fill == 0.0:
                assert float(o.float().abs().max()) == 0.0
            if fill == 10.0:
                assert float((o.float() - 100.0).abs().max()) <= 1.0     # softmax of equal logits: mean of v1*v2
    finally:
        host.default_algo = "auto"


def test_fp16_and_fp32_through_auto():
    """The reference's dtype matrix (test_correctness.py:39,154): fp16 runs on the tensor-core kernels (where they
    cover the shape), fp32 on the general kernels."""
    for dtype, tol in ((torch.float16, 1e-2), (torch.float32, 1e-4)):
        cfg, ins, outs = gu.load("tiny_sym")
        o, _, _ = _run(ins, cfg, "auto", dtype=dtype)
        assert float((o.float().cpu() - outs["o"]).abs().max()) <= tol


@pytest.mark.parametrize("name", [n for n in gu.names() if _tc_supported(gu.load(n)[0])])
def test_tensor_core_fp16_vs_reference_golden(name):
    """IEEE half through the tensor-core kernels (the golden inputs are bf16 values, exact in half)."""
    cfg, ins, outs = gu.load(name)
    o, _, grads = _run(ins, cfg, "tcgen05", dtype=torch.float16)
    assert o.dtype == torch.float16
    assert float((o.float().cpu() - outs["o"]).abs().max()) <= TOL_O_BF16
    for nm, g in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads):
        assert g.dtype == torch.float16
        assert _grad_err(g, outs[nm]) <= TOL_G_BF16, nm


@pytest.mark.parametrize("case", [ORACLE_CASES[0], ORACLE_CASES[2], ORACLE_CASES[3], ORACLE_CASES[4], ORACLE_CASES[5], ORACLE_CASES[8]])
def test_tensor_core_fp16_vs_cpu_oracle(case):
    B, N, H, Hkv, D, w1, w2, kb, vb, h1, h2 = case
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=3, seed_do=4, halo1=h1, halo2=h2)
    scale = 1.0 / math.sqrt(D)
    cfg = dict(w1=w1, w2=w2, scale=scale, k2_bias=kb, v2_bias=vb)
    ins = dict(q=q, k1=k1, k2=k2, v1=v1, v2=v2, do=do)
    o, lse, grads = _run(ins, cfg, "tcgen05", dtype=torch.float16, halo1=h1, halo2=h2)
    ref = so.forward_backward(q, k1, k2, v1, v2, do, w1, w2, scale, kb, vb, h1, h2)
    assert float((o.float().cpu() - ref[0]).abs().max()) <= TOL_O_BF16
    assert float((lse.cpu() - ref[1]).abs().max()) <= 2e-2
    for nm, g, r in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads, ref[2:]):
        assert _grad_err(g, r) <= TOL_G_BF16, nm


def test_bad_arguments_raise():
    ins = _module_inputs()
    with pytest.raises(ValueError):
        sab.two_simplicial_attention(ins[0], ins[1][:, :50], ins[2], ins[3], ins[4], 8, 8)
    with pytest.raises(TypeError):
        sab.two_simplicial_attention(ins[0], ins[1].float(), ins[2], ins[3], ins[4], 8, 8)
    from simplical_attn_b200._abi import SimplicialAttnError
    with pytest.raises(SimplicialAttnError):
        sab.two_simplicial_attention(ins[0], ins[1], ins[2], ins[3], ins[4], 0, 8)


@pytest.mark.parametrize("w1", [128, 256, 512, 1024])
@pytest.mark.parametrize("w2", [16, 32, 64])
def test_window_sweep_tensor_core_vs_general(w1, w2):
    """The window sweep of the batch x head-parallel configuration (w1 in {128..1024} x w2 in {16,32,64},
    D=128) at a reduced batch and length: both kernel families on the same bf16 inputs."""
    B, N, H, Hkv, D = 1, 1536, 2, 2, 128
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=w1 + w2)
    cfg = dict(w1=w1, w2=w2, scale=1.0 / math.sqrt(D), k2_bias=0.0, v2_bias=0.0)
    ins = dict(q=q, k1=k1, k2=k2, v1=v1, v2=v2, do=do)
    o_t, lse_t, g_t = _run(ins, cfg, "tcgen05")
    o_g, lse_g, g_g = _run(ins, cfg, "general")
    assert float((o_t.float() - o_g.float()).abs().max()) <= 3e-2
    assert float((lse_t - lse_g).abs().max()) <= 1e-2
    for nm, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), g_t, g_g):
        assert so.rel_l2(a.float().cpu(), b.float().cpu()) <= TOL_G_BF16, nm


@pytest.mark.parametrize("w2", [16, 32, 64, 128, 200])
def test_partial_gradient_requests_match_full_call(w2):
    """The reference's two backward kernels are separate calls (dQ/dK1/dV1 and dK2/dV2).  Asking the
    tensor-core path for a subset must give the tensors of the full call and None for the rest: exactly
    with 16, 32 and 64 K2 positions (the row kernel with operand / epilogue warpgroups), and to the last
    bit or two of the 16-bit results with 128 (the other row kernel sums dQ in another order when it
    keeps no dK2 / dV2 ring) and 200 (two passes over chunks of the K2 window)."""
    B, N, H, Hkv, D, w1 = 1, 700, 4, 2, 128, 200
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=11 + w2)
    cfg = dict(w1=w1, w2=w2, scale=1.0 / math.sqrt(D), k2_bias=0.0, v2_bias=0.0)
    ins = dict(q=q, k1=k1, k2=k2, v1=v1, v2=v2, do=do)
    _, _, full = _run(ins, cfg, "tcgen05")
    for need in ((True, True, False, True, False), (False, False, True, False, True), (True, False, False, False, False),
                 (False, False, False, False, True)):
        _, _, part = _run(ins, cfg, "tcgen05", need=need)
        for nm, n, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), need, part, full):
            if n and w2 <= 64:
                assert torch.equal(a, b), (nm, need)
            elif n:
                assert so.rel_l2(a.float().cpu(), b.float().cpu()) <= 2e-3, (nm, need)
            else:
                assert a is None, (nm, need)


def test_grouped_heads_full_size():
    """The grouped-head configuration (B1, 32 query heads on 2 KV heads, N=16384, D=128, w 512/32): forward
    row slices against the C loop oracle, all five gradients against the general kernels (which sum
    the 16 query heads of a group inside one warp, in a fixed order)."""
    B, N, H, Hkv, D, w1, w2 = 1, 16384, 32, 2, 128, 512, 32
    scale = 1.0 / math.sqrt(D)
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D)
    cfg = dict(w1=w1, w2=w2, scale=scale, k2_bias=0.0, v2_bias=0.0)
    ins = dict(q=q, k1=k1, k2=k2, v1=v1, v2=v2, do=do)
    o_t, lse_t, g_t = _run(ins, cfg, "tcgen05")
    assert all(bool(torch.isfinite(t.float()).all()) for t in (o_t, *g_t))
    for lo, hi in ((0, 24), (8190, 8200), (16376, 16384)):
        ro, rl = c_oracle.forward(q, k1, k2, v1, v2, w1, w2, scale, row_begin=lo, row_end=hi)
        assert float((o_t[:, lo:hi].float().cpu() - ro[:, lo:hi]).abs().max()) <= TOL_O_BF16
        assert float((lse_t[:, :, lo:hi].cpu() - rl[:, :, lo:hi]).abs().max()) <= 2e-2
    t = {k: v.to(DEV).to(torch.bfloat16) for k, v in ins.items()}
    g_g = sab.two_simplicial_attn_bwd(t["q"], t["k1"], t["k2"], t["v1"], t["v2"], o_t, lse_t, t["do"], w1, w2, scale,
                                      algo="general")
    torch.cuda.synchronize()
    for nm, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), g_t, g_g):
        assert so.rel_l2(a.float().cpu(), b.float().cpu()) <= TOL_G_BF16, nm


# B, N, H, Hkv, D, w1, w2 -- the sizes the headline figures are quoted on
FULL_SIZE_GRAD_CASES = [
    pytest.param((2, 8192, 8, 8, 128, 512, 32), id="B2_H8_N8192_w512x32"),          # single-GPU forward / headline windows
    pytest.param((1, 16384, 32, 2, 128, 512, 32), id="B1_H32_Hkv2_N16384_w512x32"), # grouped heads: 16 query heads per KV head
    pytest.param((1, 8192, 2, 2, 128, 1024, 64), id="B1_H2_N8192_w1024x64"),        # the long-sequence configuration's windows
]


@pytest.mark.parametrize("case", FULL_SIZE_GRAD_CASES)
def test_full_size_gradients_vs_oracle(case):
    """All five gradients of the tensor-core path at full sequence length against the C loop oracle
    (`simplicial/reference.py:39-74` through the pinned C port), on ranges the oracle finishes in
    seconds.  For a range of 64 K rows [k0, k0+64) the oracle is run on every query row that reaches
    it, [k0, k0+64+w1-1): that gives dK1, dV1, dK2 and dV2 of the K rows complete (the sum of the
    shares of those queries) and dQ of all those query rows.  Ranges: the sequence start, an
    unaligned range in the interior; plus dQ of the last rows."""
    B, N, H, Hkv, D, w1, w2 = case
    scale = 1.0 / math.sqrt(D)
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=17, seed_do=18)
    cfg = dict(w1=w1, w2=w2, scale=scale, k2_bias=0.0, v2_bias=0.0)
    ins = dict(q=q, k1=k1, k2=k2, v1=v1, v2=v2, do=do)
    _, _, grads = _run(ins, cfg, "tcgen05")
    dq, dk1, dk2, dv1, dv2 = (g.float().cpu() for g in grads)
    assert all(bool(torch.isfinite(g).all()) for g in (dq, dk1, dk2, dv1, dv2))
    for k0 in (0, N // 2 + 37):
        r0, r1 = k0, min(N, k0 + 64 + w1 - 1)
        ref = c_oracle.backward(q, k1, k2, v1, v2, do, w1, w2, scale, row_begin=r0, row_end=r1)
        assert so.rel_l2(dq[:, r0:r1], ref[0][:, r0:r1]) <= TOL_G_BF16, ("dq", k0)
        for nm, g, r in zip(("dk1", "dk2", "dv1", "dv2"), (dk1, dk2, dv1, dv2), ref[1:]):
            assert so.rel_l2(g[:, k0:k0 + 64], r[:, k0:k0 + 64]) <= TOL_G_BF16, (nm, k0)
    r0 = N - 24
    ref = c_oracle.backward(q, k1, k2, v1, v2, do, w1, w2, scale, row_begin=r0, row_end=N)
    assert so.rel_l2(dq[:, r0:], ref[0][:, r0:]) <= TOL_G_BF16, "dq (end)"
    # the last K rows receive gradient only from the last queries: complete in this call as well
    for nm, g, r in zip(("dk1", "dk2", "dv1", "dv2"), (dk1, dk2, dv1, dv2), ref[1:]):
        assert so.rel_l2(g[:, N - 1:], r[:, N - 1:]) <= TOL_G_BF16, (nm, "last row")


@pytest.mark.parametrize("shape", [(5, 512, 4, 2, 128, 128, 32), (1, 384, 8, 8, 128, 96, 16), (2, 256, 8, 2, 64, 64, 32)])
def test_host_pipeline_matches_device_call(shape):
    """Pinned host tensors in, pinned host results out (uploads / kernels / downloads of (sequence,
    head-group) chunks on three streams, strided copies for the head groups).  O, dQ, dK1, dV1 are
    bit-identical to one device call on the whole batch; dK2 and dV2 are sums of per-run partials whose
    run length depends on how many (batch, head) pairs a call holds, so they agree to fp32 rounding of
    the partial sums (well inside bf16 resolution)."""
    from simplical_attn_b200.host_pipeline import HostPipeline, plan_chunks
    B, N, H, Hkv, D, w1, w2 = shape
    ts = [t.to(torch.bfloat16).pin_memory() for t in so.make_inputs(B, N, H, Hkv, D, seed=9, seed_do=10)]
    scale = 1.0 / math.sqrt(D)
    chunks = plan_chunks(B, Hkv)
    assert sorted(chunks) == chunks and sum(h1 - h0 for _, h0, h1 in chunks) == B * Hkv      # every (sequence, KV head) once
    pipe = HostPipeline("cuda")
    for _ in range(2):                                   # second call reuses buffers
        res = pipe.forward_backward(*ts, w1, w2, scale)
    dev = [t.cuda() for t in ts]
    o, lse = sab.two_simplicial_attn_fwd_kernel(*dev[:5], w1, w2, scale)
    grads = sab.two_simplicial_attn_bwd(*dev[:5], o, lse, dev[5], w1, w2, scale)
    for name, a, b in zip(("o", "dq", "dk1", "dk2", "dv1", "dv2"), res, (o,) + tuple(grads)):
        assert a.is_pinned()
        if name in ("dk2", "dv2"):
            assert so.rel_l2(a.float(), b.float().cpu()) <= 2e-3, name
        else:
            assert torch.equal(a, b.cpu()), name


def test_projection_module_matches_oracle_and_trains():
    """Hidden states -> fused input projection -> attention -> output projection: the attention inside reads the
    five strided views of the projection GEMM's output directly; its result equals the CPU oracle on the same
    projected tensors, and gradients reach the projection weights."""
    torch.manual_seed(3)
    B, N, hidden, H, Hkv, D, w1, w2 = 2, 192, 256, 4, 2, 64, 48, 16
    mod = sab.TwoSimplicialSelfAttention(hidden, H, D, w1, w2, kv_heads=Hkv, device=DEV)
    x = (0.5 * torch.randn(B, N, hidden, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    y = mod(x)
    assert y.shape == (B, N, hidden) and bool(torch.isfinite(y.float()).all())
    with torch.no_grad():
        fused = mod.in_proj(x)
        parts = [t.float().cpu() for t in torch.split(fused, mod.widths, dim=-1)]
        q = parts[0].view(B, N, H, D)
        k1, k2, v1, v2 = (t.view(B, N, Hkv, D) for t in parts[1:])
        o_ref, _ = so.forward(q, k1, k2, v1, v2, w1, w2, mod.scale)
        y_ref = torch.nn.functional.linear(o_ref.reshape(B, N, H * D).to(torch.bfloat16).to(DEV), mod.out_proj.weight)
    assert float((y.float() - y_ref.float()).abs().max()) <= 3e-2
    y.float().pow(2).mean().backward()
    for prm in (mod.in_proj.weight, mod.out_proj.weight):
        assert prm.grad is not None and bool(torch.isfinite(prm.grad.float()).all()) and float(prm.grad.float().abs().sum()) > 0
    assert x.grad is not None and x.grad.shape == x.shape
