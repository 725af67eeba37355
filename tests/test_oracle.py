"""Pins the CPU oracle (torch restatement and C loop) to the reference's own outputs.

The golden files were produced by the unmodified `simplicial/reference.py` of the reference
(see tests/golden/make_golden.py); agreement here is what lets the GPU tests use the oracle
as the reference at sizes the reference loop cannot reach.
"""
import pytest
import torch

from oracle import c_oracle, simplicial_oracle as so
from tests import golden_util as gu

TOL_O = 2e-5        # fp32 reference vs fp32/fp64 restatement
TOL_G = 2e-5        # relative L2 on gradients


def _abs_or_rel(a, b):
    """Relative L2, or absolute max error when the reference gradient is zero up to the 1e-8
    epsilon of `reference.py:74` (w1=w2=1: a single pair, softmax weight 1, no logit gradient)."""
    if float(b.abs().max()) < 1e-5:
        return float((a - b).abs().max())
    return so.rel_l2(a, b)


@pytest.mark.parametrize("name", gu.names())
def test_inputs_reproducible(name):
    cfg, ins, _ = gu.load(name)
    ts = so.make_inputs(cfg["B"], cfg["N"], cfg["H"], cfg["Hkv"], cfg["D"], seed=0, seed_do=1)
    for k, t in zip(("q", "k1", "k2", "v1", "v2", "do"), ts):
        assert torch.equal(t, ins[k].float()), k


@pytest.mark.parametrize("name", gu.names())
def test_torch_restatement_matches_reference(name):
    cfg, ins, outs = gu.load(name)
    f = {k: v.float() for k, v in ins.items()}
    res = so.forward_backward(f["q"], f["k1"], f["k2"], f["v1"], f["v2"], f["do"], cfg["w1"], cfg["w2"],
                              cfg["scale"], cfg["k2_bias"], cfg["v2_bias"])
    o = res[0]
    assert float((o - outs["o"]).abs().max()) <= TOL_O
    for nm, g in zip(("dq", "dk1", "dk2", "dv1", "dv2"), res[2:]):
        if nm in outs:
            assert _abs_or_rel(g, outs[nm]) <= TOL_G, nm


@pytest.mark.parametrize("name", gu.names())
def test_c_loop_matches_reference(name):
    cfg, ins, outs = gu.load(name)
    f = {k: v.float() for k, v in ins.items()}
    args = (f["q"], f["k1"], f["k2"], f["v1"], f["v2"])
    o, lse = c_oracle.forward(*args, cfg["w1"], cfg["w2"], cfg["scale"], cfg["k2_bias"], cfg["v2_bias"])
    assert float((o - outs["o"]).abs().max()) <= TOL_O
    _, lse_t = so.forward(*args, cfg["w1"], cfg["w2"], cfg["scale"], cfg["k2_bias"], cfg["v2_bias"])
    assert float((lse - lse_t).abs().max()) <= 1e-4
    if "dq" in outs:
        grads = c_oracle.backward(*args, f["do"], cfg["w1"], cfg["w2"], cfg["scale"], cfg["k2_bias"], cfg["v2_bias"])
        for nm, g in zip(("dq", "dk1", "dk2", "dv1", "dv2"), grads):
            assert _abs_or_rel(g, outs[nm]) <= TOL_G, nm


def test_row_slices_and_halo_equal_full():
    """A shard's view (halo rows in front, a row sub-range) reproduces the rows of the full run."""
    B, N, H, Hkv, D, w1, w2 = 1, 64, 2, 1, 16, 12, 5
    q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D)
    scale = 0.25
    o_full, lse_full = so.forward(q, k1, k2, v1, v2, w1, w2, scale)
    s = 32                                           # second shard: rows [32, 64)
    h1, h2 = w1 - 1, w2 - 1
    o_sh, lse_sh = so.forward(q[:, s:], k1[:, s - h1:], k2[:, s - h2:], v1[:, s - h1:], v2[:, s - h2:],
                              w1, w2, scale, halo1=h1, halo2=h2)
    assert float((o_sh - o_full[:, s:]).abs().max()) <= 1e-6
    assert float((lse_sh - lse_full[:, :, s:]).abs().max()) <= 1e-5
    o_c, _ = c_oracle.forward(q[:, s:], k1[:, s - h1:], k2[:, s - h2:], v1[:, s - h1:], v2[:, s - h2:],
                              w1, w2, scale)
    assert float((o_c - o_full[:, s:]).abs().max()) <= 2e-5
    # gradient shares of the two shards add up to the full gradient
    full = c_oracle.backward(q, k1, k2, v1, v2, do, w1, w2, scale)
    a = c_oracle.backward(q, k1, k2, v1, v2, do, w1, w2, scale, row_begin=0, row_end=s)
    b = c_oracle.backward(q, k1, k2, v1, v2, do, w1, w2, scale, row_begin=s, row_end=N)
    for x, y, z in zip(full, a, b):
        assert float((x - (y + z)).abs().max()) <= 1e-4
