"""Generates tests/golden/*.npz from the UNMODIFIED reference loop.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference [--skip-c1-backward]

It imports `simplicial/reference.py` of the reference by file path (the package `__init__` pulls
Triton, which the oracle must not depend on), calls
`two_simplicial_attention_reference(q, k1, k2, v1, v2, w1-1, w2-1, scale, k2_bias, v2_bias)` --
`w-1` because the reference loop attends to [i-w, i] (`reference.py:41-45`) while the operator
attends to (i-w, i] -- and stores its output and the autograd gradients of sum(O*dO).
Grouped-head cases hand the reference `repeat_interleave`-expanded K/V inside the autograd graph.

Inputs come from `oracle.simplicial_oracle.make_inputs` (seeded N(0,1), rounded to bf16, kept as
fp32); each file also stores them as bf16 bit patterns so a change in the random generator cannot
silently invalidate the vectors.  Nothing at test time reads the reference checkout.
"""
import importlib.util
import math
import os
import sys
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import simplicial_oracle as so  # noqa: E402

# name: B, N, H, Hkv, D, w1, w2, k2_bias, v2_bias, backward
CASES = {
    "tiny_sym":      (2, 40, 2, 2, 16, 8, 8, 0.0, 0.0, True),
    "tiny_asym":     (1, 48, 2, 2, 32, 12, 5, 0.0, 0.0, True),
    "tiny_bias":     (1, 32, 2, 2, 16, 8, 4, 0.1, 0.2, True),
    "tiny_w1":       (1, 20, 1, 1, 16, 1, 1, 0.0, 0.0, True),
    "tiny_wbig":     (1, 24, 2, 2, 16, 100, 100, 0.0, 0.0, True),
    "tiny_gqa":      (1, 36, 4, 2, 16, 10, 6, 0.0, 0.0, True),
    "ragged_d64":    (1, 100, 2, 1, 64, 33, 7, 0.0, 0.0, True),
    "c1":            (1, 256, 2, 2, 64, 64, 16, 0.0, 0.0, True),
}


def load_reference(root):
    path = os.path.join(root, "simplicial", "reference.py")
    spec = importlib.util.spec_from_file_location("upstream_reference", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.two_simplicial_attention_reference


def bf16_bits(t):
    return t.to(torch.bfloat16).view(torch.int16).numpy()


def main():
    root = sys.argv[1]
    skip_c1_bwd = "--skip-c1-backward" in sys.argv
    only = [a for a in sys.argv[2:] if not a.startswith("--")]
    ref = load_reference(root)
    for name, (B, N, H, Hkv, D, w1, w2, kb, vb, bwd) in CASES.items():
        if only and name not in only:
            continue
        if name == "c1" and skip_c1_bwd:
            bwd = False
        t0 = time.time()
        q, k1, k2, v1, v2, do = so.make_inputs(B, N, H, Hkv, D, seed=0, seed_do=1)
        leaves = [t.clone().requires_grad_(bwd) for t in (q, k1, k2, v1, v2)]
        g = H // Hkv
        exp = [leaves[0]] + [t.repeat_interleave(g, dim=2) if g > 1 else t for t in leaves[1:]]
        scale = 1.0 / math.sqrt(D)
        with torch.set_grad_enabled(bwd):
            o = ref(*exp, so.to_reference_window(w1), so.to_reference_window(w2), scale, kb, vb)
        out = {"meta": np.array([B, N, H, Hkv, D, w1, w2], dtype=np.int64),
               "bias": np.array([kb, vb], dtype=np.float64),
               "o": o.detach().numpy()}
        if bwd:
            o.backward(do)
            for nm, t in zip(("dq", "dk1", "dk2", "dv1", "dv2"), leaves):
                out[nm] = t.grad.numpy()
        for nm, t in zip(("q", "k1", "k2", "v1", "v2", "do"), (q, k1, k2, v1, v2, do)):
            out["in_" + nm] = bf16_bits(t)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(f"{name}: {time.time() - t0:.1f}s", flush=True)


if __name__ == "__main__":
    main()
