"""Loads the committed golden vectors (outputs of the unmodified reference loop)."""
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    B, N, H, Hkv, D, w1, w2 = (int(x) for x in z["meta"])
    kb, vb = (float(x) for x in z["bias"])
    ins = {k: torch.from_numpy(z["in_" + k].copy()).view(torch.bfloat16) for k in ("q", "k1", "k2", "v1", "v2", "do")}
    outs = {k: torch.from_numpy(z[k].copy()) for k in ("o", "dq", "dk1", "dk2", "dv1", "dv2") if k in z.files}
    cfg = dict(B=B, N=N, H=H, Hkv=Hkv, D=D, w1=w1, w2=w2, k2_bias=kb, v2_bias=vb, scale=1.0 / D ** 0.5)
    return cfg, ins, outs
