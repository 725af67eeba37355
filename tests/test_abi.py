"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares, and
its argument validation and kernel selection work without a GPU (no compute is launched)."""
import ctypes
import os
import re

import pytest

from simplical_attn_b200 import _abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "simplicial_attn_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sa_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported():
    lib = _abi.load()
    syms = declared_symbols()
    assert set(_abi.EXPORTS) <= set(syms)
    for s in syms:
        assert hasattr(lib, s), s


def test_struct_layout_matches_header():
    # 11 int32 + 3 float + 12 x (3 x int64)
    assert ctypes.sizeof(_abi.Params) == 11 * 4 + 3 * 4 + 12 * 24
    assert _abi.Params.q.offset == 56


def _params(**kw):
    p = _abi.Params()
    p.B, p.N, p.H, p.Hkv, p.D, p.w1, p.w2 = 1, 64, 4, 2, 128, 16, 8
    p.dtype, p.algo, p.scale = _abi.SA_BF16, _abi.SA_ALGO_AUTO, 0.1
    for name in ("q", "k1", "k2", "v1", "v2", "o", "d_o", "dq", "dk1", "dk2", "dv1", "dv2"):
        setattr(p, name, _abi.Strides(64 * 4 * 128, 4 * 128, 128))
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def test_validation_codes():
    lib = _abi.load()
    nul = ctypes.c_void_p(0)
    args = [nul] * 8 + [0, nul]
    assert lib.sa_forward(ctypes.byref(_params(H=3)), *args) == 2            # H % Hkv
    assert lib.sa_forward(ctypes.byref(_params(w1=0)), *args) == 2
    assert lib.sa_forward(ctypes.byref(_params(halo1=-1)), *args) == 2
    assert lib.sa_forward(ctypes.byref(_params(D=512)), *args) == 4
    assert lib.sa_forward(ctypes.byref(_params(dtype=7)), *args) == 4
    assert lib.sa_forward(ctypes.byref(_params()), *args) == 1               # NULL pointers
    assert "NULL" in _abi.strerror(1)
    with pytest.raises(_abi.SimplicialAttnError):
        _abi.check("sa_forward", 2)


def test_kernel_selection():
    lib = _abi.load()
    r = lambda **kw: lib.sa_resolve_algo(ctypes.byref(_params(**kw)))
    assert r() == _abi.SA_ALGO_TCGEN05
    assert r(D=64) == _abi.SA_ALGO_TCGEN05
    assert r(D=32) == _abi.SA_ALGO_GENERAL
    assert r(dtype=_abi.SA_F32) == _abi.SA_ALGO_GENERAL
    assert r(dtype=_abi.SA_F16) == _abi.SA_ALGO_TCGEN05
    assert r(w2=200, N=4096) == _abi.SA_ALGO_TCGEN05                         # two passes over chunks of the K2 window
    assert r(w2=1025, N=4096) == _abi.SA_ALGO_GENERAL
    assert r(w2=200, N=64) == _abi.SA_ALGO_TCGEN05                           # window clipped to 64 rows
    assert r(algo=_abi.SA_ALGO_GENERAL) == _abi.SA_ALGO_GENERAL
    assert r(D=32, algo=_abi.SA_ALGO_TCGEN05) == -4
    assert r(q=_abi.Strides(1000, 100, 4)) == _abi.SA_ALGO_GENERAL           # rows not 16-byte aligned
    assert r(H=5) == -2
    assert lib.sa_forward_workspace_size(ctypes.byref(_params())) == 256
    assert lib.sa_backward_workspace_size(ctypes.byref(_params())) >= 256
    # a K2 window of more than 128 positions: room for one more O (bf16) and LSE (fp32) in the forward, for one
    # more set of gradients in the backward
    wide, narrow = _params(w2=200, N=4096), _params(w2=100, N=4096)
    assert lib.sa_forward_workspace_size(ctypes.byref(wide)) == 256 + 4096 * 4 * 128 * 2 + 4 * 4096 * 4
    extra = lib.sa_backward_workspace_size(ctypes.byref(wide)) - lib.sa_backward_workspace_size(ctypes.byref(narrow))
    assert extra >= (4096 * 4 * 128 + 4 * 4096 * 2 * 128) * 2


def test_python_layer_rejects_cpu_tensors():
    import torch
    import simplical_attn_b200 as sab
    x = torch.zeros(1, 8, 1, 16)
    with pytest.raises(RuntimeError):
        sab.two_simplicial_attention(x, x, x, x, x, 4, 4)
    m = sab.TwoSimplicialAttention(16, 4, 4)
    assert len(m.state_dict()) == 0 and abs(m.scale - 0.25) < 1e-12


def test_host_pipeline_chunk_plan():
    from simplical_attn_b200.host_pipeline import plan_chunks
    # whole sequences in the middle, a small head group first and last
    assert plan_chunks(3, 16) == [(0, 0, 4), (0, 4, 16), (1, 0, 16), (2, 0, 12), (2, 12, 16)]
    assert plan_chunks(1, 16) == [(0, 0, 4), (0, 4, 12), (0, 12, 16)]
    assert plan_chunks(2, 1) == [(0, 0, 1), (1, 0, 1)]
    assert plan_chunks(1, 2) == [(0, 0, 1), (0, 1, 2)]
    for B, Hkv in ((1, 1), (2, 2), (5, 3), (16, 16), (2, 8)):
        ch = plan_chunks(B, Hkv)
        assert sorted(ch) == ch and all(h1 > h0 for _, h0, h1 in ch)
        assert sum(h1 - h0 for _, h0, h1 in ch) == B * Hkv


def test_cpu_list_parsing_and_numa_helper_without_a_gpu():
    from simplical_attn_b200 import host_pipeline as hp
    assert hp._cpu_list("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert hp._cpu_list("") == set()
    assert hp.local_cpus("cuda:0") is None or isinstance(hp.local_cpus("cuda:0"), set)      # no GPU here: None
    with hp.near("cuda:0") as took_effect:                                                   # must be harmless
        assert took_effect in (False, True)


def test_library_staleness_follows_source_contents(tmp_path, monkeypatch):
    """The library counts as current exactly while the digest recorded at build time matches the sources,
    whatever the file times say."""
    from simplical_attn_b200 import build as b
    assert not b._stale()                                   # built by the session fixture / build step
    digest = b.source_digest()
    assert open(b.STAMP).read().strip() == digest
    monkeypatch.setattr(b, "NVCC_FLAGS", b.NVCC_FLAGS + ["-DSOMETHING_ELSE"])
    assert b.source_digest() != digest and b._stale()       # other flags (or sources): stale
