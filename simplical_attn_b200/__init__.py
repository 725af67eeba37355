"""B200-native 2-simplicial attention: hand-written sm_100a CUDA kernels behind a C ABI, with the
reference's operator interface on top (`TwoSimplicialAttention`,
`TwoSimplicialAttentionFunction` and the kernel-named launchers).

The reference's package also re-exports its loop oracle and test runners
(`simplicial/__init__.py:12-44`); those are test infrastructure and are not part of this library.
"""
from .simplicial_attn import (TwoSimplicialAttention, TwoSimplicialAttentionFunction, check_device_status, compute_D_kernel,
                              two_simplicial_attention, two_simplicial_attn_bwd, two_simplicial_attn_bwd_kv1_kernel,
                              two_simplicial_attn_bwd_kv2_kernel, two_simplicial_attn_fwd_kernel)

from .projection import TwoSimplicialSelfAttention

_REFERENCE_ONLY = ("two_simplicial_attention_reference", "TwoSimplicialAttentionReference")


def __getattr__(name):
    # The reference package re-exports its CPU loop oracle under these names
    # (`simplicial/__init__.py:15-16`, `simplicial/reference.py:8-104`).  This library ships GPU kernels
    # only; the loop stays where it is, in the reference's own `simplicial/reference.py`.
    if name in _REFERENCE_ONLY:
        raise AttributeError(f"{name} is the reference's CPU loop oracle (simplicial/reference.py); it is not part of "
                             f"simplical_attn_b200, which has no CPU path: import it from the reference package")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = [
    "TwoSimplicialAttention",
    "TwoSimplicialAttentionFunction",
    "two_simplicial_attention",
    "two_simplicial_attn_fwd_kernel",
    "two_simplicial_attn_bwd",
    "two_simplicial_attn_bwd_kv1_kernel",
    "two_simplicial_attn_bwd_kv2_kernel",
    "compute_D_kernel",
    "check_device_status",
    "TwoSimplicialSelfAttention",
]
