"""B200-native 2-simplicial attention: hand-written sm_100a CUDA kernels behind a C ABI, with the
reference's operator interface on top (`TwoSimplicialAttention`,
`TwoSimplicialAttentionFunction` and the kernel-named launchers).

The reference's package also re-exports its loop oracle and test runners
(`simplicial/__init__.py:12-44`); those are test infrastructure and are not part of this library.
"""
from .simplicial_attn import (TwoSimplicialAttention, TwoSimplicialAttentionFunction, compute_D_kernel,
                              two_simplicial_attention, two_simplicial_attn_bwd, two_simplicial_attn_bwd_kv1_kernel,
                              two_simplicial_attn_bwd_kv2_kernel, two_simplicial_attn_fwd_kernel)

__all__ = [
    "TwoSimplicialAttention",
    "TwoSimplicialAttentionFunction",
    "two_simplicial_attention",
    "two_simplicial_attn_fwd_kernel",
    "two_simplicial_attn_bwd",
    "two_simplicial_attn_bwd_kv1_kernel",
    "two_simplicial_attn_bwd_kv2_kernel",
    "compute_D_kernel",
]
