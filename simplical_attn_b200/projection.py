"""The step either side of the operator in a model: hidden states -> (Q, K1, K2, V1, V2) -> attention
-> output projection.

The reference starts at the five tensors (`simplicial/triton_impl.py:173-186`) and leaves the
projections to its caller.  This module is that caller for users who want one: a single fused input
projection (one GEMM for all five tensors, laid out so that every head's rows are contiguous and the
attention kernels read them without a copy), the operator, and the output projection.  The GEMMs are
plain library GEMMs (`torch.nn.functional.linear`); the attention in between is this library's.
Grouped heads: K1/K2/V1/V2 get `kv_heads` heads, `num_heads % kv_heads == 0`.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .simplicial_attn import two_simplicial_attention


class TwoSimplicialSelfAttention(torch.nn.Module):
    """`y = W_o . attention(W_q x, W_k1 x, W_k2 x, W_v1 x, W_v2 x)` over `[B, N, hidden]` inputs."""

    def __init__(self, hidden: int, num_heads: int, head_dim: int, w1: int = 64, w2: int = 64, kv_heads: Optional[int] = None,
                 scale: Optional[float] = None, k2_bias: float = 0.0, v2_bias: float = 0.0, bias: bool = False,
                 dtype=torch.bfloat16, device=None):
        super().__init__()
        self.num_heads = num_heads
        self.kv_heads = kv_heads if kv_heads is not None else num_heads
        if num_heads % self.kv_heads != 0:
            raise ValueError("kv_heads must divide num_heads")
        self.head_dim = head_dim
        self.w1, self.w2 = w1, w2
        self.scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)     # triton_impl.py:169
        self.k2_bias, self.v2_bias = k2_bias, v2_bias
        self.widths = (num_heads * head_dim,) + (self.kv_heads * head_dim,) * 4    # q | k1 | k2 | v1 | v2
        self.in_proj = torch.nn.Linear(hidden, sum(self.widths), bias=bias, dtype=dtype, device=device)
        self.out_proj = torch.nn.Linear(num_heads * head_dim, hidden, bias=bias, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, N, _ = x.shape
        fused = self.in_proj(x)                                   # one GEMM: [B, N, (H + 4 Hkv) * D]
        parts = torch.split(fused, self.widths, dim=-1)
        # views into the GEMM's output: row stride (H + 4 Hkv) * D, head stride D, unit inner stride --
        # the operator takes them as they are
        q = parts[0].view(B, N, self.num_heads, self.head_dim)
        k1, k2, v1, v2 = (t.view(B, N, self.kv_heads, self.head_dim) for t in parts[1:])
        o = two_simplicial_attention(q, k1, k2, v1, v2, self.w1, self.w2, self.scale, self.k2_bias, self.v2_bias)
        return self.out_proj(o.reshape(B, N, self.num_heads * self.head_dim))
