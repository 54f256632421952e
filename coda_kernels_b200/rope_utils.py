"""RoPE frequency tables in the two-term "turns" form the kernels consume.

``make_rope_frequencies`` is the helper the reference's benchmarks import from
``coda.core.ops.rope_utils`` (benchmarks/utils/operands.py:10, 562-565).  Its
contract follows from its consumers (coda/core/ops/math_utils.py:181-195,
benchmarks/backends/torch_ops.py:116-132): for rotary pair ``p`` of every head,
element ``2p`` holds ``hi`` and ``2p+1`` holds ``lo`` with
``hi + lo = inv_freq[p] / (2*pi)`` to well below fp32 precision.
"""

from __future__ import annotations

import math

import torch


def rope_inv_freq(head_dim: int, theta: float = 500000.0, device=None) -> torch.Tensor:
    """``theta ** (-2p / head_dim)`` for ``p = 0 .. head_dim/2 - 1`` in fp32."""
    p = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device)
    return 1.0 / (theta ** (p / head_dim))


def make_rope_frequencies(inv_freq: torch.Tensor, num_heads: int) -> torch.Tensor:
    """fp32 ``[num_heads * 2 * len(inv_freq)]``: per pair ``(hi, lo)`` turns, tiled over heads."""
    turns = inv_freq.to(dtype=torch.float64) / (2.0 * math.pi)
    hi = turns.to(dtype=torch.float32)
    lo = (turns - hi.to(dtype=torch.float64)).to(dtype=torch.float32)
    per_head = torch.stack((hi, lo), dim=1).reshape(-1)
    return per_head.repeat(num_heads).contiguous()
