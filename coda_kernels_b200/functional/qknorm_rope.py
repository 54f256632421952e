"""``linear_qknorm_rope``: the attention input projection with per-head RMSNorm and RoPE applied to q and k.

Drop-in for the reference operator (coda/kernels/functional/qknorm_rope.py:8-136): same nine arguments, ``(q, k, v)``
returned with ``q`` and ``k`` as two column views of one buffer, nine gradients of which the last six are ``None``.

What differs underneath:

* q, k and v come out of ONE GEMM launch over the whole ``[(hq + hk + hv) * d, K]`` weight.  A 128-column head is
  local to one epilogue thread, so the mean-square, the normalisation by ``gamma_q`` / ``gamma_k`` and the rotation of
  adjacent column pairs need no cross-thread traffic; v columns are stored as they are.
* The numbers of q and k heads may differ (grouped-query attention), which the reference's fused epilogue refuses
  (coda/core/gemm/epilogues.py:213-215).
* The backward writes ``[grad_pre | dv]`` into one buffer, so ``dx`` and ``dweight`` are one GEMM each (the reference
  runs two each and adds the ``dx`` halves through an fp32 partial).
"""

from __future__ import annotations

import torch
from torch import Tensor

from .._guards import autocast_custom_bwd, autocast_custom_fwd, input_guard
from ..ops import qknorm_rope_backward, qknorm_rope_forward


class LinearQKNormRope(torch.autograd.Function):
    """Autograd node of :func:`linear_qknorm_rope`."""

    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x: Tensor, weight: Tensor, gamma: Tensor, positions: Tensor, frequencies: Tensor, head_dim: int,
                num_heads_q: int, num_heads_k: int, eps: float):
        rotated, preact, head_mean_sq, v = qknorm_rope_forward(
            x, weight, gamma, positions, frequencies, head_dim, num_heads_q, num_heads_k, eps)  # v: zero columns without v rows
        ctx.head_dim, ctx.num_heads_q, ctx.num_heads_k, ctx.eps = head_dim, num_heads_q, num_heads_k, eps
        ctx.save_for_backward(x, weight, gamma, positions, frequencies, preact, head_mean_sq)
        width_q = head_dim * num_heads_q
        # two views of `rotated` (the backward receives their gradients separately anyway); `split` rather than two
        # slices: with slices the outputs came back wrong under torch.compile(fullgraph=True)
        q, k = rotated.split((width_q, rotated.shape[1] - width_q), dim=-1)
        return q, k, v

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, grad_q: Tensor, grad_k: Tensor, grad_v: Tensor):
        x, weight, gamma, positions, frequencies, preact, head_mean_sq = ctx.saved_tensors
        head_dim, num_heads_q, num_heads_k, eps = ctx.head_dim, ctx.num_heads_q, ctx.num_heads_k, ctx.eps
        dx, dweight, dgamma = qknorm_rope_backward(grad_q, grad_k, grad_v, x, weight, preact, head_mean_sq, gamma, positions, frequencies,
                                                   head_dim, num_heads_q, num_heads_k, eps, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return (dx, dweight, dgamma) + (None,) * 6


def linear_qknorm_rope(x: Tensor, weight: Tensor, gamma: Tensor, positions: Tensor, frequencies: Tensor, head_dim: int,
                       num_heads_q: int, num_heads_k: int, eps: float) -> tuple[Tensor, Tensor, Tensor]:
    """``x [M, K]``; ``weight`` rows ``[q | k | v]``; ``gamma [2 * head_dim] = [gamma_q | gamma_k]``; ``positions [M]`` int32 or
    fp32; ``frequencies [(hq + hk) * head_dim]`` fp32 (hi, lo) turns per rotary pair.  Returns ``(q, k, v)``."""
    return LinearQKNormRope.apply(x, weight, gamma, positions, frequencies, head_dim, num_heads_q, num_heads_k, eps)
