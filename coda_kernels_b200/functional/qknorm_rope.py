"""``linear_qknorm_rope``: fused ``[q | k | v]`` projection with per-head RMSNorm and RoPE on q, k.

Same signature and autograd behaviour as coda/kernels/functional/qknorm_rope.py:8-136
(q and k are two views of one buffer; nine gradients, the last six ``None``).
Unlike the reference's fused epilogue (coda/core/gemm/epilogues.py:213-215) the
numbers of q and k heads may differ (GQA), and q, k and v come out of one GEMM
launch; the backward runs one GEMM for ``dx`` and one for ``dweight`` over the
concatenated ``[grad_pre | dv]``.
"""

import torch

from .._guards import autocast_custom_bwd, autocast_custom_fwd, input_guard
from ..ops import gemm, gemm_qknorm_rope, qknorm_rope_bwd


class LinearQKNormRope(torch.autograd.Function):
    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x, weight, gamma, positions, frequencies, head_dim: int, num_heads_q: int, num_heads_k: int, eps: float):
        size_q = head_dim * num_heads_q
        size_qk = head_dim * (num_heads_q + num_heads_k)
        qk, preact, head_mean_sq, v = gemm_qknorm_rope(
            x, weight.mT, weight=gamma, positions=positions, frequencies=frequencies, head_dim=head_dim,
            num_heads_q=num_heads_q, num_heads_k=num_heads_k, eps=eps,
        )
        if v is None:
            v = x.new_empty(x.shape[0], 0)
        q, k = qk.split((size_q, size_qk - size_q), dim=-1)
        ctx.head_dim = head_dim
        ctx.num_heads_q = num_heads_q
        ctx.num_heads_k = num_heads_k
        ctx.eps = eps
        ctx.save_for_backward(x, weight, gamma, positions, frequencies, preact, head_mean_sq)
        return q, k, v

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, dq, dk, dv):
        x, weight, gamma, positions, frequencies, preact, head_mean_sq = ctx.saved_tensors
        grad, dgamma = qknorm_rope_bwd(
            dq=dq, dk=dk, dv=dv if dv.shape[1] > 0 else None, x=preact, head_mean_sq=head_mean_sq, gamma=gamma,
            pos=positions, freq=frequencies, head_dim=ctx.head_dim, num_heads_q=ctx.num_heads_q,
            num_heads_k=ctx.num_heads_k, eps=ctx.eps,
        )
        dx = gemm(grad, weight)  # ([grad_pre | dv]) @ W: the two row blocks of W accumulate in fp32
        dweight = gemm(grad.mT, x)
        return dx, dweight, dgamma.to(dtype=gamma.dtype), None, None, None, None, None, None


def linear_qknorm_rope(
    x: torch.Tensor,
    weight: torch.Tensor,
    gamma: torch.Tensor,
    positions: torch.Tensor,
    frequencies: torch.Tensor,
    head_dim: int,
    num_heads_q: int,
    num_heads_k: int,
    eps: float,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return LinearQKNormRope.apply(x, weight, gamma, positions, frequencies, head_dim, num_heads_q, num_heads_k, eps)
