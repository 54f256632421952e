"""``linear_swiglu``: ``silu(x @ W_gate^T) * (x @ W_up^T)`` with one interleaved weight.

Same signature and autograd behaviour as coda/kernels/functional/swiglu.py:8-30:
``weight`` is ``[2F, K]`` with gate row ``j`` at ``2j`` and up row ``j`` at ``2j+1``.
"""

import torch

from .._guards import autocast_custom_bwd, autocast_custom_fwd, input_guard
from ..ops import dswiglu_backward, gemm, gemm_swiglu


class LinearSwiGLU(torch.autograd.Function):
    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        preact, out = gemm_swiglu(x, weight.mT)
        ctx.save_for_backward(x, weight, preact)
        return out

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, dout: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        x, weight, preact = ctx.saved_tensors
        grad_pre = dswiglu_backward(preact, dout)
        dx = gemm(grad_pre, weight)  # [M, 2F] @ [2F, K]: weight consumed MN-major, no transpose copy
        dweight = gemm(grad_pre.mT, x)  # [2F, M] @ [M, K]: both operands MN-major
        return dx, dweight


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return LinearSwiGLU.apply(x, weight)
