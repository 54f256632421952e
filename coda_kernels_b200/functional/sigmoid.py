"""``linear_sigmoid(x, weight, out_dtype=None)``: ``sigmoid(x @ weight^T)``.

Drop-in for the reference operator (coda/kernels/functional/sigmoid.py:7-46).  The output dtype defaults to the input's;
fp32 is the other supported choice.  The backward differentiates through the *stored* (rounded) output, as the
reference does, and returns ``None`` for ``out_dtype``.

Forward is one launch (GEMM with the sigmoid in its epilogue; a 128-column tile is picked automatically when ``weight``
has few rows, e.g. one gate per attention head).  Backward is one HBM-bound pass ``dout * out * (1 - out)`` followed by
the two GEMMs of :func:`coda_kernels_b200.ops.linear_backward`.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
from torch import Tensor

from .._guards import autocast_custom_bwd, autocast_custom_fwd, input_guard
from ..ops import gemm, gemm_dsigmoid_dgrad, sigmoid_backward, sigmoid_forward

# CODA_B200_FUSED_DSIGMOID=1: form the sigmoid gradient inside the input-gradient GEMM (its A-operand prologue) instead
# of in a separate element-wise pass.  Off by default: measured, the fused GEMM loses more than the pass costs.
FUSED_DSIGMOID = os.environ.get("CODA_B200_FUSED_DSIGMOID", "0") == "1"


class LinearSigmoid(torch.autograd.Function):
    """Autograd node of :func:`linear_sigmoid`; saves ``(x, weight, out)``."""

    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x: Tensor, weight: Tensor, out_dtype: Optional[torch.dtype]) -> Tensor:
        result = sigmoid_forward(x, weight, out_dtype)
        ctx.save_for_backward(x, weight, result)
        return result

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, grad_out: Tensor):
        x, weight, result = ctx.saved_tensors
        need_dx, need_dw = ctx.needs_input_grad[:2]
        if FUSED_DSIGMOID and need_dx and result.dtype == x.dtype:
            dx, grad_pre = gemm_dsigmoid_dgrad(result, grad_out.to(dtype=x.dtype), weight)
            dweight = gemm(grad_pre.mT, x) if need_dw else None
            return dx, dweight, None
        dx, dweight = sigmoid_backward(result, grad_out, x, weight, need_dx, need_dw)
        return dx, dweight, None


def linear_sigmoid(x: Tensor, weight: Tensor, out_dtype: Optional[torch.dtype] = None) -> Tensor:
    """``x [M, K]``, ``weight [N, K]`` -> ``sigmoid(x @ weight^T)`` of shape ``[M, N]``."""
    return LinearSigmoid.apply(x, weight, out_dtype)
