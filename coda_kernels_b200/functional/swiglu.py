"""``linear_swiglu(x, weight)``: the gated MLP up-projection, ``silu(x @ W_gate^T) * (x @ W_up^T)``.

Drop-in for the operator of the same name in the reference (coda/kernels/functional/swiglu.py:8-30): one weight of
shape ``[2F, K]`` whose even rows are the gate projection and whose odd rows are the up projection, bf16 in and out.

Forward is ONE kernel launch: the tcgen05 GEMM whose epilogue reads each (gate, up) pair from adjacent accumulator
columns of one thread, writes the bf16 pre-activation (kept for the backward) and the activated product.  Backward is
one HBM-bound pass that turns (pre-activation, dout) into the pre-activation gradient, then the two GEMMs of
:func:`coda_kernels_b200.ops.linear_backward`.  Each direction is one call into the compiled dispatch layer.
"""

from __future__ import annotations

import torch
from torch import Tensor

from .._guards import autocast_custom_bwd, autocast_custom_fwd, input_guard
from ..ops import swiglu_backward, swiglu_forward


class LinearSwiGLU(torch.autograd.Function):
    """Autograd node of :func:`linear_swiglu`; saves ``(x, weight, preact)``."""

    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x: Tensor, weight: Tensor) -> Tensor:
        saved_preact, activated = swiglu_forward(x, weight)
        ctx.save_for_backward(x, weight, saved_preact)
        return activated

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, grad_out: Tensor):
        x, weight, saved_preact = ctx.saved_tensors
        need_dx, need_dw = ctx.needs_input_grad[:2]
        return swiglu_backward(saved_preact, grad_out, x, weight, need_dx, need_dw)


def linear_swiglu(x: Tensor, weight: Tensor) -> Tensor:
    """``x [M, K]``, ``weight [2F, K]`` (gate row ``j`` at ``2j``, up row ``j`` at ``2j + 1``) -> ``[M, F]``."""
    return LinearSwiGLU.apply(x, weight)
