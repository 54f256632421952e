"""Pieces shared by the fused-linear autograd wrappers."""

from __future__ import annotations

from torch import Tensor

from ..ops import gemm


def linear_backward(grad_pre: Tensor, x: Tensor, weight: Tensor, need_dx: bool = True, need_dw: bool = True):
    """Gradients of ``pre = x @ weight^T`` given ``grad_pre = dL/dpre``.

    ``dx = grad_pre @ weight`` reads the ``[N, K]`` weight as an MN-major B operand and
    ``dweight = grad_pre^T @ x`` reads both operands MN-major, so neither needs a transposed copy.
    """
    dx = gemm(grad_pre, weight) if need_dx else None
    dweight = gemm(grad_pre.mT, x) if need_dw else None
    return dx, dweight
