"""Pieces shared by the fused-linear autograd wrappers."""

from __future__ import annotations

from typing import Optional

from torch import Tensor

from ..ops import gemm


def linear_backward(grad_pre: Tensor, x: Tensor, weight: Tensor, need_dx: bool = True, need_dw: bool = True,
                    alpha: Optional[Tensor] = None):
    """Gradients of ``pre = x @ weight^T`` given ``grad_pre = dL/dpre`` (times the device scalar ``alpha``, if given).

    ``dx = grad_pre @ weight`` reads the ``[N, K]`` weight as an MN-major B operand and
    ``dweight = grad_pre^T @ x`` reads both operands MN-major, so neither needs a transposed copy.  ``alpha`` is
    applied in the GEMM epilogues (read from device memory: no host synchronisation).
    """
    dx = gemm(grad_pre, weight, alpha=alpha) if need_dx else None
    dweight = gemm(grad_pre.mT, x, alpha=alpha) if need_dw else None
    return dx, dweight


def masked_loss(row_losses: Tensor, target: Tensor, ignore_index: int, reduction: str):
    """``(loss, inv_count)``: per-row losses folded to the scalar loss.  For ``"mean"`` the divisor is the number of rows
    whose target is not ``ignore_index`` and ``inv_count`` (a 0-d device tensor) is kept for the backward; for ``"sum"``
    it is ``None``.  Ignored rows already carry an exact zero."""
    total = row_losses.sum()
    if reduction == "sum":
        return total, None
    inv_count = (target != ignore_index).sum().float().reciprocal()
    return total * inv_count, inv_count
