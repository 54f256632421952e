"""``linear_cross_entropy`` / ``linear_cross_entropy_forward``: LM-head loss without logits in memory.

Same signatures, asserts and autograd behaviour as
coda/kernels/functional/cross_entropy.py:97-193.  The forward GEMM's epilogue
keeps an online row max / sum-exp per column tile and stores only unnormalised
probabilities; one in-place pass turns them into ``softmax - onehot`` (zero for
ignored rows), which the two backward GEMMs scale by ``dloss / count`` read from
device memory.  ``fused_lse`` is accepted for signature parity; both values run
this fused path.
"""

import torch

from .._guards import autocast_custom_bwd, autocast_custom_fwd, input_guard
from ..ops import gemm_lse_dlogits, gemm_lse_select_logits, gemm_scalar_scale


def _backward_dlogits(x, weight, dlogits, dloss, need_dx, need_dweight):
    alpha = dloss.reshape(1).to(dtype=torch.float32)
    dx = gemm_scalar_scale(dlogits, weight, alpha=alpha) if need_dx else None
    dweight = gemm_scalar_scale(dlogits.mT, x, alpha=alpha) if need_dweight else None
    return dx, dweight


class LinearCrossEntropy(torch.autograd.Function):
    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x, weight, target, ignore_index: int, reduction: str, fused_lse: bool) -> torch.Tensor:
        losses, dlogits = gemm_lse_dlogits(x, weight.mT, target, ignore_index)
        if reduction == "mean":
            scale = 1.0 / (target != ignore_index).sum().float()
            loss = losses.sum() * scale
        else:
            scale = None
            loss = losses.sum()
        ctx.save_for_backward(x, weight, dlogits, scale)
        return loss

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, dloss: torch.Tensor):
        x, weight, dlogits, scale = ctx.saved_tensors
        dloss_scaled = dloss * scale if scale is not None else dloss
        dx, dweight = _backward_dlogits(
            x=x, weight=weight, dlogits=dlogits, dloss=dloss_scaled,
            need_dx=ctx.needs_input_grad[0], need_dweight=ctx.needs_input_grad[1],
        )
        return dx, dweight, None, None, None, None


def linear_cross_entropy(
    x: torch.Tensor,
    weight: torch.Tensor,
    target: torch.Tensor,
    ignore_index: int = -100,
    reduction: str = "mean",
    fused_lse: bool = True,
) -> torch.Tensor:
    assert reduction in ("mean", "sum")
    assert target.dtype == torch.int32
    return LinearCrossEntropy.apply(x, weight, target, ignore_index, reduction, fused_lse)


def linear_cross_entropy_forward(
    x: torch.Tensor,
    weight: torch.Tensor,
    target: torch.Tensor,
    ignore_index: int = -100,
    reduction: str = "mean",
) -> torch.Tensor:
    assert reduction in ("mean", "sum")
    assert target.dtype == torch.int32
    losses, _, _ = gemm_lse_select_logits(x.contiguous(), weight.contiguous().mT, target.contiguous(), ignore_index)
    if reduction == "mean":
        scale = 1.0 / (target != ignore_index).sum().float()
        return losses.sum() * scale
    return losses.sum()
