"""``linear_cross_entropy`` / ``linear_cross_entropy_forward``: LM-head loss without logits in memory.

Drop-in for coda/kernels/functional/cross_entropy.py:97-193 (signatures, defaults, the two asserts, autograd behaviour).

Dataflow here: the forward GEMM's epilogue keeps a row max / sum-exp per column tile and stores only unnormalised
probabilities; a per-row reduction gives the log-sum-exp and the row losses; one in-place pass turns the stored
probabilities into ``softmax - onehot`` (exactly zero for ignored rows).  That buffer is the only ``[M, V]`` tensor
and is what the node saves.  The backward is :func:`coda_kernels_b200.ops.linear_backward` over it with
``alpha = dloss / count`` read from device memory, so neither direction synchronises with the host.  ``fused_lse`` is accepted for signature parity; both
values run this path.
"""

import torch

from .._guards import autocast_custom_bwd, autocast_custom_fwd, input_guard
from ..ops import cross_entropy_backward, cross_entropy_forward


class LinearCrossEntropy(torch.autograd.Function):
    """Saves ``(x, weight, dlogits, inv_count)``; ``dlogits`` is the gradient of the SUM of the row losses."""

    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x, weight, target, ignore_index: int, reduction: str, fused_lse: bool) -> torch.Tensor:
        loss, inv_count, dlogits = cross_entropy_forward(x, weight, target, ignore_index, reduction, store_grad=True)
        ctx.save_for_backward(x, weight, dlogits, inv_count)
        return loss

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, dloss: torch.Tensor):
        x, weight, dlogits, inv_count = ctx.saved_tensors
        need_dx, need_dw = ctx.needs_input_grad[:2]
        return (*cross_entropy_backward(dloss, inv_count, dlogits, x, weight, need_dx, need_dw), None, None, None, None)


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


@input_guard
def _forward_only(x, weight, target, ignore_index: int, reduction: str) -> torch.Tensor:
    return cross_entropy_forward(x, weight, target, ignore_index, reduction, store_grad=False)[0]


def linear_cross_entropy_forward(
    x: torch.Tensor,
    weight: torch.Tensor,
    target: torch.Tensor,
    ignore_index: int = -100,
    reduction: str = "mean",
) -> torch.Tensor:
    """The loss alone: nothing of size ``[M, V]`` is written anywhere."""
    assert reduction in ("mean", "sum")
    assert target.dtype == torch.int32
    return _forward_only(x, weight, target, ignore_index, reduction)
