"""The operator names the reference's wrappers import from ``coda.core.elementwise.functional``, with its signatures,
bound to the B200 kernels (see ``coda/core/gemm/functional.py`` of this layout)."""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from coda_kernels_b200 import ops as _ops
from coda_kernels_b200 import ops_logits as _lg
from coda_kernels_b200.ops_block import partial_rmsnorm, rope_bwd_zdz  # noqa: F401


def dswiglu_backward(preact: Tensor, dout: Tensor) -> Tensor:
    """coda/core/elementwise/functional.py:202-218."""
    return _ops.dswiglu_backward(preact, dout)


def cross_entropy_fwd_bwd(logits: Tensor, lses: Tensor, target: Tensor, ignore_index: int, return_zdz: bool = False,
                          losses: Optional[Tensor] = None, zdz: Optional[Tensor] = None):
    """In place ``logits -> softmax - onehot``; returns ``(losses, None)`` (coda/core/elementwise/functional.py:286-311).
    The row dot ``zdz`` is produced by the fused ``gemm_rmsnorm_cross_entropy_fwd_bwd`` instead and is not offered here."""
    if return_zdz:
        raise NotImplementedError("use coda_kernels_b200.ops_block.gemm_rmsnorm_cross_entropy_fwd_bwd(return_zdz=True)")
    ls, _ = _lg.cross_entropy_fwd_bwd(logits, lses, target, ignore_index)
    if losses is not None:
        losses.copy_(ls)
        ls = losses
    return ls, None


def qknorm_rope_bwd(dq: Tensor, dk: Tensor, x: Tensor, head_mean_sq: Tensor, gamma: Tensor, pos: Tensor, freq: Tensor, head_dim: int,
                    num_heads_q: int, num_heads_k: int, eps: float, dx: Optional[Tensor] = None, dgamma: Optional[Tensor] = None):
    """``(grad_pre, dgamma fp32)`` (coda/core/elementwise/functional.py:421-456)."""
    g, dg = _ops.qknorm_rope_bwd(dq.contiguous(), dk.contiguous(), None, x, head_mean_sq, gamma, pos, freq, head_dim, num_heads_q,
                                 num_heads_k, eps)
    if dx is not None:
        dx.copy_(g)
        g = dx
    if dgamma is not None:
        dgamma.copy_(dg)
        dg = dgamma
    return g, dg
