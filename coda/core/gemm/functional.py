"""The operator names ``coda/kernels/functional/*.py`` and ``coda/kernels/blocks/llama3.py`` of the reference import
from ``coda.core.gemm.functional``, with the reference's signatures, bound to the B200 kernels.

With this module (and ``coda.core.elementwise.functional``) on the path, the reference's own autograd wrappers run
unchanged on sm_100a.  Arguments the B200 ops do not need (pre-allocated optional outputs) are honoured where the
reference's callers use them.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from coda_kernels_b200 import ops as _ops
from coda_kernels_b200 import ops_block as _blk
from coda_kernels_b200 import ops_logits as _lg
from coda_kernels_b200 import ops_rmsnorm as _rn
from coda_kernels_b200.ops_block import (  # noqa: F401
    gemm_residual_partial_rmsnorm,
    gemm_residual_partial_rmsnorm_bwd,
    gemm_rmsnorm_rope,
    gemm_swiglu_bwd_zdz,
)


def gemm(A: Tensor, B: Tensor, out: Optional[Tensor] = None, C: Optional[Tensor] = None) -> Tensor:
    """``out = A @ B (+ C)`` (coda/core/gemm/functional.py:54-69); ``C`` is added to the accumulator in the GEMM's epilogue."""
    if C is not None:
        assert C.shape == (A.shape[0], B.shape[1])
        C = C if C.stride(-1) == 1 else C.contiguous()
    return _ops.gemm(A, B, out=out, C=C)


def gemm_scalar_scale(A: Tensor, B: Tensor, alpha: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """``alpha * (A @ B)`` with ``alpha`` a 0-d device tensor (coda/core/gemm/functional.py:116-132)."""
    return _ops.gemm(A, B, out=out, alpha=alpha.reshape(1).to(dtype=torch.float32))


def gemm_sigmoid(A: Tensor, B: Tensor, out: Optional[Tensor] = None) -> Tensor:
    return _ops.gemm_sigmoid(A, B, out=out)


def gemm_swiglu(A: Tensor, B: Tensor) -> tuple[Tensor, Tensor]:
    return _ops.gemm_swiglu(A, B)


def gemm_rmsnorm_swiglu(A: Tensor, B: Tensor, rstd: Tensor, pre: Optional[Tensor] = None, post: Optional[Tensor] = None):
    z, y = _rn.gemm_rmsnorm_swiglu(A, B, rstd)
    if pre is not None:
        pre.copy_(z)
        z = pre
    if post is not None:
        post.copy_(y)
        y = post
    return z, y


def gemm_lse(A: Tensor, B: Tensor) -> tuple[Tensor, Tensor]:
    """``(logits, lses)`` (coda/core/gemm/functional.py:371-389)."""
    return _lg.gemm_lse(A, B)


def gemm_rmsnorm_lse(A: Tensor, B: Tensor, rstd: Tensor, logits: Optional[Tensor] = None, lses: Optional[Tensor] = None):
    lg, ls = _lg.gemm_lse(A, B, rstd=rstd)
    if logits is not None:
        logits.copy_(lg)
        lg = logits
    if lses is not None:
        lses.copy_(ls)
        ls = lses
    return lg, ls


def gemm_lse_select_logits(A: Tensor, B: Tensor, target: Tensor, ignore_index: int, return_lse: bool,
                           losses: Optional[Tensor] = None, target_logits: Optional[Tensor] = None):
    """``(losses, lses or None, target_logits)`` without storing logits (coda/core/gemm/functional.py:496-527)."""
    assert target.dtype == torch.int32
    ls, lse, tl = _ops.gemm_lse_select_logits(A, B, target, ignore_index)
    if losses is not None:
        losses.copy_(ls)
        ls = losses
    if target_logits is not None:
        target_logits.copy_(tl)
        tl = target_logits
    return ls, (lse if return_lse else None), tl


def gemm_qknorm_rope(A: Tensor, B: Tensor, weight: Tensor, positions: Tensor, frequencies: Tensor, head_dim: int, num_heads_q: int,
                     num_heads_k: int, eps: float, out: Optional[Tensor] = None, preact: Optional[Tensor] = None,
                     head_mean_sq: Optional[Tensor] = None) -> tuple[Tensor, Tensor, Tensor]:
    """``(rotated qk, preact, head_mean_sq)`` for ``B = W_qk.mT`` (coda/core/gemm/functional.py:1155-1200); unlike the
    reference's epilogue, ``num_heads_q`` and ``num_heads_k`` may differ."""
    qk, pre, ms, _ = _ops.gemm_qknorm_rope(A, B, weight, positions, frequencies, head_dim, num_heads_q, num_heads_k, eps)
    for given, got in ((out, qk), (preact, pre), (head_mean_sq, ms)):
        if given is not None:
            given.copy_(got)
    return (out if out is not None else qk), (preact if preact is not None else pre), (head_mean_sq if head_mean_sq is not None else ms)
