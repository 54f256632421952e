"""Fused Llama-3 layer blocks: whole-layer ``autograd.Function``s that chain the GEMM + epilogue operators.

Same public functions, argument order and return values as coda/kernels/blocks/llama3.py:635-775 of the reference:

* ``block_pre``:  first RMSNorm + QKV projection + RoPE of the first layer; returns ``(residual, qkv)``.
* ``block``:      attention output projection + residual + RMSNorm + SwiGLU MLP + residual + the NEXT layer's
  RMSNorm + QKV projection + RoPE; returns ``(x2, qkv)``.  Attention itself runs between two blocks, outside.
* ``block_post``: like ``block`` but ending in the final RMSNorm + LM head + cross entropy; returns the loss.

Every RMSNorm is deferred: the GEMM that produces the residual stream also emits ``rstd`` and ``x * weight``, and the
GEMM that consumes it applies ``rstd`` to its accumulator, so the normalised activations never exist in memory.  The
backward reuses ``sum(z * dz)`` row dots that the preceding backward kernel already has in registers.
Weights are ``nn.Linear``-style ``[out, in]``; the SwiGLU weight interleaves gate and up rows; ``frequencies`` has one
(hi, lo) pair per column pair of ``qkv`` and is zero on the v columns.
"""

from __future__ import annotations

import os

import torch

from .._guards import autocast_custom_bwd, autocast_custom_fwd, input_guard
from ..ops import gemm, gemm_scalar_scale
from ..ops_block import (
    gemm_residual_partial_rmsnorm,
    gemm_residual_partial_rmsnorm_bwd,
    gemm_rmsnorm_cross_entropy_fwd_bwd,
    gemm_rmsnorm_rope,
    gemm_swiglu_bwd_zdz,
    partial_rmsnorm,
    reduce_losses,
    rope_bwd_zdz,
)
from ..ops_rmsnorm import gemm_rmsnorm_swiglu

# Same switch as the reference (coda/core/ops/constants.py:10-19): accumulate into the incoming gradient buffer.
ALLOW_INPLACE_GRAD_OUTPUT = os.environ.get("CODA_ALLOW_INPLACE_GRAD_OUTPUT", "1") == "1"


# ------------------------------------------------------------------------------------------------ block_pre
def block_pre_forward(x, w, wn, positions, frequencies, eps):
    assert wn.dtype == x.dtype and x.ndim == 2
    residual, h, rstd = partial_rmsnorm(x=x, weight=wn, eps=eps)
    qkv = gemm_rmsnorm_rope(A=h, B=w.mT, rstd=rstd, positions=positions, frequencies=frequencies)
    return qkv, rstd, residual


def block_pre_backward(dx, dy, x, w, wn, qkv, rstd, positions, frequencies):
    dim = x.shape[1]
    # rotations are orthogonal: sum(z * dz) = sum(y * dy), so the row dot comes from the rotated tensors
    dz, zdz = rope_bwd_zdz(y=qkv, dy=dy, pos=positions, freq=frequencies, scale=1.0 / dim)
    dx_out = dx if ALLOW_INPLACE_GRAD_OUTPUT else dx.clone()
    dx_out, dwn, x_out = gemm_residual_partial_rmsnorm_bwd(A=dz, B=w.mT, weight=wn, pre=x, ZdZ=zdz, rstd=rstd, dX=dx_out)
    dw = gemm(dz.mT, x_out)
    return dx_out, dw, dwn.to(dtype=wn.dtype)


class BlockPre(torch.autograd.Function):
    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x, w, wn, positions, frequencies, eps: float):
        qkv, rstd, residual = block_pre_forward(x, w, wn, positions, frequencies, eps)
        ctx.save_for_backward(x, w, wn, qkv, rstd, positions, frequencies)
        # x feeds both qkv and the residual stream; returning a copy lets this backward add the two gradients in fp32
        return residual, qkv

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, dx, dy):
        x, w, wn, qkv, rstd, positions, frequencies = ctx.saved_tensors
        dx_out, dw, dwn = block_pre_backward(dx, dy, x, w, wn, qkv, rstd, positions, frequencies)
        return dx_out, dw, dwn, None, None, None


# ------------------------------------------------------------------------------------------------ shared middle part
def _mlp_forward(x0, y0, w0, w1, w2, wn0, wn1, eps):
    x1, h1, rstd1 = gemm_residual_partial_rmsnorm(A=y0, B=w0.mT, C=x0, weight=wn0, eps=eps)
    z1, y1 = gemm_rmsnorm_swiglu(h1, w1.mT, rstd1)
    x2, h2, rstd2 = gemm_residual_partial_rmsnorm(A=y1, B=w2.mT, C=x1, weight=wn1, eps=eps)
    return x1, rstd1, z1, x2, h2, rstd2


def _mlp_backward(dx_out, y0, w0, w1, w2, wn0, x1, rstd1, z1, dim):
    """From the gradient of the second residual stream ``x2`` back to ``x0``, ``y0`` and the three weights."""
    dz1, zdz1, y1 = gemm_swiglu_bwd_zdz(A=dx_out, B=w2.mT, Z=z1, scale=1.0 / dim)
    dw2 = gemm(dx_out.mT, y1)
    dx_out, dwn0, x_out1 = gemm_residual_partial_rmsnorm_bwd(A=dz1, B=w1.mT, weight=wn0, pre=x1, ZdZ=zdz1, rstd=rstd1, dX=dx_out)
    dw1 = gemm(dz1.mT, x_out1)
    dy0 = gemm(dx_out, w0)
    dw0 = gemm(dx_out.mT, y0)
    return dx_out, dy0, dw0, dw1, dw2, dwn0


# ------------------------------------------------------------------------------------------------ block
def block_forward(x0, y0, w0, w1, w2, w3, wn0, wn1, positions, frequencies, eps):
    x1, rstd1, z1, x2, h2, rstd2 = _mlp_forward(x0, y0, w0, w1, w2, wn0, wn1, eps)
    qkv = gemm_rmsnorm_rope(A=h2, B=w3.mT, rstd=rstd2, positions=positions, frequencies=frequencies)
    return qkv, x1, x2, rstd1, rstd2, z1


def block_backward(dx2, dy2, y0, w0, w1, w2, w3, wn0, wn1, qkv, x1, x2, rstd1, rstd2, z1, positions, frequencies):
    dim = x2.shape[1]
    dz2, zdz2 = rope_bwd_zdz(y=qkv, dy=dy2, pos=positions, freq=frequencies, scale=1.0 / dim)
    dx_out = dx2 if ALLOW_INPLACE_GRAD_OUTPUT else dx2.clone()
    dx_out, dwn1, x_out2 = gemm_residual_partial_rmsnorm_bwd(A=dz2, B=w3.mT, weight=wn1, pre=x2, ZdZ=zdz2, rstd=rstd2, dX=dx_out)
    dw3 = gemm(dz2.mT, x_out2)
    dx_out, dy0, dw0, dw1, dw2, dwn0 = _mlp_backward(dx_out, y0, w0, w1, w2, wn0, x1, rstd1, z1, dim)
    return dx_out, dy0, dw0, dw1, dw2, dw3, dwn0.to(dtype=wn0.dtype), dwn1.to(dtype=wn1.dtype)


class Block(torch.autograd.Function):
    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x0, y0, w0, w1, w2, w3, wn0, wn1, positions, frequencies, eps: float):
        qkv, x1, x2, rstd1, rstd2, z1 = block_forward(x0, y0, w0, w1, w2, w3, wn0, wn1, positions, frequencies, eps)
        ctx.save_for_backward(y0, w0, w1, w2, w3, wn0, wn1, qkv, x1, x2, rstd1, rstd2, z1, positions, frequencies)
        return x2, qkv

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, dx2, dy2):
        y0, w0, w1, w2, w3, wn0, wn1, qkv, x1, x2, rstd1, rstd2, z1, positions, frequencies = ctx.saved_tensors
        grads = block_backward(dx2, dy2, y0, w0, w1, w2, w3, wn0, wn1, qkv, x1, x2, rstd1, rstd2, z1, positions, frequencies)
        return (*grads, None, None, None)


# ------------------------------------------------------------------------------------------------ block_post
def block_post_forward(x0, y0, w0, w1, w2, w3, wn0, wn1, targets, eps, ignore_index, reduction):
    x1, rstd1, z1, x2, h2, rstd2 = _mlp_forward(x0, y0, w0, w1, w2, wn0, wn1, eps)
    # LM head and cross entropy in one GEMM: the logits stay in fp32 accumulators and are never stored
    losses, dlogits, zdz2 = gemm_rmsnorm_cross_entropy_fwd_bwd(A=h2, B=w3.mT, rstd=rstd2, target=targets, ignore_index=ignore_index,
                                                               return_zdz=True)
    loss, scale = reduce_losses(losses=losses, target=targets, ignore_index=ignore_index, reduction=reduction)
    return loss, x1, x2, rstd1, rstd2, z1, scale, dlogits, zdz2


def block_post_backward(dloss, y0, w0, w1, w2, w3, wn0, wn1, x1, x2, rstd1, rstd2, z1, scale, dlogits, zdz2):
    dim = x2.shape[1]
    if scale is not None:
        dloss = dloss * scale  # 1 / count of the mean reduction
    alpha = dloss.reshape(1).to(dtype=torch.float32)
    dx_out, dwn1, x_out2 = gemm_residual_partial_rmsnorm_bwd(A=dlogits, B=w3.mT, weight=wn1, pre=x2, ZdZ=zdz2 * (alpha / dim),
                                                             rstd=rstd2, alpha=alpha, dX=None)
    dw3 = gemm_scalar_scale(dlogits.mT, x_out2, alpha=alpha)
    dx_out, dy0, dw0, dw1, dw2, dwn0 = _mlp_backward(dx_out, y0, w0, w1, w2, wn0, x1, rstd1, z1, dim)
    return dx_out, dy0, dw0, dw1, dw2, dw3, dwn0.to(dtype=wn0.dtype), dwn1.to(dtype=wn1.dtype)


class BlockPost(torch.autograd.Function):
    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x0, y0, w0, w1, w2, w3, wn0, wn1, targets, eps: float, ignore_index: int, reduction: str):
        loss, x1, x2, rstd1, rstd2, z1, scale, dlogits, zdz2 = block_post_forward(
            x0, y0, w0, w1, w2, w3, wn0, wn1, targets, eps, ignore_index, reduction)
        ctx.save_for_backward(y0, w0, w1, w2, w3, wn0, wn1, x1, x2, rstd1, rstd2, z1, scale, dlogits, zdz2)
        return loss

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, dloss):
        y0, w0, w1, w2, w3, wn0, wn1, x1, x2, rstd1, rstd2, z1, scale, dlogits, zdz2 = ctx.saved_tensors
        grads = block_post_backward(dloss, y0, w0, w1, w2, w3, wn0, wn1, x1, x2, rstd1, rstd2, z1, scale, dlogits, zdz2)
        return (*grads, None, None, None, None)


# ------------------------------------------------------------------------------------------------ public functions
def block_pre(x, w, wn, positions, frequencies, eps: float):
    """``(residual, qkv)`` for ``x [M, dim]``, ``w [(hq + 2 hk) * d, dim]``, ``wn [dim]``."""
    return BlockPre.apply(x, w, wn, positions, frequencies, eps)


def block(x0, y0, w0, w1, w2, w3, wn0, wn1, positions, frequencies, eps: float):
    """``(x2, qkv)``: ``x0`` residual stream, ``y0`` attention output, ``w0`` output projection, ``w1`` interleaved
    gate/up, ``w2`` down projection, ``w3`` the next layer's QKV weight, ``wn0`` / ``wn1`` the two norm weights."""
    return Block.apply(x0, y0, w0, w1, w2, w3, wn0, wn1, positions, frequencies, eps)


def block_post(x0, y0, w0, w1, w2, w3, wn0, wn1, targets, eps: float, ignore_index: int = -100, reduction: str = "mean"):
    """The last layer's MLP half, final norm, LM head ``w3 [vocab, dim]`` and cross entropy against int32 ``targets``."""
    assert reduction in ("mean", "sum")
    assert targets.dtype == torch.int32
    return BlockPost.apply(x0, y0, w0, w1, w2, w3, wn0, wn1, targets, eps, ignore_index, reduction)
