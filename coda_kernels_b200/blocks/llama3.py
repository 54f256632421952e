"""Fused Llama-3 layer blocks: whole-layer ``autograd.Function``s that chain the GEMM + epilogue operators.

Public surface of coda/kernels/blocks/llama3.py:635-775 of the reference (same names, argument order, return values):

* ``block_pre``:  first RMSNorm + QKV projection + RoPE of the first layer; returns ``(residual, qkv)``.
* ``block``:      attention output projection + residual + RMSNorm + SwiGLU MLP + residual + the NEXT layer's
  RMSNorm + QKV projection + RoPE; returns ``(x2, qkv)``.  Attention itself runs between two blocks, outside.
* ``block_post``: like ``block`` but ending in the final RMSNorm + LM head + cross entropy; returns the loss.

Every RMSNorm is deferred: the GEMM that produces the residual stream also emits ``rstd`` and ``x * weight``, and the
GEMM that consumes it applies ``rstd`` to its accumulator, so the normalised activations never exist in memory.

How this file is organised.  A layer is a *trunk* (output projection, MLP, the two residual adds) followed by a *head*
that reads the normalised residual stream: the next layer's QKV projection with RoPE, or the LM head with the loss.
All three blocks run the same three steps backward:

1. the head hands back ``(g, zdz, alpha)``: the gradient w.r.t. its linear output, the per-row dot ``sum(z * dz)`` the
   RMSNorm VJP needs (each head has it almost for free: rotations are orthogonal; the loss GEMM sums it per tile), and
   an optional device scalar that still has to multiply ``g``;
2. :func:`_normed_linear_backward` turns that into the gradient of the residual stream (one dgrad GEMM whose epilogue
   applies the norm VJP and accumulates), the weight gradient (one wgrad GEMM) and the norm-weight gradient;
3. :func:`_trunk_backward` walks the trunk, which is again a normed linear (gate/up behind the MLP norm) between two
   plain projections.

Weights are ``nn.Linear``-style ``[out, in]``; the SwiGLU weight interleaves gate and up rows; ``frequencies`` has one
(hi, lo) pair per column pair of ``qkv`` and is zero on the v columns.  Activations may be ``[tokens, dim]`` or
``[batch, length, dim]``.
"""

from __future__ import annotations

import os
from typing import NamedTuple, Optional

import torch
from torch import Tensor

from .._guards import autocast_custom_bwd, autocast_custom_fwd, input_guard
from ..ops import gemm
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


# ------------------------------------------------------------------------------------------------ building blocks
class HeadGrad(NamedTuple):
    """What a head's backward hands to the norm in front of it."""

    g: Tensor                # gradient w.r.t. the head's linear output, [M, N]
    zdz: Tensor              # per-row sum(z * dz) / dim, fp32 [M]
    alpha: Optional[Tensor]  # device scalar still to be applied to g (and already applied to zdz), or None


class Trunk(NamedTuple):
    """Tensors the trunk keeps for its backward, plus what the head consumes (``h2``, ``rstd2``)."""

    x1: Tensor     # residual stream after the attention output projection
    rstd1: Tensor  # its deferred-norm statistic
    z1: Tensor     # gate/up pre-activation
    x2: Tensor     # residual stream after the MLP
    h2: Tensor     # x2 * wn_head (un-normalised: rstd2 is applied by the consumer)
    rstd2: Tensor


def _normed_linear_backward(head: HeadGrad, w: Tensor, wn: Tensor, stream: Tensor, rstd: Tensor, grad_stream: Optional[Tensor]):
    """Backward of ``linear(rmsnorm(stream; wn); w)`` given the gradient of its output.

    One dgrad GEMM (``g @ w``) whose epilogue applies the RMSNorm VJP at the saved ``rstd`` and adds into
    ``grad_stream`` (or starts it when that is ``None``), and one wgrad GEMM against the normalised input, which the
    same epilogue re-creates on the fly.  Returns ``(grad_stream, dw, dwn)`` with ``dwn`` in the weight's dtype.
    """
    grad_stream, dwn, normed = gemm_residual_partial_rmsnorm_bwd(
        A=head.g, B=w.mT, weight=wn, pre=stream, ZdZ=head.zdz, rstd=rstd, alpha=head.alpha, dX=grad_stream)
    dw = gemm(head.g.mT, normed, alpha=head.alpha)
    return grad_stream, dw, dwn.to(dtype=wn.dtype)


def _trunk_forward(x0, y0, w_out, w_gate_up, w_down, wn_mlp, wn_head, eps) -> Trunk:
    x1, h1, rstd1 = gemm_residual_partial_rmsnorm(A=y0, B=w_out.mT, C=x0, weight=wn_mlp, eps=eps)
    z1, y1 = gemm_rmsnorm_swiglu(h1, w_gate_up.mT, rstd1)
    x2, h2, rstd2 = gemm_residual_partial_rmsnorm(A=y1, B=w_down.mT, C=x1, weight=wn_head, eps=eps)
    return Trunk(x1, rstd1, z1, x2, h2, rstd2)


def _trunk_backward(grad_stream: Tensor, y0, w_out, w_gate_up, w_down, wn_mlp, x1, rstd1, z1):
    """From the gradient of ``x2`` to ``(dx0, dy0, dw_out, dw_gate_up, dw_down, dwn_mlp)``."""
    dim = x1.shape[1]
    # down projection: its dgrad runs the SwiGLU derivative in the epilogue and re-creates the activation for the wgrad
    dz1, zdz1, y1 = gemm_swiglu_bwd_zdz(A=grad_stream, B=w_down.mT, Z=z1, scale=1.0 / dim)
    dw_down = gemm(grad_stream.mT, y1)
    grad_stream, dw_gate_up, dwn_mlp = _normed_linear_backward(HeadGrad(dz1, zdz1, None), w_gate_up, wn_mlp, x1, rstd1, grad_stream)
    # attention output projection: the residual gradient is also the gradient of its output
    dy0 = gemm(grad_stream, w_out)
    dw_out = gemm(grad_stream.mT, y0)
    return grad_stream, dy0, dw_out, dw_gate_up, dw_down, dwn_mlp


def _rope_head_backward(qkv: Tensor, dqkv: Tensor, positions, frequencies, dim: int) -> HeadGrad:
    # rotations are orthogonal: sum(z * dz) = sum(y * dy), so the row dot comes from the rotated tensors
    dz, zdz = rope_bwd_zdz(y=qkv, dy=dqkv, pos=positions, freq=frequencies, scale=1.0 / dim)
    return HeadGrad(dz, zdz, None)


def _incoming(grad: Tensor) -> Tensor:
    return grad if ALLOW_INPLACE_GRAD_OUTPUT else grad.clone()


# ------------------------------------------------------------------------------------------------ autograd nodes
class BlockPre(torch.autograd.Function):
    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x, w, wn, positions, frequencies, eps: float):
        assert wn.dtype == x.dtype and x.ndim == 2
        # x feeds both qkv and the residual stream; returning a copy lets the backward add the two gradients in fp32
        residual, h, rstd = partial_rmsnorm(x=x, weight=wn, eps=eps)
        qkv = gemm_rmsnorm_rope(A=h, B=w.mT, rstd=rstd, positions=positions, frequencies=frequencies)
        ctx.save_for_backward(x, w, wn, qkv, rstd, positions, frequencies)
        return residual, qkv

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, d_residual, dqkv):
        x, w, wn, qkv, rstd, positions, frequencies = ctx.saved_tensors
        head = _rope_head_backward(qkv, dqkv, positions, frequencies, x.shape[1])
        dx, dw, dwn = _normed_linear_backward(head, w, wn, x, rstd, _incoming(d_residual))
        return dx, dw, dwn, None, None, None


class Block(torch.autograd.Function):
    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x0, y0, w0, w1, w2, w3, wn0, wn1, positions, frequencies, eps: float):
        t = _trunk_forward(x0, y0, w0, w1, w2, wn0, wn1, eps)
        qkv = gemm_rmsnorm_rope(A=t.h2, B=w3.mT, rstd=t.rstd2, positions=positions, frequencies=frequencies)
        ctx.save_for_backward(y0, w0, w1, w2, w3, wn0, wn1, qkv, t.x1, t.x2, t.rstd1, t.rstd2, t.z1, positions, frequencies)
        return t.x2, qkv

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, dx2, dqkv):
        y0, w0, w1, w2, w3, wn0, wn1, qkv, x1, x2, rstd1, rstd2, z1, positions, frequencies = ctx.saved_tensors
        head = _rope_head_backward(qkv, dqkv, positions, frequencies, x2.shape[1])
        grad_stream, dw3, dwn1 = _normed_linear_backward(head, w3, wn1, x2, rstd2, _incoming(dx2))
        dx0, dy0, dw0, dw1, dw2, dwn0 = _trunk_backward(grad_stream, y0, w0, w1, w2, wn0, x1, rstd1, z1)
        return dx0, dy0, dw0, dw1, dw2, dw3, dwn0, dwn1, None, None, None


class BlockPost(torch.autograd.Function):
    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x0, y0, w0, w1, w2, w3, wn0, wn1, targets, eps: float, ignore_index: int, reduction: str):
        t = _trunk_forward(x0, y0, w0, w1, w2, wn0, wn1, eps)
        # LM head and cross entropy in one GEMM: the logits stay in fp32 accumulators and are never stored
        losses, dlogits, zdz = gemm_rmsnorm_cross_entropy_fwd_bwd(A=t.h2, B=w3.mT, rstd=t.rstd2, target=targets,
                                                                  ignore_index=ignore_index, return_zdz=True)
        loss, mean_scale = reduce_losses(losses=losses, target=targets, ignore_index=ignore_index, reduction=reduction)
        ctx.save_for_backward(y0, w0, w1, w2, w3, wn0, wn1, t.x1, t.x2, t.rstd1, t.rstd2, t.z1, mean_scale, dlogits, zdz)
        return loss

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, dloss):
        y0, w0, w1, w2, w3, wn0, wn1, x1, x2, rstd1, rstd2, z1, mean_scale, dlogits, zdz = ctx.saved_tensors
        # dlogits is d(sum of row losses)/d(logits); the loss gradient (times 1 / count for "mean") stays a device scalar
        alpha = (dloss if mean_scale is None else dloss * mean_scale).reshape(1).to(dtype=torch.float32)
        head = HeadGrad(dlogits, zdz * (alpha / x2.shape[1]), alpha)
        grad_stream, dw3, dwn1 = _normed_linear_backward(head, w3, wn1, x2, rstd2, None)
        dx0, dy0, dw0, dw1, dw2, dwn0 = _trunk_backward(grad_stream, y0, w0, w1, w2, wn0, x1, rstd1, z1)
        return dx0, dy0, dw0, dw1, dw2, dw3, dwn0, dwn1, None, None, None, None


# ------------------------------------------------------------------------------------------------ public functions
def _tokens(t: Tensor) -> Tensor:
    """``[batch, length, dim]`` or ``[tokens, dim]`` -> ``[tokens, dim]`` (a view)."""
    return t.reshape(-1, t.shape[-1])


def _like(flat: Tensor, ref: Tensor) -> Tensor:
    return flat if ref.ndim == 2 else flat.reshape(*ref.shape[:-1], flat.shape[-1])


def _check_trunk_args(x0, y0, w0, w1, w2, w3, wn0, wn1):
    dim = w0.shape[0]
    assert x0.shape[-1] == dim and y0.shape == x0.shape and y0.dtype == x0.dtype
    assert w0.shape == (dim, dim) and w1.shape[1] == dim and w2.shape == (dim, w1.shape[0] // 2) and w3.shape[1] == dim
    assert wn0.shape == (dim,) and wn1.shape == (dim,)
    for w in (w0, w1, w2, w3, wn0, wn1):
        assert w.dtype == x0.dtype


def block_pre(x, w, wn, positions, frequencies, eps: float):
    """``(residual, qkv)`` for ``x [..., dim]``, ``w [(hq + 2 hk) * d, dim]``, ``wn [dim]``."""
    assert w.shape[1] == x.shape[-1] and w.dtype == x.dtype and wn.shape == (x.shape[-1],) and wn.dtype == x.dtype
    assert positions.dtype in (torch.float32, torch.int32) and frequencies.shape == (w.shape[0],) and frequencies.dtype == torch.float32
    residual, qkv = BlockPre.apply(_tokens(x), w, wn, positions, frequencies, eps)
    return _like(residual, x), _like(qkv, x)


def block(x0, y0, w0, w1, w2, w3, wn0, wn1, positions, frequencies, eps: float):
    """``(x2, qkv)``: ``x0`` residual stream, ``y0`` attention output, ``w0`` output projection, ``w1`` interleaved
    gate/up, ``w2`` down projection, ``w3`` the next layer's QKV weight, ``wn0`` / ``wn1`` the two norm weights."""
    _check_trunk_args(x0, y0, w0, w1, w2, w3, wn0, wn1)
    assert positions.dtype in (torch.float32, torch.int32) and frequencies.shape == (w3.shape[0],) and frequencies.dtype == torch.float32
    x2, qkv = Block.apply(_tokens(x0), _tokens(y0), w0, w1, w2, w3, wn0, wn1, positions, frequencies, eps)
    return _like(x2, x0), _like(qkv, x0)


def block_post(x0, y0, w0, w1, w2, w3, wn0, wn1, targets, eps: float, ignore_index: int = -100, reduction: str = "mean"):
    """The last layer's MLP half, final norm, LM head ``w3 [vocab, dim]`` and cross entropy against int32 ``targets``."""
    _check_trunk_args(x0, y0, w0, w1, w2, w3, wn0, wn1)
    assert reduction in ("mean", "sum")
    assert targets.dtype == torch.int32
    return BlockPost.apply(_tokens(x0), _tokens(y0), w0, w1, w2, w3, wn0, wn1, targets.reshape(-1), eps, ignore_index, reduction)
