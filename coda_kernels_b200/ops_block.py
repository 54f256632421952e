"""GEMMs that sit between the fused-linear operators inside a transformer layer.

Counterparts of ``gemm_residual_partial_rmsnorm``, ``gemm_residual_partial_rmsnorm_bwd`` and
``gemm_swiglu_bwd_zdz`` (coda/core/gemm/functional.py:573-952), which the reference's fused
blocks chain with the deferred-RMSNorm GEMMs of :mod:`coda_kernels_b200.ops_rmsnorm`.  ``B`` is
given as in the reference: ``[K, N]`` for the forward op, the ``[N, K]`` weight itself for the two
backward ops (they compute ``A @ B^T``).
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ._lib import check, lib
from .ops import _noop_fake, _require, _require_cuda_bf16, _stream, lse_tiles, status_word


@torch.library.custom_op(
    "coda_b200::gemm_residual_partial_rmsnorm_out", mutates_args=("pre", "post", "rstd", "scratch"), device_types="cuda"
)
def _residual_norm_out(A: Tensor, B: Tensor, C: Tensor, weight: Tensor, eps: float, pre: Tensor, post: Tensor, rstd: Tensor,
                       scratch: Tensor) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_residual_partial_rmsnorm(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), C.data_ptr(), C.stride(0),
            weight.data_ptr(), float(eps), pre.data_ptr(), pre.stride(0), post.data_ptr(), post.stride(0), rstd.data_ptr(),
            scratch.data_ptr(), M, N, K, status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_residual_partial_rmsnorm",
    )


@torch.library.custom_op(
    "coda_b200::gemm_swiglu_bwd_zdz_out", mutates_args=("dZ", "postact", "zdz", "scratch"), device_types="cuda"
)
def _swiglu_bwd_zdz_out(A: Tensor, B: Tensor, Z: Tensor, dZ: Tensor, postact: Tensor, zdz: Tensor, scale: float,
                        scratch: Tensor) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_swiglu_bwd_zdz(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), Z.data_ptr(), Z.stride(0),
            dZ.data_ptr(), dZ.stride(0), postact.data_ptr(), postact.stride(0), zdz.data_ptr(), float(scale), scratch.data_ptr(),
            M, N, K, status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_swiglu_bwd_zdz",
    )


@torch.library.custom_op(
    "coda_b200::gemm_residual_partial_rmsnorm_bwd_out", mutates_args=("dX", "dW", "normed", "scratch"), device_types="cuda"
)
def _residual_norm_bwd_out(A: Tensor, B: Tensor, weight: Tensor, pre: Tensor, zdz: Tensor, rstd: Tensor, alpha: Optional[Tensor],
                           dX: Tensor, accumulate: bool, dW: Tensor, normed: Tensor, scratch: Tensor) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_residual_partial_rmsnorm_bwd(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), weight.data_ptr(), pre.data_ptr(),
            pre.stride(0), zdz.data_ptr(), rstd.data_ptr(), alpha.data_ptr() if alpha is not None else None, dX.data_ptr(),
            dX.stride(0), int(accumulate), dW.data_ptr(), normed.data_ptr(), normed.stride(0), scratch.data_ptr(), M, N, K,
            status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_residual_partial_rmsnorm_bwd",
    )


for _op in (_residual_norm_out, _swiglu_bwd_zdz_out, _residual_norm_bwd_out):
    _op.register_fake(_noop_fake)


def gemm_residual_partial_rmsnorm(A: Tensor, B: Tensor, C: Tensor, weight: Tensor, eps: float, pre: Optional[Tensor] = None,
                                  post: Optional[Tensor] = None, rstd: Optional[Tensor] = None) -> tuple[Tensor, Tensor, Tensor]:
    """``pre = A @ B + C``, ``post = pre * weight`` and ``rstd = rsqrt(mean(pre^2) + eps)`` of the unrounded ``pre``."""
    _require_cuda_bf16(A, B, C, weight)
    M, N = A.shape[0], B.shape[1]
    _require(tuple(C.shape) == (M, N) and C.stride(1) == 1 and tuple(weight.shape) == (N,), "C must be [M, N], weight [N]")
    pre = torch.empty(M, N, dtype=A.dtype, device=A.device) if pre is None else pre
    post = torch.empty(M, N, dtype=A.dtype, device=A.device) if post is None else post
    rstd = torch.empty(M, dtype=torch.float32, device=A.device) if rstd is None else rstd
    scratch = torch.empty(M, lse_tiles(N), dtype=torch.float32, device=A.device)
    _residual_norm_out(A, B, C, weight.contiguous(), float(eps), pre, post, rstd, scratch)
    return pre, post, rstd


def gemm_swiglu_bwd_zdz(A: Tensor, B: Tensor, Z: Tensor, scale: Optional[float] = None, dZ: Optional[Tensor] = None,
                        ZdZ: Optional[Tensor] = None) -> tuple[Tensor, Tensor, Tensor]:
    """Down-projection dgrad through SwiGLU: ``A [M, K] @ B[N, K]^T`` is ``d(postact)``; returns ``(dZ, ZdZ, postact)``
    with ``dZ = dswiglu(Z, d(postact))``, ``ZdZ = scale * sum(Z * dZ, dim=1)`` and the recomputed ``postact``."""
    _require_cuda_bf16(A, B, Z)
    M, N = A.shape[0], B.shape[0]
    _require(tuple(Z.shape) == (M, 2 * N) and Z.stride(1) == 1, "Z must be [M, 2N]")
    dZ = torch.empty(M, 2 * N, dtype=A.dtype, device=A.device) if dZ is None else dZ
    ZdZ = torch.empty(M, dtype=torch.float32, device=A.device) if ZdZ is None else ZdZ
    postact = torch.empty(M, N, dtype=A.dtype, device=A.device)
    scratch = torch.empty(M, lse_tiles(N), dtype=torch.float32, device=A.device)
    _swiglu_bwd_zdz_out(A, B.mT, Z, dZ, postact, ZdZ, 1.0 if scale is None else float(scale), scratch)
    return dZ, ZdZ, postact


def gemm_residual_partial_rmsnorm_bwd(A: Tensor, B: Tensor, weight: Tensor, pre: Tensor, ZdZ: Tensor, rstd: Tensor,
                                      alpha: Optional[Tensor] = None, dX: Optional[Tensor] = None, dW: Optional[Tensor] = None,
                                      post: Optional[Tensor] = None) -> tuple[Tensor, Tensor, Tensor]:
    """RMSNorm backward fused into the next GEMM's dgrad ``A [M, K] @ B[N, K]^T``: returns ``(dX, dW, normed)``;
    a given ``dX`` is accumulated into."""
    _require_cuda_bf16(A, B, weight, pre)
    M, N = A.shape[0], B.shape[0]
    _require(tuple(pre.shape) == (M, N) and tuple(weight.shape) == (N,), "pre must be [M, N], weight [N]")
    _require(ZdZ.dtype == torch.float32 and rstd.dtype == torch.float32 and ZdZ.numel() == M and rstd.numel() == M,
             "ZdZ and rstd must be fp32 [M]")
    accumulate = dX is not None
    dX = torch.empty(M, N, dtype=A.dtype, device=A.device) if dX is None else dX
    dW = torch.empty(N, dtype=torch.float32, device=A.device) if dW is None else dW
    post = torch.empty(M, N, dtype=A.dtype, device=A.device) if post is None else post
    scratch = torch.empty((M + 31) // 32, N, dtype=torch.float32, device=A.device)
    _residual_norm_bwd_out(A, B.mT, weight.contiguous(), pre, ZdZ.contiguous(), rstd.contiguous(), alpha, dX, accumulate, dW,
                           post, scratch)
    return dX, dW, post


# ------------------------------------------------------------------------------------------------ pieces of the layer blocks
@torch.library.custom_op("coda_b200::partial_rmsnorm_out", mutates_args=("residual", "h", "rstd"), device_types="cuda")
def _partial_rmsnorm_out(x: Tensor, weight: Tensor, eps: float, residual: Optional[Tensor], h: Tensor, rstd: Tensor) -> None:
    M, N = x.shape
    check(
        lib.coda_b200_partial_rmsnorm(
            x.data_ptr(), x.stride(0), weight.data_ptr(), float(eps), residual.data_ptr() if residual is not None else None,
            residual.stride(0) if residual is not None else 0, h.data_ptr(), h.stride(0), rstd.data_ptr(), M, N, _stream(x),
        ),
        "partial_rmsnorm",
    )


@torch.library.custom_op("coda_b200::gemm_rmsnorm_rope_out", mutates_args=("out",), device_types="cuda")
def _gemm_rmsnorm_rope_out(A: Tensor, B: Tensor, rstd: Optional[Tensor], positions: Tensor, frequencies: Tensor, out: Tensor) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_rmsnorm_rope(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1),
            rstd.data_ptr() if rstd is not None else None, out.data_ptr(), out.stride(0), positions.data_ptr(),
            int(positions.dtype == torch.float32), frequencies.data_ptr(), M, N, K, status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_rmsnorm_rope",
    )


@torch.library.custom_op("coda_b200::rope_bwd_zdz_out", mutates_args=("dz", "zdz"), device_types="cuda")
def _rope_bwd_zdz_out(y: Tensor, dy: Tensor, pos: Tensor, freq: Tensor, scale: float, dz: Tensor, zdz: Tensor) -> None:
    M, N = y.shape
    check(
        lib.coda_b200_rope_bwd_zdz(
            y.data_ptr(), y.stride(0), dy.data_ptr(), dy.stride(0), pos.data_ptr(), int(pos.dtype == torch.float32),
            freq.data_ptr(), float(scale), dz.data_ptr(), dz.stride(0), zdz.data_ptr(), M, N, _stream(y),
        ),
        "rope_bwd_zdz",
    )


@torch.library.custom_op(
    "coda_b200::gemm_rmsnorm_ce_out", mutates_args=("probs", "part_max", "part_sum", "part_sz", "target_logit", "lse", "losses", "zdz"),
    device_types="cuda",
)
def _gemm_rmsnorm_ce_out(A: Tensor, B: Tensor, rstd: Tensor, target: Tensor, ignore_index: int, probs: Tensor, part_max: Tensor,
                         part_sum: Tensor, part_sz: Tensor, target_logit: Tensor, lse: Tensor, losses: Tensor, zdz: Tensor) -> None:
    M, K = A.shape
    N = B.shape[1]
    st = _stream(A)
    check(
        lib.coda_b200_gemm_rmsnorm_lse_zdz(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), rstd.data_ptr(), probs.data_ptr(),
            probs.stride(0), part_max.data_ptr(), part_sum.data_ptr(), part_sz.data_ptr(), target.data_ptr(), target_logit.data_ptr(),
            M, N, K, status_word(A.device).data_ptr(), st,
        ),
        "gemm_rmsnorm_lse_zdz",
    )
    check(
        lib.coda_b200_lse_finalize_zdz(
            part_max.data_ptr(), part_sum.data_ptr(), part_sz.data_ptr(), part_max.shape[1], target.data_ptr(),
            target_logit.data_ptr(), ignore_index, lse.data_ptr(), losses.data_ptr(), zdz.data_ptr(), M, st,
        ),
        "lse_finalize_zdz",
    )
    check(
        lib.coda_b200_ce_grad_fixup(
            probs.data_ptr(), probs.stride(0), part_max.data_ptr(), part_max.shape[1], lse.data_ptr(), target.data_ptr(),
            ignore_index, M, N, st,
        ),
        "ce_grad_fixup",
    )


for _op in (_partial_rmsnorm_out, _gemm_rmsnorm_rope_out, _rope_bwd_zdz_out, _gemm_rmsnorm_ce_out):
    _op.register_fake(_noop_fake)


def partial_rmsnorm(x: Tensor, weight: Tensor, eps: float) -> tuple[Tensor, Tensor, Tensor]:
    """``(residual, h, rstd)``: a copy of ``x``, ``h = x * weight`` and ``rstd = rsqrt(mean(x^2) + eps)`` from one read of ``x``."""
    _require_cuda_bf16(x, weight)
    _require(x.dim() == 2 and x.stride(1) == 1 and weight.numel() == x.shape[1], "x must be [M, N] row-major, weight [N]")
    residual = torch.empty_like(x)
    h = torch.empty_like(x)
    rstd = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    _partial_rmsnorm_out(x, weight.contiguous(), float(eps), residual, h, rstd)
    return residual, h, rstd


def gemm_rmsnorm_rope(A: Tensor, B: Tensor, rstd: Optional[Tensor], positions: Tensor, frequencies: Tensor,
                      out: Optional[Tensor] = None) -> Tensor:
    """``rotate((A @ B) * rstd[:, None])`` over every adjacent column pair; ``frequencies`` has one entry per column
    (zero on the v columns, which therefore pass through)."""
    _require_cuda_bf16(A, B)
    M, N = A.shape[0], B.shape[1]
    _require(N % 2 == 0 and positions.numel() == M and positions.dtype in (torch.int32, torch.float32), "bad positions / N")
    _require(frequencies.dtype == torch.float32 and frequencies.numel() == N, "frequencies must be fp32 [N]")
    out = torch.empty(M, N, dtype=A.dtype, device=A.device) if out is None else out
    _gemm_rmsnorm_rope_out(A, B, rstd, positions.contiguous(), frequencies.contiguous(), out)
    return out


def rope_bwd_zdz(y: Tensor, dy: Tensor, pos: Tensor, freq: Tensor, scale: float = 1.0) -> tuple[Tensor, Tensor]:
    """``(dz, zdz)``: the gradient rotated back and ``scale * sum(y * dy, dim=1)`` (= ``scale * sum(z * dz)``, rotations being orthogonal)."""
    _require_cuda_bf16(y, dy)
    _require(y.shape == dy.shape and y.stride(1) == 1 and dy.stride(1) == 1, "y and dy must be row-major and of one shape")
    dz = torch.empty_like(y)
    zdz = torch.empty(y.shape[0], dtype=torch.float32, device=y.device)
    _rope_bwd_zdz_out(y, dy, pos.contiguous(), freq.contiguous(), float(scale), dz, zdz)
    return dz, zdz


def gemm_rmsnorm_cross_entropy_fwd_bwd(A: Tensor, B: Tensor, rstd: Tensor, target: Tensor, ignore_index: int,
                                       return_zdz: bool = True) -> tuple[Tensor, Tensor, Optional[Tensor]]:
    """LM head + cross entropy on ``rmsnorm``-deferred input: per-row ``losses``, bf16 ``dlogits = softmax - onehot`` (zero for
    ignored rows) and ``zdz = sum(logits * dlogits, dim=1)`` taken in fp32 inside the GEMM epilogue; the logits are never stored."""
    _require_cuda_bf16(A, B)
    _require(target.dtype == torch.int32 and target.is_contiguous(), "target must be contiguous int32")
    M, N = A.shape[0], B.shape[1]
    tiles = lse_tiles(N)
    f32 = dict(dtype=torch.float32, device=A.device)
    probs = torch.empty(M, N, dtype=A.dtype, device=A.device)
    part_max, part_sum, part_sz = (torch.empty(M, tiles, **f32) for _ in range(3))
    target_logit = torch.zeros(M, **f32)
    lse, losses, zdz = (torch.empty(M, **f32) for _ in range(3))
    _gemm_rmsnorm_ce_out(A, B, rstd.contiguous(), target, int(ignore_index), probs, part_max, part_sum, part_sz, target_logit, lse,
                         losses, zdz)
    return losses, probs, (zdz if return_zdz else None)


def reduce_losses(losses: Tensor, target: Tensor, ignore_index: int, reduction: str) -> tuple[Tensor, Optional[Tensor]]:
    """``(loss, scale)``: the sum of the per-row losses, divided by the number of non-ignored rows for ``"mean"``
    (``scale = 1 / count`` stays on the device), as ``LinearCrossEntropy.forward`` does (cross_entropy.py:122-127)."""
    assert reduction in ("mean", "sum")
    if reduction == "mean":
        scale = 1.0 / (target != ignore_index).sum().float()
        return losses.sum() * scale, scale
    return losses.sum(), None
