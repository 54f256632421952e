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
