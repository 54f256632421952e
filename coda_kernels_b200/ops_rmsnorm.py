"""Deferred-RMSNorm variants of the fused GEMMs: the accumulator is scaled by a per-row fp32 ``rstd`` first.

They stand in for ``gemm_rmsnorm_swiglu``, ``gemm_rmsnorm_lse`` and the ``rstd`` form of ``gemm_qknorm_rope``
(coda/core/gemm/functional.py:283-334, 392-450; coda/core/gemm/epilogues.py:262-303), which the reference's fused
transformer blocks call with ``rstd = rsqrt(mean(x^2) + eps)`` so that the normalisation of ``x`` never has to be
materialised.  Same custom-op conventions as :mod:`coda_kernels_b200.ops`.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ._lib import check, lib
from .ops import _aligned16, _ce_grad_fixup, _noop_fake, _require, _require_cuda_bf16, _stream, lse_finalize, lse_tiles, status_word


def _check_rstd(rstd: Tensor, M: int) -> None:
    _require(rstd.dtype == torch.float32 and rstd.is_cuda and rstd.is_contiguous() and tuple(rstd.shape) == (M,),
             "rstd must be a contiguous fp32 CUDA tensor with one entry per row")


@torch.library.custom_op("coda_b200::gemm_rmsnorm_swiglu_out", mutates_args=("preact", "postact"), device_types="cuda")
def _gemm_rmsnorm_swiglu_out(A: Tensor, B: Tensor, rstd: Tensor, preact: Tensor, postact: Tensor) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_rmsnorm_swiglu(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), rstd.data_ptr(), preact.data_ptr(),
            preact.stride(0), postact.data_ptr(), postact.stride(0), M, N, K, status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_rmsnorm_swiglu",
    )


@torch.library.custom_op(
    "coda_b200::gemm_rmsnorm_lse_out", mutates_args=("probs", "part_max", "part_sum", "target_logit"), device_types="cuda"
)
def _gemm_rmsnorm_lse_out(
    A: Tensor, B: Tensor, rstd: Tensor, probs: Optional[Tensor], part_max: Tensor, part_sum: Tensor, target: Tensor,
    target_logit: Tensor,
) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_rmsnorm_lse(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), rstd.data_ptr(),
            probs.data_ptr() if probs is not None else None, probs.stride(0) if probs is not None else 0,
            part_max.data_ptr(), part_sum.data_ptr(), target.data_ptr(), target_logit.data_ptr(), M, N, K,
            status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_rmsnorm_lse",
    )


@torch.library.custom_op(
    "coda_b200::gemm_rmsnorm_qknorm_rope_out", mutates_args=("qk", "preact", "v", "mean_sq"), device_types="cuda"
)
def _gemm_rmsnorm_qknorm_rope_out(
    A: Tensor, B: Tensor, rstd: Tensor, qk: Tensor, preact: Tensor, v: Optional[Tensor], mean_sq: Tensor, gamma: Tensor,
    positions: Tensor, frequencies: Tensor, head_dim: int, num_heads_q: int, num_heads_k: int, eps: float,
) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_rmsnorm_qknorm_rope(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), rstd.data_ptr(), qk.data_ptr(),
            qk.stride(0), preact.data_ptr(), preact.stride(0), v.data_ptr() if v is not None else None,
            v.stride(0) if v is not None else 0, mean_sq.data_ptr(), gamma.data_ptr(), positions.data_ptr(),
            int(positions.dtype == torch.float32), frequencies.data_ptr(), head_dim, num_heads_q, num_heads_k, float(eps), M, N, K,
            status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_rmsnorm_qknorm_rope",
    )


for _op in (_gemm_rmsnorm_swiglu_out, _gemm_rmsnorm_lse_out, _gemm_rmsnorm_qknorm_rope_out):
    _op.register_fake(_noop_fake)


def gemm_rmsnorm_swiglu(A: Tensor, B: Tensor, rstd: Tensor) -> tuple[Tensor, Tensor]:
    """``preact = bf16((A @ B) * rstd[:, None])`` and ``postact = swiglu(preact pairs)`` from the unrounded scaled values."""
    _require_cuda_bf16(A, B)
    M, N = A.shape[0], B.shape[1]
    _require(N % 2 == 0, "gemm_rmsnorm_swiglu: N must be even")
    _check_rstd(rstd, M)
    preact = torch.empty(M, N, dtype=A.dtype, device=A.device)
    postact = torch.empty(M, N // 2, dtype=A.dtype, device=A.device)
    _gemm_rmsnorm_swiglu_out(A, B, rstd, preact, postact)
    return preact, postact


def _rmsnorm_lse_partials(A: Tensor, B: Tensor, rstd: Tensor, target: Tensor, store_probs: bool):
    _require_cuda_bf16(A, B)
    _require(target.dtype == torch.int32 and target.is_cuda and target.is_contiguous(), "target must be a contiguous int32 CUDA tensor")
    M, N = A.shape[0], B.shape[1]
    _check_rstd(rstd, M)
    tiles = lse_tiles(N)
    probs = torch.empty(M, N, dtype=A.dtype, device=A.device) if store_probs else None
    part_max = torch.empty(M, tiles, dtype=torch.float32, device=A.device)
    part_sum = torch.empty(M, tiles, dtype=torch.float32, device=A.device)
    target_logit = torch.zeros(M, dtype=torch.float32, device=A.device)
    _gemm_rmsnorm_lse_out(A, B, rstd, probs, part_max, part_sum, target, target_logit)
    return probs, part_max, part_sum, target_logit


def gemm_rmsnorm_lse_select_logits(A: Tensor, B: Tensor, rstd: Tensor, target: Tensor, ignore_index: int) -> tuple[Tensor, Tensor, Tensor]:
    """Per-row ``(loss, lse, target_logit)`` of the logits ``(A @ B) * rstd[:, None]``; nothing of size [M, N] is stored."""
    _, part_max, part_sum, target_logit = _rmsnorm_lse_partials(A, B, rstd, target, store_probs=False)
    lse, losses = lse_finalize(part_max, part_sum, target, target_logit, ignore_index)
    return losses, lse, target_logit


def gemm_rmsnorm_lse_dlogits(A: Tensor, B: Tensor, rstd: Tensor, target: Tensor, ignore_index: int) -> tuple[Tensor, Tensor, Tensor]:
    """``(losses, lse, dlogits)``: per-row loss, log-sum-exp, and ``softmax - onehot`` of the scaled logits (bf16, zero for ignored rows)."""
    probs, part_max, part_sum, target_logit = _rmsnorm_lse_partials(A, B, rstd, target, store_probs=True)
    lse, losses = lse_finalize(part_max, part_sum, target, target_logit, ignore_index)
    _ce_grad_fixup(probs, part_max, lse, target, int(ignore_index))
    return losses, lse, probs


def gemm_rmsnorm_qknorm_rope(
    A: Tensor, B: Tensor, rstd: Tensor, weight: Tensor, positions: Tensor, frequencies: Tensor, head_dim: int, num_heads_q: int,
    num_heads_k: int, eps: float,
) -> tuple[Tensor, Tensor, Tensor, Optional[Tensor]]:
    """``(qk, preact, head_mean_sq, v)`` with the q, k, v projections of ``rmsnorm(x)``: ``preact`` keeps the unscaled
    accumulator (the backward recovers the scaled value as ``rstd * preact``), ``head_mean_sq`` is that of the scaled head."""
    _require_cuda_bf16(A, B, weight)
    _require(positions.dtype in (torch.int32, torch.float32), "positions must be int32 or float32")
    _require(frequencies.dtype == torch.float32, "frequencies must be float32")
    M, N = A.shape[0], B.shape[1]
    _check_rstd(rstd, M)
    heads = num_heads_q + num_heads_k
    size_qk = heads * head_dim
    _require(weight.numel() == 2 * head_dim and frequencies.numel() == size_qk and positions.numel() == M, "bad gamma / frequencies / positions")
    qk = torch.empty(M, size_qk, dtype=A.dtype, device=A.device)
    preact = torch.empty(M, size_qk, dtype=A.dtype, device=A.device)
    mean_sq = torch.empty(M, heads, dtype=torch.float32, device=A.device)
    v = torch.empty(M, N - size_qk, dtype=A.dtype, device=A.device) if N > size_qk else None
    _gemm_rmsnorm_qknorm_rope_out(
        A, B, rstd, qk, preact, v, mean_sq, _aligned16(weight), positions.contiguous(), _aligned16(frequencies), head_dim,
        num_heads_q, num_heads_k, float(eps),
    )
    return qk, preact, mean_sq, v
