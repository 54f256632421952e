"""The reference's own cross-entropy dataflow, kept for callers that want the logits in memory.

``gemm_lse`` and ``cross_entropy_fwd_bwd`` have the signatures and semantics of the reference ops
(coda/core/gemm/functional.py:371-389; coda/core/elementwise/functional.py:286-311), so the reference's
``_forward_lse`` (coda/kernels/functional/cross_entropy.py:25-47) runs on them unchanged.
``coda_kernels_b200.functional.cross_entropy`` does not use them: it stores probabilities instead of logits.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ._lib import check, lib
from .ops import _noop_fake, _require, _require_cuda_bf16, _stream, lse_tiles, status_word


@torch.library.custom_op("coda_b200::gemm_lse_logits_out", mutates_args=("logits", "part_max", "part_sum"), device_types="cuda")
def _gemm_lse_logits_out(A: Tensor, B: Tensor, rstd: Optional[Tensor], logits: Tensor, part_max: Tensor, part_sum: Tensor) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_lse_logits(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1),
            rstd.data_ptr() if rstd is not None else None, logits.data_ptr(), logits.stride(0), part_max.data_ptr(),
            part_sum.data_ptr(), M, N, K, status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_lse_logits",
    )


@torch.library.custom_op("coda_b200::lse_reduce_out", mutates_args=("lse",), device_types="cuda")
def _lse_reduce_out(part_max: Tensor, part_sum: Tensor, lse: Tensor) -> None:
    M, tiles = part_max.shape
    check(lib.coda_b200_lse_reduce(part_max.data_ptr(), part_sum.data_ptr(), tiles, lse.data_ptr(), M, _stream(part_max)), "lse_reduce")


@torch.library.custom_op("coda_b200::cross_entropy_fwd_bwd_", mutates_args=("logits", "losses"), device_types="cuda")
def _cross_entropy_fwd_bwd(logits: Tensor, lses: Tensor, target: Tensor, ignore_index: int, losses: Tensor) -> None:
    M, N = logits.shape
    check(
        lib.coda_b200_cross_entropy_fwd_bwd(
            logits.data_ptr(), logits.stride(0), lses.data_ptr(), target.data_ptr(), ignore_index, losses.data_ptr(), M, N,
            _stream(logits),
        ),
        "cross_entropy_fwd_bwd",
    )


for _op in (_gemm_lse_logits_out, _lse_reduce_out, _cross_entropy_fwd_bwd):
    _op.register_fake(_noop_fake)


def gemm_lse(A: Tensor, B: Tensor, rstd: Optional[Tensor] = None) -> tuple[Tensor, Tensor]:
    """``(logits, lses)``: bf16 logits ``A @ B`` (times ``rstd[:, None]`` if given) and each row's fp32 log-sum-exp,
    reduced from per-tile partials taken on the unrounded accumulator."""
    _require_cuda_bf16(A, B)
    M, N = A.shape[0], B.shape[1]
    if rstd is not None:
        _require(rstd.dtype == torch.float32 and tuple(rstd.shape) == (M,) and rstd.is_contiguous(), "rstd must be contiguous fp32 [M]")
    logits = torch.empty(M, N, dtype=A.dtype, device=A.device)
    tiles = lse_tiles(N)
    part_max = torch.empty(M, tiles, dtype=torch.float32, device=A.device)
    part_sum = torch.empty(M, tiles, dtype=torch.float32, device=A.device)
    lses = torch.empty(M, dtype=torch.float32, device=A.device)
    _gemm_lse_logits_out(A, B, rstd, logits, part_max, part_sum)
    _lse_reduce_out(part_max, part_sum, lses)
    return logits, lses


def cross_entropy_fwd_bwd(logits: Tensor, lses: Tensor, target: Tensor, ignore_index: int) -> tuple[Tensor, Tensor]:
    """In place: ``logits`` becomes ``softmax - onehot`` (zero rows where ``target == ignore_index``).  Returns
    ``(losses, logits)`` with ``losses[i] = lses[i] - logit[i, target[i]]`` (0 for ignored rows)."""
    _require_cuda_bf16(logits)
    _require(logits.dim() == 2 and logits.stride(1) == 1, "logits must be a row-major matrix")
    _require(target.dtype == torch.int32 and target.is_contiguous() and lses.dtype == torch.float32 and lses.is_contiguous(),
             "target must be contiguous int32, lses contiguous fp32")
    losses = torch.zeros(logits.shape[0], dtype=torch.float32, device=logits.device)
    _cross_entropy_fwd_bwd(logits, lses, target, int(ignore_index), losses)
    return losses, logits
