"""``linear_sigmoid_glu``: ``sigmoid(x @ W_gate^T) * (x @ W_val^T)`` with one interleaved weight.

An extension with no counterpart in the reference, whose ``linear_sigmoid`` has no value branch
(coda/kernels/functional/sigmoid.py:12-28): it is the "gated projection" reading of the sigmoid benchmark configuration.
``weight`` is ``[2N, K]`` with gate row ``j`` at ``2j`` and value row ``j`` at ``2j+1``, as ``linear_swiglu`` lays out
its weight; the structure of forward and backward is that of ``linear_swiglu`` with the gate's activation swapped.
"""

import torch
from torch import Tensor

from .._guards import autocast_custom_bwd, autocast_custom_fwd, input_guard
from .._lib import check, lib
from ..ops import _noop_fake, _require, _require_cuda_bf16, _stream, gemm, status_word


@torch.library.custom_op("coda_b200::gemm_sigmoid_glu_out", mutates_args=("preact", "postact"), device_types="cuda")
def _gemm_sigmoid_glu_out(A: Tensor, B: Tensor, preact: Tensor, postact: Tensor) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_sigmoid_glu(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), preact.data_ptr(), preact.stride(0),
            postact.data_ptr(), postact.stride(0), M, N, K, status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_sigmoid_glu",
    )


@torch.library.custom_op("coda_b200::dsigmoid_glu_out", mutates_args=("grad_pre",), device_types="cuda")
def _dsigmoid_glu_out(preact: Tensor, dout: Tensor, grad_pre: Tensor) -> None:
    M, F = dout.shape
    check(
        lib.coda_b200_dsigmoid_glu(preact.data_ptr(), preact.stride(0), dout.data_ptr(), dout.stride(0), grad_pre.data_ptr(),
                                   grad_pre.stride(0), M, F, _stream(dout)),
        "dsigmoid_glu",
    )


_gemm_sigmoid_glu_out.register_fake(_noop_fake)
_dsigmoid_glu_out.register_fake(_noop_fake)


class LinearSigmoidGLU(torch.autograd.Function):
    @staticmethod
    @input_guard
    @autocast_custom_fwd
    def forward(ctx, x: Tensor, weight: Tensor) -> Tensor:
        _require_cuda_bf16(x, weight)
        _require(weight.shape[0] % 2 == 0, "weight must hold interleaved (gate, value) rows")
        M, N = x.shape[0], weight.shape[0]
        preact = torch.empty(M, N, dtype=x.dtype, device=x.device)
        out = torch.empty(M, N // 2, dtype=x.dtype, device=x.device)
        _gemm_sigmoid_glu_out(x, weight.mT, preact, out)
        ctx.save_for_backward(x, weight, preact)
        return out

    @staticmethod
    @input_guard
    @autocast_custom_bwd
    def backward(ctx, dout: Tensor):
        x, weight, preact = ctx.saved_tensors
        grad_pre = torch.empty_like(preact)
        _dsigmoid_glu_out(preact, dout, grad_pre)
        return gemm(grad_pre, weight), gemm(grad_pre.mT, x)


def linear_sigmoid_glu(x: Tensor, weight: Tensor) -> Tensor:
    return LinearSigmoidGLU.apply(x, weight)
