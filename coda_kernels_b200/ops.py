"""Device operators: ``torch.library`` custom ops over the C ABI of ``libcoda_b200.so``.

This is the layer that stands in for ``coda/core/gemm/functional.py`` and
``coda/core/elementwise/functional.py`` of the reference: every device op is a
mutating custom op that returns ``None`` (outputs are allocated by the Python
wrapper and passed in), with a no-op fake implementation so that the ops trace
under ``torch.compile(fullgraph=True)`` — the convention of
``coda/core/gemm/gemm_interface.py:78-100``.  PyTorch only provides device
memory and the current stream; all arithmetic runs in the library's kernels.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
from torch import Tensor

from . import _lib as _lib_module
from ._lib import check, lib

_BF16 = torch.bfloat16
_status_words: dict[int, Tensor] = {}
_status_views: dict[int, ctypes.c_int] = {}


def status_word(device: torch.device) -> Tensor:
    """Per-device int32 word that kernels set when a bounded wait expires.

    It lives in pinned host memory, which the device maps at the same address: a kernel writes it only on its failure
    path (one store over PCIe), and the host sees the code by reading the word, without a copy, a stream operation or
    any CUDA call.  That is what makes the check cheap enough to run in every operator call."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(idx)
    if word is None:
        with torch.cuda.device(idx):
            word = torch.zeros(1, dtype=torch.int32).pin_memory()
        _status_words[idx] = word
        _status_views[idx] = ctypes.c_int.from_address(word.data_ptr())
    return word


def check_device_status(device: Optional[torch.device] = None) -> None:
    """Wait for the device, then read the status word; raise if any kernel reported trouble."""
    device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    word = status_word(device)
    torch.cuda.synchronize(device)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise RuntimeError(f"coda_b200 kernel reported device-side error code {code} (a bounded wait expired)")


def lazy_status_check(device: Optional[torch.device] = None) -> None:
    """Report an expired device-side wait without synchronising.

    Called at the start of every operator's forward and backward: a plain read of the status word in pinned host
    memory.  A kernel that gave up is therefore reported by the first operator call after its launch has finished,
    typically the backward of the same step, instead of yielding silent garbage for the rest of a training run.  It
    costs no CUDA call and enqueues nothing, so it also runs while a CUDA graph is being captured; it is skipped
    while ``torch.compile`` traces the caller.
    """
    if torch.compiler.is_compiling():
        return
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    view = _status_views.get(idx)
    if view is None:
        status_word(torch.device("cuda", idx))
        view = _status_views[idx]
    code = view.value
    if code != 0:
        view.value = 0
        raise RuntimeError(
            f"coda_b200: a kernel on cuda:{idx} reported device-side error code {code} (a bounded wait expired); "
            "the outputs of that launch are incomplete")


def _sync_status_hook(what: str) -> None:
    torch.cuda.synchronize()
    for idx, word in list(_status_words.items()):
        code = int(word.item())
        if code != 0:
            word.zero_()
            raise RuntimeError(f"coda_b200: device-side error code {code} on cuda:{idx}, detected after {what}")


if os.environ.get("CODA_B200_SYNC_STATUS", "0") == "1":
    _lib_module.post_call_hook = _sync_status_hook


def _stream(t: Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _require_cuda_bf16(*tensors: Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("coda_b200 operators run on CUDA tensors only; there is no CPU fallback")
        if t.dtype != _BF16:
            raise NotImplementedError(f"coda_b200 operators take bfloat16 matrices, got {t.dtype}")


def _noop_fake(*args, **kwargs) -> None:
    return None


# ------------------------------------------------------------------------------------------------ custom ops


@torch.library.custom_op("coda_b200::gemm_out", mutates_args=("out",), device_types="cuda")
def _gemm_out(A: Tensor, B: Tensor, out: Tensor, alpha: Optional[Tensor], C: Optional[Tensor] = None) -> None:
    M, K = A.shape
    N = B.shape[1]
    if C is None:
        # a plain product may have its last round cut along K: the library says whether it wants the fp32 workspace
        ws_bytes = int(lib.coda_b200_gemm_workspace_bytes(M, N, K))
        ws = torch.empty(ws_bytes // 4, dtype=torch.float32, device=A.device) if ws_bytes > 0 else None
        check(
            lib.coda_b200_gemm_ws(
                A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), out.data_ptr(), out.stride(0),
                int(out.dtype == torch.float32), M, N, K, alpha.data_ptr() if alpha is not None else None,
                ws.data_ptr() if ws is not None else None, ws_bytes, status_word(A.device).data_ptr(), _stream(A),
            ),
            "gemm",
        )
        return
    check(
        lib.coda_b200_gemm_add(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1),
            C.data_ptr() if C is not None else None, C.stride(0) if C is not None else 0,
            int(C is not None and C.dtype == torch.float32), out.data_ptr(), out.stride(0),
            int(out.dtype == torch.float32), M, N, K, alpha.data_ptr() if alpha is not None else None,
            status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm",
    )


@torch.library.custom_op("coda_b200::gemm_sigmoid_out", mutates_args=("out",), device_types="cuda")
def _gemm_sigmoid_out(A: Tensor, B: Tensor, out: Tensor) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_sigmoid(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), out.data_ptr(), out.stride(0),
            int(out.dtype == torch.float32), M, N, K, status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_sigmoid",
    )


@torch.library.custom_op("coda_b200::gemm_swiglu_out", mutates_args=("preact", "postact"), device_types="cuda")
def _gemm_swiglu_out(A: Tensor, B: Tensor, preact: Tensor, postact: Tensor) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_swiglu(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), preact.data_ptr(),
            preact.stride(0), postact.data_ptr(), postact.stride(0), M, N, K, status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_swiglu",
    )


@torch.library.custom_op(
    "coda_b200::gemm_lse_out", mutates_args=("probs", "part_max", "part_sum", "target_logit"), device_types="cuda"
)
def _gemm_lse_out(
    A: Tensor, B: Tensor, probs: Optional[Tensor], part_max: Tensor, part_sum: Tensor, target: Tensor, target_logit: Tensor
) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_lse(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1),
            probs.data_ptr() if probs is not None else None, probs.stride(0) if probs is not None else 0,
            part_max.data_ptr(), part_sum.data_ptr(), target.data_ptr(), target_logit.data_ptr(), M, N, K,
            status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_lse",
    )


@torch.library.custom_op("coda_b200::lse_finalize_out", mutates_args=("lse", "losses"), device_types="cuda")
def _lse_finalize_out(
    part_max: Tensor, part_sum: Tensor, target: Tensor, target_logit: Tensor, ignore_index: int, lse: Tensor, losses: Tensor
) -> None:
    M, tiles = part_max.shape
    check(
        lib.coda_b200_lse_finalize(
            part_max.data_ptr(), part_sum.data_ptr(), tiles, target.data_ptr(), target_logit.data_ptr(), ignore_index,
            lse.data_ptr(), losses.data_ptr(), M, _stream(part_max),
        ),
        "lse_finalize",
    )


@torch.library.custom_op("coda_b200::ce_grad_fixup_", mutates_args=("probs",), device_types="cuda")
def _ce_grad_fixup(probs: Tensor, part_max: Tensor, lse: Tensor, target: Tensor, ignore_index: int) -> None:
    M, N = probs.shape
    check(
        lib.coda_b200_ce_grad_fixup(
            probs.data_ptr(), probs.stride(0), part_max.data_ptr(), part_max.shape[1], lse.data_ptr(), target.data_ptr(),
            ignore_index, M, N, _stream(probs),
        ),
        "ce_grad_fixup",
    )


@torch.library.custom_op(
    "coda_b200::gemm_qknorm_rope_out", mutates_args=("qk", "preact", "v", "mean_sq"), device_types="cuda"
)
def _gemm_qknorm_rope_out(
    A: Tensor, B: Tensor, qk: Tensor, preact: Tensor, v: Optional[Tensor], mean_sq: Tensor, gamma: Tensor, positions: Tensor,
    frequencies: Tensor, head_dim: int, num_heads_q: int, num_heads_k: int, eps: float,
) -> None:
    M, K = A.shape
    N = B.shape[1]
    check(
        lib.coda_b200_gemm_qknorm_rope(
            A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1), qk.data_ptr(), qk.stride(0),
            preact.data_ptr(), preact.stride(0), v.data_ptr() if v is not None else None, v.stride(0) if v is not None else 0,
            mean_sq.data_ptr(), gamma.data_ptr(), positions.data_ptr(), int(positions.dtype == torch.float32),
            frequencies.data_ptr(), head_dim, num_heads_q, num_heads_k, float(eps), M, N, K,
            status_word(A.device).data_ptr(), _stream(A),
        ),
        "gemm_qknorm_rope",
    )


@torch.library.custom_op("coda_b200::dswiglu_out", mutates_args=("grad_pre",), device_types="cuda")
def _dswiglu_out(preact: Tensor, dout: Tensor, grad_pre: Tensor) -> None:
    M, F = dout.shape
    check(
        lib.coda_b200_dswiglu(
            preact.data_ptr(), preact.stride(0), dout.data_ptr(), dout.stride(0), grad_pre.data_ptr(), grad_pre.stride(0), M, F,
            _stream(dout),
        ),
        "dswiglu",
    )


@torch.library.custom_op("coda_b200::dsigmoid_out", mutates_args=("grad_pre",), device_types="cuda")
def _dsigmoid_out(out: Tensor, dout: Tensor, grad_pre: Tensor) -> None:
    M, N = dout.shape
    check(
        lib.coda_b200_dsigmoid(
            out.data_ptr(), out.stride(0), int(out.dtype == torch.float32), dout.data_ptr(), dout.stride(0),
            grad_pre.data_ptr(), grad_pre.stride(0), M, N, _stream(dout),
        ),
        "dsigmoid",
    )


@torch.library.custom_op("coda_b200::qknorm_rope_bwd_out", mutates_args=("grad", "dgamma", "scratch"), device_types="cuda")
def _qknorm_rope_bwd_out(
    dq: Tensor, dk: Tensor, dv: Optional[Tensor], preact: Tensor, mean_sq: Tensor, gamma: Tensor, positions: Tensor,
    frequencies: Tensor, head_dim: int, num_heads_q: int, num_heads_k: int, eps: float, grad: Tensor, dgamma: Tensor,
    scratch: Tensor,
) -> None:
    M = preact.shape[0]
    check(
        lib.coda_b200_qknorm_rope_bwd(
            dq.data_ptr(), dq.stride(0), dk.data_ptr(), dk.stride(0), dv.data_ptr() if dv is not None else None,
            dv.stride(0) if dv is not None else 0, dv.shape[1] if dv is not None else 0, preact.data_ptr(), preact.stride(0),
            mean_sq.data_ptr(), gamma.data_ptr(), positions.data_ptr(), int(positions.dtype == torch.float32),
            frequencies.data_ptr(), head_dim, num_heads_q, num_heads_k, float(eps), grad.data_ptr(), grad.stride(0),
            dgamma.data_ptr(), scratch.data_ptr(), scratch.numel() * scratch.element_size(), M, _stream(preact),
        ),
        "qknorm_rope_bwd",
    )


@torch.library.custom_op("coda_b200::gemm_dsigmoid_dgrad_out", mutates_args=("grad_pre", "dx"), device_types="cuda")
def _gemm_dsigmoid_dgrad_out(out: Tensor, dout: Tensor, weight: Tensor, grad_pre: Tensor, dx: Tensor) -> None:
    M, N = out.shape
    K = weight.shape[1]
    check(
        lib.coda_b200_gemm_dsigmoid_dgrad(
            out.data_ptr(), out.stride(0), dout.data_ptr(), dout.stride(0), weight.data_ptr(), weight.stride(0),
            grad_pre.data_ptr(), grad_pre.stride(0), dx.data_ptr(), dx.stride(0), M, N, K, status_word(out.device).data_ptr(),
            _stream(out),
        ),
        "gemm_dsigmoid_dgrad",
    )


for _op in (
    _gemm_out, _gemm_sigmoid_out, _gemm_swiglu_out, _gemm_lse_out, _lse_finalize_out, _ce_grad_fixup, _gemm_qknorm_rope_out,
    _dswiglu_out, _dsigmoid_out, _qknorm_rope_bwd_out, _gemm_dsigmoid_dgrad_out,
):
    _op.register_fake(_noop_fake)


# ------------------------------------------------------------------------------------------------ compiled dispatch
# The same ten device operators registered from C++ (csrc_torch/torch_binding.cpp, namespace ``coda_b200n``): a
# TORCH_LIBRARY shim over the same C ABI that skips the per-launch Python work of the ctypes ops above.  Eager calls
# go through it; while ``torch.compile`` traces, the Python custom ops above are used (opaque to the tracer, and
# dispatch cost is irrelevant there).  ``CODA_B200_DISPATCH=ctypes`` keeps every call on the ctypes binding.
# The same library also holds one entry point per direction of each operator (see "whole operators" at the end).
_native = None
if os.environ.get("CODA_B200_DISPATCH", "native") != "ctypes":
    if not _lib_module.NATIVE_LIB_PATH.exists():
        raise ImportError(
            f"{_lib_module.NATIVE_LIB_PATH} is missing: build it with `python -m coda_kernels_b200.build` "
            "(or set CODA_B200_DISPATCH=ctypes to use the ctypes binding of the same kernels)")
    torch.ops.load_library(str(_lib_module.NATIVE_LIB_PATH))
    _native = torch.ops.coda_b200n
    for _name in ("gemm_out", "gemm_sigmoid_out", "gemm_swiglu_out", "gemm_lse_out", "lse_finalize_out", "ce_grad_fixup_",
                  "gemm_qknorm_rope_out", "dswiglu_out", "dsigmoid_out", "qknorm_rope_bwd_out"):
        torch.library.register_fake(f"coda_b200n::{_name}")(_noop_fake)

    def _use_native() -> bool:
        return not torch.compiler.is_compiling()

    class _Native:
        """``torch.ops.coda_b200n`` with argument errors re-raised as the package's own exception type, so both bindings
        report a rejected call the same way."""

        def __getattr__(self, name):
            op = getattr(torch.ops.coda_b200n, name)

            def call(*args):
                try:
                    return op(*args)
                except RuntimeError as ex:
                    raise _lib_module.CodaB200Error(str(ex).split("\n")[0]) from None

            setattr(self, name, call)
            return call

    _native = _Native()
    _ct_gemm_out, _ct_gemm_sigmoid_out, _ct_gemm_swiglu_out, _ct_gemm_lse_out = _gemm_out, _gemm_sigmoid_out, _gemm_swiglu_out, _gemm_lse_out
    _ct_lse_finalize_out, _ct_ce_grad_fixup, _ct_gemm_qknorm_rope_out = _lse_finalize_out, _ce_grad_fixup, _gemm_qknorm_rope_out
    _ct_dswiglu_out, _ct_dsigmoid_out, _ct_qknorm_rope_bwd_out = _dswiglu_out, _dsigmoid_out, _qknorm_rope_bwd_out

    def _gemm_out(A, B, out, alpha, C=None):  # noqa: F811
        if _use_native():
            _native.gemm_out(A, B, out, alpha, C, status_word(A.device))
        else:
            _ct_gemm_out(A, B, out, alpha, C)

    def _gemm_sigmoid_out(A, B, out):  # noqa: F811
        if _use_native():
            _native.gemm_sigmoid_out(A, B, out, status_word(A.device))
        else:
            _ct_gemm_sigmoid_out(A, B, out)

    def _gemm_swiglu_out(A, B, preact, postact):  # noqa: F811
        if _use_native():
            _native.gemm_swiglu_out(A, B, preact, postact, status_word(A.device))
        else:
            _ct_gemm_swiglu_out(A, B, preact, postact)

    def _gemm_lse_out(A, B, probs, part_max, part_sum, target, target_logit):  # noqa: F811
        if _use_native():
            _native.gemm_lse_out(A, B, probs, part_max, part_sum, target, target_logit, status_word(A.device))
        else:
            _ct_gemm_lse_out(A, B, probs, part_max, part_sum, target, target_logit)

    def _lse_finalize_out(part_max, part_sum, target, target_logit, ignore_index, lse, losses):  # noqa: F811
        if _use_native():
            _native.lse_finalize_out(part_max, part_sum, target, target_logit, ignore_index, lse, losses)
        else:
            _ct_lse_finalize_out(part_max, part_sum, target, target_logit, ignore_index, lse, losses)

    def _ce_grad_fixup(probs, part_max, lse, target, ignore_index):  # noqa: F811
        if _use_native():
            _native.ce_grad_fixup_(probs, part_max, lse, target, ignore_index)
        else:
            _ct_ce_grad_fixup(probs, part_max, lse, target, ignore_index)

    def _gemm_qknorm_rope_out(A, B, qk, preact, v, mean_sq, gamma, positions, frequencies, head_dim, num_heads_q, num_heads_k, eps):  # noqa: F811
        if _use_native():
            _native.gemm_qknorm_rope_out(A, B, qk, preact, v, mean_sq, gamma, positions, frequencies, head_dim, num_heads_q,
                                         num_heads_k, eps, status_word(A.device))
        else:
            _ct_gemm_qknorm_rope_out(A, B, qk, preact, v, mean_sq, gamma, positions, frequencies, head_dim, num_heads_q, num_heads_k, eps)

    def _dswiglu_out(preact, dout, grad_pre):  # noqa: F811
        if _use_native():
            _native.dswiglu_out(preact, dout, grad_pre)
        else:
            _ct_dswiglu_out(preact, dout, grad_pre)

    def _dsigmoid_out(out, dout, grad_pre):  # noqa: F811
        if _use_native():
            _native.dsigmoid_out(out, dout, grad_pre)
        else:
            _ct_dsigmoid_out(out, dout, grad_pre)

    def _qknorm_rope_bwd_out(dq, dk, dv, preact, mean_sq, gamma, positions, frequencies, head_dim, num_heads_q, num_heads_k, eps,  # noqa: F811
                             grad, dgamma, scratch):
        if _use_native():
            _native.qknorm_rope_bwd_out(dq, dk, dv, preact, mean_sq, gamma, positions, frequencies, head_dim, num_heads_q, num_heads_k,
                                        eps, grad, dgamma, scratch)
        else:
            _ct_qknorm_rope_bwd_out(dq, dk, dv, preact, mean_sq, gamma, positions, frequencies, head_dim, num_heads_q, num_heads_k, eps,
                                    grad, dgamma, scratch)


# ------------------------------------------------------------------------------------------------ python wrappers


def gemm(A: Tensor, B: Tensor, out: Optional[Tensor] = None, alpha: Optional[Tensor] = None,
         out_dtype: Optional[torch.dtype] = None, C: Optional[Tensor] = None) -> Tensor:
    """``out = alpha * (A @ B) + C`` for ``A[M,K]``, ``B[K,N]`` (any mix of plain and ``.mT`` views).

    Counterpart of ``gemm`` / ``gemm_scalar_scale`` (coda/core/gemm/functional.py:54-69, 116-132).
    ``alpha`` is a 0-d or 1-element fp32 device tensor (no host sync).  ``C`` (bf16 or fp32, ``[M, N]``, row-major;
    it may be ``out`` itself) is added to the fp32 accumulator inside the same kernel.
    """
    _require_cuda_bf16(A, B)
    _require(A.dim() == 2 and B.dim() == 2 and A.shape[1] == B.shape[0], "gemm: A[M,K] @ B[K,N] expected")
    if out is None:
        out = torch.empty(A.shape[0], B.shape[1], dtype=out_dtype or A.dtype, device=A.device)
    _require(out.dtype in (_BF16, torch.float32), "gemm: out must be bfloat16 or float32")
    _require(out.dim() == 2 and out.stride(1) == 1 and tuple(out.shape) == (A.shape[0], B.shape[1]), "gemm: bad out")
    if alpha is not None:
        _require(alpha.dtype == torch.float32 and alpha.numel() == 1 and alpha.is_cuda, "gemm: alpha must be a 1-element fp32 CUDA tensor")
    if C is not None:
        _require(C.is_cuda and C.dtype in (_BF16, torch.float32) and tuple(C.shape) == tuple(out.shape) and C.stride(1) == 1,
                 "gemm: C must be a row-major bf16 or fp32 CUDA tensor of the output's shape")
    _gemm_out(A, B, out, alpha, C)
    return out


def gemm_scalar_scale(A: Tensor, B: Tensor, alpha: Tensor, out: Optional[Tensor] = None) -> Tensor:
    return gemm(A, B, out=out, alpha=alpha)


def gemm_sigmoid(A: Tensor, B: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """``sigmoid(A @ B)``; counterpart of coda/core/gemm/functional.py:220-234."""
    _require_cuda_bf16(A, B)
    if out is None:
        out = torch.empty(A.shape[0], B.shape[1], dtype=A.dtype, device=A.device)
    _require(out.dtype in (_BF16, torch.float32), "gemm_sigmoid: out must be bfloat16 or float32")
    _require(out.stride(1) == 1 and tuple(out.shape) == (A.shape[0], B.shape[1]), "gemm_sigmoid: bad out")
    _gemm_sigmoid_out(A, B, out)
    return out


def gemm_swiglu(A: Tensor, B: Tensor) -> tuple[Tensor, Tensor]:
    """``(preact, postact)`` with interleaved gate/up columns; counterpart of coda/core/gemm/functional.py:261-280."""
    _require_cuda_bf16(A, B)
    M, N = A.shape[0], B.shape[1]
    _require(N % 2 == 0, "gemm_swiglu: N must be even")
    preact = torch.empty(M, N, dtype=A.dtype, device=A.device)
    postact = torch.empty(M, N // 2, dtype=A.dtype, device=A.device)
    _gemm_swiglu_out(A, B, preact, postact)
    return preact, postact


# Tiling constants of the library, read once at import so that the wrappers below are plain Python arithmetic
# (traceable by torch.compile, which cannot look into ctypes calls).
_LSE_TILE_N = (1 << 20) // int(lib.coda_b200_lse_tiles(1 << 20))
_QK_BWD_ROWS_PER_BLOCK = (1 << 20) * 2 * 128 * 4 // int(lib.coda_b200_qknorm_rope_bwd_scratch_bytes(1 << 20, 128))


def lse_tiles(N: int) -> int:
    """Number of column tiles of the LSE epilogue (= ``coda_b200_lse_tiles(N)``)."""
    return (N + _LSE_TILE_N - 1) // _LSE_TILE_N


def gemm_lse_partials(A: Tensor, B: Tensor, target: Tensor, store_probs: bool) -> tuple[Optional[Tensor], Tensor, Tensor, Tensor]:
    """Run the LSE GEMM.  Returns ``(probs or None, part_max, part_sum, target_logit)``."""
    _require_cuda_bf16(A, B)
    _require(target.dtype == torch.int32 and target.is_cuda and target.is_contiguous(), "target must be a contiguous int32 CUDA tensor")
    M, N = A.shape[0], B.shape[1]
    tiles = lse_tiles(N)
    probs = torch.empty(M, N, dtype=A.dtype, device=A.device) if store_probs else None
    part_max = torch.empty(M, tiles, dtype=torch.float32, device=A.device)
    part_sum = torch.empty(M, tiles, dtype=torch.float32, device=A.device)
    target_logit = torch.zeros(M, dtype=torch.float32, device=A.device)
    _gemm_lse_out(A, B, probs, part_max, part_sum, target, target_logit)
    return probs, part_max, part_sum, target_logit


def lse_finalize(part_max: Tensor, part_sum: Tensor, target: Tensor, target_logit: Tensor, ignore_index: int) -> tuple[Tensor, Tensor]:
    M = part_max.shape[0]
    lse = torch.empty(M, dtype=torch.float32, device=part_max.device)
    losses = torch.empty(M, dtype=torch.float32, device=part_max.device)
    _lse_finalize_out(part_max, part_sum, target, target_logit, int(ignore_index), lse, losses)
    return lse, losses


_DEBUG_CHECKS = os.environ.get("CODA_B200_SYNC_STATUS", "0") == "1" or os.environ.get("CODA_B200_DEBUG", "0") == "1"


def _debug_check_targets(target: Tensor, num_classes: int, ignore_index: int) -> None:
    """Debug mode only (it synchronises): a label outside ``[0, num_classes)`` that is not ``ignore_index`` would pick no
    logit and give a silently wrong loss (the reference does not check either)."""
    if _DEBUG_CHECKS and not torch.compiler.is_compiling():
        bad = (target != ignore_index) & ((target < 0) | (target >= num_classes))
        if bool(bad.any()):
            raise ValueError(f"target holds labels outside [0, {num_classes}) that are not ignore_index={ignore_index}")


def gemm_lse_select_logits(A: Tensor, B: Tensor, target: Tensor, ignore_index: int) -> tuple[Tensor, Tensor, Tensor]:
    """Per-row ``(loss, lse, target_logit)`` without storing anything of size [M, N].

    Counterpart of ``gemm_lse_select_logits`` (coda/core/gemm/functional.py:496-527).
    """
    _debug_check_targets(target, B.shape[1], ignore_index)
    _, part_max, part_sum, target_logit = gemm_lse_partials(A, B, target, store_probs=False)
    lse, losses = lse_finalize(part_max, part_sum, target, target_logit, ignore_index)
    return losses, lse, target_logit


def gemm_lse_dlogits(A: Tensor, B: Tensor, target: Tensor, ignore_index: int) -> tuple[Tensor, Tensor]:
    """Per-row losses and the bf16 gradient of each row's loss w.r.t. the logits.

    Counterpart of ``gemm_lse`` + ``cross_entropy_fwd_bwd``
    (coda/kernels/functional/cross_entropy.py:25-47); the [M, N] buffer holds
    unnormalised probabilities first and the gradient after the in-place pass,
    never the logits.
    """
    _debug_check_targets(target, B.shape[1], ignore_index)
    probs, part_max, part_sum, target_logit = gemm_lse_partials(A, B, target, store_probs=True)
    lse, losses = lse_finalize(part_max, part_sum, target, target_logit, ignore_index)
    _ce_grad_fixup(probs, part_max, lse, target, int(ignore_index))
    return losses, probs


def _aligned16(t: Tensor) -> Tensor:
    """Contiguous and 16-byte aligned (the kernels read small vectors such as gamma and the frequencies 16 bytes at a
    time): a view that starts at an odd offset is copied."""
    t = t.contiguous()
    if torch.compiler.is_compiling():  # addresses are not visible to the tracer; traced callers pass whole tensors
        return t
    return t if t.data_ptr() % 16 == 0 else t.clone()


def gemm_qknorm_rope(
    A: Tensor, B: Tensor, weight: Tensor, positions: Tensor, frequencies: Tensor, head_dim: int, num_heads_q: int,
    num_heads_k: int, eps: float,
) -> tuple[Tensor, Tensor, Tensor, Optional[Tensor]]:
    """Fused ``[q | k | v]`` projection: returns ``(qk, preact, head_mean_sq, v)``.

    ``B`` is ``W.mT`` of the whole ``[(hq+hk+hv)*d, K]`` weight (``v`` is ``None``
    when it has no v rows).  Counterpart of ``gemm_qknorm_rope``
    (coda/core/gemm/functional.py:1155-1200) plus the v GEMM of
    coda/kernels/functional/qknorm_rope.py:39.
    """
    _require_cuda_bf16(A, B, weight)
    _require(positions.dtype in (torch.int32, torch.float32), "positions must be int32 or float32")
    _require(frequencies.dtype == torch.float32, "frequencies must be float32")
    M, N = A.shape[0], B.shape[1]
    heads = num_heads_q + num_heads_k
    size_qk = heads * head_dim
    _require(weight.numel() == 2 * head_dim, "gamma must hold [gamma_q | gamma_k]")
    _require(frequencies.numel() == size_qk, "frequencies must have (hq + hk) * head_dim entries")
    _require(positions.numel() == M, "positions must have one entry per row")
    qk = torch.empty(M, size_qk, dtype=A.dtype, device=A.device)
    preact = torch.empty(M, size_qk, dtype=A.dtype, device=A.device)
    mean_sq = torch.empty(M, heads, dtype=torch.float32, device=A.device)
    v = torch.empty(M, N - size_qk, dtype=A.dtype, device=A.device) if N > size_qk else None
    _gemm_qknorm_rope_out(
        A, B, qk, preact, v, mean_sq, _aligned16(weight), positions.contiguous(), _aligned16(frequencies), head_dim,
        num_heads_q, num_heads_k, float(eps),
    )
    return qk, preact, mean_sq, v


def dswiglu_backward(preact: Tensor, dout: Tensor) -> Tensor:
    """Counterpart of ``dswiglu_backward`` (coda/core/elementwise/functional.py:202-218)."""
    _require_cuda_bf16(preact, dout)
    _require(preact.stride(1) == 1 and dout.stride(1) == 1 and preact.shape[1] == 2 * dout.shape[1], "dswiglu: bad shapes")
    grad_pre = torch.empty_like(preact)
    _dswiglu_out(preact, dout, grad_pre)
    return grad_pre


def dsigmoid_backward(out: Tensor, dout: Tensor) -> Tensor:
    """``dout * out * (1 - out)`` in bf16 (the ``sigmoid_backward(...).to(x.dtype)`` step of sigmoid.py:35)."""
    _require_cuda_bf16(dout)
    _require(out.dtype in (_BF16, torch.float32) and out.shape == dout.shape, "dsigmoid: bad out")
    grad_pre = torch.empty(dout.shape, dtype=_BF16, device=dout.device)
    _dsigmoid_out(out, dout, grad_pre)
    return grad_pre


def gemm_dsigmoid_dgrad(out: Tensor, dout: Tensor, weight: Tensor) -> tuple[Tensor, Tensor]:
    """``(dx, grad_pre)`` of ``out = sigmoid(x @ weight^T)``: ``grad_pre = dout * out * (1 - out)`` is formed inside the
    input-gradient GEMM ``dx = grad_pre @ weight`` (by its transform warps, as the A operand) and written once for the
    weight-gradient GEMM, instead of by a separate pass (coda/kernels/functional/sigmoid.py:33-38).  bf16 only."""
    _require_cuda_bf16(out, dout, weight)
    _require(out.shape == dout.shape and out.stride(1) == 1 and dout.stride(1) == 1 and weight.stride(1) == 1
             and weight.shape[0] == out.shape[1], "gemm_dsigmoid_dgrad: out, dout [M, N] and weight [N, K] row-major expected")
    grad_pre = torch.empty_like(out)
    dx = torch.empty(out.shape[0], weight.shape[1], dtype=_BF16, device=out.device)
    _gemm_dsigmoid_dgrad_out(out, dout, weight, grad_pre, dx)
    return dx, grad_pre


def qknorm_rope_bwd(
    dq: Tensor, dk: Tensor, dv: Optional[Tensor], x: Tensor, head_mean_sq: Tensor, gamma: Tensor, pos: Tensor, freq: Tensor,
    head_dim: int, num_heads_q: int, num_heads_k: int, eps: float,
) -> tuple[Tensor, Tensor]:
    """Returns ``(grad, dgamma)``: ``grad = [grad_pre | dv]`` (bf16 ``[M, N]``) and fp32 ``dgamma[2*head_dim]``.

    Counterpart of ``qknorm_rope_bwd`` (coda/core/elementwise/functional.py:421-456).
    """
    _require_cuda_bf16(dq, dk, x, gamma)
    M, size_qk = x.shape
    nv = dv.shape[1] if dv is not None else 0
    grad = torch.empty(M, size_qk + nv, dtype=x.dtype, device=x.device)
    dgamma = torch.empty(2 * head_dim, dtype=torch.float32, device=x.device)
    blocks = (M + _QK_BWD_ROWS_PER_BLOCK - 1) // _QK_BWD_ROWS_PER_BLOCK  # = coda_b200_qknorm_rope_bwd_scratch_bytes / (8 * head_dim)
    scratch = torch.empty(blocks * 2 * head_dim, dtype=torch.float32, device=x.device)
    _qknorm_rope_bwd_out(
        dq, dk, dv, x, head_mean_sq, _aligned16(gamma), pos.contiguous(), _aligned16(freq), head_dim, num_heads_q,
        num_heads_k, float(eps), grad, dgamma, scratch,
    )
    return grad, dgamma


# ------------------------------------------------------------------------------------------------ whole operators
# One call per direction of an autograd node.  Eagerly they are single entry points of the compiled dispatch layer
# (outputs allocated and every launch of that direction issued from C++); while ``torch.compile`` traces, or with
# ``CODA_B200_DISPATCH=ctypes``, the same sequence is composed from the wrappers above.


# CODA_B200_DISPATCH=launch keeps the compiled per-launch ops but composes each operator in Python (what the tests
# compare the whole-operator entry points against).
_WHOLE_OPERATORS = os.environ.get("CODA_B200_DISPATCH", "native") == "native"


def _fast() -> bool:
    return _WHOLE_OPERATORS and _native is not None and not torch.compiler.is_compiling()


def linear_backward(grad_pre: Tensor, x: Tensor, weight: Tensor, need_dx: bool = True, need_dw: bool = True,
                    alpha: Optional[Tensor] = None) -> tuple[Optional[Tensor], Optional[Tensor]]:
    """Gradients of ``pre = x @ weight^T`` given ``grad_pre = dL/dpre`` (times the device scalar ``alpha``, if given).

    ``dx = grad_pre @ weight`` reads the ``[N, K]`` weight as an MN-major B operand and ``dweight = grad_pre^T @ x``
    reads both operands MN-major, so neither needs a transposed copy.  ``alpha`` is applied in the GEMM epilogues (read
    from device memory: no host synchronisation).
    """
    if _fast():
        return _native.linear_backward(grad_pre, x, weight, need_dx, need_dw, alpha, status_word(x.device))
    dx = gemm(grad_pre, weight, alpha=alpha) if need_dx else None
    dweight = gemm(grad_pre.mT, x, alpha=alpha) if need_dw else None
    return dx, dweight


def swiglu_forward(x: Tensor, weight: Tensor) -> tuple[Tensor, Tensor]:
    """``(preact, postact)`` of ``x @ weight^T`` with interleaved gate/up rows in ``weight [2F, K]``."""
    _require_cuda_bf16(x, weight)
    if _fast():
        return _native.swiglu_fwd(x, weight, status_word(x.device))
    return gemm_swiglu(x, weight.mT)  # weight.mT is a view: the kernel consumes the [2F, K] rows as a K-major B operand


def swiglu_backward(preact: Tensor, dout: Tensor, x: Tensor, weight: Tensor, need_dx: bool, need_dw: bool):
    if _fast():
        return _native.swiglu_bwd(preact, dout, x, weight, need_dx, need_dw, status_word(x.device))
    return linear_backward(dswiglu_backward(preact, dout), x, weight, need_dx, need_dw)


def sigmoid_forward(x: Tensor, weight: Tensor, out_dtype: Optional[torch.dtype]) -> Tensor:
    _require_cuda_bf16(x, weight)
    out_dtype = x.dtype if out_dtype is None else out_dtype
    _require(out_dtype in (_BF16, torch.float32), "gemm_sigmoid: out must be bfloat16 or float32")
    if _fast():
        return _native.sigmoid_fwd(x, weight, out_dtype == torch.float32, status_word(x.device))
    return gemm_sigmoid(x, weight.mT, out=x.new_empty((x.shape[0], weight.shape[0]), dtype=out_dtype))


def sigmoid_backward(out: Tensor, dout: Tensor, x: Tensor, weight: Tensor, need_dx: bool, need_dw: bool):
    dout = dout.to(dtype=x.dtype)
    if _fast():
        return _native.sigmoid_bwd(out, dout, x, weight, need_dx, need_dw, status_word(x.device))
    return linear_backward(dsigmoid_backward(out, dout), x, weight, need_dx, need_dw)


def cross_entropy_forward(x: Tensor, weight: Tensor, target: Tensor, ignore_index: int, reduction: str,
                          store_grad: bool) -> tuple[Tensor, Optional[Tensor], Optional[Tensor]]:
    """``(loss, inv_count, dlogits)``.  ``inv_count`` (0-d device tensor, ``"mean"`` only) is one over the number of rows
    whose target is not ``ignore_index``; ignored rows carry an exact zero loss.  ``dlogits`` (with ``store_grad``) is
    the bf16 gradient of the SUM of the row losses w.r.t. the logits: the only ``[M, V]`` buffer of the operator."""
    _require_cuda_bf16(x, weight)
    _debug_check_targets(target, weight.shape[0], ignore_index)
    if _fast():
        return _native.cross_entropy_fwd(x, weight, target, int(ignore_index), reduction == "mean", store_grad, status_word(x.device))
    if store_grad:
        row_losses, dlogits = gemm_lse_dlogits(x, weight.mT, target, ignore_index)
    else:
        row_losses, dlogits = gemm_lse_select_logits(x, weight.mT, target, ignore_index)[0], None
    total = row_losses.sum()
    if reduction == "sum":
        return total, None, dlogits
    inv_count = (target != ignore_index).sum().float().reciprocal()
    return total * inv_count, inv_count, dlogits


def cross_entropy_backward(dloss: Tensor, inv_count: Optional[Tensor], dlogits: Tensor, x: Tensor, weight: Tensor, need_dx: bool,
                           need_dw: bool):
    if _fast():
        return _native.cross_entropy_bwd(dloss, inv_count, dlogits, x, weight, need_dx, need_dw, status_word(x.device))
    alpha = (dloss if inv_count is None else dloss * inv_count).reshape(1).to(dtype=torch.float32)
    return linear_backward(dlogits, x, weight, need_dx, need_dw, alpha=alpha)


def qknorm_rope_forward(x: Tensor, weight: Tensor, gamma: Tensor, positions: Tensor, frequencies: Tensor, head_dim: int,
                        num_heads_q: int, num_heads_k: int, eps: float) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """``(qk, preact, head_mean_sq, v)`` from ONE GEMM over the whole ``[(hq + hk + hv) * d, K]`` weight; ``v`` has zero
    columns when the weight has no v rows."""
    _require_cuda_bf16(x, weight, gamma)
    if _fast():
        return _native.qknorm_rope_fwd(x, weight, gamma, positions, frequencies, head_dim, num_heads_q, num_heads_k, float(eps),
                                       status_word(x.device))
    qk, preact, mean_sq, v = gemm_qknorm_rope(x, weight.mT, gamma, positions, frequencies, head_dim, num_heads_q, num_heads_k, eps)
    return qk, preact, mean_sq, (x.new_empty(x.shape[0], 0) if v is None else v)


def qknorm_rope_backward(dq: Tensor, dk: Tensor, dv: Tensor, x: Tensor, weight: Tensor, preact: Tensor, head_mean_sq: Tensor,
                         gamma: Tensor, positions: Tensor, frequencies: Tensor, head_dim: int, num_heads_q: int, num_heads_k: int,
                         eps: float, need_dx: bool, need_dw: bool):
    """``(dx, dweight, dgamma)``; ``dv`` with zero columns stands for "no v rows"."""
    if _fast():
        return _native.qknorm_rope_bwd(dq, dk, dv, x, weight, preact, head_mean_sq, gamma, positions, frequencies, head_dim, num_heads_q,
                                       num_heads_k, float(eps), need_dx, need_dw, status_word(x.device))
    grad_all, dgamma = qknorm_rope_bwd(dq, dk, dv if dv.shape[1] > 0 else None, preact, head_mean_sq, gamma, positions, frequencies,
                                       head_dim, num_heads_q, num_heads_k, eps)
    dx, dweight = linear_backward(grad_all, x, weight, need_dx, need_dw)
    return dx, dweight, dgamma.to(dtype=gamma.dtype)
