"""CPU/GPU-agnostic restatement of the reference's eager formulation of the hot path.

TEST INFRASTRUCTURE ONLY.  Nothing under ``coda_kernels_b200/`` imports this
module; it is the checker used by ``tests/``, by ``__graft_entry__.smoke()``
and by the CPU-baseline / reference legs of ``bench.py``.

Each function follows the PyTorch eager code the reference benchmarks use as
their own ground truth (``benchmarks/backends/torch_linear.py`` over
``benchmarks/backends/torch_ops.py``), evaluated as "fp32 math on the same bf16
inputs": inputs are converted to ``compute_dtype`` (fp32 by default, fp64 for a
tighter check) and all arithmetic, including the GEMM, runs in that type under
autograd, so gradients come from ``torch.autograd.grad``.

Pinning: the reference holds no golden vectors for this path.  This module is
pinned against the reference's own eager implementation run in this build
container; the vectors are committed under ``tests/golden/`` together with the
script that produced them (``tests/golden/make_golden.py``), and
``tests/test_oracle.py`` replays them.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _c(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return t.to(dtype=dtype)


# ---------------------------------------------------------------------------------------------- swiglu
def linear_swiglu(x: torch.Tensor, weight: torch.Tensor, compute_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``silu(gate) * up`` with gate/up interleaved along the rows of ``weight [2F, K]``.

    Follows benchmarks/backends/torch_linear.py:19-33 and torch_ops.swiglu (torch_ops.py:18-32, interleaved layout).
    """
    preact = _c(x, compute_dtype) @ _c(weight, compute_dtype).mT
    gate = preact[:, 0::2]
    up = preact[:, 1::2]
    return F.silu(gate) * up


def dswiglu(preact: torch.Tensor, grad: torch.Tensor) -> torch.Tensor:
    """Hand-written derivative of the interleaved SwiGLU (torch_ops.py:35-65)."""
    gate = preact[:, 0::2]
    up = preact[:, 1::2]
    s = torch.sigmoid(gate)
    silu = gate * s
    dgate = grad * up * (s + silu * (1 - s))
    dup = grad * silu
    return torch.stack((dgate, dup), dim=-1).reshape(preact.shape)


# ---------------------------------------------------------------------------------------------- sigmoid
def linear_sigmoid(x: torch.Tensor, weight: torch.Tensor, compute_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``sigmoid(x @ weight^T)`` (benchmarks/backends/torch_linear.py:6-16, torch_ops.py:406-417)."""
    return torch.sigmoid(_c(x, compute_dtype) @ _c(weight, compute_dtype).mT)


def linear_sigmoid_glu(x: torch.Tensor, weight: torch.Tensor, compute_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``sigmoid(gate) * value`` with gate / value rows interleaved in ``weight [2N, K]``: the gated-projection reading of the
    sigmoid benchmark configuration (no counterpart in the reference; same structure as ``linear_swiglu``)."""
    preact = _c(x, compute_dtype) @ _c(weight, compute_dtype).mT
    return torch.sigmoid(preact[:, 0::2]) * preact[:, 1::2]


# ---------------------------------------------------------------------------------------------- cross entropy
def linear_cross_entropy(
    x: torch.Tensor,
    weight: torch.Tensor,
    target: torch.Tensor,
    ignore_index: int = -100,
    reduction: str = "mean",
    compute_dtype: torch.dtype = torch.float32,
    chunk_rows: int = 1024,
) -> torch.Tensor:
    """Cross entropy of ``x @ weight^T`` (benchmarks/backends/torch_linear.py:83-104, torch_ops.py:1023-1037).

    Rows are processed ``chunk_rows`` at a time so that the ``[rows, vocab]``
    logits stay small, as the reference's oracle runner does
    (benchmarks/utils/cases.py:20-24).  ``mean`` divides by the number of rows
    whose target differs from ``ignore_index``.
    """
    assert reduction in ("mean", "sum")
    w = _c(weight, compute_dtype)
    total = None
    for r0 in range(0, x.shape[0], chunk_rows):
        logits = _c(x[r0 : r0 + chunk_rows], compute_dtype) @ w.mT
        part = F.cross_entropy(logits, target[r0 : r0 + chunk_rows].long(), ignore_index=ignore_index, reduction="sum")
        total = part if total is None else total + part
    if reduction == "mean":
        count = (target != ignore_index).sum().to(dtype=compute_dtype)
        return total / count
    return total


def cross_entropy_rows(logits: torch.Tensor, target: torch.Tensor, ignore_index: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-row losses and ``softmax - onehot`` with ignored rows zeroed (torch_ops.py:279-313)."""
    valid = target != ignore_index
    safe = torch.where(valid, target, torch.zeros_like(target)).long()
    rows = torch.arange(logits.shape[0], device=logits.device)
    lse = torch.logsumexp(logits, dim=-1)
    losses = torch.where(valid, lse - logits[rows, safe], torch.zeros_like(lse))
    d = torch.softmax(logits, dim=-1)
    d[rows, safe] -= 1
    d = torch.where(valid[:, None], d, torch.zeros_like(d))
    return losses, d


# ---------------------------------------------------------------------------------------------- qk-norm + rope
def rope_tables(positions: torch.Tensor, frequencies: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``cos``/``sin`` of ``2*pi * pos * (hi + lo)`` per rotary pair, formed in fp64 (torch_ops.py:116-132)."""
    pairs = frequencies.to(dtype=torch.float64).reshape(-1, 2)
    turns = pairs[:, 0] + pairs[:, 1]
    angles = 2 * math.pi * positions.to(dtype=torch.float64)[:, None] * turns[None, :]
    return torch.cos(angles), torch.sin(angles)


def rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate adjacent pairs ``(2p, 2p+1)``: ``(x0 c - x1 s, x1 c + x0 s)`` (torch_ops.py:148-196, interleaved layout).

    ``cos``/``sin`` are ``[M, N/2]`` (one column per pair of ``x [M, N]``).
    """
    x0 = x[:, 0::2]
    x1 = x[:, 1::2]
    c = cos.to(dtype=x.dtype)
    s = sin.to(dtype=x.dtype)
    return torch.stack((x0 * c - x1 * s, x1 * c + x0 * s), dim=-1).reshape(x.shape)


def head_mean_square(x: torch.Tensor, head_dim: int) -> torch.Tensor:
    """``[M, heads]`` mean of squares per head (torch_ops.py:199-206)."""
    return x.reshape(x.shape[0], -1, head_dim).square().mean(dim=-1)


def qknorm(x, head_mean_sq, gamma, head_dim, num_heads_q, num_heads_k, eps):
    """Each head times ``rsqrt(mean_sq + eps)`` and its gamma (q heads: ``gamma[:d]``, k heads: ``gamma[d:]``); torch_ops.py:209-230."""
    xh = x.reshape(x.shape[0], -1, head_dim)
    rstd = torch.rsqrt(head_mean_sq + eps)[..., None]
    gq, gk = gamma[:head_dim], gamma[head_dim:]
    g = torch.cat((gq.expand(num_heads_q, head_dim), gk.expand(num_heads_k, head_dim)))
    return (xh * rstd * g).reshape(x.shape)


def linear_qknorm_rope(
    x, weight, gamma, positions, frequencies, head_dim, num_heads_q, num_heads_k, eps, compute_dtype=torch.float32
):
    """``(q, k, v)`` of the fused projection (benchmarks/backends/torch_linear.py:36-80, torch_ops.py:675-722)."""
    size_q = head_dim * num_heads_q
    size_qk = head_dim * (num_heads_q + num_heads_k)
    xc = _c(x, compute_dtype)
    wc = _c(weight, compute_dtype)
    preact = xc @ wc[:size_qk].mT
    ms = head_mean_square(preact, head_dim)
    normed = qknorm(preact, ms, _c(gamma, compute_dtype), head_dim, num_heads_q, num_heads_k, eps)
    cos, sin = rope_tables(positions, frequencies)
    rotated = rope_interleaved(normed, cos, sin)
    v = xc @ wc[size_qk:].mT
    return rotated[:, :size_q], rotated[:, size_q:], v


# ---------------------------------------------------------------------------------------------- deferred-RMSNorm variants
def rmsnorm_rstd(x: torch.Tensor, eps: float, compute_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Each row's ``1 / sqrt(mean(x^2) + eps)`` (torch_ops.py:68-76)."""
    return torch.rsqrt(_c(x, compute_dtype).square().mean(dim=-1) + eps)


def gemm_rmsnorm_swiglu(A, B, rstd, compute_dtype=torch.float32):
    """``preact = (A @ B) * rstd``, ``postact = swiglu(preact)`` (torch_ops.py:442-464); ``B`` is ``[K, 2F]``."""
    preact = (_c(A, compute_dtype) @ _c(B, compute_dtype)) * _c(rstd, compute_dtype)[:, None]
    return preact, F.silu(preact[:, 0::2]) * preact[:, 1::2]


def gemm_rmsnorm_lse(A, B, rstd, compute_dtype=torch.float32):
    """Logits ``(A @ B) * rstd`` and each row's log-sum-exp (torch_ops.py:1061-1081)."""
    logits = (_c(A, compute_dtype) @ _c(B, compute_dtype)) * _c(rstd, compute_dtype)[:, None]
    return logits, torch.logsumexp(logits, dim=-1)


def gemm_rmsnorm_qknorm_rope(A, B, rstd, weight, positions, frequencies, head_dim, num_heads_q, num_heads_k, eps,
                             compute_dtype=torch.float32):
    """``(rotated, preact, head_mean_sq)`` where the statistic and the output use ``z = (A @ B) * rstd`` and ``preact``
    is saved without ``rstd`` (torch_ops.py:725-777; that code rounds ``z`` to the GEMM dtype first, this one does not)."""
    preact = _c(A, compute_dtype) @ _c(B, compute_dtype)
    z = preact * _c(rstd, compute_dtype)[:, None]
    ms = head_mean_square(z, head_dim)
    normed = qknorm(z, ms, _c(weight, compute_dtype), head_dim, num_heads_q, num_heads_k, eps)
    cos, sin = rope_tables(positions, frequencies)
    return rope_interleaved(normed, cos, sin), preact, ms


# ---------------------------------------------------------------------------------------------- GEMMs between the operators
def gemm_residual_partial_rmsnorm(A, B, C, weight, eps, compute_dtype=torch.float32):
    """``pre = A @ B + C``, ``post = pre * weight``, ``rstd`` of the unrounded ``pre`` (torch_ops.py:528-549)."""
    pre = _c(A, compute_dtype) @ _c(B, compute_dtype) + _c(C, compute_dtype)
    return pre, pre * _c(weight, compute_dtype), torch.rsqrt(pre.square().mean(dim=-1) + eps)


def gemm_swiglu_bwd_zdz(A, B, Z, scale=None, compute_dtype=torch.float32):
    """Down-projection dgrad ``A @ B^T`` through SwiGLU at the stored preact ``Z``: ``(dZ, ZdZ, postact)``
    with ``ZdZ = scale * sum(Z * dZ)`` (torch_ops.py:466-490)."""
    dpost = _c(A, compute_dtype) @ _c(B, compute_dtype).mT
    z = _c(Z, compute_dtype)
    dz = dswiglu(z, dpost)
    zdz = (z * dz).sum(dim=-1)
    if scale is not None:
        zdz = zdz * scale
    return dz, zdz, F.silu(z[:, 0::2]) * z[:, 1::2]


def gemm_residual_partial_rmsnorm_bwd(A, B, weight, pre, ZdZ, rstd, alpha=None, dX=None, compute_dtype=torch.float32):
    """The next GEMM's dgrad ``A @ B^T`` (times ``alpha``) through the RMSNorm backward at the stored ``pre`` and
    ``rstd``: ``(dpre [+ dX], dweight, normed)`` (torch_ops.py:91-113, 552-583)."""
    grad = _c(A, compute_dtype) @ _c(B, compute_dtype).mT
    if alpha is not None:
        grad = grad * _c(alpha, compute_dtype)
    r = _c(rstd, compute_dtype)[:, None]
    w = _c(weight, compute_dtype)
    n = _c(pre, compute_dtype) * r
    dpre = (grad * w - n * _c(ZdZ, compute_dtype)[:, None]) * r
    dweight = (grad * n).sum(dim=0)
    if dX is not None:
        dpre = dpre + _c(dX, compute_dtype)
    return dpre, dweight, n * w


# ---------------------------------------------------------------------------------------------- Llama-3 layer blocks
def _rms_norm(x, weight, eps):
    return x * torch.rsqrt(x.square().mean(dim=-1, keepdim=True) + eps) * weight


def _rope_all_columns(x, positions, frequencies):
    cos, sin = rope_tables(positions, frequencies)  # frequencies are zero on the v columns: identity there
    return rope_interleaved(x, cos, sin)


def llama3_block_pre(x, w, wn, positions, frequencies, eps, compute_dtype=torch.float32):
    """``(residual, qkv)``: RMSNorm, QKV projection, RoPE on q and k (benchmarks/backends/torch_blocks,py:219-250)."""
    xc = _c(x, compute_dtype)
    qkv = _rms_norm(xc, _c(wn, compute_dtype), eps) @ _c(w, compute_dtype).mT
    return xc, _rope_all_columns(qkv, positions, frequencies)


def _llama3_mlp(x0, y0, w0, w1, w2, wn0, eps, compute_dtype):
    x1 = _c(x0, compute_dtype) + _c(y0, compute_dtype) @ _c(w0, compute_dtype).mT
    preact = _rms_norm(x1, _c(wn0, compute_dtype), eps) @ _c(w1, compute_dtype).mT
    postact = F.silu(preact[:, 0::2]) * preact[:, 1::2]
    return x1 + postact @ _c(w2, compute_dtype).mT


def llama3_block(x0, y0, w0, w1, w2, w3, wn0, wn1, positions, frequencies, eps, compute_dtype=torch.float32):
    """``(x2, qkv)``: output projection + residual, SwiGLU MLP + residual, next layer's norm + QKV + RoPE
    (benchmarks/backends/torch_blocks,py:253-314)."""
    x2 = _llama3_mlp(x0, y0, w0, w1, w2, wn0, eps, compute_dtype)
    qkv = _rms_norm(x2, _c(wn1, compute_dtype), eps) @ _c(w3, compute_dtype).mT
    return x2, _rope_all_columns(qkv, positions, frequencies)


def llama3_block_post(x0, y0, w0, w1, w2, w3, wn0, wn1, targets, eps, ignore_index=-100, reduction="mean",
                      compute_dtype=torch.float32):
    """The loss after the last layer's MLP, final norm and LM head (benchmarks/backends/torch_blocks,py:317-377)."""
    x2 = _llama3_mlp(x0, y0, w0, w1, w2, wn0, eps, compute_dtype)
    logits = _rms_norm(x2, _c(wn1, compute_dtype), eps) @ _c(w3, compute_dtype).mT
    total = F.cross_entropy(logits, targets.long(), ignore_index=ignore_index, reduction="sum")
    if reduction == "mean":
        return total / (targets != ignore_index).sum().to(dtype=compute_dtype)
    return total


# ---------------------------------------------------------------------------------------------- fwd + bwd helpers
def fwd_bwd(fn, inputs: dict, grad_names: list[str], cotangents):
    """Run ``fn(**inputs)`` with autograd on ``grad_names`` and return ``(outputs, grads)``.

    ``cotangents`` is one tensor or a tuple matching ``fn``'s outputs; they are cast to the outputs' dtype.
    """
    work = dict(inputs)
    leaves = []
    for name in grad_names:
        leaf = work[name].detach().clone().to(dtype=torch.float32 if work[name].dtype != torch.float64 else torch.float64)
        leaf.requires_grad_(True)
        work[name] = leaf
        leaves.append(leaf)
    out = fn(**work)
    outs = out if isinstance(out, tuple) else (out,)
    cots = cotangents if isinstance(cotangents, tuple) else (cotangents,)
    cots = tuple(c.to(dtype=o.dtype) for c, o in zip(cots, outs))
    grads = torch.autograd.grad(outs, leaves, cots)
    return tuple(o.detach() for o in outs), dict(zip(grad_names, grads))


# ---------------------------------------------------------------------------------------------- error metrics
def max_rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """``max|a - b| / max|b|``: the tolerance metric of the parity tests (b = oracle).  Evaluated where ``b`` lives."""
    a = a.detach().to(device=b.device, dtype=torch.float64)
    b = b.detach().to(dtype=torch.float64)
    denom = b.abs().max().item()
    num = (a - b).abs().max().item()
    return float(num) if denom == 0.0 else float(num / denom)


def rel_l2_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """``||a - b|| / ||b||``: the metric the reference's harness reports (benchmarks/utils/numerics.py:20-29)."""
    a = a.detach().to(device=b.device, dtype=torch.float64)
    b = b.detach().to(dtype=torch.float64)
    denom = b.norm().item()
    num = (a - b).norm().item()
    return float(num) if denom == 0.0 else float(num / denom)


def rounding_floor(b: torch.Tensor, dtype: torch.dtype) -> float:
    """Relative L2 error of the exact answer ``b`` once rounded to ``dtype``: the least error any implementation that
    returns ``dtype`` can have (the reference's ``errors_minimum``, benchmarks/utils/numerics.py:81-85)."""
    b64 = b.detach().to(dtype=torch.float64)
    return rel_l2_err(b64.to(dtype=dtype), b64)


def max_elementwise_err(a: torch.Tensor, b: torch.Tensor, atol_frac: float = 1e-6) -> float:
    """``max |a - b| / (|b| + atol)`` with ``atol = atol_frac * max|b|``: an element-wise relative error with an absolute
    floor, which sees a wrong small-magnitude entry that ``max_rel_err`` (one global scale) cannot."""
    a = a.detach().to(device=b.device, dtype=torch.float64)
    b = b.detach().to(dtype=torch.float64)
    atol = atol_frac * b.abs().max().item()
    if atol == 0.0:
        return float((a - b).abs().max().item())
    return float(((a - b).abs() / (b.abs() + atol)).max().item())
