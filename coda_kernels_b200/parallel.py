"""Sharding of the fused-linear operators over the GPUs of one box (one process per GPU).

The reference has no distributed code; this module adds what the operators
need to run column-, head- or vocab-parallel over ``torch.distributed``:

* ``linear_swiglu`` / ``linear_sigmoid``: column-parallel over the output
  features (gate/up pairs stay together).  The forward needs no communication;
  each rank's ``dx`` is a partial sum.  :func:`column_parallel_linear_swiglu` /
  :func:`column_parallel_linear_sigmoid` fold it inside the backward, with the
  all-reduce in flight while the weight-gradient GEMM runs
  (:func:`linear_backward_overlapped`); :func:`allreduce_partial_dx` is the
  plain fold for callers that run the unsharded operator on a weight shard.
* ``linear_qknorm_rope``: head-parallel (whole q heads, with the k and v heads
  of their group), :func:`head_parallel_linear_qknorm_rope`.  ``dgamma`` is
  summed over ranks, ``dx`` as above.
* ``linear_cross_entropy``: vocab-parallel.  Each rank runs the fused GEMM on
  its vocabulary slice; one all-gather of per-row ``(lse, target logit)``
  (8 bytes per row per rank) gives every rank the global log-sum-exp, and the
  gradient pass uses it directly, so logits never exist anywhere.

Host-side pieces (:func:`shard_bounds`, :func:`combine_lse`, the target
re-basing) are plain tensor code and are exercised on CPU with the ``gloo``
backend; the GEMMs and element-wise passes are the library's CUDA kernels.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor

# CODA_B200_OVERLAP_DX=0 issues the input-gradient all-reduce synchronously (after it, then the weight-gradient GEMM)
# instead of letting the two overlap: a switch for measurements.
OVERLAP_DX_ALLREDUCE = os.environ.get("CODA_B200_OVERLAP_DX", "1") == "1"
# CTAs the weight-gradient GEMM may use while an all-reduce is in flight beside it.  The GEMM is a persistent kernel of
# one 224 KB CTA per SM with a static share of the tiles each: an SM that the collective's CTAs hold cannot take one, and
# the CTA that did not fit starts only when the collective has finished and then still runs its whole share, so an
# uncapped GEMM ends no earlier than if the two had run one after the other (measured on 8 GPUs, linear_swiglu with the
# 134 MB all-reduce: 1.50 ms serial, 1.59 ms overlapped with all 148 CTAs or with 132 or 124, 1.34 ms with 116 = 148 minus
# the collective's 32; on 4 GPUs 2.68 serial, 2.69 uncapped, 2.61 with 116).  A grid that leaves the collective its SMs
# keeps every CTA resident, at the price of a GEMM that is 148/116 times longer.  So only as much of the weight gradient
# as the all-reduce lasts runs capped (its first rows, a launch of its own); the rest runs on all SMs afterwards.
# CODA_B200_OVERLAP_MAX_CTAS: "auto" (default: the plan below), 0 = never cap, n = cap the whole GEMM at n CTAs.
_OVERLAP_MAX_CTAS = os.environ.get("CODA_B200_OVERLAP_MAX_CTAS", "auto")
_COLLECTIVE_CTAS = 32
_GEMM_FLOPS_PER_S = 1.2e15      # sustained rate of one GPU, for the estimate only
_ALLREDUCE_BUS_BYTES_PER_S = 7.0e11
_SPLIT_ROWS = 256               # the capped part ends on a tile boundary
# CODA_B200_OVERLAP_SPLIT=1: cap only the first rows of a long weight gradient (a launch of its own) instead of all or
# nothing.  Off by default: on 4 GPUs it lost to the all-or-nothing plan (2.71 vs 2.56 ms per linear_swiglu step); when the
# transfer outlasts the estimate, the uncapped remainder meets the same wall as an uncapped GEMM.
_OVERLAP_SPLIT = os.environ.get("CODA_B200_OVERLAP_SPLIT", "0") == "1"


def overlap_plan(flops: float, rows: int, allreduce_bytes: int, world: int, sms: int) -> tuple[int, int]:
    """``(cap, capped_rows)`` for a weight-gradient GEMM of ``flops`` with ``rows`` output rows that starts while an all-reduce
    of ``allreduce_bytes`` over ``world`` ranks is in flight: its first ``capped_rows`` rows run on ``cap`` CTAs, the rest
    uncapped.  ``(0, 0)``: no cap at all; ``capped_rows == rows``: one capped launch."""
    if _OVERLAP_MAX_CTAS != "auto":
        cap = int(_OVERLAP_MAX_CTAS)
        return (cap, rows) if cap > 0 else (0, 0)
    capped = sms - _COLLECTIVE_CTAS
    if capped < sms // 2 or world < 2:
        return 0, 0
    gemm_capped = flops / _GEMM_FLOPS_PER_S * sms / capped  # duration of the whole GEMM on the capped grid
    allreduce = allreduce_bytes * 2.0 * (world - 1) / world / _ALLREDUCE_BUS_BYTES_PER_S
    fraction = allreduce / gemm_capped
    if not _OVERLAP_SPLIT:
        # all or nothing: cap when the 148/116 stretch of the whole GEMM is shorter than the transfer
        return (capped, rows) if gemm_capped * (1.0 - capped / sms) < 0.9 * allreduce else (0, 0)
    if fraction >= 0.85:
        return capped, rows
    if fraction < 0.1:
        return 0, 0  # a transfer this short is not worth a second launch
    part = int(round(fraction * rows / _SPLIT_ROWS)) * _SPLIT_ROWS
    if part < _SPLIT_ROWS or rows - part < _SPLIT_ROWS:
        return (capped, rows) if fraction >= 0.5 else (0, 0)
    return capped, part


def shard_bounds(total: int, rank: int, world: int, multiple: int = 1) -> tuple[int, int]:
    """Contiguous slice ``[lo, hi)`` of ``total`` items for ``rank``, in units of ``multiple`` items.

    The first ``(total / multiple) % world`` ranks get one extra unit, so any
    ``total`` that is a multiple of ``multiple`` is covered without gaps.
    """
    if total % multiple != 0:
        raise ValueError(f"{total} is not a multiple of {multiple}")
    units = total // multiple
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo * multiple, hi * multiple


def shard_swiglu_weight(weight: Tensor, rank: int, world: int) -> Tensor:
    """Rows of the interleaved ``[2F, K]`` weight owned by ``rank``: whole (gate, up) pairs, 8 pairs at a time."""
    lo, hi = shard_bounds(weight.shape[0], rank, world, multiple=16)
    return weight[lo:hi]


def shard_rows(weight: Tensor, rank: int, world: int, multiple: int = 8) -> Tensor:
    """Output-feature rows ``[N/g]`` of a ``[N, K]`` weight owned by ``rank``."""
    lo, hi = shard_bounds(weight.shape[0], rank, world, multiple=multiple)
    return weight[lo:hi]


def shard_qkv_weight(
    weight: Tensor, frequencies: Tensor, head_dim: int, num_heads_q: int, num_heads_k: int, num_heads_v: int, rank: int, world: int
) -> tuple[Tensor, Tensor, int, int, int]:
    """Local ``[q_r | k_r | v_r]`` weight rows, the matching frequency slice and the local head counts."""
    if num_heads_q % world or num_heads_k % world or num_heads_v % world:
        raise ValueError("head counts must be divisible by the number of ranks")
    d = head_dim
    hq, hk, hv = num_heads_q // world, num_heads_k // world, num_heads_v // world
    q0 = rank * hq * d
    k0 = num_heads_q * d + rank * hk * d
    v0 = (num_heads_q + num_heads_k) * d + rank * hv * d
    local_w = torch.cat((weight[q0 : q0 + hq * d], weight[k0 : k0 + hk * d], weight[v0 : v0 + hv * d])).contiguous()
    fq0 = rank * hq * d
    fk0 = num_heads_q * d + rank * hk * d
    local_f = torch.cat((frequencies[fq0 : fq0 + hq * d], frequencies[fk0 : fk0 + hk * d])).contiguous()
    return local_w, local_f, hq, hk, hv


def allreduce_partial_dx(dx: Tensor, group: Optional[dist.ProcessGroup] = None) -> Tensor:
    """Sum the per-rank partial input gradients in place (bf16 on the wire, NCCL over NVLink)."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(dx, op=dist.ReduceOp.SUM, group=group)
    return dx


def _several_ranks(group: Optional[dist.ProcessGroup]) -> bool:
    return dist.is_initialized() and dist.get_world_size(group) > 1


def linear_backward_overlapped(grad_pre: Tensor, x: Tensor, weight_shard: Tensor, need_dx: bool, need_dw: bool,
                               group: Optional[dist.ProcessGroup], reduce_dx: bool, alpha: Optional[Tensor] = None,
                               also_reduce: Optional[Tensor] = None):
    """``(dx, dweight)`` of ``pre = x @ weight_shard^T`` on a rank that holds a slice of the weight's rows.

    ``dx = grad_pre @ weight_shard`` is this rank's partial sum.  With ``reduce_dx`` its all-reduce (bf16 on the wire)
    is started right after the GEMM that produced it, asynchronously on the communicator's stream, and joined only
    after the weight-gradient GEMM ``grad_pre^T @ x`` has been enqueued on this stream: the transfer over NVLink runs
    under that GEMM.  ``also_reduce`` (e.g. a ``dgamma`` partial) is summed over the ranks the same way.
    """
    from . import ops

    pending = []
    several = _several_ranks(group)
    if also_reduce is not None and several:
        pending.append(dist.all_reduce(also_reduce, op=dist.ReduceOp.SUM, group=group, async_op=True))
    dx = dweight = None
    if need_dx:
        dx = ops.gemm(grad_pre, weight_shard, alpha=alpha)
        if reduce_dx and several:
            pending.append(dist.all_reduce(dx, op=dist.ReduceOp.SUM, group=group, async_op=True))
            if not OVERLAP_DX_ALLREDUCE:
                pending.pop().wait()
    if need_dw:
        cap = part = 0
        rows = grad_pre.shape[1]
        if dx is not None and pending and OVERLAP_DX_ALLREDUCE and reduce_dx:
            sms = torch.cuda.get_device_properties(x.device).multi_processor_count if x.is_cuda else 148
            cap, part = overlap_plan(2.0 * grad_pre.shape[0] * rows * x.shape[1], rows, dx.numel() * dx.element_size(),
                                     dist.get_world_size(group), sms)
        if cap > 0:
            from ._lib import option_override

            if part >= rows:
                with option_override("max_ctas", cap):
                    dweight = ops.gemm(grad_pre.mT, x, alpha=alpha)
            else:
                # rows [0, part) beside the collective on the SMs it leaves, rows [part, rows) on all SMs once it is done
                dweight = torch.empty(rows, x.shape[1], dtype=x.dtype, device=x.device)
                with option_override("max_ctas", cap):
                    ops.gemm(grad_pre[:, :part].mT, x, out=dweight[:part], alpha=alpha)
                ops.gemm(grad_pre[:, part:].mT, x, out=dweight[part:], alpha=alpha)
        else:
            dweight = ops.gemm(grad_pre.mT, x, alpha=alpha)
    for work in pending:
        work.wait()
    return dx, dweight


def rebase_target(target: Tensor, vocab_start: int, vocab_local: int, ignore_index: int) -> tuple[Tensor, int]:
    """Targets in the index space of a vocabulary slice.

    Rows whose label lives on another rank get a sentinel that matches no column
    and differs from ``ignore_index``; ignored rows keep ``ignore_index``.
    Returns ``(local_target, local_ignore_index)``.
    """
    sentinel = -1 if ignore_index != -1 else -2
    local_ignore = ignore_index if ignore_index < 0 else -3  # keep the ignore marker outside [0, vocab_local)
    local = target - vocab_start
    owned = (local >= 0) & (local < vocab_local)
    ignored = target == ignore_index
    out = torch.where(owned, local, torch.full_like(local, sentinel))
    out = torch.where(ignored, torch.full_like(local, local_ignore), out)
    return out.to(dtype=torch.int32), local_ignore


def combine_lse(local_lse: Tensor, local_target_logit: Tensor, group: Optional[dist.ProcessGroup] = None) -> tuple[Tensor, Tensor]:
    """Global per-row ``(lse, target_logit)`` from each rank's slice values: one all-gather of ``[M, 2]`` fp32.

    ``local_target_logit`` must be zero on ranks that do not own the row's label.
    """
    packed = torch.stack((local_lse, local_target_logit), dim=1).contiguous()
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        world = dist.get_world_size(group)
        gathered = torch.empty((world,) + tuple(packed.shape), dtype=packed.dtype, device=packed.device)
        dist.all_gather(list(gathered.unbind(0)), packed, group=group)
    else:
        gathered = packed[None]
    lse = torch.logsumexp(gathered[:, :, 0], dim=0)
    target_logit = gathered[:, :, 1].sum(dim=0)
    return lse, target_logit


class VocabParallelLinearCrossEntropy(torch.autograd.Function):
    """``linear_cross_entropy`` with ``weight`` sharded over the vocabulary; every rank returns the same loss."""

    @staticmethod
    def forward(ctx, x, weight_shard, target, vocab_start: int, ignore_index: int, reduction: str, group, reduce_dx: bool):
        from . import ops

        ops.lazy_status_check(x.device)
        x = x.contiguous()
        weight_shard = weight_shard.contiguous()
        local_target, local_ignore = rebase_target(target, vocab_start, weight_shard.shape[0], ignore_index)
        probs, part_max, part_sum, target_logit = ops.gemm_lse_partials(x, weight_shard.mT, local_target, store_probs=True)
        local_lse, _ = ops.lse_finalize(part_max, part_sum, local_target, target_logit, local_ignore)
        lse, tlogit = combine_lse(local_lse, target_logit, group)
        valid = target != ignore_index
        losses = torch.where(valid, lse - tlogit, torch.zeros_like(lse))
        ops._ce_grad_fixup(probs, part_max, lse, local_target, int(local_ignore))
        if reduction == "mean":
            scale = 1.0 / valid.sum().float()
            loss = losses.sum() * scale
        else:
            scale = None
            loss = losses.sum()
        ctx.save_for_backward(x, weight_shard, probs, scale)
        ctx.group = group
        ctx.reduce_dx = reduce_dx
        return loss

    @staticmethod
    def backward(ctx, dloss):
        from . import ops

        x, weight_shard, dlogits, scale = ctx.saved_tensors
        ops.lazy_status_check(x.device)
        alpha = (dloss * scale if scale is not None else dloss).reshape(1).to(dtype=torch.float32)
        dx, dweight = linear_backward_overlapped(dlogits, x, weight_shard, ctx.needs_input_grad[0], ctx.needs_input_grad[1],
                                                 ctx.group, ctx.reduce_dx, alpha=alpha)
        return dx, dweight, None, None, None, None, None, None


def vocab_parallel_linear_cross_entropy(
    x: Tensor,
    weight_shard: Tensor,
    target: Tensor,
    vocab_start: int,
    ignore_index: int = -100,
    reduction: str = "mean",
    group: Optional[dist.ProcessGroup] = None,
    reduce_dx: bool = True,
) -> Tensor:
    """Loss of ``x @ W^T`` against ``target`` where this rank holds rows ``[vocab_start, vocab_start + len(shard))`` of ``W``."""
    assert reduction in ("mean", "sum")
    assert target.dtype == torch.int32
    return VocabParallelLinearCrossEntropy.apply(x, weight_shard, target, vocab_start, ignore_index, reduction, group, reduce_dx)


class ColumnParallelLinearSwiGLU(torch.autograd.Function):
    """``linear_swiglu`` on a slice of the gate/up pairs; the output is this rank's slice of the features."""

    @staticmethod
    def forward(ctx, x, weight_shard, group, reduce_dx: bool):
        from . import ops

        ops.lazy_status_check(x.device)
        x, weight_shard = x.contiguous(), weight_shard.contiguous()
        preact, out = ops.swiglu_forward(x, weight_shard)
        ctx.save_for_backward(x, weight_shard, preact)
        ctx.group, ctx.reduce_dx = group, reduce_dx
        return out

    @staticmethod
    def backward(ctx, grad_out):
        from . import ops

        x, weight_shard, preact = ctx.saved_tensors
        ops.lazy_status_check(x.device)
        grad_pre = ops.dswiglu_backward(preact, grad_out.contiguous())
        dx, dweight = linear_backward_overlapped(grad_pre, x, weight_shard, ctx.needs_input_grad[0], ctx.needs_input_grad[1],
                                                 ctx.group, ctx.reduce_dx)
        return dx, dweight, None, None


class ColumnParallelLinearSigmoid(torch.autograd.Function):
    """``linear_sigmoid`` on a slice of the output features."""

    @staticmethod
    def forward(ctx, x, weight_shard, out_dtype, group, reduce_dx: bool):
        from . import ops

        ops.lazy_status_check(x.device)
        x, weight_shard = x.contiguous(), weight_shard.contiguous()
        out = ops.sigmoid_forward(x, weight_shard, out_dtype)
        ctx.save_for_backward(x, weight_shard, out)
        ctx.group, ctx.reduce_dx = group, reduce_dx
        return out

    @staticmethod
    def backward(ctx, grad_out):
        from . import ops

        x, weight_shard, out = ctx.saved_tensors
        ops.lazy_status_check(x.device)
        grad_pre = ops.dsigmoid_backward(out, grad_out.contiguous().to(dtype=x.dtype))
        dx, dweight = linear_backward_overlapped(grad_pre, x, weight_shard, ctx.needs_input_grad[0], ctx.needs_input_grad[1],
                                                 ctx.group, ctx.reduce_dx)
        return dx, dweight, None, None, None


class HeadParallelLinearQKNormRope(torch.autograd.Function):
    """``linear_qknorm_rope`` on this rank's q heads with the k and v heads of their groups (:func:`shard_qkv_weight`)."""

    @staticmethod
    def forward(ctx, x, weight_shard, gamma, positions, frequencies_shard, head_dim: int, num_heads_q: int, num_heads_k: int, eps: float,
                group, reduce_dx: bool):
        from . import ops

        ops.lazy_status_check(x.device)
        x, weight_shard = x.contiguous(), weight_shard.contiguous()
        rotated, preact, head_mean_sq, v = ops.qknorm_rope_forward(x, weight_shard, gamma, positions, frequencies_shard, head_dim,
                                                                   num_heads_q, num_heads_k, eps)
        ctx.save_for_backward(x, weight_shard, gamma, positions, frequencies_shard, preact, head_mean_sq)
        ctx.args = (head_dim, num_heads_q, num_heads_k, eps)
        ctx.group, ctx.reduce_dx = group, reduce_dx
        width_q = head_dim * num_heads_q
        q, k = rotated.split((width_q, rotated.shape[1] - width_q), dim=-1)
        return q, k, v

    @staticmethod
    def backward(ctx, grad_q, grad_k, grad_v):
        from . import ops

        x, weight_shard, gamma, positions, frequencies_shard, preact, head_mean_sq = ctx.saved_tensors
        ops.lazy_status_check(x.device)
        grad_v = grad_v.contiguous()
        grad_all, dgamma = ops.qknorm_rope_bwd(grad_q.contiguous(), grad_k.contiguous(), grad_v if grad_v.shape[1] > 0 else None, preact,
                                               head_mean_sq, gamma, positions, frequencies_shard, *ctx.args)
        # gamma is shared by every head, so its gradient is summed over the ranks (fp32, 2 * head_dim values)
        dx, dweight = linear_backward_overlapped(grad_all, x, weight_shard, ctx.needs_input_grad[0], ctx.needs_input_grad[1],
                                                 ctx.group, ctx.reduce_dx, also_reduce=dgamma)
        return (dx, dweight, dgamma.to(dtype=gamma.dtype)) + (None,) * 8


def column_parallel_linear_swiglu(x: Tensor, weight_shard: Tensor, group: Optional[dist.ProcessGroup] = None,
                                  reduce_dx: bool = True) -> Tensor:
    """``linear_swiglu(x, weight)[:, this rank's features]`` for ``weight_shard = shard_swiglu_weight(weight, rank, world)``.
    With ``reduce_dx`` the returned ``dx`` is the full input gradient on every rank."""
    return ColumnParallelLinearSwiGLU.apply(x, weight_shard, group, reduce_dx)


def column_parallel_linear_sigmoid(x: Tensor, weight_shard: Tensor, out_dtype: Optional[torch.dtype] = None,
                                   group: Optional[dist.ProcessGroup] = None, reduce_dx: bool = True) -> Tensor:
    """``linear_sigmoid(x, weight)[:, this rank's features]`` for ``weight_shard = shard_rows(weight, rank, world)``."""
    return ColumnParallelLinearSigmoid.apply(x, weight_shard, out_dtype, group, reduce_dx)


def head_parallel_linear_qknorm_rope(x: Tensor, weight_shard: Tensor, gamma: Tensor, positions: Tensor, frequencies_shard: Tensor,
                                     head_dim: int, num_heads_q: int, num_heads_k: int, eps: float,
                                     group: Optional[dist.ProcessGroup] = None, reduce_dx: bool = True):
    """``(q, k, v)`` of this rank's heads; the head counts are the LOCAL ones, ``weight_shard`` and ``frequencies_shard`` come
    from :func:`shard_qkv_weight`.  ``dgamma`` is summed over the ranks, and with ``reduce_dx`` so is ``dx``."""
    return HeadParallelLinearQKNormRope.apply(x, weight_shard, gamma, positions, frequencies_shard, head_dim, num_heads_q, num_heads_k,
                                              eps, group, reduce_dx)
