"""The call sequences of the reference's own autograd wrappers (coda/kernels/functional/qknorm_rope.py:27-112 and
cross_entropy.py:25-47, 73-89), issued against the drop-in modules ``coda.core.gemm.functional`` /
``coda.core.elementwise.functional``: row-sliced weight views, ``out=`` slices, an fp32 partial and ``C=`` accumulation."""

import functools

import pytest
import torch

from oracle import eager, inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2


def close(a, b, what, tol=TOL):
    err = eager.max_rel_err(a, b)
    assert err <= tol, f"{what}: max rel err {err:.3e} > {tol}"


def test_qknorm_rope_wrapper_sequence():
    from coda.core.elementwise.functional import qknorm_rope_bwd
    from coda.core.gemm.functional import gemm, gemm_qknorm_rope

    hd, hq, hk, hv = 128, 4, 2, 2
    d = {k: v.to(DEV) for k, v in inputs.qknorm_rope_inputs(300, 264, hd, hq, hk, hv, seq_len=64).items()}
    x, weight, gamma = d["x"], d["weight"], d["gamma"]
    size_q, size_qk = hd * hq, hd * (hq + hk)
    # forward, as LinearQKNormRope.forward does
    qk, preact, head_mean_sq = gemm_qknorm_rope(x, weight[:size_qk, :].mT, weight=gamma, positions=d["positions"],
                                                frequencies=d["frequencies"], head_dim=hd, num_heads_q=hq, num_heads_k=hk, eps=1e-6)
    v = gemm(x, weight[size_qk:, :].mT)
    q, k = qk.split((size_q, size_qk - size_q), dim=-1)
    # backward, as LinearQKNormRope.backward does
    grad_pre, dgamma = qknorm_rope_bwd(dq=d["dq"], dk=d["dk"], x=preact, head_mean_sq=head_mean_sq, gamma=gamma, pos=d["positions"],
                                       freq=d["frequencies"], head_dim=hd, num_heads_q=hq, num_heads_k=hk, eps=1e-6)
    partial = torch.empty_like(x, dtype=torch.float32)
    gemm(grad_pre, weight[:size_qk, :], out=partial)
    dx = gemm(d["dv"], weight[size_qk:, :], C=partial)
    dweight = torch.empty_like(weight)
    gemm(grad_pre.mT, x, out=dweight[:size_qk, :])
    gemm(d["dv"].mT, x, out=dweight[size_qk:, :])
    dgamma = dgamma.to(dtype=gamma.dtype)

    fn = functools.partial(eager.linear_qknorm_rope, positions=d["positions"], frequencies=d["frequencies"], head_dim=hd,
                           num_heads_q=hq, num_heads_k=hk, eps=1e-6)
    outs, g = eager.fwd_bwd(fn, {n: d[n] for n in ("x", "weight", "gamma")}, ["x", "weight", "gamma"], (d["dq"], d["dk"], d["dv"]))
    for a, b, n in zip((q, k, v), outs, "qkv"):
        close(a, b, n)
    close(dx, g["x"], "dx")
    close(dweight, g["weight"], "dweight")
    close(dgamma, g["gamma"], "dgamma")


def test_cross_entropy_wrapper_sequence():
    from coda.core.elementwise.functional import cross_entropy_fwd_bwd
    from coda.core.gemm.functional import gemm_lse, gemm_lse_select_logits, gemm_scalar_scale

    d = {k: v.to(DEV) for k, v in inputs.cross_entropy_inputs(520, 264, 1000, ignore_frac=0.1).items()}
    x, weight, target = d["x"], d["weight"], d["target"]
    # _forward_lse
    logits, lses = gemm_lse(x, weight.mT)
    losses, _ = cross_entropy_fwd_bwd(logits=logits, lses=lses, target=target, ignore_index=-100)
    scale = 1.0 / (target != -100).sum().float()
    loss = losses.sum() * scale
    # _backward_dlogits with dloss = 1
    dloss_scaled = torch.ones((), device=DEV) * scale
    dx = gemm_scalar_scale(logits, weight, alpha=dloss_scaled)
    dweight = gemm_scalar_scale(logits.mT, x, alpha=dloss_scaled)
    # linear_cross_entropy_forward
    sel_losses, sel_lse, _ = gemm_lse_select_logits(x, weight.mT, target=target, ignore_index=-100, return_lse=False)
    assert sel_lse is None

    fn = functools.partial(eager.linear_cross_entropy, target=target)
    (rl,), g = eager.fwd_bwd(fn, {"x": x, "weight": weight}, ["x", "weight"], torch.tensor(1.0, device=DEV))
    assert abs(float(loss) - float(rl)) <= 5e-3 * abs(float(rl))  # target logit read from bf16 logits, as in the reference
    assert abs(float(sel_losses.sum() * scale) - float(rl)) <= 1e-3 * abs(float(rl))
    close(dx, g["x"], "dx")
    close(dweight, g["weight"], "dweight")
