"""The operators trace under ``torch.compile(fullgraph=True)``, as the reference's harness runs every implementation
(benchmarks/utils/cases.py:312-343): custom ops with fake implementations inside ``autograd.Function``s."""

import pytest
import torch

from oracle import eager, inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_swiglu_and_cross_entropy_under_compile():
    import coda_kernels_b200 as ck

    d = inputs.swiglu_inputs(256, 128, 128)
    x = d["x"].to(DEV).requires_grad_(True)
    w = d["weight"].to(DEV).requires_grad_(True)

    # forward compiled as one graph, backward through the graph AOTAutograd built from the Function's backward
    fwd = torch.compile(ck.linear_swiglu, fullgraph=True, dynamic=False)
    out = fwd(x, w)
    dx, dw = torch.autograd.grad(out, (x, w), d["dout"].to(DEV))
    (ro,), g = eager.fwd_bwd(eager.linear_swiglu, {"x": d["x"].to(DEV), "weight": d["weight"].to(DEV)}, ["x", "weight"], d["dout"].to(DEV))
    assert eager.max_rel_err(out, ro) <= 2e-2
    assert eager.max_rel_err(dx, g["x"]) <= 2e-2
    assert eager.max_rel_err(dw, g["weight"]) <= 2e-2

    c = inputs.cross_entropy_inputs(128, 128, 512)
    loss_fn = torch.compile(ck.linear_cross_entropy_forward, fullgraph=True, dynamic=False)
    loss = loss_fn(c["x"].to(DEV), c["weight"].to(DEV), c["target"].to(DEV))
    ref = eager.linear_cross_entropy(c["x"].to(DEV), c["weight"].to(DEV), c["target"].to(DEV))
    assert abs(float(loss) - float(ref)) <= 1e-3 * abs(float(ref))


def test_cross_entropy_qknorm_sigmoid_under_compile():
    """The remaining operators: forward compiled as one graph, backward through the graph built from their ``backward``."""
    import functools

    import coda_kernels_b200 as ck

    # cross entropy with autograd
    c = inputs.cross_entropy_inputs(192, 128, 520, ignore_frac=0.1)
    x = c["x"].to(DEV).requires_grad_(True)
    w = c["weight"].to(DEV).requires_grad_(True)
    t = c["target"].to(DEV)
    ce = torch.compile(ck.linear_cross_entropy, fullgraph=True, dynamic=False)
    loss = ce(x, w, t)
    dx, dw = torch.autograd.grad(loss, (x, w))
    fn = functools.partial(eager.linear_cross_entropy, target=t)
    (rl,), g = eager.fwd_bwd(fn, {"x": c["x"].to(DEV), "weight": c["weight"].to(DEV)}, ["x", "weight"], torch.tensor(1.0, device=DEV))
    assert abs(float(loss) - float(rl)) <= 1e-3 * abs(float(rl))
    assert eager.max_rel_err(dx, g["x"]) <= 2e-2 and eager.max_rel_err(dw, g["weight"]) <= 2e-2

    # qk-norm + rope (GQA) with autograd
    d = inputs.qknorm_rope_inputs(160, 128, 128, 2, 1, 1, seq_len=64)
    x, w, gm = (d[n].to(DEV).requires_grad_(True) for n in ("x", "weight", "gamma"))
    qk = torch.compile(ck.linear_qknorm_rope, fullgraph=True, dynamic=False)
    q, k, v = qk(x, w, gm, d["positions"].to(DEV), d["frequencies"].to(DEV), 128, 2, 1, 1e-6)
    grads = torch.autograd.grad((q, k, v), (x, w, gm), (d["dq"].to(DEV), d["dk"].to(DEV), d["dv"].to(DEV)))
    fn = functools.partial(eager.linear_qknorm_rope, positions=d["positions"].to(DEV), frequencies=d["frequencies"].to(DEV),
                           head_dim=128, num_heads_q=2, num_heads_k=1, eps=1e-6)
    outs, g = eager.fwd_bwd(fn, {n: d[n].to(DEV) for n in ("x", "weight", "gamma")}, ["x", "weight", "gamma"],
                            (d["dq"].to(DEV), d["dk"].to(DEV), d["dv"].to(DEV)))
    for a, b in zip((q, k, v), outs):
        assert eager.max_rel_err(a, b) <= 2e-2
    for a, n in zip(grads, ("x", "weight", "gamma")):
        assert eager.max_rel_err(a, g[n]) <= 2e-2

    # sigmoid
    s = inputs.sigmoid_inputs(128, 128, 136)
    x, w = s["x"].to(DEV).requires_grad_(True), s["weight"].to(DEV).requires_grad_(True)
    sg = torch.compile(ck.linear_sigmoid, fullgraph=True, dynamic=False)
    out = sg(x, w)
    dx, dw = torch.autograd.grad(out, (x, w), s["dout"].to(DEV))
    (ro,), g = eager.fwd_bwd(eager.linear_sigmoid, {"x": s["x"].to(DEV), "weight": s["weight"].to(DEV)}, ["x", "weight"], s["dout"].to(DEV))
    assert eager.max_rel_err(out, ro) <= 2e-2 and eager.max_rel_err(dx, g["x"]) <= 2e-2 and eager.max_rel_err(dw, g["weight"]) <= 2e-2
