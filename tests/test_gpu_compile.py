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
