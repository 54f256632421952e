"""The four benchmark configurations at FULL size against the oracle evaluated in fp32 on the same GPU.

These are the shapes the throughput numbers are quoted on.  The oracle runs as
plain PyTorch fp32 matmuls + autograd on the device (TF32 off), so the check
covers every row and column, including the tile-scheduler's whole range.
"""

import functools
import gc

import pytest
import torch

from oracle import eager, inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2


@pytest.fixture(autouse=True)
def _fp32_matmul_and_cleanup():
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = prev
    gc.collect()
    torch.cuda.empty_cache()


def leaf(t):
    return t.to(DEV).detach().requires_grad_(True)


def check(pairs):
    """Normalised max-abs error within TOL, and relative L2 error within 2 x (outputs) or 3 x (gradients, which pass through
    one more bf16 tensor) the bf16 rounding floor of the oracle (benchmarks/utils/numerics.py:20-29, 81-85 of the reference)."""
    worst = {}
    for name, (a, b) in pairs.items():
        err = eager.max_rel_err(a, b)
        l2 = eager.rel_l2_err(a, b)
        worst[name] = (err, l2)
        assert err <= TOL, f"{name}: max rel err {err:.3e} > {TOL}"
        floor = eager.rounding_floor(b, torch.bfloat16)
        factor = 3.0 if name.startswith("d") else 2.0
        assert l2 <= factor * floor + 1e-6, f"{name}: rel L2 {l2:.3e} > {factor} x the bf16 rounding floor {floor:.3e}"
    return worst


def test_swiglu_llama3_8b_mlp():
    import coda_kernels_b200 as ck

    d = inputs.swiglu_inputs(16384, 4096, 14336)
    x, w = leaf(d["x"]), leaf(d["weight"])
    out = ck.linear_swiglu(x, w)
    dx, dw = torch.autograd.grad(out, (x, w), d["dout"].to(DEV))
    (ro,), g = eager.fwd_bwd(eager.linear_swiglu, {"x": d["x"].to(DEV), "weight": d["weight"].to(DEV)}, ["x", "weight"], d["dout"].to(DEV))
    check({"out": (out, ro), "dx": (dx, g["x"]), "dweight": (dw, g["weight"])})
    ck.ops.check_device_status(torch.device(DEV))


def test_sigmoid_large():
    import coda_kernels_b200 as ck

    d = inputs.sigmoid_inputs(32768, 5120, 5120)
    x, w = leaf(d["x"]), leaf(d["weight"])
    out = ck.linear_sigmoid(x, w)
    dx, dw = torch.autograd.grad(out, (x, w), d["dout"].to(DEV))
    (ro,), g = eager.fwd_bwd(eager.linear_sigmoid, {"x": d["x"].to(DEV), "weight": d["weight"].to(DEV)}, ["x", "weight"], d["dout"].to(DEV))
    check({"out": (out, ro), "dx": (dx, g["x"]), "dweight": (dw, g["weight"])})


def test_cross_entropy_llama3_vocab():
    import coda_kernels_b200 as ck

    d = inputs.cross_entropy_inputs(8192, 4096, 128256)
    t = d["target"].to(DEV)
    x, w = leaf(d["x"]), leaf(d["weight"])
    loss = ck.linear_cross_entropy(x, w, t, -100, "mean")
    dx, dw = torch.autograd.grad(loss, (x, w))
    fwd_only = ck.linear_cross_entropy_forward(x.detach(), w.detach(), t, -100, "mean")
    fn = functools.partial(eager.linear_cross_entropy, target=t, reduction="mean")
    (rl,), g = eager.fwd_bwd(fn, {"x": d["x"].to(DEV), "weight": d["weight"].to(DEV)}, ["x", "weight"], torch.tensor(1.0, device=DEV))
    assert abs(float(loss) - float(rl)) <= 1e-3 * abs(float(rl)), f"loss {float(loss)} vs {float(rl)}"
    assert abs(float(fwd_only) - float(rl)) <= 1e-3 * abs(float(rl)), f"forward-only loss {float(fwd_only)} vs {float(rl)}"
    check({"dx": (dx, g["x"]), "dweight": (dw, g["weight"])})
    # masking stays exact at full size: weight rows never used as a label and ignored rows do not leak
    losses, dlogits = ck.ops.gemm_lse_dlogits(d["x"].to(DEV), d["weight"].to(DEV).mT, t, -100)
    ignored = t == -100
    assert int(ignored.sum()) > 0
    assert (losses[ignored] == 0).all() and (dlogits[ignored].view(torch.int16) == 0).all()
    del dlogits


def test_qknorm_rope_llama3_8b_gqa():
    import coda_kernels_b200 as ck

    hd, hq, hk, hv = 128, 32, 8, 8
    d = inputs.qknorm_rope_inputs(16384, 4096, hd, hq, hk, hv, seq_len=4096)
    x, w, gm = leaf(d["x"]), leaf(d["weight"]), leaf(d["gamma"])
    q, k, v = ck.linear_qknorm_rope(x, w, gm, d["positions"].to(DEV), d["frequencies"].to(DEV), hd, hq, hk, 1e-6)
    dx, dw, dg = torch.autograd.grad((q, k, v), (x, w, gm), (d["dq"].to(DEV), d["dk"].to(DEV), d["dv"].to(DEV)))
    fn = functools.partial(eager.linear_qknorm_rope, positions=d["positions"].to(DEV), frequencies=d["frequencies"].to(DEV),
                           head_dim=hd, num_heads_q=hq, num_heads_k=hk, eps=1e-6)
    outs, g = eager.fwd_bwd(fn, {n: d[n].to(DEV) for n in ("x", "weight", "gamma")}, ["x", "weight", "gamma"],
                            (d["dq"].to(DEV), d["dk"].to(DEV), d["dv"].to(DEV)))
    check({"q": (q, outs[0]), "k": (k, outs[1]), "v": (v, outs[2]), "dx": (dx, g["x"]), "dweight": (dw, g["weight"]),
           "dgamma": (dg, g["gamma"])})
    ck.ops.check_device_status(torch.device(DEV))
