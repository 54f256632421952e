"""The reference's accuracy shapes (benchmarks/utils/data.py:215-304: odd token counts, ragged ffn / vocabulary,
head_dim 64 and 128, GQA, RoPE from position 2^20) with hard value distributions, all four operators, against the
oracle in fp32 on the same GPU.  The distributions are this repository's own stand-ins for the reference's
"diffuse / outlier / floor / stress" labels, whose generators are not part of the reference tree."""

import functools

import pytest
import torch

from oracle import eager, inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2

SHAPES = {
    "gqa64": dict(tokens=1025, dim=512, ffn=1152, heads=8, kv_heads=2, head_dim=64, vocab=1000, offset=0, dist="random"),
    "mha128-far": dict(tokens=777, dim=1024, ffn=1408, heads=8, kv_heads=8, head_dim=128, vocab=4104, offset=2**20, dist="diffuse"),
    "mha128-outlier": dict(tokens=1031, dim=1024, ffn=1408, heads=8, kv_heads=8, head_dim=128, vocab=4104, offset=0, dist="outlier"),
    "mha128-floor": dict(tokens=1027, dim=1024, ffn=1408, heads=8, kv_heads=8, head_dim=128, vocab=4104, offset=0, dist="floor"),
    "mha128-stress": dict(tokens=1029, dim=1024, ffn=1408, heads=8, kv_heads=8, head_dim=128, vocab=4104, offset=0, dist="stress"),
}


def shape_x(x: torch.Tensor, dist: str) -> torch.Tensor:
    """Re-shape the activation distribution: a few huge entries, values near eps, or both signs of extreme."""
    g = torch.Generator().manual_seed(123)
    x = x.float()
    if dist == "diffuse":
        x = x * 0.05
    elif dist == "outlier":
        mask = torch.rand(x.shape, generator=g) < 1e-3
        x = torch.where(mask, x * 60.0, x)
    elif dist == "floor":
        x = x * 1e-3
    elif dist == "stress":
        mask = torch.rand(x.shape, generator=g) < 1e-3
        x = torch.where(mask, x * 200.0, x * 4.0)
    return x.to(torch.bfloat16)


def leaf(t):
    return t.to(DEV).detach().requires_grad_(True)


def check(pairs, tol=TOL):
    for name, (a, b) in pairs.items():
        assert torch.isfinite(a.float()).all(), f"{name}: non-finite values"
        err = eager.max_rel_err(a, b)
        assert err <= tol, f"{name}: max rel err {err:.3e} > {tol}"


@pytest.mark.parametrize("name", list(SHAPES))
def test_swiglu_and_sigmoid(name):
    import coda_kernels_b200 as ck

    s = SHAPES[name]
    d = inputs.swiglu_inputs(s["tokens"], s["dim"], s["ffn"])
    d["x"] = shape_x(d["x"], s["dist"])
    x, w = leaf(d["x"]), leaf(d["weight"])
    out = ck.linear_swiglu(x, w)
    dx, dw = torch.autograd.grad(out, (x, w), d["dout"].to(DEV))
    (ro,), g = eager.fwd_bwd(eager.linear_swiglu, {"x": d["x"].to(DEV), "weight": d["weight"].to(DEV)}, ["x", "weight"], d["dout"].to(DEV))
    check({"swiglu out": (out, ro), "swiglu dx": (dx, g["x"]), "swiglu dweight": (dw, g["weight"])})
    # sigmoid gate with N = number of heads (the skinny shape the reference benches) and with N = ffn
    for n_out in (s["heads"], s["ffn"]):
        sg = inputs.sigmoid_inputs(s["tokens"], s["dim"], n_out)
        sg["x"] = d["x"]
        x, w = leaf(sg["x"]), leaf(sg["weight"])
        out = ck.linear_sigmoid(x, w)
        dx, dw = torch.autograd.grad(out, (x, w), sg["dout"].to(DEV))
        (ro,), g = eager.fwd_bwd(eager.linear_sigmoid, {"x": sg["x"].to(DEV), "weight": sg["weight"].to(DEV)}, ["x", "weight"], sg["dout"].to(DEV))
        check({f"sigmoid[{n_out}] out": (out, ro), f"sigmoid[{n_out}] dx": (dx, g["x"]), f"sigmoid[{n_out}] dweight": (dw, g["weight"])})
    ck.ops.check_device_status(torch.device(DEV))


@pytest.mark.parametrize("name", list(SHAPES))
def test_cross_entropy(name):
    import coda_kernels_b200 as ck

    s = SHAPES[name]
    d = inputs.cross_entropy_inputs(s["tokens"], s["dim"], s["vocab"], ignore_frac=0.05)
    d["x"] = shape_x(d["x"], s["dist"])
    if s["dist"] in ("floor", "stress"):
        d["weight"] = (d["weight"].float() * 6.0).to(torch.bfloat16)  # confident predictions: logits far apart
    t = d["target"].to(DEV)
    for reduction in ("mean", "sum"):
        x, w = leaf(d["x"]), leaf(d["weight"])
        loss = ck.linear_cross_entropy(x, w, t, -100, reduction)
        dx, dw = torch.autograd.grad(loss, (x, w))
        fwd = ck.linear_cross_entropy_forward(x.detach(), w.detach(), t, -100, reduction)
        fn = functools.partial(eager.linear_cross_entropy, target=t, reduction=reduction)
        (rl,), g = eager.fwd_bwd(fn, {"x": d["x"].to(DEV), "weight": d["weight"].to(DEV)}, ["x", "weight"], torch.tensor(1.0, device=DEV))
        assert abs(float(loss) - float(rl)) <= 1e-3 * abs(float(rl)), f"{reduction} loss {float(loss)} vs {float(rl)}"
        assert abs(float(fwd) - float(rl)) <= 1e-3 * abs(float(rl)), f"{reduction} forward-only loss {float(fwd)} vs {float(rl)}"
        check({"ce dx": (dx, g["x"]), "ce dweight": (dw, g["weight"])})
    ck.ops.check_device_status(torch.device(DEV))


@pytest.mark.parametrize("name", list(SHAPES))
def test_qknorm_rope(name):
    import coda_kernels_b200 as ck

    s = SHAPES[name]
    hd, hq, hk = s["head_dim"], s["heads"], s["kv_heads"]
    d = inputs.qknorm_rope_inputs(s["tokens"], s["dim"], hd, hq, hk, hk, seq_len=4096, pos_offset=s["offset"])
    d["x"] = shape_x(d["x"], s["dist"])
    gen = torch.Generator().manual_seed(5)
    d["gamma"] = torch.exp(torch.empty(2 * hd).uniform_(-1.6, 1.4, generator=gen)).to(torch.bfloat16)  # 0.2 .. 4
    eps = 1e-6
    x, w, gm = leaf(d["x"]), leaf(d["weight"]), leaf(d["gamma"])
    q, k, v = ck.linear_qknorm_rope(x, w, gm, d["positions"].to(DEV), d["frequencies"].to(DEV), hd, hq, hk, eps)
    dx, dw, dg = torch.autograd.grad((q, k, v), (x, w, gm), (d["dq"].to(DEV), d["dk"].to(DEV), d["dv"].to(DEV)))
    fn = functools.partial(eager.linear_qknorm_rope, positions=d["positions"].to(DEV), frequencies=d["frequencies"].to(DEV),
                           head_dim=hd, num_heads_q=hq, num_heads_k=hk, eps=eps)
    outs, g = eager.fwd_bwd(fn, {n: d[n].to(DEV) for n in ("x", "weight", "gamma")}, ["x", "weight", "gamma"],
                            (d["dq"].to(DEV), d["dk"].to(DEV), d["dv"].to(DEV)))
    check({"q": (q, outs[0]), "k": (k, outs[1]), "v": (v, outs[2]), "dx": (dx, g["x"]), "dweight": (dw, g["weight"]), "dgamma": (dg, g["gamma"])})
    ck.ops.check_device_status(torch.device(DEV))
