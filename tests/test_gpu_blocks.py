"""Fused Llama-3 layer blocks (block_pre / block / block_post) on the GPU: golden vectors from the reference's eager
blocks, then a larger ragged GQA layer against the oracle, every output and every gradient."""

import functools

import pytest
import torch

from oracle import eager, inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2
NAMES = ["x0", "y0", "w0", "w1", "w2", "w3", "wn0", "wn1"]


def close(a, b, what, tol=TOL):
    err = eager.max_rel_err(a, b)
    assert err <= tol, f"{what}: max rel err {err:.3e} > {tol}"


def leaf(t):
    return t.to(DEV).detach().requires_grad_(True)


def run_pre(d, eps):
    from coda_kernels_b200.blocks import llama3

    x, w, wn = leaf(d["x0"]), leaf(d["w_qkv"]), leaf(d["wn0"])
    res, qkv = llama3.block_pre(x, w, wn, d["positions"].to(DEV), d["frequencies"].to(DEV), eps)
    grads = torch.autograd.grad((res, qkv), (x, w, wn), (d["dx"].to(DEV).clone(), d["dqkv"].to(DEV)))
    return res, qkv, grads


def run_block(d, eps):
    from coda_kernels_b200.blocks import llama3

    lv = [leaf(d[{"w3": "w_qkv"}.get(n, n)]) for n in NAMES]
    x2, qkv = llama3.block(*lv, d["positions"].to(DEV), d["frequencies"].to(DEV), eps)
    grads = torch.autograd.grad((x2, qkv), lv, (d["dx"].to(DEV).clone(), d["dqkv"].to(DEV)))
    return x2, qkv, dict(zip(NAMES, grads))


def run_post(d, eps, reduction):
    from coda_kernels_b200.blocks import llama3

    lv = [leaf(d[{"w3": "w_vocab"}.get(n, n)]) for n in NAMES]
    loss = llama3.block_post(*lv, d["targets"].to(DEV), eps, -100, reduction)
    grads = torch.autograd.grad(loss, lv)
    return loss, dict(zip(NAMES, grads))


def test_golden(golden_dir):
    from coda_kernels_b200 import ops

    g = torch.load(golden_dir / "llama3_blocks.pt", weights_only=False)
    d = g["inputs"]
    res, qkv, (dx, dw, dwn) = run_pre(d, 1e-5)
    assert res.data_ptr() != d["x0"].data_ptr()
    close(res, g["pre"]["residual"], "pre residual")
    close(qkv, g["pre"]["qkv"], "pre qkv")
    close(dx, g["pre"]["dx"], "pre dx")
    close(dw, g["pre"]["dw"], "pre dw")
    close(dwn, g["pre"]["dwn"], "pre dwn")

    x2, qkv, grads = run_block(d, 1e-5)
    close(x2, g["block"]["x2"], "block x2")
    close(qkv, g["block"]["qkv"], "block qkv")
    for n in NAMES:
        close(grads[n], g["block"]["grads"][{"w3": "w_qkv"}.get(n, n)], f"block d{n}")

    for reduction in ("mean", "sum"):
        loss, grads = run_post(d, 1e-5, reduction)
        ref = g[f"post_{reduction}"]
        assert abs(float(loss.detach()) - float(ref["loss"])) <= 2e-3 * abs(float(ref["loss"])), f"{reduction} loss {float(loss.detach())} vs {float(ref['loss'])}"
        for n in NAMES:
            close(grads[n], ref["grads"][{"w3": "w_vocab"}.get(n, n)], f"post[{reduction}] d{n}")
    torch.cuda.synchronize()
    ops.check_device_status(torch.device(DEV))


def test_gqa_layer_vs_oracle():
    """515 tokens, dim 512, ffn 1032, GQA 8/2 x 64, vocabulary 1000: ragged in every dimension."""
    from coda_kernels_b200 import ops

    eps = 1e-6
    d = inputs.llama3_block_inputs(515, 512, 1032, 64, 8, 2, 1000, seq_len=128, seed=3)
    dev = {k: v.to(DEV) for k, v in d.items()}

    res, qkv, (dx, dw, dwn) = run_pre(d, eps)
    fn = functools.partial(eager.llama3_block_pre, positions=dev["positions"], frequencies=dev["frequencies"], eps=eps)
    outs, g = eager.fwd_bwd(fn, {"x": dev["x0"], "w": dev["w_qkv"], "wn": dev["wn0"]}, ["x", "w", "wn"], (dev["dx"], dev["dqkv"]))
    close(res, outs[0], "pre residual")
    close(qkv, outs[1], "pre qkv")
    close(dx, g["x"], "pre dx")
    close(dw, g["w"], "pre dw")
    close(dwn, g["wn"], "pre dwn")

    x2, qkv, grads = run_block(d, eps)
    fn = functools.partial(eager.llama3_block, positions=dev["positions"], frequencies=dev["frequencies"], eps=eps)
    outs, g = eager.fwd_bwd(fn, {n: dev[{"w3": "w_qkv"}.get(n, n)] for n in NAMES}, NAMES, (dev["dx"], dev["dqkv"]))
    close(x2, outs[0], "block x2")
    close(qkv, outs[1], "block qkv")
    for n in NAMES:
        close(grads[n], g[n], f"block d{n}")

    loss, grads = run_post(d, eps, "mean")
    fn = functools.partial(eager.llama3_block_post, targets=dev["targets"], eps=eps)
    (rl,), g = eager.fwd_bwd(fn, {n: dev[{"w3": "w_vocab"}.get(n, n)] for n in NAMES}, NAMES, torch.tensor(1.0, device=DEV))
    assert abs(float(loss.detach()) - float(rl)) <= 2e-3 * abs(float(rl)), f"loss {float(loss.detach())} vs {float(rl)}"
    for n in NAMES:
        close(grads[n], g[n], f"post d{n}")
    torch.cuda.synchronize()
    ops.check_device_status(torch.device(DEV))
