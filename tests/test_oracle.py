"""The oracle (oracle/eager.py) against the golden vectors produced by the reference's own eager code."""

import functools

import pytest
import torch

from oracle import eager

F64 = torch.float64
CASES_SWIGLU = ["swiglu_small", "swiglu_ragged"]
CASES_CE = ["ce_mean", "ce_sum"]
CASES_QK = ["qk_gqa_d64", "qk_gqa_d128_far", "qk_mha_d64_fpos"]


def load(golden_dir, name):
    return torch.load(golden_dir / f"{name}.pt", weights_only=False)


def close(a, b, tol):
    err = eager.max_rel_err(a, b)
    assert err <= tol, f"max rel err {err:.3e} > {tol:.1e}"


@pytest.mark.parametrize("name", CASES_SWIGLU)
@pytest.mark.parametrize("dtype,tol", [(F64, 1e-12), (torch.float32, 2e-5)])
def test_swiglu(golden_dir, name, dtype, tol):
    g = load(golden_dir, name)
    d = g["inputs"]
    fn = functools.partial(eager.linear_swiglu, compute_dtype=dtype)
    (out,), grads = eager.fwd_bwd(fn, {"x": d["x"].to(dtype), "weight": d["weight"].to(dtype)}, ["x", "weight"], d["dout"])
    close(out, g["out"], tol)
    close(grads["x"], g["dx"], tol)
    close(grads["weight"], g["dweight"], tol)
    # hand-written derivative used by the kernels
    close(eager.dswiglu(g["preact"], d["dout"].to(F64)), g["dpreact"], 1e-12)


def test_sigmoid(golden_dir):
    g = load(golden_dir, "sigmoid_small")
    d = g["inputs"]
    for dtype, tol in ((F64, 1e-12), (torch.float32, 2e-5)):
        fn = functools.partial(eager.linear_sigmoid, compute_dtype=dtype)
        (out,), grads = eager.fwd_bwd(fn, {"x": d["x"].to(dtype), "weight": d["weight"].to(dtype)}, ["x", "weight"], d["dout"])
        close(out, g["out"], tol)
        close(grads["x"], g["dx"], tol)
        close(grads["weight"], g["dweight"], tol)


@pytest.mark.parametrize("name", CASES_CE)
def test_cross_entropy(golden_dir, name):
    g = load(golden_dir, name)
    d = g["inputs"]
    for dtype, tol in ((F64, 1e-12), (torch.float32, 2e-5)):
        fn = functools.partial(eager.linear_cross_entropy, target=d["target"], reduction=g["reduction"], compute_dtype=dtype, chunk_rows=16)
        (loss,), grads = eager.fwd_bwd(fn, {"x": d["x"].to(dtype), "weight": d["weight"].to(dtype)}, ["x", "weight"], torch.tensor(1.0))
        close(loss, g["loss"], tol)
        close(grads["x"], g["dx"], tol)
        close(grads["weight"], g["dweight"], tol)
    logits = d["x"].to(F64) @ d["weight"].to(F64).mT
    losses, dlogits = eager.cross_entropy_rows(logits, d["target"], -100)
    close(losses, g["row_losses"], 1e-12)
    close(dlogits, g["dlogits"], 1e-12)
    close(losses, g["select_losses"], 1e-12)
    # masking is exact: ignored rows give exactly zero loss and gradient
    ignored = d["target"] == -100
    assert ignored.any()
    assert (losses[ignored] == 0).all() and (dlogits[ignored] == 0).all()
    assert (g["row_losses"][ignored] == 0).all() and (g["dlogits"][ignored] == 0).all()


@pytest.mark.parametrize("name", CASES_QK)
def test_qknorm_rope(golden_dir, name):
    g = load(golden_dir, name)
    d, cfg = g["inputs"], g["cfg"]
    for dtype, tol in ((F64, 1e-9), (torch.float32, 5e-5)):  # fp64 at position 2^20: the order of the angle product shows at 1e-10
        fn = functools.partial(
            eager.linear_qknorm_rope, positions=d["positions"], frequencies=d["frequencies"], head_dim=cfg["head_dim"],
            num_heads_q=cfg["hq"], num_heads_k=cfg["hk"], eps=cfg["eps"], compute_dtype=dtype,
        )
        outs, grads = eager.fwd_bwd(
            fn, {"x": d["x"].to(dtype), "weight": d["weight"].to(dtype), "gamma": d["gamma"].to(dtype)}, ["x", "weight", "gamma"],
            (d["dq"], d["dk"], d["dv"]),
        )
        for o, ref in zip(outs, (g["q"], g["k"], g["v"])):
            close(o, ref, tol)
        close(grads["x"], g["dx"], tol)
        close(grads["weight"], g["dweight"], tol)
        close(grads["gamma"], g["dgamma"], tol)
    # the reference's hand-written backward agrees with autograd on dgamma
    close(g["dgamma_bwd"], g["dgamma"], 1e-10)


def test_rstd_variants(golden_dir):
    """Deferred-RMSNorm forms of the three fused GEMMs against the reference's eager ops."""
    g = load(golden_dir, "rstd_variants")
    cfg, qk = g["cfg"], g["qk_inputs"]
    for dtype, tol in ((F64, 1e-9), (torch.float32, 5e-5)):
        pre, post = eager.gemm_rmsnorm_swiglu(g["x"], g["w_swiglu"].mT, g["rstd"], compute_dtype=dtype)
        close(pre, g["swiglu_pre"], tol)
        close(post, g["swiglu_post"], tol)
        logits, lse = eager.gemm_rmsnorm_lse(g["x"], g["w_vocab"].mT, g["rstd"], compute_dtype=dtype)
        close(lse, g["lse"], tol)
        losses, dlogits = eager.cross_entropy_rows(logits, g["target"], -100)
        close(losses, g["row_losses"], tol)
        close(dlogits, g["dlogits"], tol)
        rot, preact, ms = eager.gemm_rmsnorm_qknorm_rope(
            g["x"], qk["weight"].mT, g["rstd"], qk["gamma"], qk["positions"], qk["frequencies"], cfg["head_dim"], cfg["hq"], cfg["hk"],
            cfg["eps"], compute_dtype=dtype)
        close(rot, g["qk_rotated"], tol)
        close(preact, g["qk_preact"], tol)
        close(ms, g["qk_mean_sq"], tol)
    assert torch.allclose(eager.rmsnorm_rstd(g["x"], 1e-5, F64).float(), g["rstd"])


def test_block_gemms(golden_dir):
    """Residual + partial RMSNorm (forward, backward) and the SwiGLU dgrad against the reference's eager ops."""
    g = load(golden_dir, "block_gemms")
    for dtype, tol in ((F64, 1e-10), (torch.float32, 5e-5)):
        pre, post, rstd = eager.gemm_residual_partial_rmsnorm(g["A"], g["B"], g["C"], g["weight"], g["eps"], compute_dtype=dtype)
        close(pre, g["pre"], tol)
        close(post, g["post"], tol)
        close(rstd, g["rstd"], tol)
        for key, al, dx in (("plain", None, None), ("alpha_accum", g["alpha"], g["dX0"])):
            dX, dW, normed = eager.gemm_residual_partial_rmsnorm_bwd(
                g["A2"], g["B2"], g["weight"], g["pre_bf16"], g["zdz"], g["rstd32"], alpha=al, dX=dx, compute_dtype=dtype)
            close(dX, g["bwd"][key]["dX"], tol)
            close(dW, g["bwd"][key]["dW"], tol)
            close(normed, g["bwd"][key]["normed"], tol)
        for key, sc in (("plain", None), ("scaled", 0.125)):
            dZ, ZdZ, postact = eager.gemm_swiglu_bwd_zdz(g["A3"], g["B3"], g["Z"], scale=sc, compute_dtype=dtype)
            close(dZ, g["swiglu_bwd"][key]["dZ"], tol)
            close(ZdZ, g["swiglu_bwd"][key]["ZdZ"], tol)
            close(postact, g["swiglu_bwd"][key]["postact"], tol)


def test_llama3_blocks(golden_dir):
    """The oracle's Llama-3 layer blocks against the reference's eager blocks (forward and every gradient)."""
    g = load(golden_dir, "llama3_blocks")
    d = g["inputs"]
    pos, freq = d["positions"], d["frequencies"]
    for dtype, tol in ((F64, 1e-9), (torch.float32, 1e-4)):
        fn = functools.partial(eager.llama3_block_pre, positions=pos, frequencies=freq, eps=1e-5, compute_dtype=dtype)
        outs, grads = eager.fwd_bwd(fn, {"x": d["x0"].to(dtype), "w": d["w_qkv"].to(dtype), "wn": d["wn0"].to(dtype)}, ["x", "w", "wn"],
                                    (d["dx"], d["dqkv"]))
        close(outs[0], g["pre"]["residual"], tol)
        close(outs[1], g["pre"]["qkv"], tol)
        close(grads["x"], g["pre"]["dx"], tol)
        close(grads["w"], g["pre"]["dw"], tol)
        close(grads["wn"], g["pre"]["dwn"], tol)

        names = ["x0", "y0", "w0", "w1", "w2", "w3", "wn0", "wn1"]
        src = {"w3": "w_qkv"}
        fn = functools.partial(eager.llama3_block, positions=pos, frequencies=freq, eps=1e-5, compute_dtype=dtype)
        outs, grads = eager.fwd_bwd(fn, {n: d[src.get(n, n)].to(dtype) for n in names}, names, (d["dx"], d["dqkv"]))
        close(outs[0], g["block"]["x2"], tol)
        close(outs[1], g["block"]["qkv"], tol)
        for n in names:
            close(grads[n], g["block"]["grads"][src.get(n, n)], tol)

        src = {"w3": "w_vocab"}
        for reduction in ("mean", "sum"):
            fn = functools.partial(eager.llama3_block_post, targets=d["targets"], eps=1e-5, reduction=reduction, compute_dtype=dtype)
            (loss,), grads = eager.fwd_bwd(fn, {n: d[src.get(n, n)].to(dtype) for n in names}, names, torch.tensor(1.0))
            close(loss, g[f"post_{reduction}"]["loss"], tol)
            for n in names:
                close(grads[n], g[f"post_{reduction}"]["grads"][src.get(n, n)], tol)
