"""Generates the golden vectors under tests/golden/ from the reference's own eager implementation.

Run where the reference tree is available, passing its path:

    python tests/golden/make_golden.py /path/to/reference

It imports ``benchmarks/backends/torch_linear.py`` and ``torch_ops.py`` of the
reference unmodified, evaluates every operator of the hot path forward and
backward in fp64 on small seeded bf16 inputs, and stores inputs, outputs and
gradients in one ``.pt`` file per case.  The files are small (tens of KB) and
are committed; the reference itself is never copied.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("CODA_REFERENCE", "reference")).resolve()
sys.path.insert(0, str(REF))
sys.path.insert(0, str(REPO))

from benchmarks.backends import torch_linear, torch_ops  # noqa: E402  (reference code)

from oracle import inputs as synth  # noqa: E402

F64 = torch.float64
IL = torch_ops.PairLayout.interleaved


def leaf(t):
    return t.detach().to(dtype=F64).requires_grad_(True)


def save(name, payload):
    torch.save(payload, HERE / f"{name}.pt")
    print(f"wrote {name}.pt")


def swiglu_case(name, M, K, Fdim, seed):
    d = synth.swiglu_inputs(M, K, Fdim, seed)
    x, w = leaf(d["x"]), leaf(d["weight"])
    out = torch_linear.linear_swiglu(x, w, layout=IL)
    dx, dw = torch.autograd.grad(out, (x, w), d["dout"].to(F64))
    preact = (x @ w.mT).detach()
    dpre, post = torch_ops.dswiglu(preact, d["dout"].to(F64), IL)
    save(name, {"inputs": d, "out": out.detach(), "dx": dx, "dweight": dw, "preact": preact, "dpreact": dpre, "postact": post})


def sigmoid_case(name, M, K, N, seed):
    d = synth.sigmoid_inputs(M, K, N, seed)
    x, w = leaf(d["x"]), leaf(d["weight"])
    out = torch_linear.linear_sigmoid(x, w)
    dx, dw = torch.autograd.grad(out, (x, w), d["dout"].to(F64))
    save(name, {"inputs": d, "out": out.detach(), "dx": dx, "dweight": dw})


def ce_case(name, M, K, V, seed, reduction, ignore_frac):
    d = synth.cross_entropy_inputs(M, K, V, seed, ignore_frac=ignore_frac)
    x, w = leaf(d["x"]), leaf(d["weight"])
    tgt = d["target"].long()
    loss = torch_linear.linear_cross_entropy(x, w, tgt, logits_dtype=F64, ignore_index=-100, reduction=reduction)
    dx, dw = torch.autograd.grad(loss, (x, w))
    logits = (x @ w.mT).detach()
    losses, dlogits = torch_ops.cross_entropy(logits, tgt, -100)
    margins, lses, tlog = torch_ops.gemm_lse_select_logits(x.detach(), w.detach().mT, tgt, -100, logits_dtype=F64)
    save(name, {"inputs": d, "reduction": reduction, "loss": loss.detach(), "dx": dx, "dweight": dw, "row_losses": losses,
                "dlogits": dlogits, "select_losses": margins, "lse": lses, "target_logit": tlog})


def qk_case(name, M, K, d_, hq, hk, hv, seq, seed, pos_offset, float_pos=False):
    d = synth.qknorm_rope_inputs(M, K, d_, hq, hk, hv, seq, seed=seed, pos_offset=pos_offset)
    if float_pos:
        d["positions"] = d["positions"].to(torch.float32)
    x, w, g = leaf(d["x"]), leaf(d["weight"]), leaf(d["gamma"])
    freq = d["frequencies"].to(F64)
    pos = d["positions"].to(F64)
    q, k, v = torch_linear.linear_qknorm_rope(x, w, g, cos=None, sin=None, positions=pos, frequencies=freq, head_dim=d_,
                                              num_heads_q=hq, num_heads_k=hk, eps=1e-6, layout=IL)
    dx, dw, dg = torch.autograd.grad((q, k, v), (x, w, g), (d["dq"].to(F64), d["dk"].to(F64), d["dv"].to(F64)))
    size_qk = (hq + hk) * d_
    preact = (x @ w[:size_qk].mT).detach()
    ms = torch_ops.head_mean_square(preact, d_)
    gpre, dgam = torch_ops.qknorm_rope_bwd(d["dq"].to(F64), d["dk"].to(F64), preact, ms, g.detach(), cos=None, sin=None, pos=pos,
                                           freq=freq, head_dim=d_, num_heads_q=hq, num_heads_k=hk, eps=1e-6, layout=IL)
    save(name, {"inputs": d, "cfg": {"head_dim": d_, "hq": hq, "hk": hk, "hv": hv, "eps": 1e-6}, "q": q.detach(), "k": k.detach(),
                "v": v.detach(), "dx": dx, "dweight": dw, "dgamma": dg, "preact": preact, "mean_sq": ms, "grad_pre": gpre,
                "dgamma_bwd": dgam})


def rstd_case(name, M, K, Fdim, V, d_, hq, hk, seed):
    """The deferred-RMSNorm variants of the three fused GEMMs, from the reference's eager ops (run in fp64)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    rstd = torch_ops.rmsnorm_rstd(x.to(F64), 1e-5).to(torch.float32)
    w_sw = (torch.randn(2 * Fdim, K, generator=g) / K**0.5).to(torch.bfloat16)
    w_v = (torch.randn(V, K, generator=g) / K**0.5).to(torch.bfloat16)
    qk = synth.qknorm_rope_inputs(M, K, d_, hq, hk, 0, seq_len=M, seed=seed + 1)
    target = torch.randint(0, V, (M,), generator=g).to(torch.int32)
    target[::5] = -100
    pre, post = torch_ops.gemm_rmsnorm_swiglu(x.to(F64), w_sw.to(F64).mT, rstd.to(F64), IL)
    logits, lses = torch_ops.gemm_rmsnorm_lse(x.to(F64), w_v.to(F64).mT, rstd.to(F64), logits_dtype=F64)
    losses, dlogits = torch_ops.cross_entropy(logits, target.long(), -100)
    rot, preact, ms = torch_ops.gemm_rmsnorm_qknorm_rope(
        x.to(F64), qk["weight"].to(F64).mT, rstd.to(F64), qk["gamma"].to(F64), cos=None, sin=None, positions=qk["positions"].to(F64),
        frequencies=qk["frequencies"].to(F64), head_dim=d_, num_heads_q=hq, num_heads_k=hk, eps=1e-6, layout=IL)
    save(name, {"x": x, "rstd": rstd, "w_swiglu": w_sw, "w_vocab": w_v, "target": target, "qk_inputs": qk,
                "cfg": {"head_dim": d_, "hq": hq, "hk": hk, "eps": 1e-6}, "swiglu_pre": pre, "swiglu_post": post, "lse": lses,
                "row_losses": losses, "dlogits": dlogits, "qk_rotated": rot, "qk_preact": preact, "qk_mean_sq": ms})


def block_case(name, M, K, N, Fdim, seed):
    """The GEMMs between the operators: residual + partial RMSNorm (forward, backward) and the SwiGLU dgrad."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s_, std=1.0: (torch.randn(*s_, generator=g) * std).to(torch.bfloat16)  # noqa: E731
    A, B, C = rn(M, K), rn(K, N, std=K**-0.5), rn(M, N)
    weight = (1.0 + 0.1 * torch.randn(N, generator=g)).to(torch.bfloat16)
    pre, post, rstd = torch_ops.gemm_residual_partial_rmsnorm(A.to(F64), B.to(F64), C.to(F64), weight.to(F64), 1e-5)
    # backward: dgrad of the next GEMM, A2 [M, K2] @ B2 [N, K2]^T
    A2, B2 = rn(M, K), rn(N, K, std=K**-0.5)
    zdz = torch.randn(M, generator=g).to(torch.float32)
    alpha = torch.tensor(0.37, dtype=torch.float32)
    dX0 = rn(M, N)
    pre_bf = pre.to(torch.bfloat16)
    rstd32 = rstd.to(torch.float32)
    outs = {}
    for key, al, dx in (("plain", None, None), ("alpha_accum", alpha, dX0)):
        dpre, dw, normed = torch_ops.gemm_residual_partial_rmsnorm_bwd(
            A2.to(F64), B2.to(F64), weight.to(F64), pre_bf.to(F64), zdz.to(F64), rstd32.to(F64),
            alpha=None if al is None else al.to(F64), dX=None if dx is None else dx.to(F64))
        outs[key] = {"dX": dpre, "dW": dw, "normed": normed}
    # swiglu dgrad: A3 [M, K] @ B3 [F, K]^T, Z [M, 2F]
    A3, B3, Z = rn(M, K), rn(Fdim, K, std=K**-0.5), rn(M, 2 * Fdim)
    sw = {}
    for key, sc in (("plain", None), ("scaled", 0.125)):
        dZ, ZdZ, postact = torch_ops.gemm_swiglu_bwd_zdz(A3.to(F64), B3.to(F64), Z.to(F64), IL, scale=sc)
        sw[key] = {"dZ": dZ, "ZdZ": ZdZ, "postact": postact}
    save(name, {"A": A, "B": B, "C": C, "weight": weight, "eps": 1e-5, "pre": pre, "post": post, "rstd": rstd, "A2": A2, "B2": B2,
                "zdz": zdz, "alpha": alpha, "dX0": dX0, "pre_bf16": pre_bf, "rstd32": rstd32, "bwd": outs, "A3": A3, "B3": B3,
                "Z": Z, "swiglu_bwd": sw})


def llama3_blocks_case(name, M, dim, ffn, head_dim, heads, vocab, seed):
    """block_pre / block / block_post of a Llama-3 layer from the reference's eager blocks (MHA: that code splits qkv in thirds)."""
    import importlib.machinery
    import importlib.util

    # the file's name ends in ",py" (a comma), so it has to be loaded by path with an explicit source loader
    loader = importlib.machinery.SourceFileLoader("ref_torch_blocks", str(REF / "benchmarks" / "backends" / "torch_blocks,py"))
    spec = importlib.util.spec_from_loader("ref_torch_blocks", loader)
    tb = importlib.util.module_from_spec(spec)
    loader.exec_module(tb)
    d = synth.llama3_block_inputs(M, dim, ffn, head_dim, heads, heads, vocab, seq_len=M, seed=seed)
    cos, sin = torch_ops.rope_tables(d["positions"].to(F64), d["frequencies"][:head_dim].to(F64))
    n_qk = 2 * heads * head_dim
    out = {"inputs": d, "cfg": {"head_dim": head_dim, "heads": heads, "eps": 1e-5}}

    x, w, wn = leaf(d["x0"]), leaf(d["w_qkv"]), leaf(d["wn0"])
    res, qk, v = tb.block_pre(x, w, wn, cos, sin, head_dim, IL, 1e-5)
    grads = torch.autograd.grad((res, qk, v), (x, w, wn), (d["dx"].to(F64), d["dqkv"][:, :n_qk].to(F64), d["dqkv"][:, n_qk:].to(F64)))
    out["pre"] = {"residual": res.detach(), "qkv": torch.cat((qk, v), dim=1).detach(), "dx": grads[0], "dw": grads[1], "dwn": grads[2]}

    names = ("x0", "y0", "w0", "w1", "w2", "w_qkv", "wn0", "wn1")
    lv = [leaf(d[n]) for n in names]
    x2, qk, v = tb.block(*lv, cos, sin, head_dim, IL, IL, 1e-5)
    grads = torch.autograd.grad((x2, qk, v), lv, (d["dx"].to(F64), d["dqkv"][:, :n_qk].to(F64), d["dqkv"][:, n_qk:].to(F64)))
    out["block"] = {"x2": x2.detach(), "qkv": torch.cat((qk, v), dim=1).detach(), "grads": dict(zip(names, grads))}

    names = ("x0", "y0", "w0", "w1", "w2", "w_vocab", "wn0", "wn1")
    for reduction in ("mean", "sum"):
        lv = [leaf(d[n]) for n in names]
        lv3 = [lv[0][None], lv[1][None]] + lv[2:]
        loss = tb.block_post(*lv3, d["targets"][None].long(), IL, 1e-5, F64, -100, reduction)
        grads = torch.autograd.grad(loss, lv)
        out[f"post_{reduction}"] = {"loss": loss.detach(), "grads": dict(zip(names, grads))}
    save(name, out)


if __name__ == "__main__":
    torch.manual_seed(0)
    swiglu_case("swiglu_small", 48, 64, 40, seed=1)
    swiglu_case("swiglu_ragged", 37, 72, 24, seed=2)
    sigmoid_case("sigmoid_small", 40, 64, 48, seed=3)
    ce_case("ce_mean", 40, 64, 304, seed=4, reduction="mean", ignore_frac=0.2)
    ce_case("ce_sum", 33, 72, 520, seed=5, reduction="sum", ignore_frac=0.1)
    qk_case("qk_gqa_d64", 24, 64, 64, 4, 2, 2, seq=12, seed=6, pos_offset=0)
    qk_case("qk_gqa_d128_far", 20, 72, 128, 2, 1, 1, seq=10, seed=7, pos_offset=1 << 20)
    qk_case("qk_mha_d64_fpos", 16, 64, 64, 2, 2, 2, seq=16, seed=8, pos_offset=5, float_pos=True)
    rstd_case("rstd_variants", 24, 64, 24, 264, 64, 2, 1, seed=9)
    block_case("block_gemms", 45, 64, 72, 40, seed=10)
    llama3_blocks_case("llama3_blocks", 36, 64, 48, 16, 4, 200, seed=11)
