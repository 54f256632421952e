"""Parity of the CUDA operators (called through the public API, i.e. through the C ABI) with the oracle.

Tolerances are the ones the task states: bf16 outputs and gradients
``max|a-b| / max|b| <= 2e-2`` (a normalised max-abs error), loss relative error
``<= 1e-3``, ignore-index masking and label indexing bit-exact.  On top of
that every bf16 tensor is held to the reference harness's own metric: its
relative L2 error against the oracle must stay within ``L2_FACTOR`` times the
rounding floor (the error of the oracle itself once rounded to bf16,
benchmarks/utils/numerics.py:20-29, 81-85); gradients that pass through one
more bf16 tensor (the saved pre-activation gradient) get ``L2_FACTOR_GRAD``.
"""

import functools

import pytest
import torch

from oracle import eager, inputs

pytestmark = pytest.mark.gpu

TOL = 2e-2
LOSS_TOL = 1e-3
L2_FACTOR = 2.0       # outputs computed from the fp32 accumulator
L2_FACTOR_GRAD = 3.0  # gradients formed from a bf16-rounded intermediate (dx, dweight, dgamma)
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ck():
    import coda_kernels_b200 as ck

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return ck


def load(golden_dir, name):
    return torch.load(golden_dir / f"{name}.pt", weights_only=False)


def close(a, b, tol=TOL, what=""):
    err = eager.max_rel_err(a, b)
    l2 = eager.rel_l2_err(a, b)
    assert err <= tol, f"{what}: max rel err {err:.3e} > {tol:.1e} (rel L2 {l2:.3e})"
    if a.dtype == torch.bfloat16:
        floor = eager.rounding_floor(b, torch.bfloat16)
        factor = L2_FACTOR_GRAD if what.startswith("d") else L2_FACTOR
        assert l2 <= factor * floor + 1e-6, f"{what}: rel L2 {l2:.3e} > {factor} x the bf16 rounding floor {floor:.3e}"
    return err


def leaf(t):
    return t.to(DEV).detach().requires_grad_(True)


def status_ok(ck):
    torch.cuda.synchronize()
    ck.ops.check_device_status(torch.device(DEV))


# ------------------------------------------------------------------------------------------------ swiglu
def run_swiglu(ck, d):
    x, w = leaf(d["x"]), leaf(d["weight"])
    out = ck.linear_swiglu(x, w)
    dx, dw = torch.autograd.grad(out, (x, w), d["dout"].to(DEV))
    return out, dx, dw


@pytest.mark.parametrize("name", ["swiglu_small", "swiglu_ragged"])
def test_swiglu_golden(ck, golden_dir, name):
    g = load(golden_dir, name)
    out, dx, dw = run_swiglu(ck, g["inputs"])
    status_ok(ck)
    assert out.dtype == torch.bfloat16 and dx.dtype == torch.bfloat16 and dw.dtype == torch.bfloat16
    close(out, g["out"], what="out")
    close(dx, g["dx"], what="dx")
    close(dw, g["dweight"], what="dweight")


def oracle_swiglu(d, dev=DEV):
    (out,), grads = eager.fwd_bwd(eager.linear_swiglu, {"x": d["x"].to(dev), "weight": d["weight"].to(dev)}, ["x", "weight"], d["dout"].to(dev))
    return out, grads["x"], grads["weight"]


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("shape", [(256, 512, 1024), (1000, 1032, 1544), (130, 64, 8)])
def test_swiglu_vs_oracle(ck, shape, cta_group):
    """(256, 512, 1024) is the CPU-runnable benchmark configuration; the others have ragged row, column and depth tiles."""
    ck.set_option("cta_group", cta_group)
    try:
        d = inputs.swiglu_inputs(*shape)
        out, dx, dw = run_swiglu(ck, d)
        status_ok(ck)
    finally:
        ck.set_option("cta_group", 2)
    ro, rdx, rdw = oracle_swiglu(d)
    close(out, ro, what="out")
    close(dx, rdx, what="dx")
    close(dw, rdw, what="dweight")


def test_swiglu_strided_and_repeatable(ck):
    """Non-contiguous inputs are accepted (made contiguous by the guard) and a second call gives the same bits."""
    d = inputs.swiglu_inputs(192, 256, 128)
    xw = torch.empty(192, 512, dtype=torch.bfloat16, device=DEV)
    xw[:, ::2] = d["x"].to(DEV)
    x = xw[:, ::2]
    w = d["weight"].to(DEV)
    a = ck.linear_swiglu(x, w)
    b = ck.linear_swiglu(x, w)
    status_ok(ck)
    assert torch.equal(a, b)
    close(a, oracle_swiglu(d)[0], what="out")


# ------------------------------------------------------------------------------------------------ sigmoid
def test_sigmoid_golden(ck, golden_dir):
    g = load(golden_dir, "sigmoid_small")
    d = g["inputs"]
    x, w = leaf(d["x"]), leaf(d["weight"])
    out = ck.linear_sigmoid(x, w)
    dx, dw = torch.autograd.grad(out, (x, w), d["dout"].to(DEV))
    status_ok(ck)
    close(out, g["out"], what="out")
    close(dx, g["dx"], what="dx")
    close(dw, g["dweight"], what="dweight")


@pytest.mark.parametrize("out_dtype", [None, torch.float32])
def test_sigmoid_vs_oracle(ck, out_dtype):
    d = inputs.sigmoid_inputs(520, 328, 264)
    x, w = leaf(d["x"]), leaf(d["weight"])
    out = ck.linear_sigmoid(x, w, out_dtype)
    assert out.dtype == (out_dtype or torch.bfloat16)
    dx, dw = torch.autograd.grad(out, (x, w), d["dout"].to(DEV).to(out.dtype))
    status_ok(ck)
    (ro,), grads = eager.fwd_bwd(eager.linear_sigmoid, {"x": d["x"].to(DEV), "weight": d["weight"].to(DEV)}, ["x", "weight"], d["dout"].to(DEV))
    close(out, ro, what="out", tol=TOL if out_dtype is None else 1e-4)
    close(dx, grads["x"], what="dx")
    close(dw, grads["weight"], what="dweight")


# ------------------------------------------------------------------------------------------------ cross entropy
def run_ce(ck, d, reduction):
    x, w = leaf(d["x"]), leaf(d["weight"])
    t = d["target"].to(DEV)
    loss = ck.linear_cross_entropy(x, w, t, -100, reduction)
    dx, dw = torch.autograd.grad(loss, (x, w))
    return loss, dx, dw


def rel(a, b):
    return abs(float(a) - float(b)) / abs(float(b))


@pytest.mark.parametrize("name", ["ce_mean", "ce_sum"])
def test_cross_entropy_golden(ck, golden_dir, name):
    g = load(golden_dir, name)
    d = g["inputs"]
    loss, dx, dw = run_ce(ck, d, g["reduction"])
    status_ok(ck)
    assert loss.dtype == torch.float32 and loss.dim() == 0
    assert rel(loss, g["loss"]) <= LOSS_TOL
    close(dx, g["dx"], what="dx")
    close(dw, g["dweight"], what="dweight")
    fwd = ck.linear_cross_entropy_forward(d["x"].to(DEV), d["weight"].to(DEV), d["target"].to(DEV), -100, g["reduction"])
    assert rel(fwd, g["loss"]) <= LOSS_TOL
    # the inner ops: per-row losses, and the gradient w.r.t. the logits with exact masking / label indexing
    losses, dlogits = ck.ops.gemm_lse_dlogits(d["x"].to(DEV), d["weight"].to(DEV).mT, d["target"].to(DEV), -100)
    status_ok(ck)
    close(losses, g["row_losses"], tol=LOSS_TOL, what="row losses")
    close(dlogits, g["dlogits"], what="dlogits")
    # element-wise: tiny softmax entries pass two bf16 roundings (the stored probability, then the rescaled gradient)
    ew = eager.max_elementwise_err(dlogits, g["dlogits"])
    assert ew <= 2e-2, f"dlogits: element-wise relative error {ew:.3e}"
    ignored = (d["target"] == -100).to(DEV)
    assert ignored.any()
    assert (losses[ignored] == 0).all(), "ignored rows must have exactly zero loss"
    assert (dlogits[ignored].view(torch.int16) == 0).all(), "ignored rows must have exactly +0 gradient"
    valid = ~ignored
    assert torch.equal(dlogits[valid].float().argmin(dim=1).int(), d["target"].to(DEV)[valid]), "the one negative entry of a row sits at its label"
    assert (dlogits[valid].float().min(dim=1).values < 0).all()


def test_cross_entropy_second_call_and_inputs_untouched(ck):
    """The gradient buffer is rewritten in place inside the forward; a second step on the same inputs must give the same
    bits, and the inputs must come out unchanged (the reference harness reads the second call for this reason,
    benchmarks/utils/numerics.py:48-57)."""
    d = inputs.cross_entropy_inputs(520, 264, 1544, seed=9, ignore_frac=0.1)
    x0, w0 = d["x"].to(DEV), d["weight"].to(DEV)
    xc, wc = x0.clone(), w0.clone()
    first = run_ce(ck, {"x": x0, "weight": w0, "target": d["target"]}, "mean")
    second = run_ce(ck, {"x": x0, "weight": w0, "target": d["target"]}, "mean")
    status_ok(ck)
    assert torch.equal(x0, xc) and torch.equal(w0, wc), "inputs were clobbered"
    for a, b, n in zip(first, second, ("loss", "dx", "dweight")):
        assert torch.equal(a, b), f"{n} differs between two calls on the same inputs"


@pytest.mark.parametrize("reduction", ["mean", "sum"])
def test_cross_entropy_vs_oracle_ragged_vocab(ck, reduction):
    """Vocabulary 5000 = 19 full column tiles + 136 columns; 777 rows = ragged row tile."""
    d = inputs.cross_entropy_inputs(777, 264, 5000, seed=3, ignore_frac=0.1)
    loss, dx, dw = run_ce(ck, d, reduction)
    status_ok(ck)
    fn = functools.partial(eager.linear_cross_entropy, target=d["target"].to(DEV), reduction=reduction)
    (rl,), grads = eager.fwd_bwd(fn, {"x": d["x"].to(DEV), "weight": d["weight"].to(DEV)}, ["x", "weight"], torch.tensor(1.0, device=DEV))
    assert rel(loss, rl) <= LOSS_TOL
    close(dx, grads["x"], what="dx")
    close(dw, grads["weight"], what="dweight")


def test_cross_entropy_all_ignored_and_grad_flags(ck):
    d = inputs.cross_entropy_inputs(64, 64, 512, seed=5)
    t = torch.full((64,), -100, dtype=torch.int32, device=DEV)
    x, w = leaf(d["x"]), leaf(d["weight"])
    s = ck.linear_cross_entropy(x, w, t, -100, "sum")
    m = ck.linear_cross_entropy(x, w, t, -100, "mean")
    dx, dw = torch.autograd.grad(s, (x, w))
    status_ok(ck)
    assert float(s) == 0.0 and torch.isnan(m), "sum of no rows is 0, mean of no rows is NaN (as torch.nn.functional.cross_entropy)"
    assert (dx == 0).all() and (dw == 0).all()
    # only the requested gradient is produced
    x2 = d["x"].to(DEV)
    loss = ck.linear_cross_entropy(x2, w, d["target"].to(DEV))
    (dw2,) = torch.autograd.grad(loss, (w,))
    assert dw2.shape == w.shape
    # non-default ignore_index: label 7 is masked, -100 never appears
    t7 = torch.randint(0, 512, (64,), dtype=torch.int32, device=DEV)
    t7[::3] = 7
    l7 = ck.linear_cross_entropy_forward(d["x"].to(DEV), d["weight"].to(DEV), t7, 7, "mean")
    r7 = eager.linear_cross_entropy(d["x"].to(DEV), d["weight"].to(DEV), t7, ignore_index=7)
    assert rel(l7, r7) <= LOSS_TOL


# ------------------------------------------------------------------------------------------------ qk-norm + rope
def run_qk(ck, d, cfg):
    x, w, g = leaf(d["x"]), leaf(d["weight"]), leaf(d["gamma"])
    q, k, v = ck.linear_qknorm_rope(x, w, g, d["positions"].to(DEV), d["frequencies"].to(DEV), cfg["head_dim"], cfg["hq"], cfg["hk"], cfg["eps"])
    grads = torch.autograd.grad((q, k, v), (x, w, g), (d["dq"].to(DEV), d["dk"].to(DEV), d["dv"].to(DEV)))
    return (q, k, v), grads


@pytest.mark.parametrize("name", ["qk_gqa_d64", "qk_gqa_d128_far", "qk_mha_d64_fpos"])
def test_qknorm_rope_golden(ck, golden_dir, name):
    g = load(golden_dir, name)
    (q, k, v), (dx, dw, dg) = run_qk(ck, g["inputs"], g["cfg"])
    status_ok(ck)
    assert q.data_ptr() + q.shape[1] * 2 == k.data_ptr(), "q and k are two views of one buffer"
    close(q, g["q"], what="q")
    close(k, g["k"], what="k")
    close(v, g["v"], what="v")
    close(dx, g["dx"], what="dx")
    close(dw, g["dweight"], what="dweight")
    close(dg, g["dgamma"], what="dgamma")
    # element-wise, with an absolute floor of a tenth of the largest entry: every entry is a sum of rows x heads signed
    # terms, so one that happens to lie near zero still carries the absolute error of the whole sum
    ew = eager.max_elementwise_err(dg, g["dgamma"], atol_frac=0.1)
    assert ew <= 5e-2, f"dgamma: element-wise relative error {ew:.3e}"
    assert dg.dtype == torch.bfloat16


@pytest.mark.parametrize("cfg,M,K,offset", [
    ({"head_dim": 128, "hq": 8, "hk": 2, "hv": 2, "eps": 1e-6}, 1000, 520, 1 << 20),
    ({"head_dim": 128, "hq": 4, "hk": 1, "hv": 1, "eps": 1e-6}, 300, 256, 0),  # one GPU's share of 32/8/8 heads: a tile straddles k and v
    ({"head_dim": 64, "hq": 6, "hk": 3, "hv": 3, "eps": 1e-5}, 515, 136, 77),
])
def test_qknorm_rope_vs_oracle(ck, cfg, M, K, offset):
    d = inputs.qknorm_rope_inputs(M, K, cfg["head_dim"], cfg["hq"], cfg["hk"], cfg["hv"], seq_len=4096, pos_offset=offset)
    # gamma over the range of trained norm weights rather than near 1
    gen = torch.Generator().manual_seed(1)
    d["gamma"] = torch.exp(torch.empty(2 * cfg["head_dim"]).uniform_(-1.6, 1.4, generator=gen)).to(torch.bfloat16)
    (q, k, v), (dx, dw, dg) = run_qk(ck, d, cfg)
    status_ok(ck)
    fn = functools.partial(eager.linear_qknorm_rope, positions=d["positions"].to(DEV), frequencies=d["frequencies"].to(DEV),
                           head_dim=cfg["head_dim"], num_heads_q=cfg["hq"], num_heads_k=cfg["hk"], eps=cfg["eps"])
    outs, grads = eager.fwd_bwd(fn, {n: d[n].to(DEV) for n in ("x", "weight", "gamma")}, ["x", "weight", "gamma"],
                                (d["dq"].to(DEV), d["dk"].to(DEV), d["dv"].to(DEV)))
    for a, b, n in zip((q, k, v), outs, "qkv"):
        close(a, b, what=n)
    close(dx, grads["x"], what="dx")
    close(dw, grads["weight"], what="dweight")
    close(dg, grads["gamma"], what="dgamma")


# ------------------------------------------------------------------------------------------------ plain GEMM, every operand layout
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_operand_layouts(ck, a_t, b_t):
    gen = torch.Generator().manual_seed(7)
    M, K, N = 392, 328, 520
    A = torch.randn((K, M) if a_t else (M, K), generator=gen).to(torch.bfloat16).to(DEV)
    B = torch.randn((N, K) if b_t else (K, N), generator=gen).to(torch.bfloat16).to(DEV)
    Av = A.mT if a_t else A
    Bv = B.mT if b_t else B
    ref = Av.float() @ Bv.float()
    alpha = torch.tensor([0.25], device=DEV)
    out = ck.ops.gemm(Av, Bv)
    out32 = ck.ops.gemm(Av, Bv, out_dtype=torch.float32, alpha=alpha)
    status_ok(ck)
    close(out, ref, what="bf16 out")
    close(out32, 0.25 * ref, tol=1e-5, what="fp32 out with alpha")


@pytest.mark.parametrize("M,N,K,a_t,b_t", [
    (512, 1024, 8192, False, False),   # 8 tiles, long contraction: every tile is accumulated in nine parts
    (768, 1024, 4096, True, True),     # weight-gradient layout (both operands MN-major), 12 tiles
    (300, 520, 8200, False, True),     # input-gradient layout; ragged in M, N and K
    (9728, 512, 2048, False, False),   # 76 tiles: one full round of whole tiles, then two tiles cut in four
])
def test_gemm_tail_split_matches_the_whole_tile_schedule(ck, M, N, K, a_t, b_t):
    """With a workspace the plain GEMM cuts the tiles of its last, mostly idle round along K: they are accumulated in
    parts that a follow-up kernel adds in a fixed order.  Same product as the whole-tile launch up to fp32 summation
    order, and reproducible run to run."""
    from coda_kernels_b200 import _lib

    assert _lib.lib.coda_b200_gemm_workspace_bytes(M, N, K) > 0, "this shape should have its last round cut"
    gen = torch.Generator().manual_seed(11)
    A = torch.randn((K, M) if a_t else (M, K), generator=gen).to(torch.bfloat16).to(DEV)
    B = torch.randn((N, K) if b_t else (K, N), generator=gen).to(torch.bfloat16).to(DEV)
    Av, Bv = (A.mT if a_t else A), (B.mT if b_t else B)
    ref = Av.float() @ Bv.float()
    alpha = torch.tensor([0.5], device=DEV)
    split = ck.ops.gemm(Av, Bv)
    split32 = ck.ops.gemm(Av, Bv, out_dtype=torch.float32, alpha=alpha)
    again = torch.empty_like(split)
    ck.ops._ct_gemm_out(Av, Bv, again, None, None)                  # the ctypes binding offers the workspace too
    assert _lib.lib.coda_b200_set_option(b"split_tail", 0) == 0
    try:
        whole = ck.ops.gemm(Av, Bv)                                 # whole tiles only
    finally:
        assert _lib.lib.coda_b200_set_option(b"split_tail", 1) == 0
    status_ok(ck)
    assert torch.equal(split, again), "parts are added in a fixed order, whichever binding launches"
    close(split, ref, what="tail-split bf16 out")
    close(split32, 0.5 * ref, tol=1e-5, what="tail-split fp32 out with alpha")
    assert eager.max_rel_err(split, whole) <= 1e-2, "cut vs whole tiles: one bf16 rounding of a differently ordered fp32 sum"
    assert _lib.lib.coda_b200_gemm_workspace_bytes(16384, 4096, 28672) == 0, "62 tail tiles cannot be cut profitably"


def test_bad_arguments_raise(ck):
    x = torch.zeros(64, 60, dtype=torch.bfloat16, device=DEV)  # K = 60 is not a multiple of 8
    w = torch.zeros(32, 60, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ck.CodaB200Error):
        ck.linear_swiglu(x, w)
    with pytest.raises(NotImplementedError):
        ck.linear_swiglu(x.half(), w.half())


# ------------------------------------------------------------------------------------------------ deferred-RMSNorm variants
def test_rstd_variants_golden_and_oracle(ck, golden_dir):
    from coda_kernels_b200 import ops_rmsnorm as R

    g = load(golden_dir, "rstd_variants")
    cfg, qk = g["cfg"], g["qk_inputs"]
    x, rstd = g["x"].to(DEV), g["rstd"].to(DEV)
    pre, post = R.gemm_rmsnorm_swiglu(x, g["w_swiglu"].to(DEV).mT, rstd)
    close(pre, g["swiglu_pre"], what="swiglu preact")
    close(post, g["swiglu_post"], what="swiglu postact")
    t = g["target"].to(DEV)
    losses, lse, dlogits = R.gemm_rmsnorm_lse_dlogits(x, g["w_vocab"].to(DEV).mT, rstd, t, -100)
    sel_losses, sel_lse, _ = R.gemm_rmsnorm_lse_select_logits(x, g["w_vocab"].to(DEV).mT, rstd, t, -100)
    close(lse, g["lse"], tol=LOSS_TOL, what="lse")
    close(sel_lse, g["lse"], tol=LOSS_TOL, what="lse (select)")
    close(losses, g["row_losses"], tol=LOSS_TOL, what="row losses")
    close(sel_losses, g["row_losses"], tol=LOSS_TOL, what="row losses (select)")
    close(dlogits, g["dlogits"], what="dlogits")
    assert (dlogits[t == -100].view(torch.int16) == 0).all()
    w = qk["weight"].to(DEV)
    rot, preact, ms, v = R.gemm_rmsnorm_qknorm_rope(
        x, w.mT, rstd, qk["gamma"].to(DEV), qk["positions"].to(DEV), qk["frequencies"].to(DEV), cfg["head_dim"], cfg["hq"], cfg["hk"], cfg["eps"])
    status_ok(ck)
    assert v is None
    close(rot, g["qk_rotated"], what="rotated qk")
    close(preact, g["qk_preact"], what="preact (unscaled)")
    close(ms, g["qk_mean_sq"], tol=1e-3, what="head mean square")
    # a larger, ragged case with v columns against the oracle: v = (x @ Wv^T) * rstd
    d = inputs.qknorm_rope_inputs(700, 264, 128, 4, 2, 2, seq_len=512, pos_offset=9)
    xg = d["x"].to(DEV)
    r2 = eager.rmsnorm_rstd(xg, 1e-5)
    size_qk = 6 * 128
    rot, preact, ms, v = R.gemm_rmsnorm_qknorm_rope(xg, d["weight"].to(DEV).mT, r2, d["gamma"].to(DEV), d["positions"].to(DEV),
                                                    d["frequencies"].to(DEV), 128, 4, 2, 1e-6)
    ro, rp, rms = eager.gemm_rmsnorm_qknorm_rope(xg, d["weight"].to(DEV)[:size_qk].mT, r2, d["gamma"].to(DEV), d["positions"].to(DEV),
                                                 d["frequencies"].to(DEV), 128, 4, 2, 1e-6)
    status_ok(ck)
    close(rot, ro, what="rotated qk (large)")
    close(preact, rp, what="preact (large)")
    close(ms, rms, tol=1e-3, what="mean square (large)")
    close(v, (xg.float() @ d["weight"].to(DEV)[size_qk:].float().mT) * r2[:, None], what="v (large)")


# ------------------------------------------------------------------------------------------------ logits dataflow of the reference
@pytest.mark.parametrize("name", ["ce_mean", "ce_sum"])
def test_gemm_lse_and_cross_entropy_fwd_bwd(ck, golden_dir, name):
    """``gemm_lse`` + ``cross_entropy_fwd_bwd`` chained as in the reference's ``_forward_lse``."""
    from coda_kernels_b200 import ops_logits as L

    g = load(golden_dir, name)
    d = g["inputs"]
    x, w, t = d["x"].to(DEV), d["weight"].to(DEV), d["target"].to(DEV)
    logits, lses = L.gemm_lse(x, w.mT)
    ref_logits = x.float() @ w.float().mT
    close(logits, ref_logits, what="logits")
    close(lses, g["lse"], tol=LOSS_TOL, what="lse")
    losses, dlogits = L.cross_entropy_fwd_bwd(logits, lses, t, -100)
    status_ok(ck)
    assert dlogits.data_ptr() == logits.data_ptr(), "the gradient overwrites the logits in place"
    # the target logit is read from the bf16-rounded logits here, as in the reference: looser than the fused path
    close(losses, g["row_losses"], tol=5e-3, what="row losses")
    close(dlogits, g["dlogits"], what="dlogits")
    ignored = t == -100
    assert (losses[ignored] == 0).all() and (dlogits[ignored].view(torch.int16) == 0).all()


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, True)])
def test_gemm_narrow_tile(ck, a_t, b_t, cta_group):
    """The 128-column tile (chosen automatically for narrow or few-tile outputs) forced on, in the three layouts the operators use."""
    gen = torch.Generator().manual_seed(11)
    M, K, N = 520, 264, 392
    A = torch.randn((K, M) if a_t else (M, K), generator=gen).to(torch.bfloat16).to(DEV)
    B = torch.randn((N, K) if b_t else (K, N), generator=gen).to(torch.bfloat16).to(DEV)
    Av, Bv = (A.mT if a_t else A), (B.mT if b_t else B)
    ref = Av.float() @ Bv.float()
    ck.set_option("cta_group", cta_group)
    ck.set_option("tile_n", 128)
    try:
        out = ck.ops.gemm(Av, Bv)
        sig = ck.ops.gemm_sigmoid(Av, Bv, out=torch.empty(M, N, dtype=torch.float32, device=DEV))
        status_ok(ck)
    finally:
        ck.set_option("tile_n", 0)
        ck.set_option("cta_group", 2)
    close(out, ref, what="bf16 out, 128-column tiles")
    close(sig, torch.sigmoid(ref), tol=1e-3, what="sigmoid fp32 out, 128-column tiles")
    # automatic choice: a skinny output (N = 32 gate heads) takes the narrow tile and stays correct
    W = torch.randn(32, K, generator=gen).to(torch.bfloat16).to(DEV)
    x = A.mT if a_t else A
    close(ck.ops.gemm_sigmoid(x, W.mT), torch.sigmoid(x.float() @ W.float().mT), what="skinny sigmoid")


# ------------------------------------------------------------------------------------------------ extension: sigmoid-gated projection
@pytest.mark.parametrize("shape", [(333, 264, 136), (1024, 512, 1024)])
def test_sigmoid_glu_vs_oracle(ck, shape):
    """``sigmoid(x W_gate^T) * (x W_val^T)``: the gated-projection reading of the sigmoid benchmark configuration."""
    from coda_kernels_b200.functional.sigmoid_glu import linear_sigmoid_glu

    M, K, N = shape
    d = inputs.swiglu_inputs(M, K, N)  # same interleaved weight layout and distributions
    x, w = leaf(d["x"]), leaf(d["weight"])
    out = linear_sigmoid_glu(x, w)
    dx, dw = torch.autograd.grad(out, (x, w), d["dout"].to(DEV))
    status_ok(ck)
    (ro,), g = eager.fwd_bwd(eager.linear_sigmoid_glu, {"x": d["x"].to(DEV), "weight": d["weight"].to(DEV)}, ["x", "weight"], d["dout"].to(DEV))
    close(out, ro, what="out")
    close(dx, g["x"], what="dx")
    close(dw, g["weight"], what="dweight")


# ------------------------------------------------------------------------------------------------ epilogue store paths, fused addend, 64-column tile
@pytest.mark.parametrize("epi_tma", [0, 1])
def test_store_paths_agree_bitwise(ck, epi_tma):
    """Staged TMA stores and per-thread stores write the same bits, on ragged shapes where the hardware clips the boxes."""
    d = inputs.swiglu_inputs(333, 264, 136)
    dq = inputs.qknorm_rope_inputs(300, 256, 128, 4, 1, 1, seq_len=512)
    dc = inputs.cross_entropy_inputs(300, 256, 1000, ignore_frac=0.1)
    cfg = {"head_dim": 128, "hq": 4, "hk": 1, "eps": 1e-6}

    def run_all():
        a = run_swiglu(ck, d)
        (q, k, v), gq = run_qk(ck, dq, cfg)
        c = run_ce(ck, dc, "mean")
        s32 = ck.linear_sigmoid(d["x"].to(DEV), d["weight"].to(DEV), torch.float32)
        status_ok(ck)
        return [*a, q, k, v, *gq, *c, s32]

    ck.set_option("epi_tma", epi_tma)
    try:
        got = run_all()
    finally:
        ck.set_option("epi_tma", 1)
    ref = run_all()
    for i, (a, b) in enumerate(zip(got, ref)):
        assert torch.equal(a, b), f"output {i} differs between epi_tma={epi_tma} and the default"


@pytest.mark.parametrize("c_dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16), (torch.float32, torch.float32)])
def test_gemm_with_addend_is_one_kernel(ck, c_dtype, out_dtype):
    """``gemm(A, B, C=...)``: the addend joins the fp32 accumulator in the epilogue (the reference's ``quack_gemm_add`` form,
    coda/core/gemm/functional.py:54-69), also in place (``out is C``) and through the reference-shaped shim."""
    from coda.core.gemm.functional import gemm as shim_gemm

    gen = torch.Generator().manual_seed(21)
    M, K, N = 392, 264, 520
    A = torch.randn(M, K, generator=gen).to(torch.bfloat16).to(DEV)
    W = torch.randn(N, K, generator=gen).to(torch.bfloat16).to(DEV)
    C = torch.randn(M, N, generator=gen).to(c_dtype).to(DEV)
    ref = A.float() @ W.float().mT + C.float()
    out = ck.ops.gemm(A, W.mT, C=C, out_dtype=out_dtype)
    status_ok(ck)
    assert out.dtype == out_dtype
    close(out, ref, tol=TOL if out_dtype == torch.bfloat16 else 1e-5, what="A @ B + C")
    if c_dtype == out_dtype:
        buf = C.clone()
        ck.ops.gemm(A, W.mT, out=buf, C=buf)
        status_ok(ck)
        assert torch.equal(buf, out), "accumulating in place must give the same bits"
    if out_dtype == torch.bfloat16:
        assert torch.equal(shim_gemm(A, W.mT, C=C), out)


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("n_gates", [8, 32, 64])
def test_skinny_sigmoid_uses_the_64_column_tile(ck, n_gates, cta_group):
    """``linear_sigmoid`` with one gate per attention head (the shape the reference benchmarks, benchmarks/linear.py:28-42)."""
    d = inputs.sigmoid_inputs(1000, 520, n_gates)
    ck.set_option("cta_group", cta_group)
    try:
        x, w = leaf(d["x"]), leaf(d["weight"])
        out = ck.linear_sigmoid(x, w)
        dx, dw = torch.autograd.grad(out, (x, w), d["dout"].to(DEV))
        out32 = ck.linear_sigmoid(d["x"].to(DEV), d["weight"].to(DEV), torch.float32)
        status_ok(ck)
    finally:
        ck.set_option("cta_group", 2)
    (ro,), grads = eager.fwd_bwd(eager.linear_sigmoid, {"x": d["x"].to(DEV), "weight": d["weight"].to(DEV)}, ["x", "weight"], d["dout"].to(DEV))
    close(out, ro, what="out")
    close(out32, ro, tol=1e-4, what="out fp32")
    close(dx, grads["x"], what="dx")
    close(dw, grads["weight"], what="dweight")


@pytest.mark.parametrize("shape", [(520, 328, 264), (1000, 520, 1032), (4096, 512, 2048)])
def test_fused_sigmoid_gradient_dgrad(ck, shape):
    """``dx`` and ``grad_pre`` from the input-gradient GEMM whose transform warps form ``dout * out * (1 - out)`` as its
    A operand, against the separate pass + plain GEMM and against the oracle (ragged rows, columns and contraction)."""
    M, K, N = shape
    d = inputs.sigmoid_inputs(M, K, N)
    x, w, dout = d["x"].to(DEV), d["weight"].to(DEV), d["dout"].to(DEV)
    out = ck.ops.gemm_sigmoid(x, w.mT)
    dx, g = ck.ops.gemm_dsigmoid_dgrad(out, dout, w)
    g_ref = ck.ops.dsigmoid_backward(out, dout)
    dx_ref = ck.ops.gemm(g_ref, w)
    status_ok(ck)
    # the fused kernel forms grad_pre in packed bf16 (three roundings), the separate pass in fp32 (one): they agree to a
    # few bf16 ulps, and both sit within the gradient tolerance of the exact value
    assert eager.max_rel_err(g, g_ref.float()) <= 1e-2
    assert eager.max_rel_err(dx, dx_ref.float()) <= 1e-2
    exact_g = dout.float() * out.float() * (1.0 - out.float())
    close(g, exact_g, what="dgrad_pre")
    (ro,), grads = eager.fwd_bwd(eager.linear_sigmoid, {"x": x, "weight": w}, ["x", "weight"], dout)
    close(dx, grads["x"], what="dx")
    dw = ck.ops.gemm(g.mT, x)
    close(dw, grads["weight"], what="dweight")
