"""The GEMMs between the fused-linear operators (residual + partial RMSNorm forward / backward, SwiGLU dgrad):
golden vectors from the reference's eager ops, then ragged larger shapes against the oracle."""

import pytest
import torch

from oracle import eager

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2


def close(a, b, what, tol=TOL):
    err = eager.max_rel_err(a, b)
    assert err <= tol, f"{what}: max rel err {err:.3e} > {tol}"


def rn(gen, *shape, std=1.0):
    return (torch.randn(*shape, generator=gen) * std).to(torch.bfloat16).to(DEV)


def test_golden(golden_dir):
    from coda_kernels_b200 import ops, ops_block as Bk

    g = torch.load(golden_dir / "block_gemms.pt", weights_only=False)
    dev = lambda t: t.to(DEV)  # noqa: E731
    pre, post, rstd = Bk.gemm_residual_partial_rmsnorm(dev(g["A"]), dev(g["B"]), dev(g["C"]), dev(g["weight"]), g["eps"])
    close(pre, g["pre"], "pre")
    close(post, g["post"], "post")
    close(rstd, g["rstd"], "rstd", tol=1e-3)
    for key, al, dx in (("plain", None, None), ("alpha_accum", g["alpha"], g["dX0"])):
        dX, dW, normed = Bk.gemm_residual_partial_rmsnorm_bwd(
            dev(g["A2"]), dev(g["B2"]), dev(g["weight"]), dev(g["pre_bf16"]), dev(g["zdz"]), dev(g["rstd32"]),
            alpha=None if al is None else dev(al).reshape(1), dX=None if dx is None else dev(dx).clone())
        close(dX, g["bwd"][key]["dX"], f"{key} dX")
        close(dW, g["bwd"][key]["dW"], f"{key} dW")
        close(normed, g["bwd"][key]["normed"], f"{key} normed")
    for key, sc in (("plain", None), ("scaled", 0.125)):
        dZ, ZdZ, postact = Bk.gemm_swiglu_bwd_zdz(dev(g["A3"]), dev(g["B3"]), dev(g["Z"]), scale=sc)
        close(dZ, g["swiglu_bwd"][key]["dZ"], f"{key} dZ")
        close(ZdZ, g["swiglu_bwd"][key]["ZdZ"], f"{key} ZdZ")
        close(postact, g["swiglu_bwd"][key]["postact"], f"{key} postact")
    torch.cuda.synchronize()
    ops.check_device_status(torch.device(DEV))


@pytest.mark.parametrize("M,K,N", [(777, 264, 1032), (2050, 512, 520)])
def test_vs_oracle_ragged(M, K, N):
    from coda_kernels_b200 import ops, ops_block as Bk

    gen = torch.Generator().manual_seed(M)
    A, B, C = rn(gen, M, K), rn(gen, K, N, std=K**-0.5), rn(gen, M, N)
    weight = (1.0 + 0.2 * torch.randn(N, generator=gen)).to(torch.bfloat16).to(DEV)
    pre, post, rstd = Bk.gemm_residual_partial_rmsnorm(A, B, C, weight, 1e-6)
    rp, rpost, rr = eager.gemm_residual_partial_rmsnorm(A, B, C, weight, 1e-6)
    close(pre, rp, "pre")
    close(post, rpost, "post")
    close(rstd, rr, "rstd", tol=1e-3)
    # in place: the residual stream is overwritten by `pre`
    C2 = C.clone()
    pre2, _, _ = Bk.gemm_residual_partial_rmsnorm(A, B, C2, weight, 1e-6, pre=C2)
    assert pre2.data_ptr() == C2.data_ptr() and torch.equal(pre2, pre)

    A2, W2 = rn(gen, M, K), rn(gen, N, K, std=K**-0.5)
    zdz = torch.randn(M, generator=gen).to(DEV)
    alpha = torch.tensor([0.5], device=DEV)
    dX0 = rn(gen, M, N)
    dX, dW, normed = Bk.gemm_residual_partial_rmsnorm_bwd(A2, W2, weight, pre, zdz, rstd, alpha=alpha, dX=dX0.clone())
    rdx, rdw, rn_ = eager.gemm_residual_partial_rmsnorm_bwd(A2, W2, weight, pre, zdz, rstd, alpha=alpha, dX=dX0)
    close(dX, rdx, "dX (accumulated)")
    close(dW, rdw, "dW")
    close(normed, rn_, "normed")

    Fd = N  # treat N as the ffn width: Z is [M, 2N]
    Z = rn(gen, M, 2 * Fd)
    dZ, ZdZ, postact = Bk.gemm_swiglu_bwd_zdz(A2, W2, Z, scale=0.25)
    rdz, rzdz, rpa = eager.gemm_swiglu_bwd_zdz(A2, W2, Z, scale=0.25)
    close(dZ, rdz, "dZ")
    close(ZdZ, rzdz, "ZdZ")
    close(postact, rpa, "postact")
    torch.cuda.synchronize()
    ops.check_device_status(torch.device(DEV))
