"""The compiled dispatch shim (TORCH_LIBRARY ops in libcoda_b200_torch.so) and the ctypes custom ops are two bindings of the
same C ABI: same bits, and the shim is what eager calls use."""

import pytest
import torch

from oracle import inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_native_and_ctypes_bindings_agree():
    import coda_kernels_b200 as ck
    from coda_kernels_b200 import ops

    assert ops._native is not None, "the compiled dispatch shim should be loaded by default"
    d = inputs.swiglu_inputs(333, 264, 136)
    x, w, dout = d["x"].to(DEV), d["weight"].to(DEV), d["dout"].to(DEV)

    def run(gemm_swiglu_out, dswiglu_out, gemm_out):
        pre = torch.empty(333, 272, dtype=torch.bfloat16, device=DEV)
        post = torch.empty(333, 136, dtype=torch.bfloat16, device=DEV)
        gemm_swiglu_out(x, w.mT, pre, post)
        g = torch.empty_like(pre)
        dswiglu_out(pre, dout, g)
        dx = torch.empty(333, 264, dtype=torch.bfloat16, device=DEV)
        gemm_out(g, w, dx, None, None)
        return pre, post, g, dx

    a = run(ops._gemm_swiglu_out, ops._dswiglu_out, ops._gemm_out)
    b = run(ops._ct_gemm_swiglu_out, ops._ct_dswiglu_out, ops._ct_gemm_out)
    torch.cuda.synchronize()
    ops.check_device_status(torch.device(DEV))
    for u, v in zip(a, b):
        assert torch.equal(u, v)
    # host-side argument errors surface as exceptions through the shim too
    with pytest.raises(RuntimeError, match="multiple of 8|failed"):
        ck.linear_swiglu(torch.zeros(64, 60, dtype=torch.bfloat16, device=DEV), torch.zeros(32, 60, dtype=torch.bfloat16, device=DEV))


def test_dispatch_cost_of_the_shim_is_below_the_ctypes_ops():
    """Host time per launch, measured on a tiny GEMM where the GPU is never the limiter."""
    import time

    from coda_kernels_b200 import ops

    A = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    B = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    out = torch.empty(128, 128, dtype=torch.bfloat16, device=DEV)

    def per_call(fn, n=300):
        for _ in range(20):
            fn(A, B.mT, out, None, None)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            fn(A, B.mT, out, None, None)
        dt = (time.perf_counter() - t0) / n
        torch.cuda.synchronize()
        return dt

    native, ct = per_call(ops._gemm_out), per_call(ops._ct_gemm_out)
    print(f"host time per launch: compiled shim {native * 1e6:.1f} us, ctypes custom op {ct * 1e6:.1f} us")
    assert native < ct


def test_whole_operator_entry_points_match_the_composed_path(monkeypatch):
    """Forward and backward of the four operators through the one-call-per-direction entry points of the compiled layer
    against the same launches composed in Python: the same kernels on the same inputs, so the same bits."""
    import coda_kernels_b200 as ck
    from coda_kernels_b200 import ops

    dev = torch.device(DEV)

    def leaf(t):
        return t.to(dev).detach().requires_grad_(True)

    def swiglu():
        d = inputs.swiglu_inputs(333, 264, 136)
        x, w = leaf(d["x"]), leaf(d["weight"])
        y = ck.linear_swiglu(x, w)
        y.backward(d["dout"].to(dev))
        return y, x.grad, w.grad

    def sigmoid(out_dtype=None):
        d = inputs.sigmoid_inputs(300, 136, 72)
        x, w = leaf(d["x"]), leaf(d["weight"])
        y = ck.linear_sigmoid(x, w, out_dtype)
        y.backward(d["dout"].to(dev).to(y.dtype))
        return y, x.grad, w.grad

    def cross_entropy(reduction):
        d = inputs.cross_entropy_inputs(257, 136, 1000)
        x, w = leaf(d["x"]), leaf(d["weight"])
        loss = ck.linear_cross_entropy(x, w, d["target"].to(dev), reduction=reduction)
        (loss * 3.0).backward()
        only = ck.linear_cross_entropy_forward(x.detach(), w.detach(), d["target"].to(dev), reduction=reduction)
        return loss, only, x.grad, w.grad

    def qknorm(hv):
        d = inputs.qknorm_rope_inputs(200, 136, 128, 4, 2, hv, 64)
        x, w, g = leaf(d["x"]), leaf(d["weight"]), leaf(d["gamma"])
        q, k, v = ck.linear_qknorm_rope(x, w, g, d["positions"].to(dev), d["frequencies"].to(dev), 128, 4, 2, 1e-6)
        torch.autograd.backward((q, k, v), (d["dq"].to(dev), d["dk"].to(dev), d["dv"].to(dev)))
        return q, k, v, x.grad, w.grad, g.grad

    cases = [swiglu, sigmoid, lambda: sigmoid(torch.float32), lambda: cross_entropy("mean"), lambda: cross_entropy("sum"),
             lambda: qknorm(2), lambda: qknorm(0)]
    assert ops._fast(), "eager calls should use the whole-operator entry points by default"
    whole = [case() for case in cases]
    monkeypatch.setattr(ops, "_WHOLE_OPERATORS", False)
    composed = [case() for case in cases]
    torch.cuda.synchronize()
    ops.check_device_status(dev)
    for a, b in zip(whole, composed):
        for u, v in zip(a, b):
            assert u.dtype == v.dtype and u.shape == v.shape and torch.equal(u, v)
