"""``coda_b200_qknorm_rope_bwd_noalloc``: the workspace-free variant of the QK-norm + RoPE backward.

It serves hosts that have no buffer to lend the library: a bare C / ctypes
program holding only its inputs and outputs, or a process that claimed all of
its device memory up front and must not call ``cudaMalloc`` later.  The test
calls it through the C ABI twice in a row and compares with the regular entry
point, which takes the scratch buffer from the caller.  The file name sorts
last so that a run that stops at the first failure has already run every
other test.
"""

import ctypes

import pytest
import torch

from oracle import eager, inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call(lib, noalloc, d, pre, ms, cfg, M, scratch=None):
    heads = cfg["hq"] + cfg["hk"]
    N = (heads + cfg["hv"]) * cfg["head_dim"]
    grad = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    dgamma = torch.full((2 * cfg["head_dim"],), float("nan"), dtype=torch.float32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    common = [
        d["dq"].data_ptr(), d["dq"].stride(0), d["dk"].data_ptr(), d["dk"].stride(0), d["dv"].data_ptr(), d["dv"].stride(0),
        d["dv"].shape[1], pre.data_ptr(), pre.stride(0), ms.data_ptr(), d["gamma"].data_ptr(), d["positions"].data_ptr(), 0,
        d["frequencies"].data_ptr(), cfg["head_dim"], cfg["hq"], cfg["hk"], ctypes.c_float(cfg["eps"]), grad.data_ptr(),
        grad.stride(0), dgamma.data_ptr(),
    ]
    if noalloc:
        rc = lib.coda_b200_qknorm_rope_bwd_noalloc(*common, M, stream)
    else:
        rc = lib.coda_b200_qknorm_rope_bwd(*common, scratch.data_ptr(), scratch.numel() * 4, M, stream)
    torch.cuda.synchronize()
    return rc, grad, dgamma


def test_noalloc_matches_workspace_entry_point_twice():
    from coda_kernels_b200 import _lib

    lib = _lib.lib
    cfg = {"head_dim": 128, "hq": 4, "hk": 2, "hv": 2, "eps": 1e-6}
    M = 333
    host = inputs.qknorm_rope_inputs(M, 64, cfg["head_dim"], cfg["hq"], cfg["hk"], cfg["hv"], seq_len=128)
    d = {k: v.to(DEV) for k, v in host.items()}
    size_qk = (cfg["hq"] + cfg["hk"]) * cfg["head_dim"]
    pre32 = d["x"].float() @ d["weight"][:size_qk].float().mT
    pre = pre32.to(torch.bfloat16)
    ms = eager.head_mean_square(pre32, cfg["head_dim"]).contiguous()

    nbytes = lib.coda_b200_qknorm_rope_bwd_scratch_bytes(M, cfg["head_dim"])
    scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=DEV)
    rc, ref_grad, ref_dgamma = _call(lib, False, d, pre, ms, cfg, M, scratch)
    assert rc == 0, lib.coda_b200_last_error()

    for attempt in range(2):
        before = torch.cuda.memory_allocated()
        rc, grad, dgamma = _call(lib, True, d, pre, ms, cfg, M)
        assert rc == 0, lib.coda_b200_last_error()
        assert not torch.isnan(grad.float()).any() and not torch.isnan(dgamma).any(), f"call {attempt}: unwritten output"
        assert eager.max_rel_err(grad, ref_grad) <= 2e-2, f"call {attempt}: grad differs"
        assert eager.max_rel_err(dgamma, ref_dgamma) <= 2e-2, f"call {attempt}: dgamma differs"
        assert torch.equal(grad, ref_grad) and torch.equal(dgamma, ref_dgamma), f"call {attempt}: same kernels, same order: bits must match"
        del grad, dgamma
        assert torch.cuda.memory_allocated() == before

    # and against the oracle's backward, so that both entry points are right, not merely equal
    fn = lambda x, weight, gamma: eager.linear_qknorm_rope(  # noqa: E731
        x, weight, gamma, d["positions"], d["frequencies"], cfg["head_dim"], cfg["hq"], cfg["hk"], cfg["eps"])
    _, g = eager.fwd_bwd(fn, {n: d[n] for n in ("x", "weight", "gamma")}, ["x", "weight", "gamma"], (d["dq"], d["dk"], d["dv"]))
    assert eager.max_rel_err(ref_dgamma, g["gamma"]) <= 2e-2


def test_noalloc_rejects_oversized_batch():
    from coda_kernels_b200 import _lib

    lib = _lib.lib
    rc = lib.coda_b200_qknorm_rope_bwd_noalloc(None, 0, None, 0, None, 0, 0, None, 0, None, None, None, 0, None, 128, 1, 1,
                                               ctypes.c_float(1e-6), None, 0, None, 16385, None)
    assert rc == -1
    assert b"at most 16384 rows" in lib.coda_b200_last_error()
