"""Failure detection without a GPU fault: a device-side wait that nothing satisfies ends by itself within its limit,
the kernel returns normally, the status word carries the code, Python raises, and the context stays usable."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_bounded_wait_expires_and_reports():
    import coda_kernels_b200 as ck
    from coda_kernels_b200 import _lib, ops

    dev = torch.device(DEV)
    word = ops.status_word(dev)
    torch.cuda.synchronize()
    assert int(word.item()) == 0
    waited = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = _lib.lib.coda_b200_selftest_wait_timeout(word.data_ptr(), 2000, waited.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.lib.coda_b200_last_error()
    torch.cuda.synchronize()  # returns: the wait gave up by itself
    us = int(waited.item())
    assert 2000 <= us < 200000, f"the wait should end shortly after its 2 ms limit, took {us} us"
    assert int(word.item()) > 0
    with pytest.raises(RuntimeError, match="device-side error code"):
        ops.check_device_status(dev)
    assert int(word.item()) == 0, "reading the status clears it"
    # the context is still healthy: a real operator runs and is correct afterwards
    x = torch.randn(256, 128, device=dev).to(torch.bfloat16)
    w = torch.randn(256, 128, device=dev).to(torch.bfloat16)
    out = ck.ops.gemm(x, w.mT)
    ref = x.float() @ w.float().mT
    torch.cuda.synchronize()
    ops.check_device_status(dev)
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
    # bad arguments are refused on the host
    assert _lib.lib.coda_b200_selftest_wait_timeout(None, 10, None, None) == -1
    assert _lib.lib.coda_b200_selftest_wait_timeout(word.data_ptr(), 0, None, None) == -1


def test_operator_path_reports_an_expired_wait_without_sync():
    """A kernel that gave up is reported by a later operator call on its own (no explicit status read, no
    CODA_B200_SYNC_STATUS): the status word sits in pinned host memory, the failing kernel writes it there, and the
    guards read it as plain memory."""
    import coda_kernels_b200 as ck
    from coda_kernels_b200 import _lib, ops

    dev = torch.device(DEV)
    word = ops.status_word(dev)
    torch.cuda.synchronize()
    ops.check_device_status(dev)  # start clean
    x = torch.randn(256, 128, device=dev).to(torch.bfloat16).requires_grad_(True)
    w = torch.randn(256, 128, device=dev).to(torch.bfloat16).requires_grad_(True)
    ck.linear_swiglu(x, w).sum().backward()  # healthy step: nothing is raised, snapshots read zero
    torch.cuda.synchronize()
    rc = _lib.lib.coda_b200_selftest_wait_timeout(word.data_ptr(), 2000, None, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    with pytest.raises(RuntimeError, match="device-side error code"):
        for _ in range(4):  # the first guard that runs after the failed launch has finished sees the code
            out = ck.linear_swiglu(x, w)
            torch.cuda.synchronize()
            out.sum().backward()
            torch.cuda.synchronize()
    # the report cleared the word; the next steps run normally
    torch.cuda.synchronize()
    ck.linear_swiglu(x, w).sum().backward()
    torch.cuda.synchronize()
    ck.linear_swiglu(x, w).sum().backward()
    torch.cuda.synchronize()
    ops.check_device_status(dev)


def test_status_poll_reports_a_device_resident_word_without_sync():
    """`coda_b200_status_poll` is the same lazy check for callers that keep the status word in device memory: snapshot,
    event query, report once, clear."""
    from coda_kernels_b200 import _lib

    lib = _lib.lib
    dev = torch.device(DEV)
    word = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    assert lib.coda_b200_status_poll(word.data_ptr(), stream) == 0  # takes a snapshot of a clean word
    torch.cuda.synchronize()
    assert lib.coda_b200_selftest_wait_timeout(word.data_ptr(), 2000, None, stream) == 0
    codes = []
    for _ in range(3):  # 1st: old snapshot was clean, takes a new one; 2nd (after the kernel ended): reports; 3rd: clean again
        torch.cuda.synchronize()
        codes.append(lib.coda_b200_status_poll(word.data_ptr(), stream))
    assert codes[0] == 0 and codes[1] > 0 and codes[2] == 0, codes
    torch.cuda.synchronize()
    assert int(word.item()) == 0, "reporting clears the device word"
    assert lib.coda_b200_status_poll(None, None) == -1
