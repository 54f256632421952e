"""Host-side logic: RoPE frequency tables, shard bounds, target re-basing, and the 2-rank LSE exchange over gloo."""

import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from coda_kernels_b200 import parallel, rope_utils
from oracle import eager, inputs


def test_make_rope_frequencies_contract():
    inv = rope_utils.rope_inv_freq(128, theta=500000.0)
    f = rope_utils.make_rope_frequencies(inv, num_heads=5)
    assert f.dtype == torch.float32 and f.shape == (5 * 128,)
    pairs = f[:128].reshape(-1, 2).to(torch.float64)
    turns = inv.to(torch.float64) / (2 * math.pi)
    assert torch.allclose(pairs.sum(dim=1), turns, rtol=1e-13, atol=0)
    assert torch.equal(f[:128], f[128:256])
    # same table as the synthetic-input generator of the oracle
    d = inputs.qknorm_rope_inputs(4, 16, 128, 3, 2, 2, 4)
    assert torch.equal(d["frequencies"], f)


def test_shard_bounds_cover_everything():
    for total, world, mult in [(28672, 8, 16), (128256, 8, 8), (5120, 4, 8), (48, 5, 16)]:
        spans = [parallel.shard_bounds(total, r, world, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a, b), (c, d) in zip(spans, spans[1:]):
            assert b == c and (b - a) % mult == 0
    with pytest.raises(ValueError):
        parallel.shard_bounds(100, 0, 2, 16)


def test_shard_qkv_weight_layout():
    d, hq, hk, hv, K = 4, 4, 2, 2, 3
    w = torch.arange((hq + hk + hv) * d * K, dtype=torch.float32).reshape(-1, K)
    f = torch.arange((hq + hk) * d, dtype=torch.float32)
    lw, lf, lq, lk, lv = parallel.shard_qkv_weight(w, f, d, hq, hk, hv, rank=1, world=2)
    assert (lq, lk, lv) == (2, 1, 1)
    assert torch.equal(lw[: 2 * d], w[2 * d : 4 * d])
    assert torch.equal(lw[2 * d : 3 * d], w[hq * d + d : hq * d + 2 * d])
    assert torch.equal(lw[3 * d :], w[(hq + hk) * d + d : (hq + hk) * d + 2 * d])
    assert torch.equal(lf, torch.cat((f[2 * d : 4 * d], f[hq * d + d : hq * d + 2 * d])))


def test_rebase_target():
    t = torch.tensor([0, 5, 9, -100, 10, 19], dtype=torch.int32)
    local, ign = parallel.rebase_target(t, vocab_start=10, vocab_local=10, ignore_index=-100)
    assert ign == -100
    assert local.tolist() == [-1, -1, -1, -100, 0, 9]
    local, ign = parallel.rebase_target(torch.tensor([0, 3, 12], dtype=torch.int32), 10, 10, ignore_index=0)
    assert ign == -3 and local.tolist() == [-3, -1, 2]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _lse_worker(rank: int, world: int, port: int, result_path: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d = inputs.cross_entropy_inputs(24, 32, 80, seed=11, ignore_frac=0.25)
        x, w, t = d["x"].float(), d["weight"].float(), d["target"]
        lo, hi = parallel.shard_bounds(w.shape[0], rank, world, 8)
        logits = x @ w[lo:hi].T
        local_t, ign = parallel.rebase_target(t, lo, hi - lo, -100)
        local_lse = torch.logsumexp(logits, dim=1)
        owned = local_t >= 0
        tl = torch.where(owned, logits[torch.arange(24), local_t.clamp(min=0).long()], torch.zeros(24))
        lse, tlogit = parallel.combine_lse(local_lse, tl)
        valid = t != -100
        losses = torch.where(valid, lse - tlogit, torch.zeros_like(lse))
        loss = losses.sum() / valid.sum()
        ref = eager.linear_cross_entropy(d["x"], d["weight"], t)
        dx_partial = torch.full((4, 4), float(rank + 1))
        parallel.allreduce_partial_dx(dx_partial)
        ok = abs(loss.item() - ref.item()) < 1e-5 and torch.equal(dx_partial, torch.full((4, 4), 3.0))
        if rank == 0:
            with open(result_path, "w") as f:
                f.write(f"{int(ok)} {loss.item()} {ref.item()}")
    finally:
        dist.destroy_process_group()


def _overlap_worker(rank: int, world: int, port: int, result_path: str):
    """The shared sharded backward on CPU ranks: the GEMMs are stood in for by torch matmuls (this test is about the
    host-side sequencing: partial dx, asynchronous all-reduce joined after the weight gradient, dgamma summed)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from coda_kernels_b200 import ops

        def fake_gemm(A, B, out=None, alpha=None, out_dtype=None, C=None):
            res = A.float() @ B.float()
            res = res * alpha if alpha is not None else res
            if out is not None:
                out.copy_(res)
                return out
            return res

        real_gemm, ops.gemm = ops.gemm, fake_gemm
        try:
            g = torch.Generator().manual_seed(5)
            x, weight, grad_pre = torch.randn(12, 8, generator=g), torch.randn(16, 8, generator=g), torch.randn(12, 16, generator=g)
            lo, hi = parallel.shard_bounds(16, rank, world, 8)
            dgamma = torch.full((4,), float(rank + 1))
            alpha = torch.tensor([0.5])
            dx, dw = parallel.linear_backward_overlapped(grad_pre[:, lo:hi], x, weight[lo:hi], True, True, None, True, alpha=alpha,
                                                         also_reduce=dgamma)
            dx_keep, _ = parallel.linear_backward_overlapped(grad_pre[:, lo:hi], x, weight[lo:hi], True, False, None, False)
            # the weight gradient in two launches (first rows capped beside the collective, the rest afterwards)
            real_plan, parallel.overlap_plan = parallel.overlap_plan, (lambda *a: (116, 4))
            try:
                _, dw_two = parallel.linear_backward_overlapped(grad_pre[:, lo:hi].bfloat16(), x.bfloat16(), weight[lo:hi].bfloat16(), True, True,
                                                                None, True)
            finally:
                parallel.overlap_plan = real_plan
            ref_two = grad_pre[:, lo:hi].bfloat16().float().T @ x.bfloat16().float()
            ok_two = dw_two.shape == ref_two.shape and torch.allclose(dw_two.float(), ref_two, atol=5e-2, rtol=2e-2)
            ok = ok_two and (torch.allclose(dx, 0.5 * grad_pre @ weight, atol=1e-5) and torch.allclose(dw, 0.5 * grad_pre[:, lo:hi].T @ x, atol=1e-5)
                  and torch.equal(dgamma, torch.full((4,), 3.0)) and torch.allclose(dx_keep, grad_pre[:, lo:hi] @ weight[lo:hi], atol=1e-5))
        finally:
            ops.gemm = real_gemm
        if rank == 0:
            with open(result_path, "w") as f:
                f.write(str(int(ok)))
    finally:
        dist.destroy_process_group()


def test_sharded_backward_reduces_dx_and_dgamma_two_ranks(tmp_path):
    out = tmp_path / "result.txt"
    mp.spawn(_overlap_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    assert out.read_text() == "1"


def test_overlap_plan_estimate(monkeypatch):
    """The weight-gradient GEMM that starts beside the dx all-reduce gives up the collective's SMs where that costs less than
    the transfer lasts (default: all of the GEMM or nothing); with the split switched on, only its first rows do."""
    dx_bytes = 16384 * 4096 * 2
    swiglu8 = (2.0 * 16384 * 3584 * 4096, 3584, dx_bytes, 8, 148)
    swiglu4 = (2.0 * 16384 * 7168 * 4096, 7168, dx_bytes, 4, 148)
    swiglu2 = (2.0 * 16384 * 14336 * 4096, 14336, dx_bytes, 2, 148)
    ce8 = (2.0 * 8192 * 16032 * 4096, 16032, 8192 * 4096 * 2, 8, 148)
    monkeypatch.setattr(parallel, "_OVERLAP_SPLIT", False)
    assert parallel.overlap_plan(*swiglu8) == (116, 3584) and parallel.overlap_plan(*swiglu4) == (116, 7168)
    assert parallel.overlap_plan(*swiglu2) == (0, 0) and parallel.overlap_plan(*ce8) == (0, 0)
    assert parallel.overlap_plan(1e9, 1024, dx_bytes, 1, 148) == (0, 0)
    assert parallel.overlap_plan(1e9, 1024, dx_bytes, 8, 40) == (0, 0), "never below half of the SMs"
    monkeypatch.setattr(parallel, "_OVERLAP_SPLIT", True)
    assert parallel.overlap_plan(*swiglu8) == (116, 2304)
    assert parallel.overlap_plan(2.0 * 16384 * 768 * 4096, 768, dx_bytes, 8, 148) == (116, 768)   # qknorm_rope, share of 8: all of it
    cap, part = parallel.overlap_plan(*swiglu4)
    assert cap == 116 and 0 < part < 7168 // 2 and part % 256 == 0
    assert parallel.overlap_plan(*swiglu2) == (0, 0)                                            # a tenth of the GEMM: no second launch
    cap, part = parallel.overlap_plan(*ce8)
    assert cap == 116 and 2048 <= part <= 4096 and part % 256 == 0
    assert parallel.overlap_plan(2.0 * 16384 * 14336 * 4096, 14336, 1 << 20, 8, 148) == (0, 0), "a 1 MB transfer is not worth a launch"


def test_vocab_parallel_lse_exchange_two_ranks(tmp_path):
    out = tmp_path / "result.txt"
    mp.spawn(_lse_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    ok, loss, ref = out.read_text().split()
    assert ok == "1", f"sharded loss {loss} vs oracle {ref}"


def test_block_wrappers_flatten_and_restore_batched_activations():
    """The layer blocks take ``[batch, length, dim]`` activations as the reference does and hand the kernels 2-D views."""
    from coda_kernels_b200.blocks import llama3

    x = torch.zeros(2, 3, 8, dtype=torch.bfloat16)
    flat = llama3._tokens(x)
    assert flat.shape == (6, 8) and flat.data_ptr() == x.data_ptr()
    assert llama3._like(torch.zeros(6, 5), x).shape == (2, 3, 5)
    assert llama3._like(torch.zeros(6, 5), flat).shape == (6, 5)
    with pytest.raises(AssertionError):  # LM-head targets must be int32, as in the reference
        w = torch.zeros(8, 8, dtype=torch.bfloat16)
        llama3.block_post(x, x, w, torch.zeros(16, 8, dtype=torch.bfloat16), w, w, torch.zeros(8, dtype=torch.bfloat16),
                          torch.zeros(8, dtype=torch.bfloat16), torch.zeros(6, dtype=torch.int64), 1e-5)


def test_runtime_reads_model_args_like_the_reference():
    import types

    from coda.runtime import CodaRuntime

    rt = CodaRuntime(types.SimpleNamespace(n_heads=32, n_kv_heads=None, dim=4096, norm_eps=1e-5, n_layers=4))
    assert (rt.num_heads, rt.num_kv_heads, rt.head_dim, rt.num_layers) == (32, 32, 128, 4)
    rt = CodaRuntime(types.SimpleNamespace(n_heads=32, n_kv_heads=8, dim=4096, norm_eps=1e-5, n_layers=4))
    assert rt.num_kv_heads == 8 and abs(rt.attention_scale - 128 ** -0.5) < 1e-12
