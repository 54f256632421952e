"""Sharded operators on 2 GPUs (one process per GPU, NCCL) against the unsharded oracle.  Skipped with fewer than 2 GPUs."""

import functools
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import coda_kernels_b200 as ck
    from coda_kernels_b200 import parallel
    from oracle import eager, inputs

    failures = []

    def close(a, b, what, tol=TOL):
        err = eager.max_rel_err(a, b)
        if not err <= tol:
            failures.append(f"rank {rank} {what}: {err:.3e}")

    def leaf(t):
        return t.to(dev).detach().requires_grad_(True)

    try:
        # ---- swiglu, column-parallel
        d = inputs.swiglu_inputs(512, 256, 512)
        (ro,), g = eager.fwd_bwd(eager.linear_swiglu, {"x": d["x"].to(dev), "weight": d["weight"].to(dev)}, ["x", "weight"], d["dout"].to(dev))
        lo, hi = parallel.shard_bounds(d["weight"].shape[0], rank, world, 16)
        x, w = leaf(d["x"]), leaf(parallel.shard_swiglu_weight(d["weight"], rank, world).contiguous())
        out = ck.linear_swiglu(x, w)
        dx, dw = torch.autograd.grad(out, (x, w), d["dout"][:, lo // 2 : hi // 2].contiguous().to(dev))
        dx32 = dx.float()
        dist.all_reduce(dx32)
        close(out, ro[:, lo // 2 : hi // 2], "swiglu out")
        close(dw, g["weight"][lo:hi], "swiglu dweight")
        close(dx32, g["x"], "swiglu dx (sum of partials)")

        # ---- cross entropy, vocab-parallel (ragged vocabulary split, ignored rows)
        d = inputs.cross_entropy_inputs(300, 256, 1000, ignore_frac=0.1)
        t = d["target"].to(dev)
        fn = functools.partial(eager.linear_cross_entropy, target=t)
        (rl,), g = eager.fwd_bwd(fn, {"x": d["x"].to(dev), "weight": d["weight"].to(dev)}, ["x", "weight"], torch.tensor(1.0, device=dev))
        lo, hi = parallel.shard_bounds(1000, rank, world, 8)
        x, w = leaf(d["x"]), leaf(d["weight"][lo:hi].contiguous())
        loss = parallel.vocab_parallel_linear_cross_entropy(x, w, t, lo)
        dx, dw = torch.autograd.grad(loss, (x, w))
        if abs(float(loss) - float(rl)) > 1e-3 * abs(float(rl)):
            failures.append(f"rank {rank} ce loss {float(loss)} vs {float(rl)}")
        close(dx, g["x"], "ce dx (all-reduced)")
        close(dw, g["weight"][lo:hi], "ce dweight")

        # ---- qk-norm + rope, head-parallel
        hd, hq, hk, hv = 128, 4, 2, 2
        d = inputs.qknorm_rope_inputs(200, 256, hd, hq, hk, hv, seq_len=64)
        fn = functools.partial(eager.linear_qknorm_rope, positions=d["positions"].to(dev), frequencies=d["frequencies"].to(dev),
                               head_dim=hd, num_heads_q=hq, num_heads_k=hk, eps=1e-6)
        outs, g = eager.fwd_bwd(fn, {n: d[n].to(dev) for n in ("x", "weight", "gamma")}, ["x", "weight", "gamma"],
                                (d["dq"].to(dev), d["dk"].to(dev), d["dv"].to(dev)))
        lw, lf, lq, lk, lv = parallel.shard_qkv_weight(d["weight"], d["frequencies"], hd, hq, hk, hv, rank, world)
        x, w, gm = leaf(d["x"]), leaf(lw), leaf(d["gamma"])
        sl = lambda t, n: t[:, rank * n * hd : (rank + 1) * n * hd].contiguous().to(dev)  # noqa: E731
        q, k, v = ck.linear_qknorm_rope(x, w, gm, d["positions"].to(dev), lf.to(dev), hd, lq, lk, 1e-6)
        dx, dw, dg = torch.autograd.grad((q, k, v), (x, w, gm), (sl(d["dq"], lq), sl(d["dk"], lk), sl(d["dv"], lv)))
        dx32, dg32 = dx.float(), dg.float()
        dist.all_reduce(dx32)
        dist.all_reduce(dg32)
        for a, b, n, cnt in ((q, outs[0], "q", lq), (k, outs[1], "k", lk), (v, outs[2], "v", lv)):
            close(a, b[:, rank * cnt * hd : (rank + 1) * cnt * hd], f"qk {n}")
        close(dx32, g["x"], "qk dx (sum of partials)")
        close(dg32, g["gamma"], "qk dgamma (sum over ranks)")

        # ---- the sharded wrappers: same slices, dx all-reduced inside the backward (under the weight-gradient GEMM)
        d = inputs.swiglu_inputs(512, 256, 512)
        (ro,), g = eager.fwd_bwd(eager.linear_swiglu, {"x": d["x"].to(dev), "weight": d["weight"].to(dev)}, ["x", "weight"], d["dout"].to(dev))
        lo, hi = parallel.shard_bounds(d["weight"].shape[0], rank, world, 16)
        x, w = leaf(d["x"]), leaf(parallel.shard_swiglu_weight(d["weight"], rank, world).contiguous())
        out = parallel.column_parallel_linear_swiglu(x, w)
        dx, dw = torch.autograd.grad(out, (x, w), d["dout"][:, lo // 2 : hi // 2].contiguous().to(dev))
        close(out, ro[:, lo // 2 : hi // 2], "column-parallel swiglu out")
        close(dw, g["weight"][lo:hi], "column-parallel swiglu dweight")
        close(dx, g["x"], "column-parallel swiglu dx (all-reduced in the backward)")

        d = inputs.sigmoid_inputs(300, 256, 256)
        (ro,), g = eager.fwd_bwd(eager.linear_sigmoid, {"x": d["x"].to(dev), "weight": d["weight"].to(dev)}, ["x", "weight"], d["dout"].to(dev))
        lo, hi = parallel.shard_bounds(256, rank, world, 8)
        x, w = leaf(d["x"]), leaf(parallel.shard_rows(d["weight"], rank, world).contiguous())
        out = parallel.column_parallel_linear_sigmoid(x, w)
        dx, dw = torch.autograd.grad(out, (x, w), d["dout"][:, lo:hi].contiguous().to(dev))
        close(out, ro[:, lo:hi], "column-parallel sigmoid out")
        close(dw, g["weight"][lo:hi], "column-parallel sigmoid dweight")
        close(dx, g["x"], "column-parallel sigmoid dx (all-reduced in the backward)")
        keep = parallel.column_parallel_linear_sigmoid(x, w, reduce_dx=False)
        (dx_partial,) = torch.autograd.grad(keep, (x,), d["dout"][:, lo:hi].contiguous().to(dev))
        dx32 = dx_partial.float()
        dist.all_reduce(dx32)
        close(dx32, g["x"], "column-parallel sigmoid dx (partials kept, summed here)")

        d = inputs.qknorm_rope_inputs(200, 256, hd, hq, hk, hv, seq_len=64)
        x, w, gm = leaf(d["x"]), leaf(lw), leaf(d["gamma"])
        q, k, v = parallel.head_parallel_linear_qknorm_rope(x, w, gm, d["positions"].to(dev), lf.to(dev), hd, lq, lk, 1e-6)
        dx, dw, dg = torch.autograd.grad((q, k, v), (x, w, gm), (sl(d["dq"], lq), sl(d["dk"], lk), sl(d["dv"], lv)))
        fn = functools.partial(eager.linear_qknorm_rope, positions=d["positions"].to(dev), frequencies=d["frequencies"].to(dev),
                               head_dim=hd, num_heads_q=hq, num_heads_k=hk, eps=1e-6)
        outs, g = eager.fwd_bwd(fn, {n: d[n].to(dev) for n in ("x", "weight", "gamma")}, ["x", "weight", "gamma"],
                                (d["dq"].to(dev), d["dk"].to(dev), d["dv"].to(dev)))
        for a, b, n, cnt in ((q, outs[0], "q", lq), (k, outs[1], "k", lk), (v, outs[2], "v", lv)):
            close(a, b[:, rank * cnt * hd : (rank + 1) * cnt * hd], f"head-parallel {n}")
        close(dx, g["x"], "head-parallel dx (all-reduced in the backward)")
        close(dg, g["gamma"], "head-parallel dgamma (summed over ranks in the backward)")
        torch.cuda.synchronize()
        ck.ops.check_device_status(dev)
    except Exception as ex:  # noqa: BLE001
        failures.append(f"rank {rank} raised {type(ex).__name__}: {ex}")
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("\n".join(failures))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_ops_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    problems = [(tmp_path / f"rank{r}.txt").read_text() for r in range(2)]
    assert not any(problems), "\n".join(p for p in problems if p)
