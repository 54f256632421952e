"""Benchmark of the fused-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--op NAME]

A step is one forward + backward pass of one operator over one batch of seeded
synthetic input.  The headline workload is ``linear_swiglu`` at the Llama-3-8B
MLP shape (x [16384, 4096], interleaved weight [28672, 4096]).  Without
``--op`` the same JSON line also carries an ``ops`` object with the other
operators of the path (``cross_entropy``, ``qknorm_rope``, ``sigmoid``) at their
benchmark shapes and, on more than one GPU, ``swiglu_with_dx_allreduce``; with
``--op NAME`` only that operator is measured, as the headline.  With
``--gpus N`` (one process per GPU under ``torch.distributed.run``) each operator
is sharded column-, head- or vocab-parallel and the total work stays fixed.

Timing: W warm-up steps, then windows of exactly K steps, each window bracketed
by a barrier + synchronize and timed with CUDA events, the maximum over ranks
taken per window; enough windows are run to cover about a second (at least 5)
and the MEDIAN window is reported (the per-iteration-median protocol of the
reference's harness, benchmarks/bench_utils.py:45-82, at window granularity).
``nvidia-smi`` samples clocks every 20 ms meanwhile.

Rank 0 prints ONE JSON line.  ``value`` is whole-job TFLOP/s (algorithmic GEMM
flops only) with inputs resident in HBM; ``e2e`` is the same metric with
host-to-device copies of the inputs and device-to-host copies of the results
inside the timed region; ``roofline`` describes the dominant kernel (the fused
forward GEMM) timed alone; ``cpu_baseline`` is the oracle's eager formulation
timed on the host cores for a bounded row sample.  ``--impl reference`` times
that CPU formulation alone, on the same sample, as the reference arm.
"""

from __future__ import annotations

import argparse
import gc
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

METRIC = "fused GEMM+epilogue TFLOP/s (% of B200 bf16 peak), fwd+bwd, at 1/2/4/8 GPUs"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# Benchmark shapes (the operator configurations of the task): see oracle/inputs.py for the distributions.
SHAPES = {
    "swiglu": {"M": 16384, "K": 4096, "F": 14336},
    "sigmoid": {"M": 32768, "K": 5120, "N": 5120},
    # the sigmoid configuration read literally: sigmoid(X W_gate) * (X W_val), an extension op (the reference's
    # linear_sigmoid has no value branch); F = width of each of the two projections
    "sigmoid_glu": {"M": 32768, "K": 5120, "F": 5120},
    "cross_entropy": {"M": 8192, "K": 4096, "V": 128256},
    "qknorm_rope": {"M": 16384, "K": 4096, "head_dim": 128, "hq": 32, "hk": 8, "hv": 8, "seq_len": 4096},
    # one whole Llama-3-8B layer as the fused block (attention itself sits between two blocks, outside)
    "llama3_block": {"M": 16384, "dim": 4096, "ffn": 14336, "head_dim": 128, "heads": 32, "kv_heads": 8, "seq_len": 4096},
}


# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum from one ncu capture).
# swiglu: 893.4 MB (561.5 read + 331.9 written) measured at 4096 rows (the committed ncu summary of the swiglu GEMMs), x4 for the 16384-row launch,
# since the traffic grows in proportion to the rows.
NCU_TRAFFIC = {"swiglu": 3.574e9}


def algorithmic_flops(op: str, s: dict) -> float:
    """Forward + backward GEMM flops (3 GEMMs of 2*M*K*N each); recomputation never counts."""
    if op == "llama3_block":
        qd, nqkv = s["heads"] * s["head_dim"], (s["heads"] + 2 * s["kv_heads"]) * s["head_dim"]
        per_row = s["dim"] * qd + s["dim"] * 2 * s["ffn"] + s["ffn"] * s["dim"] + s["dim"] * nqkv  # o-proj, gate/up, down, next qkv
        return 3.0 * 2.0 * s["M"] * per_row
    if op in ("swiglu", "sigmoid_glu"):
        n = 2 * s["F"]
    elif op == "sigmoid":
        n = s["N"]
    elif op == "cross_entropy":
        n = s["V"]
    else:
        n = (s["hq"] + s["hk"] + s["hv"]) * s["head_dim"]
    return 3.0 * 2.0 * s["M"] * s["K"] * n


def load_peaks() -> tuple[dict, str]:
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples ``nvidia-smi`` clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self, wait_s: float = 8.0):
        """Launch nvidia-smi and wait for its first sample: its start-up stalls CUDA launches for a while, so it
        has to be over before anything is timed."""
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        t0 = time.perf_counter()
        while not self.rows and time.perf_counter() - t0 < wait_s:
            time.sleep(0.05)

    def mark(self) -> int:
        return len(self.rows)

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 7:
                self.rows.append(parts)

    def stop(self) -> None:
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        self.proc = None

    def summary(self, first: int = 0, last: int | None = None) -> dict | None:
        """Summarise the samples taken between the two marks (a timed region); sampling goes on."""
        if self.proc is None and not self.rows:
            return None
        sm = []
        reasons = set()
        sm_max = None
        power = []
        rows = self.rows[first:last] if (last is not None and last > first) else self.rows[first:]
        if not rows:
            rows = self.rows[-1:]
        for r in rows:
            try:
                sm.append(float(r[0]))
                sm_max = float(r[1])
                power.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": sm_max,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


# ------------------------------------------------------------------------------------------------ workloads
class Workload:
    """One operator at its benchmark shape, sharded for ``world`` ranks; inputs live on ``device``."""

    def __init__(self, op: str, rank: int, world: int, device: torch.device, pinned_host: bool, rows: int = 0, share_of: int = 0):
        import coda_kernels_b200 as ck
        from coda_kernels_b200 import parallel
        from oracle import inputs

        self.op, self.device, self.ck, self.parallel = op, device, ck, parallel
        # `share_of` = W on one GPU: the weights are cut as for rank 0 of W ranks and this process times that share
        # alone, without any communication (`self.world` stays 1; `self.share` scales the flops that are counted)
        self.rank, self.world, self.share = rank, world, 1.0
        if share_of > 1:
            if world != 1:
                raise SystemExit("--share-of times one rank's share on one GPU")
            self.share = 1.0 / share_of
            rank, world = 0, share_of
        s = dict(SHAPES[op])
        if rows:
            s["M"] = rows  # reduced-row variant of the same workload (profiling captures)
        self.shape = s
        if op in ("swiglu", "sigmoid_glu"):
            d = inputs.swiglu_inputs(s["M"], s["K"], s["F"])
            lo, hi = parallel.shard_bounds(2 * s["F"], rank, world, 16)
            host = {"x": d["x"], "weight": d["weight"][lo:hi].contiguous(), "dout": d["dout"][:, lo // 2 : hi // 2].contiguous()}
            self.kernels_per_step = 4  # fused GEMM, dswiglu, dgrad GEMM, wgrad GEMM
        elif op == "sigmoid":
            d = inputs.sigmoid_inputs(s["M"], s["K"], s["N"])
            lo, hi = parallel.shard_bounds(s["N"], rank, world, 8)
            host = {"x": d["x"], "weight": d["weight"][lo:hi].contiguous(), "dout": d["dout"][:, lo:hi].contiguous()}
            self.kernels_per_step = 4
        elif op == "cross_entropy":
            d = inputs.cross_entropy_inputs(s["M"], s["K"], s["V"])
            lo, hi = parallel.shard_bounds(s["V"], rank, world, 8)
            self.vocab_start = lo
            host = {"x": d["x"], "weight": d["weight"][lo:hi].contiguous(), "target": d["target"]}
            self.kernels_per_step = 5  # LSE GEMM, finalize, gradient fix-up, dgrad GEMM, wgrad GEMM
        elif op == "qknorm_rope":
            d = inputs.qknorm_rope_inputs(s["M"], s["K"], s["head_dim"], s["hq"], s["hk"], s["hv"], s["seq_len"])
            w, f, hq, hk, hv = parallel.shard_qkv_weight(d["weight"], d["frequencies"], s["head_dim"], s["hq"], s["hk"], s["hv"], rank, world)
            self.local_heads = (hq, hk, hv)
            dh = s["head_dim"]
            host = {
                "x": d["x"], "weight": w, "gamma": d["gamma"], "positions": d["positions"], "frequencies": f,
                "dq": d["dq"][:, rank * hq * dh : (rank + 1) * hq * dh].contiguous(),
                "dk": d["dk"][:, rank * hk * dh : (rank + 1) * hk * dh].contiguous(),
                "dv": d["dv"][:, rank * hv * dh : (rank + 1) * hv * dh].contiguous(),
            }
            self.kernels_per_step = 5  # fused GEMM, qk backward, partial fold, dgrad GEMM, wgrad GEMM
        elif op == "llama3_block":
            if world != 1 or share_of > 1:
                raise SystemExit("the fused block benchmark runs on one GPU")
            d = inputs.llama3_block_inputs(s["M"], s["dim"], s["ffn"], s["head_dim"], s["heads"], s["kv_heads"], 1024, s["seq_len"])
            host = {k: d[k] for k in ("x0", "y0", "w0", "w1", "w2", "w_qkv", "wn0", "wn1", "positions", "frequencies", "dx", "dqkv")}
            self.kernels_per_step = 18  # 12 GEMMs, 2 rstd + 1 zdz row reductions, 2 dweight column reductions, rope backward
        else:
            raise ValueError(op)
        if op != "llama3_block":
            # a plain GEMM whose last round is cut along K is followed by the kernel that adds the parts: count it
            from coda_kernels_b200._lib import lib

            n_local, m, k = host["weight"].shape[0], s["M"], s["K"]
            self.kernels_per_step += sum(1 for shape in ((m, k, n_local), (n_local, k, m)) if lib.coda_b200_gemm_workspace_bytes(*shape) > 0)
        self.dev = {k: v.to(device) for k, v in host.items()}
        # End-to-end leg on several GPUs: the replicated activation `x` is uploaded as one row slice per rank and
        # all-gathered over NVLink, so the host bytes summed over ranks do not grow with the number of GPUs.
        self.rows_lo, self.rows_hi = parallel.shard_bounds(s["M"], self.rank, self.world, 1)
        if self.world > 1 and op != "llama3_block":
            host["x"] = host["x"][self.rows_lo:self.rows_hi].contiguous()
        self.host = {k: (v.pin_memory() if pinned_host else v) for k, v in host.items()}
        self.h2d_bytes = sum(v.numel() * v.element_size() for v in self.host.values())
        self.host_out: dict[str, torch.Tensor] = {}

    def upload(self, dst: dict | None = None):
        """Enqueue the host-to-device copies of one step's inputs on the current stream (plus, on several GPUs, the
        all-gather that completes `x`)."""
        dst = self.dev if dst is None else dst
        for k, v in self.host.items():
            if k == "x" and self.world > 1:
                dst[k][self.rows_lo:self.rows_hi].copy_(v, non_blocking=True)
            else:
                dst[k].copy_(v, non_blocking=True)
        if self.world > 1:
            torch.distributed.all_gather_into_tensor(dst["x"], dst["x"][self.rows_lo:self.rows_hi])

    def scatter_dx(self, results: dict) -> dict:
        """On several GPUs: sum the per-rank partial `dx` over ranks, each rank keeping its own row slice."""
        if self.world == 1 or "dx" not in results:
            return results
        dx = results["dx"]
        mine = torch.empty_like(dx[self.rows_lo:self.rows_hi])
        torch.distributed.reduce_scatter_tensor(mine, dx)
        out = dict(results)
        out["dx"] = mine
        return out

    def step(self, dev_inputs: dict | None = None, reduce_dx: bool | None = None):
        """Forward + backward through the public operator API.  Returns the result tensors.

        ``reduce_dx``: all-reduce the input gradient over ranks inside the step (the sharded wrappers start it right
        after the input-gradient GEMM, so that it runs under the weight-gradient GEMM).  ``None`` = off for the column-
        and head-parallel operators (each rank keeps its partial sum), on for the vocab-parallel cross entropy."""
        ck, d = self.ck, (self.dev if dev_inputs is None else dev_inputs)
        if reduce_dx is None:
            reduce_dx = self.op == "cross_entropy"
        return self._step(ck, d, reduce_dx)

    def _step(self, ck, d, reduce_dx: bool):
        if self.op == "llama3_block":
            from coda_kernels_b200.blocks import llama3

            names = ("x0", "y0", "w0", "w1", "w2", "w_qkv", "wn0", "wn1")
            lv = [d[n].detach().requires_grad_(True) for n in names]
            x2, qkv = llama3.block(*lv, d["positions"], d["frequencies"], 1e-5)
            grads = torch.autograd.grad((x2, qkv), lv, (d["dx"], d["dqkv"]))  # d["dx"] is accumulated into, as in training
            return {"x2": x2, "qkv": qkv, **{"d" + n: g_ for n, g_ in zip(names, grads)}}
        x = d["x"].detach().requires_grad_(True)
        w = d["weight"].detach().requires_grad_(True)
        several = self.world > 1
        if self.op in ("swiglu", "sigmoid_glu"):
            if self.op == "sigmoid_glu":
                out = ck.functional.linear_sigmoid_glu(x, w)
            else:
                out = self.parallel.column_parallel_linear_swiglu(x, w, reduce_dx=reduce_dx) if several else ck.linear_swiglu(x, w)
            dx, dw = torch.autograd.grad(out, (x, w), d["dout"])
            if self.op == "sigmoid_glu" and several and reduce_dx:
                self.parallel.allreduce_partial_dx(dx)
            return {"out": out, "dx": dx, "dweight": dw}
        if self.op == "sigmoid":
            out = self.parallel.column_parallel_linear_sigmoid(x, w, reduce_dx=reduce_dx) if several else ck.linear_sigmoid(x, w)
            dx, dw = torch.autograd.grad(out, (x, w), d["dout"])
            return {"out": out, "dx": dx, "dweight": dw}
        if self.op == "cross_entropy":
            if self.world == 1:
                loss = ck.linear_cross_entropy(x, w, d["target"], -100, "mean")
            else:
                loss = self.parallel.vocab_parallel_linear_cross_entropy(x, w, d["target"], self.vocab_start, -100, "mean",
                                                                         reduce_dx=reduce_dx)
            dx, dw = torch.autograd.grad(loss, (x, w))
            return {"loss": loss, "dx": dx, "dweight": dw}
        g = d["gamma"].detach().requires_grad_(True)
        hq, hk, _ = self.local_heads
        if several:  # dgamma is summed over the ranks inside the wrapper
            q, k, v = self.parallel.head_parallel_linear_qknorm_rope(x, w, g, d["positions"], d["frequencies"], self.shape["head_dim"],
                                                                     hq, hk, 1e-6, reduce_dx=reduce_dx)
        else:
            q, k, v = ck.linear_qknorm_rope(x, w, g, d["positions"], d["frequencies"], self.shape["head_dim"], hq, hk, 1e-6)
        dx, dw, dg = torch.autograd.grad((q, k, v), (x, w, g), (d["dq"], d["dk"], d["dv"]))
        return {"q": q, "k": k, "v": v, "dx": dx, "dweight": dw, "dgamma": dg}

    def download(self, results: dict) -> int:
        nbytes = 0
        for k, v in results.items():
            buf = self.host_out.get(k)
            if buf is None:
                buf = torch.empty(v.shape, dtype=v.dtype, device="cpu").pin_memory()
                self.host_out[k] = buf
            buf.copy_(v, non_blocking=True)
            nbytes += v.numel() * v.element_size()
        return nbytes

    def dominant_kernel(self):
        """(label, callable, flops per launch): the fused forward GEMM of this rank's shard, launched alone."""
        ck, d, s = self.ck, self.dev, self.shape
        if self.op == "llama3_block":
            from coda_kernels_b200 import ops_rmsnorm

            h = d["x0"]
            rstd = torch.ones(h.shape[0], dtype=torch.float32, device=h.device)
            flops = 2.0 * h.shape[0] * h.shape[1] * d["w1"].shape[0]
            return "gemm_kernel<EpiSwiGLU> (deferred RMSNorm)", (lambda: ops_rmsnorm.gemm_rmsnorm_swiglu(h, d["w1"].mT, rstd)), flops
        x, w = d["x"], d["weight"]
        flops = 2.0 * x.shape[0] * x.shape[1] * w.shape[0]
        if self.op == "swiglu":
            return "gemm_kernel<EpiSwiGLU>", (lambda: ck.ops.gemm_swiglu(x, w.mT)), flops
        if self.op == "sigmoid_glu":
            return "gemm_kernel<EpiSigmoidGLU>", (lambda: ck.functional.linear_sigmoid_glu(x, w)), flops
        if self.op == "sigmoid":
            return "gemm_kernel<EpiStore<sigmoid>>", (lambda: ck.ops.gemm_sigmoid(x, w.mT)), flops
        if self.op == "cross_entropy":
            return "gemm_kernel<EpiLse<store>>", (lambda: ck.ops.gemm_lse_partials(x, w.mT, d["target"], True)), flops
        hq, hk, _ = self.local_heads
        return "gemm_kernel<EpiQKNormRope>", (
            lambda: ck.ops.gemm_qknorm_rope(x, w.mT, d["gamma"], d["positions"], d["frequencies"], s["head_dim"], hq, hk, 1e-6)), flops


# ------------------------------------------------------------------------------------------------ CPU formulation (oracle) timing
def cpu_eager_step(op: str, rows: int, seed_inputs: dict | None = None):
    """Build a callable that runs the oracle's eager formulation fwd+bwd on ``rows`` rows of the workload on the CPU."""
    import functools

    from oracle import eager, inputs

    s = dict(SHAPES[op])
    if op == "sigmoid_glu":
        d = inputs.swiglu_inputs(rows, s["K"], s["F"])
        fn = lambda: eager.fwd_bwd(eager.linear_sigmoid_glu, {"x": d["x"], "weight": d["weight"]}, ["x", "weight"], d["dout"])
    elif op == "swiglu":
        d = inputs.swiglu_inputs(rows, s["K"], s["F"])
        fn = lambda: eager.fwd_bwd(eager.linear_swiglu, {"x": d["x"], "weight": d["weight"]}, ["x", "weight"], d["dout"])
    elif op == "sigmoid":
        d = inputs.sigmoid_inputs(rows, s["K"], s["N"])
        fn = lambda: eager.fwd_bwd(eager.linear_sigmoid, {"x": d["x"], "weight": d["weight"]}, ["x", "weight"], d["dout"])
    elif op == "llama3_block":
        d = inputs.llama3_block_inputs(rows, s["dim"], s["ffn"], s["head_dim"], s["heads"], s["kv_heads"], 1024, s["seq_len"])
        names = ["x0", "y0", "w0", "w1", "w2", "w3", "wn0", "wn1"]
        blk = functools.partial(eager.llama3_block, positions=d["positions"], frequencies=d["frequencies"], eps=1e-5)
        fn = lambda: eager.fwd_bwd(blk, {n: d[{"w3": "w_qkv"}.get(n, n)] for n in names}, names, (d["dx"], d["dqkv"]))
    elif op == "cross_entropy":
        d = inputs.cross_entropy_inputs(rows, s["K"], s["V"])
        ce = functools.partial(eager.linear_cross_entropy, target=d["target"])
        fn = lambda: eager.fwd_bwd(ce, {"x": d["x"], "weight": d["weight"]}, ["x", "weight"], torch.tensor(1.0))
    else:
        d = inputs.qknorm_rope_inputs(rows, s["K"], s["head_dim"], s["hq"], s["hk"], s["hv"], s["seq_len"])
        qk = functools.partial(eager.linear_qknorm_rope, positions=d["positions"], frequencies=d["frequencies"],
                               head_dim=s["head_dim"], num_heads_q=s["hq"], num_heads_k=s["hk"], eps=1e-6)
        fn = lambda: eager.fwd_bwd(qk, {"x": d["x"], "weight": d["weight"], "gamma": d["gamma"]}, ["x", "weight", "gamma"],
                                   (d["dq"], d["dk"], d["dv"]))
    s["M"] = rows
    return fn, algorithmic_flops(op, s)


def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs are meant to use every core the process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(n, 1))
    return torch.get_num_threads()


def time_cpu(op: str, rows: int, steps: int, warmup: int) -> tuple[float, float]:
    """Returns (TFLOP/s, seconds per step) of the CPU eager formulation on a ``rows``-row sample."""
    use_all_host_threads()
    fn, flops = cpu_eager_step(op, rows)
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    return flops / dt / 1e12, dt


CPU_SAMPLE_ROWS = 4096  # one sample size for the in-line cpu_baseline and for the reference arm


def cpu_sample_text(op: str, rows: int) -> str:
    return (f"rows 0..{rows - 1} of {SHAPES[op]['M']} (full K and output width), fwd+bwd, "
            "oracle eager formulation in fp32 on bf16 inputs")


def run_reference_arm(args, rank: int) -> None:
    if rank != 0:
        return
    op = args.op or "swiglu"
    s = SHAPES[op]
    rows = args.cpu_rows or CPU_SAMPLE_ROWS
    tflops, dt = time_cpu(op, rows, args.steps, max(args.warmup, 1))
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(op), **s, "parallelism": f"cpu x{cores} threads", "l2": "n/a (host)"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": cpu_sample_text(op, rows)},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit_result(line)


def workload_name(op: str) -> str:
    return {
        "swiglu": "linear_swiglu fwd+bwd, Llama-3-8B MLP: x[16384,4096] W[28672,4096] interleaved gate/up",
        "sigmoid": "linear_sigmoid fwd+bwd: x[32768,5120] W[5120,5120]",
        "cross_entropy": "linear_cross_entropy fwd+bwd: x[8192,4096] W[128256,4096], 5% ignored, mean",
        "qknorm_rope": "linear_qknorm_rope fwd+bwd: x[16384,4096] W[6144,4096], GQA 32/8/8 x128, theta 5e5",
        "sigmoid_glu": "linear_sigmoid_glu (extension) fwd+bwd: x[32768,5120], W_gate and W_val [5120,5120] interleaved into [10240,5120]",
        "llama3_block": "fused Llama-3-8B layer block fwd+bwd: 16384 tokens, dim 4096, ffn 14336, GQA 32/8 x128 (o-proj, MLP, next QKV + RoPE)",
    }[op]


PARALLELISM = {"swiglu": "column", "sigmoid": "column", "cross_entropy": "vocab", "qknorm_rope": "head", "llama3_block": "no",
               "sigmoid_glu": "column"}


# ------------------------------------------------------------------------------------------------ result line
_RESULT_FD = None


def _claim_stdout() -> None:
    """Point fd 1 at stderr for the rest of the process and keep the real stdout for the one result line:
    libraries (NCCL's version banner, for one) write to fd 1 behind Python's back."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit_result(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


# ------------------------------------------------------------------------------------------------ timing
class Bench:
    """What every measurement of one run shares: ranks, the clock sampler, the CUDA graphs to drop before teardown."""

    def __init__(self, args, rank: int, local_rank: int, world: int, device: torch.device):
        self.args, self.rank, self.local_rank, self.world, self.device = args, rank, local_rank, world, device
        self.sampler = ClockSampler(local_rank)
        self.graphs: list = []
        self.peaks, self.peak_kind = load_peaks()
        self.peak = float(self.peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        self.peak_sustained = float(self.peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))

    def barrier(self) -> None:
        if self.world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, ms: float) -> float:
        if self.world == 1:
            return ms
        t = torch.tensor([ms], device=self.device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    def capture(self, step_fn):
        """One step (forward, backward, collectives) captured into a CUDA graph: the same public-API calls, minus the
        per-launch host work.  Returns the replay callable, or None when capture is off or failed."""
        if self.args.no_graph:
            return None
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                keep = step_fn()  # the graph's output tensors stay alive with it
            graph.replay()
            torch.cuda.synchronize()
            self.graphs.append((graph, keep))
            return graph.replay
        except Exception as ex:  # noqa: BLE001
            print(f"[bench] CUDA graph capture failed ({type(ex).__name__}: {ex}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
            return None

    def drop_graphs(self) -> None:
        """Destroy every captured graph.  A communicator cannot be torn down while a graph that holds its collectives
        is alive: that, not NCCL itself, is what blocked destroy_process_group() forever."""
        while self.graphs:
            graph, keep = self.graphs.pop()
            del keep
            graph.reset()
            del graph
        gc.collect()
        torch.cuda.synchronize()

    def time_windows(self, run_step, steps: int, min_windows: int = 5, target_s: float = 1.0, max_windows: int = 200):
        """Windows of exactly ``steps`` steps, each bracketed by barrier + synchronize, CUDA events on the launching
        stream, max over ranks per window.  Returns (median ms per step, per-window ms per step, clock summary)."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        per_window: list[float] = []
        total_ms = 0.0
        mark0 = self.sampler.mark()
        while len(per_window) < min_windows or (total_ms < target_s * 1e3 and len(per_window) < max_windows):
            self.barrier()
            e0.record()
            for _ in range(steps):
                run_step()
            e1.record()
            self.barrier()
            ms = self.max_over_ranks(e0.elapsed_time(e1))
            per_window.append(ms / steps)
            total_ms += ms
        mark1 = self.sampler.mark()
        clocks = self.sampler.summary(mark0, mark1) if self.rank == 0 else None
        return statistics.median(per_window), per_window, clocks


def measure_device(b: Bench, wl: Workload, reduce_dx: bool | None = None, with_eager: bool = True) -> dict:
    """Device-resident throughput of one operator: inputs already in HBM when the timed region starts."""
    args = b.args
    step_fn = lambda: wl.step(reduce_dx=reduce_dx)  # noqa: E731
    for _ in range(args.warmup):
        step_fn()
    b.barrier()
    replay = b.capture(step_fn)
    run_step = replay if replay is not None else step_fn
    b.barrier()
    ms_step, windows, clocks = b.time_windows(run_step, args.steps)
    flops = algorithmic_flops(wl.op, wl.shape) * wl.share
    value = flops / (ms_step * 1e-3) / 1e12
    res = {
        "value": value, "unit": "TFLOP/s", "ms_per_step": ms_step, "windows": len(windows),
        "ms_per_step_min": min(windows), "ms_per_step_max": max(windows),
        "tokens_per_s": wl.shape["M"] / (ms_step * 1e-3),
        "frac_of_peak": value / (b.world * b.peak), "frac_of_sustained_peak": value / (b.world * b.peak_sustained),
        "cuda_graph": replay is not None, "clocks": clocks,
        "ms_x_sm_mhz": (ms_step * clocks["sm_mhz"]) if (clocks and clocks.get("sm_mhz")) else None,
        "kernels_per_step": wl.kernels_per_step, "gpu_launches": wl.kernels_per_step * args.steps * len(windows),
    }
    if with_eager and replay is not None:
        # the same step with every launch dispatched from Python: what a training loop that does not replay a graph sees
        ms_eager, w_eager, _ = b.time_windows(step_fn, args.steps, min_windows=3, target_s=0.3)
        res["value_no_graph"] = flops / (ms_eager * 1e-3) / 1e12
        res["ms_per_step_no_graph"] = ms_eager
    return res


def measure_e2e(b: Bench, wl: Workload) -> dict:
    """Host buffers in, host buffers out, every step.  The copies of step i+1 / i-1 run on their own streams while
    step i computes (double-buffered inputs), as an input pipeline would.  On several GPUs every rank uploads its row
    slice of `x` (completed by an all-gather) and downloads its row slice of the summed `dx` (reduce-scatter)."""
    args, world = b.args, b.world
    compute = torch.cuda.current_stream()
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    bufs = [wl.dev, {k: torch.empty_like(v) for k, v in wl.dev.items()}]
    ev_up = [torch.cuda.Event(), torch.cuda.Event()]
    ev_free = [torch.cuda.Event(), torch.cuda.Event()]
    ev_done = torch.cuda.Event()

    def loop(n):
        nbytes = 0
        with torch.cuda.stream(up):
            wl.upload(bufs[0])
            ev_up[0].record(up)
        for i in range(n):
            k = i % 2
            if i + 1 < n:
                with torch.cuda.stream(up):
                    if i >= 1:
                        up.wait_event(ev_free[1 - k])
                    wl.upload(bufs[1 - k])
                    ev_up[1 - k].record(up)
            compute.wait_event(ev_up[k])
            res = wl.scatter_dx(wl.step(bufs[k], reduce_dx=False))
            ev_free[k].record(compute)
            ev_done.record(compute)
            with torch.cuda.stream(down):
                down.wait_event(ev_done)
                nbytes = wl.download(res)
                for t_ in res.values():
                    t_.record_stream(down)
        compute.wait_stream(down)
        compute.wait_stream(up)
        return nbytes

    loop(3)
    b.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    d2h = loop(args.steps)
    e1.record()
    b.barrier()
    ms = b.max_over_ranks(e0.elapsed_time(e1)) / args.steps
    flops = algorithmic_flops(wl.op, wl.shape)
    h2d = wl.h2d_bytes
    if world > 1:  # bytes of the whole job: sum over ranks
        t = torch.tensor([float(h2d), float(d2h)], device=b.device, dtype=torch.float64)
        torch.distributed.all_reduce(t)
        h2d, d2h = int(t[0].item()), int(t[1].item())
    return {"value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h,
            "bytes_are": "summed over ranks" if world > 1 else "of the one rank",
            "dx": "reduce-scattered on the device, each rank downloads its row slice" if world > 1 else "downloaded whole"}


def measure_kernel(b: Bench, wl: Workload) -> dict:
    """The dominant kernel (the fused forward GEMM of this rank's shard) launched alone, for the roofline."""
    label, launch, k_flops = wl.dominant_kernel()
    for _ in range(3):
        launch()
    torch.cuda.synchronize()
    n_k = max(b.args.steps, 10)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_k):
        launch()
    e1.record()
    torch.cuda.synchronize()
    k_ms = e0.elapsed_time(e1) / n_k
    achieved = k_flops / (k_ms * 1e-3) / 1e12
    traffic = NCU_TRAFFIC.get(wl.op) if (b.world == 1 and not b.args.rows and not b.args.share_of) else None
    return {"bound": "tensor", "kernel": label, "achieved": achieved, "peak": b.peak, "unit": "TFLOP/s", "frac": achieved / b.peak,
            "peak_kind": f"{b.peak_kind} burst bf16 (kernel timed alone)", "ms_per_launch": k_ms, "flops_per_launch": k_flops,
            "traffic": traffic}


def measure_op(b: Bench, op: str, headline: bool) -> tuple[dict, dict]:
    """Everything reported for one operator, plus (headline, several GPUs) its variant with the dx all-reduce.  The
    headline operator also gets the end-to-end leg."""
    args = b.args
    wl = Workload(op, b.rank, b.world, b.device, pinned_host=headline and not args.no_e2e, rows=args.rows, share_of=args.share_of)
    res = measure_device(b, wl, with_eager=not args.no_eager)
    res["workload"] = (workload_name(op) + (f" [rows reduced to {args.rows}]" if args.rows else "")
                       + (f" [rank 0's share of a {args.share_of}-GPU job, alone on one GPU, no communication]" if args.share_of > 1 else ""))
    res["shape"] = dict(wl.shape)
    res["parallelism"] = f"{PARALLELISM[op]}-parallel x{b.world}"
    if b.world > 1:
        res["dx_reduction"] = ("bf16 all-reduce inside the operator, issued before the weight-gradient GEMM so that the two overlap"
                               if op == "cross_entropy" else "none: every rank keeps its partial dx (see swiglu_with_dx_allreduce)")
    else:
        res["dx_reduction"] = "n/a (one GPU)"
    extra = {}
    if headline and b.world > 1 and op != "cross_entropy" and op != "llama3_block":
        with_ar = measure_device(b, wl, reduce_dx=True, with_eager=False)
        with_ar["dx_reduction"] = ("bf16 all-reduce (NCCL) of the [M, K] input gradient inside every step, issued before the "
                                   "weight-gradient GEMM so that the two overlap")
        extra[f"{op}_with_dx_allreduce"] = with_ar
    if headline and not args.no_e2e:
        res["e2e"] = measure_e2e(b, wl)
    res["roofline"] = measure_kernel(b, wl)
    res["l2"] = (f"no flush: every step streams {wl.h2d_bytes / 1e6:.0f} MB of inputs per rank plus larger intermediates, "
                 "more than the 126 MB L2")
    from coda_kernels_b200 import ops

    torch.cuda.synchronize()
    ops.check_device_status(b.device)
    b.drop_graphs()
    del wl
    gc.collect()
    torch.cuda.empty_cache()
    return res, extra


def _native_dispatch() -> bool:
    from coda_kernels_b200 import ops

    return ops._native is not None


def main() -> None:
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--op", default=None, choices=list(SHAPES),
                    help="measure this operator only (as the headline); default: linear_swiglu as the headline plus the other operators under `ops`")
    ap.add_argument("--cpu-rows", type=int, default=0, help="rows of the CPU-baseline sample (0 = default)")
    ap.add_argument("--rows", type=int, default=0, help="override the number of rows M (small captures under ncu); 0 = benchmark shape")
    ap.add_argument("--share-of", type=int, default=0, help="on one GPU: time rank 0's share of a job sharded over this many GPUs "
                    "(weights cut as for that job, no communication); implies --no-e2e and no CPU baseline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-clocks", action="store_true", help="do not sample nvidia-smi during the timed region")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from Python instead of replaying a CUDA graph of one step")
    ap.add_argument("--no-eager", action="store_true", help="skip the extra per-launch-dispatch timing (value_no_graph)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.share_of > 1:
        args.no_e2e = args.no_cpu_baseline = True

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU fallback")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep NCCL's banner off stdout: rank 0 prints one JSON line there
        torch.distributed.init_process_group("nccl", device_id=device)

    b = Bench(args, rank, local_rank, world, device)
    if rank == 0 and not args.no_clocks:
        b.sampler.start()

    head_op = args.op or "swiglu"
    head, extra = measure_op(b, head_op, headline=True)
    others = {}
    if args.op is None:
        for op in ("cross_entropy", "qknorm_rope", "sigmoid"):
            others[op], _ = measure_op(b, op, headline=False)
    others.update(extra)
    b.sampler.stop()

    # ---- CPU baseline (rank 0, single GPU run only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rows = args.cpu_rows or CPU_SAMPLE_ROWS
        tf, dt = time_cpu(head_op, rows, steps=3, warmup=1)
        cpu = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "seconds_per_sample_step": dt,
               "sample": cpu_sample_text(head_op, rows) + ", 1 warm-up + 3 timed"}

    if rank == 0:
        s = head["shape"]
        line = {
            "metric": METRIC, "value": head["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": head["workload"], **s, "global_batch_tokens": s["M"], "parallelism": head["parallelism"],
                       "dx_reduction": head["dx_reduction"], "cuda_graph": head["cuda_graph"], "l2": head["l2"],
                       "dispatch": "TORCH_LIBRARY shim (libcoda_b200_torch.so)" if _native_dispatch() else "ctypes custom ops",
                       "timing": f"median of {head['windows']} windows of {args.steps} steps, max over ranks per window"},
            "tokens_per_s": head["tokens_per_s"], "frac_of_peak": head["frac_of_peak"],
            "frac_of_sustained_peak": head["frac_of_sustained_peak"],
            "windows": head["windows"], "ms_per_step_min": head["ms_per_step_min"], "ms_per_step_max": head["ms_per_step_max"],
            "ms_x_sm_mhz": head["ms_x_sm_mhz"], "value_no_graph": head.get("value_no_graph"),
            "clocks": head["clocks"], "e2e": head.get("e2e"), "gpu_launches": head["gpu_launches"], "roofline": head["roofline"],
            "cpu_baseline": cpu, "ops": others,
        }
        emit_result(line)

    # ---- teardown: graphs are gone (measure_op dropped them), so the communicator can be destroyed and the
    # interpreter can exit normally.  The timer only ends a process whose teardown still blocked.
    torch.cuda.synchronize()
    sys.stderr.flush()
    if world > 1:
        watchdog = threading.Timer(60.0, lambda: (print("[bench] teardown blocked for 60 s; leaving", file=sys.stderr), os._exit(0)))
        watchdog.daemon = True
        watchdog.start()
        torch.distributed.barrier()
        torch.cuda.synchronize()
        torch.distributed.destroy_process_group()
        watchdog.cancel()


if __name__ == "__main__":
    main()
