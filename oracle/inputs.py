"""Seeded synthetic inputs with the shapes and distributions of the benchmark configurations.

TEST / BENCH INFRASTRUCTURE.  Tensors are drawn on the CPU from one
``torch.Generator`` seeded with 0, so the oracle and the kernels see the same
bits wherever they run.  The second parameter of every normal distribution is
a standard deviation, as in the reference's ``Sampler`` (benchmarks/utils/data.py:95-107).
"""

from __future__ import annotations

import math

import torch

BF16 = torch.bfloat16


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def _randn(g, *shape, std=1.0, dtype=BF16):
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * std).to(dtype=dtype)


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """``[K, F]`` gate and up matrices -> the operator's ``[2F, K]`` weight (row 2j = gate j, row 2j+1 = up j)."""
    return torch.stack((w_gate.T, w_up.T), dim=1).reshape(2 * w_gate.shape[1], w_gate.shape[0]).contiguous()


def swiglu_inputs(M: int, K: int, F: int, seed: int = 0) -> dict:
    g = _gen(seed)
    x = _randn(g, M, K)
    w_gate = _randn(g, K, F, std=1.0 / math.sqrt(K))
    w_up = _randn(g, K, F, std=1.0 / math.sqrt(K))
    dout = _randn(g, M, F)
    return {"x": x, "weight": interleave_gate_up(w_gate, w_up), "dout": dout}


def sigmoid_inputs(M: int, K: int, N: int, seed: int = 0) -> dict:
    g = _gen(seed)
    return {"x": _randn(g, M, K), "weight": _randn(g, N, K, std=1.0 / math.sqrt(K)), "dout": _randn(g, M, N)}


def cross_entropy_inputs(M: int, K: int, V: int, seed: int = 0, ignore_frac: float = 0.05, ignore_index: int = -100) -> dict:
    g = _gen(seed)
    x = _randn(g, M, K)
    weight = _randn(g, V, K, std=1.0 / math.sqrt(K))
    target = torch.randint(0, V, (M,), generator=g, dtype=torch.int64).to(dtype=torch.int32)
    ignored = torch.rand(M, generator=g) < ignore_frac
    target = torch.where(ignored, torch.full_like(target, ignore_index), target)
    return {"x": x, "weight": weight, "target": target}


def qknorm_rope_inputs(M: int, K: int, head_dim: int, hq: int, hk: int, hv: int, seq_len: int, theta: float = 500000.0,
                       seed: int = 0, pos_offset: int = 0) -> dict:
    g = _gen(seed)
    x = _randn(g, M, K)
    weight = _randn(g, (hq + hk + hv) * head_dim, K, std=1.0 / math.sqrt(K))
    gamma = (1.0 + 0.02 * torch.randn(2 * head_dim, generator=g)).to(dtype=BF16)
    positions = (torch.arange(M, dtype=torch.int64) % seq_len + pos_offset).to(dtype=torch.int32)
    p = torch.arange(0, head_dim, 2, dtype=torch.float32)
    inv_freq = 1.0 / (theta ** (p / head_dim))
    turns = inv_freq.to(dtype=torch.float64) / (2.0 * math.pi)
    hi = turns.to(dtype=torch.float32)
    lo = (turns - hi.to(dtype=torch.float64)).to(dtype=torch.float32)
    frequencies = torch.stack((hi, lo), dim=1).reshape(-1).repeat(hq + hk).contiguous()
    return {
        "x": x, "weight": weight, "gamma": gamma, "positions": positions, "frequencies": frequencies,
        "dq": _randn(g, M, hq * head_dim), "dk": _randn(g, M, hk * head_dim), "dv": _randn(g, M, hv * head_dim),
    }


def llama3_block_inputs(M: int, dim: int, ffn: int, head_dim: int, heads: int, kv_heads: int, vocab: int, seq_len: int,
                        theta: float = 500000.0, seed: int = 0) -> dict:
    """Inputs of the three Llama-3 layer blocks: residual stream, attention output, nn.Linear-style weights (SwiGLU weight
    interleaved), norm weights near 1, QKV frequencies that are zero on the v columns, and cotangents."""
    g = _gen(seed)
    n_qkv = (heads + 2 * kv_heads) * head_dim
    p = torch.arange(0, head_dim, 2, dtype=torch.float32)
    turns = (1.0 / (theta ** (p / head_dim))).to(dtype=torch.float64) / (2.0 * math.pi)
    hi = turns.to(dtype=torch.float32)
    lo = (turns - hi.to(dtype=torch.float64)).to(dtype=torch.float32)
    per_head = torch.stack((hi, lo), dim=1).reshape(-1)
    frequencies = torch.cat((per_head.repeat(heads + kv_heads), torch.zeros(kv_heads * head_dim))).contiguous()
    norm = lambda: (1.0 + 0.1 * torch.randn(dim, generator=g)).to(dtype=BF16)  # noqa: E731
    targets = torch.randint(0, vocab, (M,), generator=g, dtype=torch.int64).to(dtype=torch.int32)
    targets[::7] = -100
    return {
        "x0": _randn(g, M, dim), "y0": _randn(g, M, heads * head_dim),
        "w_qkv": _randn(g, n_qkv, dim, std=dim**-0.5), "w0": _randn(g, dim, heads * head_dim, std=(heads * head_dim) ** -0.5),
        "w1": _randn(g, 2 * ffn, dim, std=dim**-0.5), "w2": _randn(g, dim, ffn, std=ffn**-0.5),
        "w_vocab": _randn(g, vocab, dim, std=dim**-0.5), "wn0": norm(), "wn1": norm(),
        "positions": (torch.arange(M, dtype=torch.int64) % seq_len).to(dtype=torch.int32), "frequencies": frequencies,
        "targets": targets, "dx": _randn(g, M, dim), "dqkv": _randn(g, M, n_qkv),
    }
