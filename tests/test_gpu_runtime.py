"""The whole-model driver over the fused blocks: a two-layer GQA Llama-3 stand-in, token ids in, loss and weight
gradients out, against the same model written out in plain fp32 PyTorch."""

import types

import pytest
import torch
import torch.nn as nn

from oracle import eager, inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class _Norm(nn.Module):
    def __init__(self, dim, gen):
        super().__init__()
        self.weight = nn.Parameter((1.0 + 0.05 * torch.randn(dim, generator=gen)).to(torch.bfloat16))


class _Lin(nn.Module):
    def __init__(self, out_f, in_f, gen):
        super().__init__()
        self.weight = nn.Parameter((torch.randn(out_f, in_f, generator=gen) / in_f ** 0.5).to(torch.bfloat16))


class _Layer(nn.Module):
    def __init__(self, dim, ffn, nqkv, gen):
        super().__init__()
        self.attention = nn.Module()
        self.attention.wqkv = _Lin(nqkv, dim, gen)
        self.attention.wo = _Lin(dim, dim, gen)
        self.feed_forward = nn.Module()
        self.feed_forward.wgu = _Lin(2 * ffn, dim, gen)
        self.feed_forward.wd = _Lin(dim, ffn, gen)
        self.attention_norm = _Norm(dim, gen)
        self.ffn_norm = _Norm(dim, gen)


class _Model(nn.Module):
    def __init__(self, args, vocab, ffn, gen):
        super().__init__()
        d = args.dim // args.n_heads
        nqkv = (args.n_heads + 2 * args.n_kv_heads) * d
        self.tok_embeddings = nn.Embedding(vocab, args.dim)
        self.tok_embeddings.weight.data = torch.randn(vocab, args.dim, generator=gen).to(torch.bfloat16)
        self.layers = nn.ModuleDict({str(i): _Layer(args.dim, ffn, nqkv, gen) for i in range(args.n_layers)})
        self.norm = _Norm(args.dim, gen)
        self.output = _Lin(vocab, args.dim, gen)


def _reference_loss(model, args, tokens, targets, positions, frequencies):
    """The same network in fp32, unfused: RMSNorm, projections, interleaved-pair RoPE, causal GQA attention, SwiGLU."""
    hq, hk, d, eps = args.n_heads, args.n_kv_heads, args.dim // args.n_heads, args.norm_eps
    b, t = tokens.shape
    f = lambda p: p.float()  # noqa: E731

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * f(w)

    cos, sin = eager.rope_tables(positions, frequencies)
    h = f(model.tok_embeddings.weight)[tokens].reshape(b * t, -1)
    for i in range(args.n_layers):
        L = model.layers[str(i)]
        qkv = eager.rope_interleaved(norm(h, L.attention_norm.weight) @ f(L.attention.wqkv.weight).T, cos, sin)
        q, k, v = qkv.split((hq * d, hk * d, hk * d), dim=-1)
        q = q.reshape(b, t, hq, d).transpose(1, 2)
        k = k.reshape(b, t, hk, d).transpose(1, 2).repeat_interleave(hq // hk, dim=1)
        v = v.reshape(b, t, hk, d).transpose(1, 2).repeat_interleave(hq // hk, dim=1)
        att = (q @ k.transpose(-1, -2)) * d ** -0.5
        att = att.masked_fill(torch.ones(t, t, device=att.device, dtype=torch.bool).triu(1), float("-inf")).softmax(-1)
        o = (att @ v).transpose(1, 2).reshape(b * t, hq * d)
        h = h + o @ f(L.attention.wo.weight).T
        z = norm(h, L.ffn_norm.weight) @ f(L.feed_forward.wgu.weight).T
        h = h + (torch.nn.functional.silu(z[:, 0::2]) * z[:, 1::2]) @ f(L.feed_forward.wd.weight).T
    logits = norm(h, model.norm.weight) @ f(model.output.weight).T
    return torch.nn.functional.cross_entropy(logits, targets.long(), ignore_index=-100, reduction="sum")


def test_two_layer_gqa_model_matches_plain_pytorch():
    from coda.runtime import CodaRuntime
    from coda_kernels_b200 import ops
    from coda_kernels_b200.rope_utils import make_rope_frequencies

    gen = torch.Generator().manual_seed(3)
    args = types.SimpleNamespace(n_heads=4, n_kv_heads=2, dim=512, norm_eps=1e-5, n_layers=2)
    vocab, ffn, b, t = 1000, 768, 2, 96
    d = args.dim // args.n_heads
    model = _Model(args, vocab, ffn, gen).to(DEV)
    tokens = torch.randint(0, vocab, (b, t), generator=gen).to(DEV)
    targets = torch.randint(0, vocab, (b * t,), generator=gen, dtype=torch.int64).to(torch.int32)
    targets[::7] = -100
    targets = targets.to(DEV)
    positions = torch.arange(t, dtype=torch.int32).repeat(b).to(DEV)
    inv_freq = 500000.0 ** (-torch.arange(0, d, 2, dtype=torch.float32) / d)
    freq_qk = make_rope_frequencies(inv_freq, args.n_heads + args.n_kv_heads)
    frequencies = torch.cat((freq_qk, torch.zeros(args.n_kv_heads * d))).to(DEV)  # v columns are not rotated

    runtime = CodaRuntime(args)
    loss = runtime.forward(model, tokens, targets, positions, frequencies)
    watched = [model.layers["0"].attention.wqkv.weight, model.layers["1"].feed_forward.wgu.weight, model.output.weight,
               model.layers["0"].ffn_norm.weight]
    grads = torch.autograd.grad(loss, watched)
    torch.cuda.synchronize()
    ops.check_device_status(torch.device(DEV))

    ref = _reference_loss(model, args, tokens, targets, positions, frequencies)
    ref_grads = torch.autograd.grad(ref, watched)
    assert abs(float(loss) - float(ref)) <= 2e-3 * abs(float(ref)), f"loss {float(loss)} vs {float(ref)}"
    for g, r, name in zip(grads, ref_grads, ("d wqkv[0]", "d wgu[1]", "d output", "d ffn_norm[0]")):
        err = eager.max_rel_err(g, r)
        assert err <= 3e-2, f"{name}: max rel err {err:.3e}"  # two layers of bf16 activations between loss and the first weights
