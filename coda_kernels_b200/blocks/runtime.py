"""Whole-model driver over the fused Llama-3 blocks: token ids in, loss out.

Counterpart of ``CodaRuntime`` (benchmarks/torchtitan/llama3_coda.py:12-97 of the reference): the same constructor
argument (anything that carries ``n_heads``, ``n_kv_heads``, ``dim``, ``norm_eps``, ``n_layers``, i.e. TorchTitan's
``TransformerModelArgs``), the same ``forward(model, tokens, targets, positions, frequencies)`` and the same module
layout of ``model``::

    model.tok_embeddings                      nn.Embedding
    model.layers[str(i)].attention.wqkv       [(hq + 2 hk) * d, dim]   q, k, v rows
    model.layers[str(i)].attention.wo         [dim, dim]
    model.layers[str(i)].attention_norm       RMSNorm weight [dim]
    model.layers[str(i)].feed_forward.wgu     [2 * ffn, dim]           gate / up rows interleaved
    model.layers[str(i)].feed_forward.wd      [dim, ffn]
    model.layers[str(i)].ffn_norm             RMSNorm weight [dim]
    model.norm, model.output                  final RMSNorm weight, LM head [vocab, dim]

The layers are walked as ``block_pre`` -> (attention, ``block``) x (n_layers - 1) -> attention, ``block_post``: every
projection, norm, RoPE and the loss run in the fused blocks; only the attention core sits between them.  The reference
calls FlashAttention-3 there, a Hopper kernel; here it is ``torch.nn.functional.scaled_dot_product_attention`` (causal,
grouped-query), a library call outside this package's hot path.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

from .llama3 import block, block_post, block_pre

_IGNORE_INDEX = -100


class Llama3Runtime:
    def __init__(self, model_args) -> None:
        self.num_heads = model_args.n_heads
        kv = getattr(model_args, "n_kv_heads", None)
        self.num_kv_heads = self.num_heads if kv is None else kv
        self.head_dim = model_args.dim // model_args.n_heads
        self.norm_eps = model_args.norm_eps
        self.num_layers = model_args.n_layers
        self.attention_scale = self.head_dim ** -0.5

    def attention(self, qkv: Tensor) -> Tensor:
        """Causal grouped-query attention on the packed ``[batch, length, (hq + 2 hk) * d]`` projection."""
        b, t, _ = qkv.shape
        hq, hk, d = self.num_heads, self.num_kv_heads, self.head_dim
        q, k, v = qkv.split((hq * d, hk * d, hk * d), dim=-1)
        q = q.reshape(b, t, hq, d).transpose(1, 2)
        k = k.reshape(b, t, hk, d).transpose(1, 2)
        v = v.reshape(b, t, hk, d).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=self.attention_scale, enable_gqa=hq != hk)
        return o.transpose(1, 2).reshape(b, t, hq * d)

    def forward(self, model: torch.nn.Module, tokens: Tensor, targets: Tensor, positions: Tensor, frequencies: Tensor) -> Tensor:
        """Sum of the per-token losses (``reduction="sum"``, as the reference runtime returns it)."""
        layers = [model.layers[str(i)] for i in range(self.num_layers)]
        h = model.tok_embeddings(tokens)
        h, qkv = block_pre(x=h, w=layers[0].attention.wqkv.weight, wn=layers[0].attention_norm.weight, positions=positions,
                           frequencies=frequencies, eps=self.norm_eps)
        for this, nxt in zip(layers[:-1], layers[1:]):
            h, qkv = block(x0=h, y0=self.attention(qkv), w0=this.attention.wo.weight, w1=this.feed_forward.wgu.weight,
                           w2=this.feed_forward.wd.weight, w3=nxt.attention.wqkv.weight, wn0=this.ffn_norm.weight,
                           wn1=nxt.attention_norm.weight, positions=positions, frequencies=frequencies, eps=self.norm_eps)
        last = layers[-1]
        return block_post(x0=h, y0=self.attention(qkv), w0=last.attention.wo.weight, w1=last.feed_forward.wgu.weight,
                          w2=last.feed_forward.wd.weight, w3=model.output.weight, wn0=last.ffn_norm.weight, wn1=model.norm.weight,
                          targets=targets, eps=self.norm_eps, ignore_index=_IGNORE_INDEX, reduction="sum")


# the reference's name for the same thing
CodaRuntime = Llama3Runtime
