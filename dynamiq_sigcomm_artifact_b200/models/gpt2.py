"""GPT-2 causal LM (default: GPT-2 small - 12 layers, d_model 768, 12 heads, MLP 3072,
vocab 50257, context 1024), random-init, pre-LayerNorm, tied output embedding."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.embedding import TiedEmbedding
from ..ops.layers import LayerNorm, fused_cross_entropy, shift_labels
from .common import GeluMLP, SelfAttention, init_linear


@dataclass
class GPT2Config:
    n_layer: int = 12
    d_model: int = 768
    n_head: int = 12
    d_mlp: int = 3072
    vocab: int = 50257
    context: int = 1024
    eps: float = 1e-5

    @classmethod
    def tiny(cls) -> "GPT2Config":
        return cls(n_layer=2, d_model=128, n_head=4, d_mlp=512, vocab=1024, context=128)


class GPT2Block(nn.Module):
    def __init__(self, c: GPT2Config):
        super().__init__()
        self.ln1, self.ln2 = LayerNorm(c.d_model, c.eps), LayerNorm(c.d_model, c.eps)
        self.attn = SelfAttention(c.d_model, c.n_head, causal=True)
        self.mlp = GeluMLP(c.d_model, c.d_mlp)

    def forward(self, x):
        x = x + self.attn(self.ln1(x))
        return x + self.mlp(self.ln2(x))


class GPT2(nn.Module):
    def __init__(self, c: GPT2Config = GPT2Config()):
        super().__init__()
        self.config = c
        self.wte = TiedEmbedding(c.vocab, c.d_model)
        self.wpe = nn.Embedding(c.context, c.d_model)
        self.blocks = nn.ModuleList(GPT2Block(c) for _ in range(c.n_layer))
        self.ln_f = LayerNorm(c.d_model, c.eps)
        self.apply(init_linear)
        for b in self.blocks:  # GPT-2's scaled init of the residual projections
            nn.init.normal_(b.attn.proj.weight, std=0.02 / (2 * c.n_layer) ** 0.5)
            nn.init.normal_(b.mlp.proj.weight, std=0.02 / (2 * c.n_layer) ** 0.5)

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None):
        B, S = input_ids.shape
        pos = torch.arange(S, device=input_ids.device)
        x = self.wte(input_ids) + self.wpe(pos)
        if torch.is_autocast_enabled(x.device.type):
            x = x.to(torch.get_autocast_dtype(x.device.type))
        for blk in self.blocks:
            x = blk(x)
        h = self.ln_f(x)
        if labels is None:
            return F.linear(h, self.wte.weight)
        logits = self.wte.logits(h)
        return fused_cross_entropy(logits, shift_labels(labels).reshape(-1), self.config.vocab)
