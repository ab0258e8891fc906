"""Llama-style causal LM (default: the 1.2 B shape of Llama-3.2-1B - 16 layers, d_model 2048,
32 query / 8 KV heads, SwiGLU 8192, RMSNorm, RoPE theta 500000, vocab 128256, tied embeddings)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.embedding import TiedEmbedding
from ..ops.layers import fused_cross_entropy, padded_vocab_logits, shift_labels, RMSNorm, rope_tables
from .common import SelfAttention, SwiGLU, init_linear


@dataclass
class LlamaConfig:
    n_layer: int = 16
    d_model: int = 2048
    n_head: int = 32
    n_kv_head: int = 8
    d_ffn: int = 8192
    vocab: int = 128256
    context: int = 2048
    rope_theta: float = 500000.0
    eps: float = 1e-5
    tie_embeddings: bool = True

    @classmethod
    def tiny(cls) -> "LlamaConfig":
        return cls(n_layer=2, d_model=128, n_head=4, n_kv_head=2, d_ffn=256, vocab=1024, context=128)


class LlamaBlock(nn.Module):
    def __init__(self, c: LlamaConfig):
        super().__init__()
        self.norm1, self.norm2 = RMSNorm(c.d_model, c.eps), RMSNorm(c.d_model, c.eps)
        self.attn = SelfAttention(c.d_model, c.n_head, c.n_kv_head, bias=False, causal=True, rope=True)
        self.mlp = SwiGLU(c.d_model, c.d_ffn)

    def forward(self, x, cos, sin):
        x = x + self.attn(self.norm1(x), cos, sin)
        return x + self.mlp(self.norm2(x))


class Llama(nn.Module):
    def __init__(self, c: LlamaConfig = LlamaConfig()):
        super().__init__()
        self.config = c
        self.embed = TiedEmbedding(c.vocab, c.d_model)
        self.blocks = nn.ModuleList(LlamaBlock(c) for _ in range(c.n_layer))
        self.norm = RMSNorm(c.d_model, c.eps)
        self.lm_head = None if c.tie_embeddings else nn.Linear(c.d_model, c.vocab, bias=False)
        self.apply(init_linear)
        self._rope = None

    def _tables(self, S: int, device):
        if self._rope is None or self._rope[0].device != device or self._rope[0].size(0) < S:
            self._rope = rope_tables(max(S, self.config.context), self.config.d_model // self.config.n_head,
                                     self.config.rope_theta, device)
        return self._rope

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None):
        B, S = input_ids.shape
        cos, sin = self._tables(S, input_ids.device)
        x = self.embed(input_ids)
        if torch.is_autocast_enabled(x.device.type):
            x = x.to(torch.get_autocast_dtype(x.device.type))
        for blk in self.blocks:
            x = blk(x, cos, sin)
        w = self.embed.weight if self.lm_head is None else self.lm_head.weight
        h = self.norm(x)
        if labels is None:
            return F.linear(h, w)
        logits = self.embed.logits(h) if self.lm_head is None else padded_vocab_logits(h, w)
        return fused_cross_entropy(logits, shift_labels(labels).reshape(-1), self.config.vocab)
