"""Pieces shared by the model families: attention, MLPs, initialisation, configs.

Random-init re-implementations of the architectures the reference fine-tunes from Hugging Face
checkpoints (testbed_evaluation/train_llm_causal.py:490-497 for causal LMs,
train_llm_maskedlm_bert.py for BERT).  GEMMs and attention use the library kernels (they are
off the measured communication path); norms, rotary embedding and the optimizer are this
package's kernels (ops/layers.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.layers import apply_rope, swiglu
from ..ops.linear import MasterLinear


def init_linear(m: nn.Module, std: float = 0.02) -> None:
    if isinstance(m, (nn.Linear, MasterLinear)):
        nn.init.normal_(m.weight, mean=0.0, std=std)
        if m.bias is not None:
            nn.init.zeros_(m.bias)
    elif isinstance(m, nn.Embedding):
        nn.init.normal_(m.weight, mean=0.0, std=std)


class SelfAttention(nn.Module):
    """Multi-head / grouped-query attention over [B, S, H] with optional rotary embedding."""

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int | None = None, bias: bool = True,
                 causal: bool = True, rope: bool = False):
        super().__init__()
        self.n_heads, self.n_kv = n_heads, n_kv_heads or n_heads
        self.head_dim = hidden // n_heads
        self.causal, self.rope = causal, rope
        self.qkv = MasterLinear(hidden, (self.n_heads + 2 * self.n_kv) * self.head_dim, bias=bias)
        self.proj = MasterLinear(hidden, hidden, bias=bias)

    def forward(self, x: torch.Tensor, cos=None, sin=None) -> torch.Tensor:
        B, S, _ = x.shape
        qkv = self.qkv(x)
        q, k, v = qkv.split([self.n_heads * self.head_dim, self.n_kv * self.head_dim, self.n_kv * self.head_dim], -1)
        q = q.reshape(B, S, self.n_heads, self.head_dim)
        k = k.reshape(B, S, self.n_kv, self.head_dim)
        v = v.reshape(B, S, self.n_kv, self.head_dim)
        if self.rope:
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                           is_causal=self.causal, enable_gqa=self.n_kv != self.n_heads)
        return self.proj(o.transpose(1, 2).reshape(B, S, -1))


class GeluMLP(nn.Module):
    def __init__(self, hidden: int, inner: int, approximate: str = "tanh"):
        super().__init__()
        self.fc = MasterLinear(hidden, inner)
        self.proj = MasterLinear(inner, hidden)
        self.approximate = approximate

    def forward(self, x):
        return self.proj(F.gelu(self.fc(x), approximate=self.approximate))


class SwiGLU(nn.Module):
    def __init__(self, hidden: int, inner: int):
        super().__init__()
        self.gate_up = MasterLinear(hidden, 2 * inner, bias=False)
        self.down = MasterLinear(inner, hidden, bias=False)

    def forward(self, x):
        return self.down(swiglu(self.gate_up(x)))


def count_params(m: nn.Module) -> int:
    return sum(p.numel() for p in m.parameters())
