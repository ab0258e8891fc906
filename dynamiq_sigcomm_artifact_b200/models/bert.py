"""BERT masked LM (default: BERT-base - 12 layers, hidden 768, 12 heads, intermediate 3072,
vocab 30522, 512 positions), random-init, post-LayerNorm, tied decoder."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.embedding import TiedEmbedding
from ..ops.layers import LayerNorm, fused_cross_entropy, padded_vocab_logits, shift_labels
from ..ops.linear import MasterLinear
from .common import GeluMLP, SelfAttention, init_linear


@dataclass
class BertConfig:
    n_layer: int = 12
    hidden: int = 768
    n_head: int = 12
    intermediate: int = 3072
    vocab: int = 30522
    max_pos: int = 512
    type_vocab: int = 2
    eps: float = 1e-12
    mask_token_id: int = 103

    @classmethod
    def tiny(cls) -> "BertConfig":
        return cls(n_layer=2, hidden=128, n_head=4, intermediate=256, vocab=1024, max_pos=128, mask_token_id=3)

    @classmethod
    def large(cls) -> "BertConfig":
        return cls(n_layer=24, hidden=1024, n_head=16, intermediate=4096)


class BertLayer(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.attn = SelfAttention(c.hidden, c.n_head, causal=False)
        self.ln1, self.ln2 = LayerNorm(c.hidden, c.eps), LayerNorm(c.hidden, c.eps)
        self.mlp = GeluMLP(c.hidden, c.intermediate, approximate="none")

    def forward(self, x):
        x = self.ln1(x + self.attn(x))
        return self.ln2(x + self.mlp(x))


class BertMLM(nn.Module):
    def __init__(self, c: BertConfig = BertConfig()):
        super().__init__()
        self.config = c
        self.tok = TiedEmbedding(c.vocab, c.hidden)
        self.pos = nn.Embedding(c.max_pos, c.hidden)
        self.typ = nn.Embedding(c.type_vocab, c.hidden)
        self.ln_emb = LayerNorm(c.hidden, c.eps)
        self.layers = nn.ModuleList(BertLayer(c) for _ in range(c.n_layer))
        self.head_dense = MasterLinear(c.hidden, c.hidden)
        self.head_ln = LayerNorm(c.hidden, c.eps)
        self.head_bias = nn.Parameter(torch.zeros(c.vocab))
        self.apply(init_linear)

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None):
        B, S = input_ids.shape
        pos = torch.arange(S, device=input_ids.device)
        x = self.tok(input_ids) + self.pos(pos) + self.typ.weight[0]
        if torch.is_autocast_enabled(x.device.type):
            x = x.to(torch.get_autocast_dtype(x.device.type))
        x = self.ln_emb(x)
        for layer in self.layers:
            x = layer(x)
        h = self.head_ln(F.gelu(self.head_dense(x)))
        if labels is None:
            return F.linear(h, self.tok.weight.to(h.dtype), self.head_bias.to(h.dtype))
        logits = self.tok.logits(h, self.head_bias)
        return fused_cross_entropy(logits, labels.reshape(-1), self.config.vocab)


def mask_tokens(input_ids: torch.Tensor, vocab: int, mask_token_id: int, generator: torch.Generator | None = None,
                mlm_probability: float = 0.15):
    """BERT masking: 15% of positions become targets; of those 80% -> [MASK], 10% -> a random
    token, 10% unchanged (testbed_evaluation/train_llm_maskedlm_bert.py:354-385)."""
    dev = input_ids.device
    labels = input_ids.clone()
    r = torch.rand(input_ids.shape, generator=generator, device=dev)
    masked = r < mlm_probability
    labels[~masked] = -100
    r2 = torch.rand(input_ids.shape, generator=generator, device=dev)
    out = input_ids.clone()
    out[masked & (r2 < 0.8)] = mask_token_id
    rand_sel = masked & (r2 >= 0.8) & (r2 < 0.9)
    rnd = torch.randint(0, vocab, input_ids.shape, generator=generator, device=dev)
    out[rand_sel] = rnd[rand_sel]
    return out, labels
