"""Token embedding tied to the output projection, with a resident bf16 working copy.

A tied embedding matrix is read twice per step (row gather at the bottom of the network, the
vocabulary GEMM at the top) and receives two gradient contributions (the weight gradient of
that GEMM at the start of backward, a row scatter at its end).  Under plain autocast this costs
a cast + pad of the whole fp32 matrix every step, a dense zero matrix for the scatter and two
dense additions.  ``TiedEmbedding`` keeps a bf16 copy padded to a multiple of 128 rows (written
by the fused AdamW kernel together with the fp32 parameter, like ``MasterLinear``'s), gathers bf16
rows from it, and - when a gradient arena is attached (``weight._dq_grad_padded``, see
parallel/reducer.py) - lets the GEMM write the fp32 weight gradient straight into the arena and
the scatter add its rows on top, so no dense temporary is ever made.

The reference takes Hugging Face's tied embeddings as they are
(testbed_evaluation/train_llm_causal.py:490-497); the parameter seen by hooks, optimizer state and
checkpoints here is still the fp32 ``weight`` of shape [vocab, hidden].
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

PAD_ROWS = 128


class _LookupFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, shadow):
        ctx.save_for_backward(ids)
        ctx.rows = weight.shape[0]
        ctx.direct = getattr(weight, "_dq_grad_padded", None)
        ctx.sparse = getattr(weight, "_dq_sparse", None)
        return F.embedding(ids, shadow)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        if ctx.sparse is not None:
            # multi-rank runs: keep the token rows; the reducer exchanges them and adds every rank's rows
            # after the dense (output-projection) part of the gradient has been reduced
            ctx.sparse["ids"] = ids.reshape(-1)
            ctx.sparse["rows"] = dy.reshape(-1, dy.shape[-1]).contiguous()
            return None, None, None
        rows = dy.reshape(-1, dy.shape[-1]).float()
        if ctx.direct is not None:
            # the output projection's weight gradient was written earlier in this backward pass
            ctx.direct.index_add_(0, ids.reshape(-1), rows)
            return None, None, None
        dw = torch.zeros(ctx.rows, dy.shape[-1], dtype=torch.float32, device=dy.device)
        dw.index_add_(0, ids.reshape(-1), rows)
        return None, dw, None


class _HeadFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, weight, shadow):
        ctx.save_for_backward(h, shadow)
        ctx.rows = weight.shape[0]
        ctx.direct = getattr(weight, "_dq_grad_padded", None)
        return h.reshape(-1, h.shape[-1]) @ shadow.t()

    @staticmethod
    def backward(ctx, dy):
        h, shadow = ctx.saved_tensors
        h2 = h.reshape(-1, h.shape[-1])
        dh = (dy @ shadow).reshape(h.shape) if ctx.needs_input_grad[0] else None
        if ctx.direct is not None:
            torch.mm(dy.t(), h2, out_dtype=torch.float32, out=ctx.direct)  # overwrites: first contribution
            return dh, None, None
        dw = torch.mm(dy.t(), h2, out_dtype=torch.float32)[: ctx.rows]
        return dh, dw, None


class TiedEmbedding(nn.Embedding):
    """``nn.Embedding`` whose weight also serves as the output projection.

    ``lookup(ids)`` returns rows (bf16 from the working copy when it exists, else the parameter's
    dtype); ``logits(h)`` returns ``h @ W^T`` as [N, Vp] with the vocabulary padded to a multiple of
    128 (columns >= ``num_embeddings`` are zero weights; pair with ``fused_cross_entropy``).
    """

    def __init__(self, num_embeddings: int, embedding_dim: int):
        super().__init__(num_embeddings, embedding_dim)
        self.padded_rows = (num_embeddings + PAD_ROWS - 1) // PAD_ROWS * PAD_ROWS
        self.shadow: Optional[torch.Tensor] = None
        # a gradient arena reserves this many elements so that the padded GEMM can write in place
        self.weight._dq_padded_shape = (self.padded_rows, embedding_dim)

    def enable_shadow(self) -> torch.Tensor:
        w = self.weight
        w._dq_padded_shape = (self.padded_rows, self.embedding_dim)
        if self.shadow is None or self.shadow.device != w.device:
            self.shadow = torch.zeros(self.padded_rows, self.embedding_dim, dtype=torch.bfloat16, device=w.device)
        with torch.no_grad():
            self.shadow[: self.num_embeddings].copy_(w)
        return self.shadow

    def _use_shadow(self, device_type: str) -> bool:
        return self.shadow is not None and device_type == "cuda" and torch.is_autocast_enabled("cuda") \
            and torch.get_autocast_dtype("cuda") == torch.bfloat16

    def lookup(self, ids: torch.Tensor) -> torch.Tensor:
        if self._use_shadow(ids.device.type):
            return _LookupFn.apply(ids, self.weight, self.shadow)
        return F.embedding(ids, self.weight)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return self.lookup(ids)

    def logits(self, h: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self._use_shadow(h.device.type) and h.dtype == torch.bfloat16:
            out = _HeadFn.apply(h, self.weight, self.shadow)
            if bias is not None:
                out = out + F.pad(bias.to(out.dtype), (0, self.padded_rows - self.num_embeddings))
            return out
        from .layers import padded_vocab_logits

        return padded_vocab_logits(h, self.weight, bias, PAD_ROWS)
