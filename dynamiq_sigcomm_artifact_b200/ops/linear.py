"""Linear layer with fp32 master weights and a resident bf16 working copy.

Under ``torch.autocast`` every ``nn.Linear`` re-casts its fp32 weight to bf16 on every forward
(one read of 4 and one write of 2 bytes per parameter per step, and one kernel launch per layer).
``MasterLinear`` keeps the bf16 copy alive instead: the fused AdamW kernel writes it together
with the fp32 parameter (``FusedAdamW(shadows=...)``), the forward and the input-gradient GEMM
read it, and the weight-gradient GEMM writes fp32 directly (bf16 x bf16 -> fp32 output), so no
cast kernel runs on the weight path at all.  The parameter seen by DDP, the hooks, the optimizer
state and checkpoints is still the fp32 ``weight``.
"""
from __future__ import annotations

import math
from typing import Dict

import torch
import torch.nn as nn
import torch.nn.functional as F


class _ShadowLinearFn(torch.autograd.Function):
    """Gradients of `weight` / `bias` go to ``weight._dq_grad`` / ``bias._dq_grad`` when a gradient arena
    attached them (parallel/reducer.py): the GEMM then writes its fp32 output in place and autograd sees
    ``None`` (no temporary, no accumulate kernel).  In that mode a backward pass overwrites."""

    @staticmethod
    def forward(ctx, x, weight, shadow, bias):
        ctx.save_for_backward(x, shadow)
        ctx.has_bias = bias is not None
        ctx.wg = getattr(weight, "_dq_grad", None)
        ctx.bg = getattr(bias, "_dq_grad", None) if bias is not None else None
        return F.linear(x, shadow, None if bias is None else bias.to(x.dtype))

    @staticmethod
    def backward(ctx, dy):
        x, shadow = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = (dy2 @ shadow).reshape(x.shape) if ctx.needs_input_grad[0] else None
        dw = db = None
        if ctx.wg is not None:
            torch.mm(dy2.t(), x2, out_dtype=torch.float32, out=ctx.wg)
        elif ctx.needs_input_grad[1]:
            dw = torch.mm(dy2.t(), x2, out_dtype=torch.float32)
        if ctx.has_bias and (ctx.bg is not None or ctx.needs_input_grad[3]):
            if dy2.shape[1] % 4 == 0 and dy2.is_contiguous() and dy2.data_ptr() % 16 == 0:
                from . import require  # native column sum (csrc/kernels/colsum.cu)
                from ..utils import counters

                db = require().colsum(dy2, ctx.bg)
                counters.add("colsum", 2)
            elif ctx.bg is not None:
                db = torch.sum(dy2, dim=0, dtype=torch.float32, out=ctx.bg)
            else:
                db = dy2.sum(dim=0, dtype=torch.float32)
            if ctx.bg is not None:
                db = None
        return dx, dw, None, db


class MasterLinear(nn.Module):
    """y = x W^T + b with W fp32 (the parameter) and a bf16 working copy used on bf16 CUDA inputs."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        self.shadow = None  # bf16 copy, created by enable_shadows()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.shadow is not None and x.is_cuda:
            if x.dtype != torch.bfloat16 and torch.is_autocast_enabled("cuda") \
                    and torch.get_autocast_dtype("cuda") == torch.bfloat16:
                x = x.to(torch.bfloat16)
            if x.dtype == torch.bfloat16:
                return _ShadowLinearFn.apply(x, self.weight, self.shadow, self.bias)
        return F.linear(x, self.weight, self.bias)


def enable_shadows(model: nn.Module) -> Dict[nn.Parameter, torch.Tensor]:
    """Create (or refresh) the bf16 copy of every MasterLinear / TiedEmbedding weight; returns {weight: copy}
    (a TiedEmbedding's copy has extra zero rows after the parameter's)."""
    from .embedding import TiedEmbedding

    out: Dict[nn.Parameter, torch.Tensor] = {}
    for m in model.modules():
        if isinstance(m, TiedEmbedding):
            out[m.weight] = m.enable_shadow()
        elif isinstance(m, MasterLinear):
            if m.shadow is None or m.shadow.device != m.weight.device:
                m.shadow = torch.empty_like(m.weight, dtype=torch.bfloat16)
            with torch.no_grad():
                m.shadow.copy_(m.weight)
            out[m.weight] = m.shadow
    return out
