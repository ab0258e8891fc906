"""Autograd wrappers of the model-side kernels (csrc/kernels/model_ops.cu).

The reference uses Hugging Face's LayerNorm / RMSNorm / rotary modules and
``torch.optim.AdamW`` (testbed_evaluation/train_llm_causal.py:490-497,614).  These classes have
the same maths; on CUDA tensors they call the native kernels, on CPU tensors (tests without a
GPU) they fall back to the equivalent PyTorch expression.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import require
from ..utils import counters


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps: float, rms: bool):
        ops = require()
        xc = x.contiguous()
        y, mean, rstd = ops.norm_fwd(xc, w, b, eps, rms)
        counters.add("norm_fwd")
        ctx.save_for_backward(xc, w, mean, rstd)
        ctx.rms = rms
        ctx.has_bias = b is not None
        # gradient-arena views (parallel/reducer.py): written in place, autograd then sees None
        ctx.wg = getattr(w, "_dq_grad", None)
        ctx.bg = getattr(b, "_dq_grad", None) if b is not None else None
        return y

    @staticmethod
    def backward(ctx, dy):
        ops = require()
        x, w, mean, rstd = ctx.saved_tensors
        # with gradient-arena views the reduction kernel writes the parameter gradients in place
        dx, dw, db = ops.norm_bwd(dy.contiguous(), x, w, mean, rstd, ctx.rms, ctx.wg,
                                  ctx.bg if ctx.has_bias else None)
        counters.add("norm_bwd", 2)
        if ctx.wg is not None:
            dw = None
        if ctx.has_bias and ctx.bg is not None:
            db = None
        return dx, dw, (db if ctx.has_bias else None), None, None


class LayerNorm(nn.Module):
    """LayerNorm over the last dimension with fp32 parameters and statistics."""

    def __init__(self, hidden: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden))
        self.bias = nn.Parameter(torch.zeros(hidden))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda:
            return _NormFn.apply(x, self.weight.float(), self.bias.float(), self.eps, False)
        return F.layer_norm(x.float(), (x.shape[-1],), self.weight.float(), self.bias.float(), self.eps).to(x.dtype)


class RMSNorm(nn.Module):
    def __init__(self, hidden: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda:
            return _NormFn.apply(x, self.weight.float(), None, self.eps, True)
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        counters.add("rope")
        return require().rope(x.contiguous(), cos, sin, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        counters.add("rope")
        return require().rope(dy.contiguous(), cos, sin, True), None, None


def rope_tables(seq_len: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [S, D/2] in fp32 for the rotate-half convention."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float64), inv)
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, S, heads, D]; rotate-half: (x1 cos - x2 sin, x2 cos + x1 sin)."""
    if x.is_cuda:
        return _RopeFn.apply(x, cos, sin)
    S, D = x.shape[1], x.shape[3]
    c, s = cos[:S].view(1, S, 1, D // 2), sin[:S].view(1, S, 1, D // 2)
    x1, x2 = x.float()[..., : D // 2], x.float()[..., D // 2:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        counters.add("swiglu_fwd")
        return require().swiglu_fwd(x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        counters.add("swiglu_bwd")
        return require().swiglu_bwd(dy.contiguous(), x)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for gate_up = (gate | up) along the last dimension; one kernel each way."""
    if gate_up.is_cuda and gate_up.shape[-1] % 16 == 0:
        return _SwiGLUFn.apply(gate_up.contiguous())
    g, u = gate_up.chunk(2, dim=-1)
    return F.silu(g) * u


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, vocab: int, ignore_index: int):
        ops = require()
        lse, rows = ops.ce_fwd(logits, labels, vocab, ignore_index)
        counters.add("ce_fwd")
        n_valid = (labels != ignore_index).sum().to(torch.float32).clamp_(min=1.0).view(1)
        ctx.save_for_backward(logits, labels, lse, n_valid)
        ctx.vocab, ctx.ignore_index = vocab, ignore_index
        return rows.sum() / n_valid[0]

    @staticmethod
    def backward(ctx, g):
        logits, labels, lse, n_valid = ctx.saved_tensors
        counters.add("ce_bwd")
        grad = require().ce_bwd(logits, labels, lse, g.to(torch.float32).reshape(1).contiguous(), n_valid, ctx.vocab,
                                ctx.ignore_index)
        return grad, None, None, None


def fused_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, vocab: int, ignore_index: int = -100
                        ) -> torch.Tensor:
    """Mean cross-entropy over rows whose label is not `ignore_index`.

    `logits` is [N, Vp] with Vp >= vocab; columns >= vocab are padding.  On CUDA the backward
    pass overwrites `logits` with its gradient (the caller must not use `logits` afterwards).
    """
    if logits.is_cuda:
        return _CrossEntropyFn.apply(logits, labels.contiguous(), vocab, ignore_index)
    return F.cross_entropy(logits[:, :vocab].float(), labels, ignore_index=ignore_index)


def padded_vocab_logits(x: torch.Tensor, weight: torch.Tensor, bias=None, multiple: int = 128) -> torch.Tensor:
    """x @ weight.T with the vocabulary dimension zero-padded to a multiple of `multiple`.

    An unaligned vocabulary (50257, 30522) sends the projection GEMM and both of its backward
    GEMMs down the library's unaligned legacy path; padding the bf16 copy of the weight (made
    every step anyway under autocast) keeps the parameter shape and the maths unchanged.
    Returns [N, Vp]; use :func:`fused_cross_entropy` with ``vocab=weight.shape[0]``.
    """
    V = weight.shape[0]
    pad = (-V) % multiple
    w = weight.to(x.dtype)
    if pad:
        w = F.pad(w, (0, 0, 0, pad))
    out = x.reshape(-1, x.shape[-1]) @ w.t()
    if bias is not None:
        b = bias.to(x.dtype)
        out = out + (F.pad(b, (0, pad)) if pad else b)
    return out


def shift_labels(labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Next-token targets: position t predicts labels[t+1]; the last position is ignored."""
    out = torch.full_like(labels, ignore_index)
    out[:, :-1] = labels[:, 1:]
    return out


class FusedAdamW(torch.optim.Optimizer):
    """AdamW with one kernel launch per step for all parameters of a dtype pair (fp32 state)."""

    CHUNK = 4096

    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, shadows: Optional[dict] = None):
        """`shadows` maps a parameter to a bf16 tensor of the same shape that the kernel keeps equal
        to the updated parameter (see ops/linear.py)."""
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._tables = {}
        self._step = 0
        self._shadows = dict(shadows or {})

    def _table(self, gi, group) -> list:
        """Per (param dtype, grad dtype) metadata; rebuilt when a gradient buffer moves.  `gi` is any
        hashable key, `group["params"]` the parameters it covers."""
        ps: List[torch.Tensor] = [p for p in group["params"] if p.grad is not None]
        key = tuple((p.data_ptr(), p.grad.data_ptr(), self._shadow_ptr(p)) for p in ps)
        cached = self._tables.get(gi)
        if cached is not None and cached[0] == key:
            return cached[1]
        buckets = {}
        for p in ps:
            st = self.state[p]
            if "exp_avg" not in st:
                st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.contiguous_format)
                st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.contiguous_format)
            if not (p.is_contiguous() and p.grad.is_contiguous()):
                raise ValueError("FusedAdamW needs contiguous parameters and gradients")
            buckets.setdefault((p.dtype, p.grad.dtype), []).append(p)
        out = []
        for (pd, gd), plist in buckets.items():
            dev = plist[0].device
            rows, numel, starts, c = [], [], [], 0
            for p in plist:
                st = self.state[p]
                rows.append([p.data_ptr(), p.grad.data_ptr(), st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr(),
                             self._shadow_ptr(p)])
                numel.append(p.numel())
                starts.append(c)
                c += (p.numel() + self.CHUNK - 1) // self.CHUNK
            out.append((torch.tensor(rows, dtype=torch.int64, device=dev),
                        torch.tensor(numel, dtype=torch.int64, device=dev),
                        torch.tensor(starts, dtype=torch.int32, device=dev), c,
                        pd == torch.bfloat16, gd == torch.bfloat16, plist))
        self._tables[gi] = (key, out)
        return out

    def _shadow_ptr(self, p) -> int:
        sh = self._shadows.get(p)
        if sh is None:
            return 0
        if sh.dtype != torch.bfloat16 or not sh.is_contiguous() or sh.numel() < p.numel() \
                or sh.shape[1:] != p.shape[1:]:
            raise ValueError("a shadow must be a contiguous bf16 tensor whose leading rows have the parameter's shape")
        return sh.data_ptr()

    def advance(self) -> int:
        """Start optimizer step t+1 for callers that update parameter subsets with :meth:`step_params`."""
        self._step += 1
        return self._step

    @torch.no_grad()
    def step_params(self, key, params: List[torch.Tensor], grad_scale: float = 1.0) -> None:
        """AdamW update of `params` only (all from one param group), at the step count set by
        :meth:`advance`.  `key` identifies the subset (its pointer table is cached under it).  Used by
        the bucket reducer to update a bucket as soon as its gradients are reduced."""
        if not params:
            return
        group = self._group_of(params[0])
        b1, b2 = group["betas"]
        if params[0].is_cuda:
            ops = require()
            for table, numel, starts, chunks, pbf, gbf, _ in self._table(("subset", key), {"params": params}):
                ops.adamw_step(table, numel, starts, chunks, pbf, gbf, group["lr"], b1, b2, group["eps"],
                               group["weight_decay"], self._step, grad_scale)
                counters.add("adamw")
        else:
            self._step_cpu([p for p in params if p.grad is not None], group, grad_scale)

    def _group_of(self, p) -> dict:
        idx = getattr(self, "_pgroup", None)
        if idx is None:
            idx = self._pgroup = {id(q): g for g in self.param_groups for q in g["params"]}
        return idx[id(p)]

    def _step_cpu(self, params, group, grad_scale: float) -> None:
        b1, b2 = group["betas"]
        for p in params:
            st = self.state[p]
            if "exp_avg" not in st:
                st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
            g = p.grad.float() * grad_scale
            st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
            st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
            bc1, bc2 = 1 - b1 ** self._step, 1 - b2 ** self._step
            pf = p.float()
            pf.mul_(1 - group["lr"] * group["weight_decay"])
            pf.addcdiv_(st["exp_avg"], (st["exp_avg_sq"] / bc2).sqrt_().add_(group["eps"]),
                        value=-group["lr"] / bc1)
            p.copy_(pf)
            if p in self._shadows:
                self._shadows[p].view(-1)[: p.numel()].view_as(p).copy_(pf)

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        loss = closure() if closure is not None else None
        self._step += 1
        for gi, group in enumerate(self.param_groups):
            b1, b2 = group["betas"]
            params = [p for p in group["params"] if p.grad is not None]
            if not params:
                continue
            if params[0].is_cuda:
                ops = require()
                for table, numel, starts, chunks, pbf, gbf, _ in self._table(gi, group):
                    ops.adamw_step(table, numel, starts, chunks, pbf, gbf, group["lr"], b1, b2, group["eps"],
                                   group["weight_decay"], self._step, grad_scale)
                    counters.add("adamw")
            else:
                self._step_cpu(params, group, grad_scale)
        return loss

    def state_dict(self):
        d = super().state_dict()
        d["fused_step"] = self._step
        return d

    def load_state_dict(self, d):
        d = dict(d)
        self._step = d.pop("fused_step", 0)
        super().load_state_dict(d)
        self._tables.clear()
