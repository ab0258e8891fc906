"""Randomized Walsh-Hadamard transform of 1024-element blocks.

``fwht1024`` runs the tcgen05 / TMEM kernel (csrc/kernels/fwht_tcgen05.cu) on CUDA tensors and
a PyTorch butterfly on CPU tensors.  Reference counterparts: ``eden_utils.Hadamard*``
(cuda_kernels/src/srrcomp/eden_utils/eden_utils.cpp:56-105) and ``EdenHadamardRHT``
(testbed_evaluation/new_comm_hooks/thc_hooks.py:124-149).
"""
from __future__ import annotations

import torch

from ..utils import counters, philox
from . import require

BLOCK = 1024
TILE = 4 * BLOCK


class FwhtError(RuntimeError):
    pass


def fwht1024(x: torch.Tensor, seed: int = 0, step: int = 0, bucket: int = 0, signs: bool = True,
             normalize: bool = True, check: bool = True) -> torch.Tensor:
    """y = H_1024 (s * x) [/ 32] blockwise; x is padded with zeros to a multiple of 4096 elements."""
    n = x.numel()
    flat = x.reshape(-1).float()
    pad = (-n) % TILE
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    scale = 1.0 / 32.0 if normalize else 1.0
    if flat.is_cuda:
        y, status = require().fwht1024_tcgen05(flat.contiguous(), seed, step, bucket, signs, scale, 0)
        counters.add("fwht1024_tcgen05")
        if check and int(status.item()) != 0:
            raise FwhtError(f"fwht1024_tcgen05 gave up on a wait (status {int(status.item())})")
    else:
        s = torch.from_numpy(philox.sign_vector(step, bucket, seed)) if signs else torch.ones(BLOCK)
        v = torch.nan_to_num(flat.view(-1, BLOCK), nan=0.0, posinf=0.0, neginf=0.0) * s
        h = 1
        while h < BLOCK:
            w = v.view(-1, BLOCK // (2 * h), 2, h)
            a, b = w[:, :, 0, :].clone(), w[:, :, 1, :].clone()
            w[:, :, 0, :], w[:, :, 1, :] = a + b, a - b
            h *= 2
        y = (v * scale).reshape(-1)
    return y[:n].reshape(x.shape)


def ifwht1024(y: torch.Tensor, seed: int = 0, step: int = 0, bucket: int = 0, signs: bool = True) -> torch.Tensor:
    """Inverse of :func:`fwht1024` with ``normalize=True``: x = s * H y / 32."""
    x = fwht1024(y, seed, step, bucket, signs=False, normalize=True)
    if not signs:
        return x
    s = torch.from_numpy(philox.sign_vector(step, bucket, seed)).to(x.device)
    n = x.numel()
    reps = (n + BLOCK - 1) // BLOCK
    return (x.reshape(-1) * s.repeat(reps)[:n]).reshape(y.shape)


def fwht_pow2(x: torch.Tensor, normalize: bool = False) -> torch.Tensor:
    """Walsh-Hadamard transform (Sylvester order) of a flat tensor whose length d is a power of two.

    CUDA, d >= 4096: the tcgen05 kernel transforms the 1024-blocks (levels 0..9), then
    ``fwht_levels_`` (csrc/kernels/fwht_strided.cu) applies the remaining log2(d) - 10 levels five at a
    time, each pass streaming the array once.  Shorter CUDA tensors use ``fwht_levels_`` alone; CPU
    tensors a PyTorch butterfly.  No host synchronisation.  ``normalize`` divides by sqrt(d)."""
    d = x.numel()
    if d & (d - 1):
        raise ValueError(f"length must be a power of two, got {d}")
    k = d.bit_length() - 1
    scale = (1.0 / (2.0 ** (k / 2.0))) if normalize else 1.0
    if not x.is_cuda:
        v = x.reshape(-1).float().clone()
        h = 1
        while h < d:
            w = v.view(d // (2 * h), 2, h)
            a, b = w[:, 0, :].clone(), w[:, 1, :].clone()
            w[:, 0, :], w[:, 1, :] = a + b, a - b
            h *= 2
        return (v * scale).reshape(x.shape)
    ops = require()
    if d >= TILE:
        y = fwht1024(x.reshape(-1), signs=False, normalize=False, check=False).contiguous()
        level = 10
    else:
        y = x.reshape(-1).float().clone()
        level = 0
    if level == k:
        return (y * scale).reshape(x.shape) if scale != 1.0 else y.reshape(x.shape)
    while level < k:
        step = min(5, k - level)
        ops.fwht_levels_(y, level, step, scale if level + step == k else 1.0)
        counters.add("fwht_levels")
        level += step
    return y.reshape(x.shape)
