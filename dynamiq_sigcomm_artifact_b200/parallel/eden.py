"""EDEN: rotate, quantise to the Lloyd-Max centroids of a normal distribution, scale unbiasedly.

The codec the reference inherits from its upstream package
(cuda_kernels/src/srrcomp/srrcomp.py:293-447): a randomized Hadamard transform, 1..8-bit
quantisation to the optimal (Lloyd-Max) levels of N(0, 1) (:364-447), bit-plane packing of the
bins (csrc/cuda_packing.cu) and the scale ``||x||^2 / <R x, c>`` that makes the estimate unbiased
under the random rotation.  The rotation here is blockwise over 1024 elements (the tcgen05
kernel on GPUs); bins are packed by ``torch.ops.dq.bins_to_bits`` on GPUs and by the same plane
layout in PyTorch on CPU.
"""
from __future__ import annotations

import functools
import math
from typing import Tuple

import torch

from .. import ops as _ops
from ..ops.fwht import BLOCK, fwht1024, ifwht1024


@functools.lru_cache(maxsize=None)
def lloyd_max_normal(bits: int, iters: int = 500) -> Tuple[torch.Tensor, torch.Tensor]:
    """(centroids [2^bits], boundaries [2^bits - 1]) of the optimal scalar quantiser of N(0, 1)."""
    n = 1 << bits
    pdf = lambda t: torch.exp(-0.5 * t * t) / math.sqrt(2 * math.pi)  # noqa: E731
    cdf = lambda t: 0.5 * (1 + torch.erf(t / math.sqrt(2)))  # noqa: E731
    c = torch.linspace(-2.5, 2.5, n, dtype=torch.float64) if n > 1 else torch.zeros(1, dtype=torch.float64)
    for _ in range(iters):
        b = 0.5 * (c[1:] + c[:-1])
        lo = torch.cat([torch.tensor([-40.0], dtype=torch.float64), b])
        hi = torch.cat([b, torch.tensor([40.0], dtype=torch.float64)])
        mass = (cdf(hi) - cdf(lo)).clamp_min(1e-300)
        new = (pdf(lo) - pdf(hi)) / mass  # conditional mean of N(0,1) on [lo, hi]
        if float((new - c).abs().max()) < 1e-12:
            c = new
            break
        c = new
    return c.float(), (0.5 * (c[1:] + c[:-1])).float()


def pack_bins(bins: torch.Tensor, bits: int) -> torch.Tensor:
    """uint8 bins [n] -> int32 words [bits, ceil(n / 32)], plane-major."""
    if bins.is_cuda:
        return _ops.require().bins_to_bits(bins.contiguous(), bits)
    n = bins.numel()
    nw = (n + 31) // 32
    pad = torch.zeros(nw * 32, dtype=torch.int64)
    pad[:n] = bins.long()
    planes = (pad.view(nw, 32).unsqueeze(0) >> torch.arange(bits).view(-1, 1, 1)) & 1
    words = (planes << torch.arange(32).view(1, 1, 32)).sum(dim=2)
    return torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)


def unpack_bins(words: torch.Tensor, bits: int, n: int) -> torch.Tensor:
    if words.is_cuda:
        return _ops.require().bits_to_bins(words.contiguous(), bits, n)
    w = words.long() & 0xFFFFFFFF
    planes = (w.unsqueeze(2) >> torch.arange(32).view(1, 1, 32)) & 1  # [bits, nw, 32]
    vals = (planes << torch.arange(bits).view(-1, 1, 1)).sum(dim=0).reshape(-1)[:n]
    return vals.to(torch.uint8)


class Eden:
    """``compress`` -> (packed words, scale per 1024-block, n); ``decompress`` inverts it."""

    def __init__(self, bits: int, seed: int = 0):
        if not 1 <= bits <= 8:
            raise ValueError("EDEN supports 1..8 bits")
        self.bits, self.seed = bits, seed
        self.centroids, self.boundaries = lloyd_max_normal(bits)

    def compress(self, x: torch.Tensor, step: int = 0):
        n = x.numel()
        y = fwht1024(x.reshape(-1).float(), self.seed, step, 0, signs=True, normalize=True)
        pad = (-n) % BLOCK
        yb = torch.cat([y, y.new_zeros(pad)]).view(-1, BLOCK) if pad else y.view(-1, BLOCK)
        norm = yb.pow(2).sum(dim=1, keepdim=True)  # = ||x_block||^2 (orthonormal rotation)
        unit = yb * torch.rsqrt(norm.clamp_min(1e-30) / BLOCK)  # ~ N(0, 1) coordinates
        bins = torch.bucketize(unit, self.boundaries.to(x.device)).to(torch.uint8)
        c = self.centroids.to(x.device)[bins.long()]
        scale = norm / (yb * c).sum(dim=1, keepdim=True).clamp_min(1e-30)  # ||x||^2 / <Rx, c>
        return pack_bins(bins.reshape(-1), self.bits), scale.reshape(-1), n

    def decompress(self, msg, step: int = 0) -> torch.Tensor:
        words, scale, n = msg
        nb = scale.numel()
        bins = unpack_bins(words, self.bits, nb * BLOCK)
        y = self.centroids.to(scale.device)[bins.long()].view(nb, BLOCK) * scale.view(nb, 1)
        return ifwht1024(y.reshape(-1), self.seed, step, 0, signs=True)[:n]

    def wire_bits_per_element(self) -> float:
        return self.bits + 32.0 / BLOCK
