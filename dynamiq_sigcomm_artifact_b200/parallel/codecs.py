"""Codecs in PyTorch ops for the device-agnostic backend (``torch_backend.allreduce_torch``).

* :class:`SuperchunkCodec` - the reference's hierarchical "scaling quantisation": 256-element
  superchunks of 16 chunks of 16 values, linear (AEE) or logarithmic-lattice (MEE) codes of
  2 / 4 / 8 bits, a uint8 round-up scale per chunk and a bf16 scale per superchunk; the wire
  layout is the reference's byte for byte (spec
  cuda_kernels/documentation/scaling_quantization_algorithm.md:347-388, kernels
  cuda_kernels/src/srrcomp/eden_utils/csrc/cuda_hierarchical_mee.cu:203-343, size formula
  eden_utils.cpp:33-40).  Differences: partial sums stay fp32 between hops, and the rounding
  uniforms come from the counter-based generator instead of a pool.
* :class:`CastCodec` - identity wires bf16 / fp16 / fp32 (utils_aggregation.py:575-686).
* :class:`BlockFloatCodec` - MXFP8 (E4M3), FP6 (E3M2) and FP4 (E2M1) with one power-of-two
  scale byte per 32 values (clean spec in simulations_llm/new_comm_hooks/comm_hooks.py:138-275,
  991-1161; the testbed's fp4/fp6 only truncate the message, comm_hooks.py:214-248).
* :class:`IntBinsCodec` - THC's integer bins summed exactly along the schedule
  (``Direct_Summation``, thc_hooks.py:152-223).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .torch_backend import TorchCodec, uniform_bytes

MEE_EPS = {1: 0.23, 2: 0.23, 3: 0.18, 4: 0.18, 5: 0.18, 6: 0.10, 7: 0.10, 8: 0.10}  # cuda_hadamard.cu:878-897
SUPERCHUNK = 256
CHUNK = 16


def superchunk_bytes(bits: int) -> int:
    """Bytes of one 256-element superchunk on the wire: 16 * (2 b + 1) + 2."""
    return CHUNK * (CHUNK * bits // 8 + 1) + 2


def mee_lattice(level: torch.Tensor, eps: float) -> torch.Tensor:
    """Decode lattice ((1+2e^2)^|l| - 1) / (2 e^2) * (1 + e^2), odd in l."""
    mag = (torch.pow(torch.tensor(1.0 + 2.0 * eps * eps, dtype=torch.float32, device=level.device), level.abs())
           - 1.0) / (2.0 * eps * eps) * (1.0 + eps * eps)
    return torch.sign(level) * mag


class SuperchunkCodec(TorchCodec):
    align = SUPERCHUNK

    def __init__(self, bits: int, lattice: str = "aee", seed: int = 0, step: int = 0, bucket: int = 0):
        if bits not in (2, 4, 8):
            raise ValueError("the superchunk codec has 2, 4 and 8 bit codes")
        if lattice not in ("aee", "mee"):
            raise ValueError("lattice must be 'aee' or 'mee'")
        self.bits, self.lattice, self.seed, self.step, self.bucket = bits, lattice, seed, step, bucket
        self.R = (1 << (bits - 1)) - 1
        self.eps = MEE_EPS[bits]
        self.c1 = (1.0 + self.eps ** 2) / (2.0 * self.eps ** 2)
        self.c2 = math.log2(1.0 + 2.0 * self.eps ** 2)
        self.lattice_max = float(mee_lattice(torch.tensor(float(self.R)), self.eps)) if lattice == "mee" else float(self.R)

    def message_bytes(self, numel: int) -> int:
        assert numel % SUPERCHUNK == 0
        return numel // SUPERCHUNK * superchunk_bytes(self.bits)

    # -- encode --------------------------------------------------------------------------
    def encode(self, v: torch.Tensor, first: int, tag: int) -> torch.Tensor:
        b, R = self.bits, self.R
        nsc = v.numel() // SUPERCHUNK
        x = torch.nan_to_num(v.float().reshape(nsc, CHUNK, CHUNK), nan=0.0, posinf=0.0, neginf=0.0)
        s = (x.abs().amax(dim=2) / self.lattice_max + 1e-7).clamp_min(1e-30)  # chunk scales [nsc, 16]
        S = s.amax(dim=1, keepdim=True)  # superchunk scale
        unit_bf16 = (S / 255.0).clamp_min(1e-30).to(torch.bfloat16)
        unit = unit_bf16.float().clamp_min(1e-30)
        q = torch.ceil(s / S * 255.0).clamp_(1, 255)  # uint8 round-up chunk scale
        dec = (q * unit).clamp_min(1e-30)
        y = x / dec.unsqueeze(2)
        if self.lattice == "mee":
            y = torch.sign(y) * torch.log2(y.abs() / self.c1 + 1.0) / self.c2
        stream = ((self.bucket & 0xFFFF) << 16) | (tag & 0xFFFF)
        r = (uniform_bytes(v.numel(), stream, self.step, self.seed, v.device, offset=first // 16).float() + 0.5) / 256.0
        fl = torch.floor(y)
        code = (fl + ((y - fl) > r.reshape(nsc, CHUNK, CHUNK)).float()).clamp_(-R, R) + R
        code = code.to(torch.uint8)
        per = 8 // b  # codes per byte, little end first
        packed = torch.zeros(nsc, CHUNK, CHUNK // per, dtype=torch.uint8, device=v.device)
        c = code.reshape(nsc, CHUNK, CHUNK // per, per)
        for k in range(per):
            packed |= c[..., k] << (k * b)
        out = torch.empty(nsc, superchunk_bytes(b), dtype=torch.uint8, device=v.device)
        body = out[:, : CHUNK * (2 * b + 1)].reshape(nsc, CHUNK, 2 * b + 1)
        body[:, :, : 2 * b] = packed
        body[:, :, 2 * b] = q.to(torch.uint8)
        out[:, CHUNK * (2 * b + 1):] = unit_bf16.reshape(nsc, 1).view(torch.uint8).reshape(nsc, 2)
        return out.reshape(-1)

    # -- decode --------------------------------------------------------------------------
    def decode(self, msg: torch.Tensor, numel: int) -> torch.Tensor:
        b, R = self.bits, self.R
        nsc = numel // SUPERCHUNK
        m = msg.reshape(nsc, superchunk_bytes(b))
        body = m[:, : CHUNK * (2 * b + 1)].reshape(nsc, CHUNK, 2 * b + 1)
        packed = body[:, :, : 2 * b]
        q = body[:, :, 2 * b].float()
        unit = m[:, CHUNK * (2 * b + 1):].contiguous().view(torch.bfloat16).float().clamp_min(1e-30)
        per = 8 // b
        mask = (1 << b) - 1
        codes = torch.stack([(packed >> (k * b)) & mask for k in range(per)], dim=-1).reshape(nsc, CHUNK, CHUNK)
        level = codes.float() - R
        if self.lattice == "mee":
            level = mee_lattice(level, self.eps)
        dec = (q * unit).clamp_min(1e-30)
        return (level * dec.unsqueeze(2)).reshape(-1)


SIM_EPS = {2: 0.27, 4: 0.20, 5: 0.18, 7: 0.10, 8: 0.08}  # simulations_llm/new_comm_hooks/utils_aggregation.py:8


class SimHierarchicalCodec(TorchCodec):
    """The simulation stack's hierarchical compressor (``Mee_Dynamic_Range_Hierarchical``,
    simulations_llm/new_comm_hooks/utils_aggregation.py:176-357), which differs from the testbed's superchunk
    format in three ways that this class keeps:

    * any code width in 2..8 with the simulation's own epsilon table (``SIM_EPS``); codes are the lattice
      indices -2^(b-1) .. 2^(b-1), rounded stochastically between the two neighbouring lattice values in
      proportion to the position between them (unbiased also on the logarithmic lattice);
    * the scale of a chunk, max|chunk| / lattice(2^(b-1)), is itself quantised to 8 bits relative to the
      largest scale of its supergroup with stochastic rounding, floor(s / s_max * 255 + u);
    * no mean-centring and no superchunk byte format: the message carries the codes, one byte per
      chunk scale and one fp32 per supergroup (the simulation keeps them as bf16 numbers in one tensor).

    Rounding offsets come from the counter-based generator (the reference slides an LCG window over a
    pre-generated pool), so runs are reproducible from the seed."""

    def __init__(self, bits: int, lattice: str = "mee", chunk: int = 16, supergroup: int = 16, seed: int = 0,
                 step: int = 0, bucket: int = 0):
        if bits not in SIM_EPS:
            raise ValueError(f"the simulation compressor has widths {sorted(SIM_EPS)}")
        self.bits, self.lattice, self.chunk, self.supergroup = bits, lattice, chunk, supergroup
        self.seed, self.step, self.bucket = seed, step, bucket
        self.eps = SIM_EPS[bits]
        self.half = 1 << (bits - 1)
        self.align = chunk * supergroup
        levels = torch.arange(-(1 << bits), (1 << bits) + 1, dtype=torch.float32)
        self.table = mee_lattice(levels, self.eps) if lattice == "mee" else levels
        self.top = float(self.table[(1 << bits) + self.half])  # lattice value of the largest code

    def message_bytes(self, numel: int) -> int:
        nchunk = numel // self.chunk
        return 2 * numel + nchunk + 4 * (nchunk // self.supergroup)

    def _u(self, n: int, tag: int, device) -> torch.Tensor:
        stream = ((self.bucket & 0xFFFF) << 16) | (tag & 0xFFFF)
        return (uniform_bytes(n, stream, self.step, self.seed, device).float() + 0.5) / 256.0

    def encode(self, v, first, tag):
        assert v.numel() % self.align == 0
        x = torch.nan_to_num(v.float(), nan=0.0, posinf=0.0, neginf=0.0).view(-1, self.chunk)
        tab = self.table.to(x.device)
        scale = x.abs().amax(dim=1, keepdim=True) / self.top + 1e-23
        y = x / scale
        idx = torch.searchsorted(tab, y.contiguous(), right=True).clamp(1, tab.numel() - 1)
        left, right = tab[idx - 1], tab[idx]
        prob = (y - left) / (right - left)
        u = self._u(x.numel(), tag, x.device).view_as(x)
        code = torch.where(u < prob, idx, idx - 1) - (1 << self.bits)
        code = code.clamp(-self.half, self.half)
        sg = scale.view(-1, self.supergroup)
        sg_max = sg.amax(dim=1, keepdim=True) + 1e-23
        q = sg / sg_max * 255.0
        qf = torch.floor(q)
        u2 = self._u(sg.numel(), tag ^ 0x5A5A, x.device).view_as(sg)
        qf = (qf + (u2 < (q - qf)).float()).clamp_(0, 255)
        return torch.cat([code.to(torch.int16).reshape(-1).contiguous().view(torch.uint8),
                          qf.to(torch.uint8).reshape(-1), sg_max.reshape(-1).contiguous().view(torch.uint8)])

    def decode(self, msg, numel):
        nchunk = numel // self.chunk
        nsg = nchunk // self.supergroup
        code = msg[: 2 * numel].contiguous().view(torch.int16).long().view(nchunk, self.chunk)
        q = msg[2 * numel: 2 * numel + nchunk].float().view(nsg, self.supergroup)
        sg_max = msg[2 * numel + nchunk: 2 * numel + nchunk + 4 * nsg].contiguous().view(torch.float32).view(nsg, 1)
        scale = (q * sg_max / 255.0).view(nchunk, 1)
        tab = self.table.to(msg.device)
        return (tab[code + (1 << self.bits)] * scale).reshape(-1)


class CastCodec(TorchCodec):
    """Values travel as bf16 / fp16 / fp32; partial sums are rounded to the wire type per hop."""

    def __init__(self, dtype: torch.dtype):
        self.dtype = dtype
        self.itemsize = torch.tensor([], dtype=dtype).element_size()
        self.align = 16 // self.itemsize

    def message_bytes(self, numel: int) -> int:
        return numel * self.itemsize

    def encode(self, v, first, tag):
        return v.to(self.dtype).contiguous().view(torch.uint8).reshape(-1)

    def decode(self, msg, numel):
        return msg.view(self.dtype)[:numel].float()


_FORMATS = {  # name: (exponent bits, mantissa bits, largest finite magnitude)
    "fp8": (4, 3, 448.0),
    "fp6": (3, 2, 28.0),
    "fp4": (2, 1, 6.0),
}


def _round_to_minifloat(x: torch.Tensor, ebits: int, mbits: int, vmax: float) -> torch.Tensor:
    """Round-to-nearest-even onto the (ebits, mbits) grid with subnormals, saturating at vmax
    (what ``cvt.rn.satfinite`` does on the device).  Exponents come from ``frexp``: exact."""
    bias = (1 << (ebits - 1)) - 1
    ax = x.abs().clamp_max(vmax)
    e = (torch.frexp(ax.clamp_min(1e-38)).exponent - 1).clamp_min(1 - bias)  # floor(log2 |x|), at least emin
    step = torch.ldexp(torch.ones_like(ax), e - mbits)
    return torch.sign(x) * torch.round(ax / step) * step


class BlockFloatCodec(TorchCodec):
    """MXFP8 (E4M3) / FP6 (E3M2) / FP4 (E2M1): 32-value blocks with one power-of-two scale byte.

    Layout, shared with the fused kernel (csrc/common/mx_codec.cuh): per 1024 values, 32 lanes x 4 w
    code bytes (the 32 codes of a lane as a little-endian stream of w-bit codes, a code being the
    format's sign | exponent | mantissa bit pattern), then the 32 scale bytes (biased exponent of the
    scale).  8.25 / 6.25 / 4.25 bit per value - the figures the reference's bandwidth emulation charges
    (comm_hooks.py:239-241).
    """

    BLOCK = 32

    def __init__(self, fmt: str):
        self.fmt = fmt
        self.ebits, self.mbits, self.vmax = _FORMATS[fmt]
        self.width = 1 + self.ebits + self.mbits
        self.align = 1024
        mags = [0.0]
        bias = (1 << (self.ebits - 1)) - 1
        for e in range(1 << self.ebits):
            for m in range(1 << self.mbits):
                val = (m / (1 << self.mbits)) * 2.0 ** (1 - bias) if e == 0 else (1 + m / (1 << self.mbits)) * 2.0 ** (e - bias)
                if 0 < val <= self.vmax:
                    mags.append(val)
        # sorted magnitudes: the index of a magnitude is its exponent | mantissa bit pattern
        self.table = torch.tensor(sorted(set(mags)), dtype=torch.float32)

    def block_bytes(self) -> int:
        return 128 * self.width + 32

    def message_bytes(self, numel: int) -> int:
        return (numel + 1023) // 1024 * self.block_bytes()

    def _table(self, device):
        if self.table.device != device:
            self.table = self.table.to(device)
        return self.table

    def encode(self, v, first, tag):
        n, w = v.numel(), self.width
        nblk = (n + 1023) // 1024
        x = torch.zeros(nblk * 1024, dtype=torch.float32, device=v.device)
        x[:n] = torch.nan_to_num(v.float(), nan=0.0, posinf=0.0, neginf=0.0)
        x = x.reshape(nblk, 32, 32)  # [block, lane, value]
        amax = x.abs().amax(dim=2)
        r = amax / torch.tensor(self.vmax, dtype=torch.float32, device=v.device)
        fr = torch.frexp(r.clamp_min(1e-38))
        e = torch.where(fr.mantissa > 0.5, fr.exponent, fr.exponent - 1).clamp(-127, 127)  # ceil(log2 r), exact
        e = torch.where(amax >= 1e-30, e, torch.full_like(e, -127))
        y = _round_to_minifloat(torch.ldexp(x, -e.unsqueeze(2)), self.ebits, self.mbits, self.vmax)
        t = self._table(v.device)
        idx = torch.bucketize(y.abs(), t).clamp_max(t.numel() - 1)  # |y| is on the grid: first entry >= |y| is |y|
        code = (idx | ((y < 0) | ((y == 0) & torch.signbit(y))).long() << (w - 1)).to(torch.int64)
        bits = ((code.unsqueeze(3) >> torch.arange(w, device=v.device)) & 1).to(torch.uint8)  # [blk, lane, value, w]
        bits = bits.reshape(nblk, 32, 32 * w // 8, 8)
        weights = (1 << torch.arange(8, device=v.device)).to(torch.uint8)
        payload = (bits * weights).sum(dim=3).to(torch.uint8).reshape(nblk, 32 * 4 * w)
        scales = (e + 127).to(torch.uint8)
        return torch.cat([payload, scales], dim=1).reshape(-1)

    def decode(self, msg, numel):
        w = self.width
        nblk = (numel + 1023) // 1024
        m = msg.reshape(nblk, self.block_bytes())
        payload = m[:, : 128 * w].reshape(nblk, 32, 4 * w)
        e = m[:, 128 * w:].to(torch.int32) - 127
        bits = ((payload.unsqueeze(3) >> torch.arange(8, device=msg.device)) & 1).reshape(nblk, 32, 32, w)
        code = (bits.long() << torch.arange(w, device=msg.device)).sum(dim=3)
        sign = 1.0 - 2.0 * ((code >> (w - 1)) & 1).float()
        mag = self._table(msg.device)[(code & ((1 << (w - 1)) - 1)).clamp_max(self.table.numel() - 1)]
        y = torch.ldexp(sign * mag, e.unsqueeze(2))
        return y.reshape(-1)[:numel]


class MinifloatCodec(TorchCodec):
    """Values already normalised by the caller travel as bare FP8 / FP6 / FP4 numbers: every hop rounds its
    partial sum to the format's grid and saturates at its largest magnitude, with no scale of its own - the
    arithmetic of the reference's simulated ``Fpx_arithmetics`` under the shared-scale hook
    (simulations_llm/new_comm_hooks/comm_hooks.py:1026-1046).  One byte per value on this executor's wire."""

    align = 16

    def __init__(self, fmt: str):
        self.fmt = fmt
        self.ebits, self.mbits, self.vmax = _FORMATS[fmt]
        self.width = 1 + self.ebits + self.mbits

    def message_bytes(self, numel: int) -> int:
        return numel * 4

    def encode(self, v, first, tag):
        y = _round_to_minifloat(torch.nan_to_num(v.float(), nan=0.0, posinf=self.vmax, neginf=-self.vmax), self.ebits,
                                self.mbits, self.vmax)
        return y.contiguous().view(torch.uint8).reshape(-1)

    def decode(self, msg, numel):
        return msg.view(torch.float32)[:numel].clone()


class IntBinsCodec(TorchCodec):
    """Integer bins carried exactly (int16 on the wire): sums of bins stay integers."""

    align = 8

    def message_bytes(self, numel: int) -> int:
        return numel * 2

    def encode(self, v, first, tag):
        return torch.round(v).clamp_(-32768, 32767).to(torch.int16).contiguous().view(torch.uint8).reshape(-1)

    def decode(self, msg, numel):
        return msg.view(torch.int16)[:numel].float()
