"""CPU oracle of the `rht` codec family: a NumPy restatement of what the CUDA kernels compute.

Follows the reference's strongest test idea - a scalar restatement of the codec fed the
same random numbers as the kernel (cuda_kernels/tests/test_scaling_quantization_functional.py:122-259)
- but for the rotation codec that this framework's `dynamiQ_aee_{b}bit` methods use:

    block of 1024 values
      -> Rademacher diagonal (1024 sign bits from Philox, shared by all ranks)
      -> Walsh-Hadamard H_1024 = H_32 (x) H_32, left unnormalised (the 1/1024 of the round
         trip is folded into the final scale, so no pass multiplies by 1/32)
      -> per-block fp32 scale  absmax / R,  R = 2^(b-1) - 1
      -> stochastic rounding  floor(y * R/absmax + u),  u = (byte + 0.5) / 256 from Philox-4x32-7
         (evaluated as floor(fma(y, 256 R/absmax, 2^15 + byte + 0.5) / 256) - 128, the kernel's form)
      -> b-bit codes, b in 2..8, packed without padding (8 codes of 5 bits in 5 bytes)

A hop adds the decoded incoming block to the locally rotated block with one fp32 fma per
value, v <- fma(code - R, scale, v), and encodes the sum again (the reference rounds the sum to bf16 first,
cuda_kernels/src/srrcomp/eden_utils/csrc/cuda_hierarchical_mee.cu:567-568).

All arithmetic is float32 in the order the kernel uses (fused multiply-adds where the kernel
fuses: the rounding argument and the hop accumulation), so that the kernel's bytes can be
compared with ``==``.

Layouts (shared with ``csrc/common/rht_codec.cuh`` and ``csrc/kernels/fused_rht_tc.cuh``)
* A warp owns a block; after the rotation lane ``l`` holds, in register ``k``, the
  coefficient with index ``RHO[l, k] = (l & 3) + 4 k + 128 (l >> 2)`` when the rotation ran as register
  butterflies (layout ``"simt"``) and ``RHO_TC[l, k] = 32 k + l`` when it ran on the tensor cores
  (layout ``"tc"``: lane = accumulator row, register = accumulator column).
* The 32 codes of a lane form a little-endian bit stream of ``b`` 32-bit words; word ``j`` of
  lane ``l`` is stored at word ``j * 32 + l`` of the block's ``128 b`` code bytes, so each of
  the ``b`` warp-wide stores is one contiguous 128-byte line.
* A shard's message is ``[codes: nb * 128 b bytes][scales: nb * 4 bytes]``.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np

from .utils import philox

BLOCK = 1024
_L = np.arange(32).reshape(32, 1)
_K = np.arange(32).reshape(1, 32)
RHO = ((_L & 3) + 4 * _K + 128 * (_L >> 2)).astype(np.int64)  # [lane, reg] -> coefficient index
RHO_TC = (32 * _K + _L).astype(np.int64)
LAYOUTS = {"simt": RHO, "tc": RHO_TC}
FWD_STAGES = (0, 1, 7, 8, 9, 2, 3, 4, 5, 6)  # bit of the element index handled by each butterfly stage
INV_STAGES = (2, 3, 4, 5, 6, 0, 1, 7, 8, 9)
F32 = np.float32


def fma32(a, b, c) -> np.ndarray:
    """float32 fused multiply-add: the product of two float32 is exact in float64, the sum is
    rounded once to float64 and once more to float32 (a double rounding that differs from a
    true fma only on exact ties, ~2^-29 of the inputs)."""
    return (np.asarray(a, np.float64) * np.asarray(b, np.float64) + np.asarray(c, np.float64)).astype(F32)


def qmax(bits: int) -> int:
    if not 2 <= bits <= 8:
        raise ValueError("bits must be in 2..8")
    return (1 << (bits - 1)) - 1


def payload_bytes(nblocks: int, bits: int) -> int:
    """Bytes of one message: packed codes then one fp32 scale per block."""
    return nblocks * (128 * bits + 4)


def wire_bits_per_element(bits: int) -> float:
    return (128 * bits + 4) * 8 / BLOCK


def to_blocks(x: np.ndarray) -> np.ndarray:
    """Flat fp32 vector -> [nblocks, 1024], zero padded.  Non-finite inputs are kept: the rotation
    spreads them over their block, and ``quantize`` then sends that block as zeros."""
    x = np.asarray(x, dtype=F32).reshape(-1)
    nb = (x.size + BLOCK - 1) // BLOCK
    out = np.zeros(nb * BLOCK, dtype=F32)
    out[: x.size] = x
    return out.reshape(nb, BLOCK)


def _butterflies(v: np.ndarray, stages) -> np.ndarray:
    v = v.astype(F32, copy=True)
    idx = np.arange(BLOCK)
    with np.errstate(invalid="ignore", over="ignore"):
        for bit in stages:
            lo = idx[(idx >> bit) & 1 == 0]
            hi = lo | (1 << bit)
            a, b = v[:, lo], v[:, hi]
            v[:, lo], v[:, hi] = a + b, a - b
    return v


def rotate_fwd(x: np.ndarray, signs: np.ndarray) -> np.ndarray:
    """y = H_1024 (s * x) (unnormalised) for every row of x [nb, 1024]."""
    return _butterflies(x * signs[None, :], FWD_STAGES)


def rotate_inv(y: np.ndarray, signs: np.ndarray, post_scale: float = 1.0) -> np.ndarray:
    """x = s * H_1024 y * post_scale / 1024 (post_scale = 1/world for the mean)."""
    v = _butterflies(y, INV_STAGES)
    return (v * F32(post_scale / 1024.0)) * signs[None, :]


TAG_STRATIFIED = 0x4000


def quantize(y: np.ndarray, bits: int, block_idx: np.ndarray, tag: int, step: int, seed: int,
             rank: int = 0, world: int = 1, layout: str = "simt") -> Tuple[np.ndarray, np.ndarray]:
    """Rotated blocks [nb, 1024] -> (codes uint8 [nb, 32 lanes, 32 regs], scale f32 [nb]).

    A block whose largest magnitude is NaN, infinite or below 1e-30 is sent as zeros: scale 0 and
    every code equal to R.

    With TAG_STRATIFIED set in `tag` the uniform of value k is the rank's stratum of a uniform all
    ranks share: u = (((rank + shift) mod W) * 256 + byte_k + 0.5) / (256 W), where shift is the
    byte of the neighbouring value ((k + 1) mod 32 of the same lane)."""
    R = qmax(bits)
    y = y.astype(F32, copy=False)
    rho = LAYOUTS[layout]
    absmax = np.max(np.abs(y), axis=1)  # NaN if any coefficient is NaN
    with np.errstate(divide="ignore", invalid="ignore"):
        ok = (absmax >= F32(1e-30)) & np.isfinite(absmax)
        scale = np.where(ok, absmax / F32(R), F32(0)).astype(F32)
        inv = np.where(ok, F32(R) / absmax, F32(0)).astype(F32)
    y = np.where(ok[:, None], y, F32(0))
    r8 = philox.block_uniforms8(block_idx, tag & ~TAG_STRATIFIED, step, seed)  # [nb, 32, 32]
    if tag & TAG_STRATIFIED and world > 1:
        shift = np.roll(r8, -1, axis=2).astype(np.int64)
        stratum = ((rank + shift) % world).astype(F32)
        u = ((stratum * F32(256.0) + r8.astype(F32)) + F32(0.5)) * F32(1.0 / (256.0 * world))
        t = fma32(y[:, rho], inv[:, None, None], u)
        code = np.floor(t).astype(np.int32) + R
    else:
        a = r8.astype(F32) + F32(32768.5)  # 2^15 + byte + 0.5, exact in fp32
        t = fma32(y[:, rho], (inv * F32(256.0))[:, None, None], a)
        code = np.floor(t * F32(1.0 / 256.0)).astype(np.int32) - 128 + R
    # |y| <= absmax keeps the code inside [0, 2 R]: no clamp
    assert code.min(initial=R) >= 0 and code.max(initial=R) <= 2 * R
    return code.astype(np.uint8), scale


def dequantize_add(codes: np.ndarray, scale: np.ndarray, bits: int, acc: np.ndarray,
                   layout: str = "simt") -> np.ndarray:
    """acc [nb, 1024] (coefficient order) + decoded block, one fma per value."""
    R = qmax(bits)
    f = (codes.astype(np.int32) - R).astype(F32)
    out = acc.astype(F32, copy=True)
    flat = LAYOUTS[layout].reshape(-1)
    with np.errstate(invalid="ignore", over="ignore"):
        out[:, flat] = fma32(f.reshape(codes.shape[0], BLOCK), scale[:, None], acc[:, flat])
    return out


def dequantize(codes: np.ndarray, scale: np.ndarray, bits: int, layout: str = "simt") -> np.ndarray:
    """(codes [nb,32,32], scale [nb]) -> rotated blocks [nb, 1024] in coefficient order."""
    R = qmax(bits)
    vals = (codes.astype(np.int32) - R).astype(F32) * scale[:, None, None].astype(F32)
    y = np.empty((codes.shape[0], BLOCK), dtype=F32)
    y[:, LAYOUTS[layout].reshape(-1)] = vals.reshape(codes.shape[0], BLOCK)
    return y


def pack(codes: np.ndarray, bits: int) -> np.ndarray:
    """codes [nb, 32 lanes, 32 regs] -> uint32 words [nb, bits, 32 lanes]."""
    nb = codes.shape[0]
    acc = np.zeros((nb, 32, bits), dtype=np.uint64)
    for k in range(32):
        off = k * bits
        w, sh = off >> 5, off & 31
        val = codes[:, :, k].astype(np.uint64) << np.uint64(sh)
        acc[:, :, w] |= val & np.uint64(0xFFFFFFFF)
        if sh + bits > 32:
            acc[:, :, w + 1] |= val >> np.uint64(32)
    return acc.astype(np.uint32).transpose(0, 2, 1).copy()


def unpack(words: np.ndarray, bits: int) -> np.ndarray:
    """uint32 words [nb, bits, 32] -> codes uint8 [nb, 32, 32]."""
    nb = words.shape[0]
    w64 = words.transpose(0, 2, 1).astype(np.uint64)  # [nb, lane, word]
    codes = np.empty((nb, 32, 32), dtype=np.uint8)
    mask = np.uint64((1 << bits) - 1)
    for k in range(32):
        off = k * bits
        w, sh = off >> 5, off & 31
        val = w64[:, :, w] >> np.uint64(sh)
        if sh + bits > 32:
            val = val | (w64[:, :, w + 1] << np.uint64(32 - sh))
        codes[:, :, k] = (val & mask).astype(np.uint8)
    return codes


def to_message(words: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """Serialise one shard's blocks into the wire layout (uint8)."""
    return np.concatenate([words.reshape(-1).view(np.uint8), scale.astype(F32).view(np.uint8)])


def from_message(msg: np.ndarray, nblocks: int, bits: int) -> Tuple[np.ndarray, np.ndarray]:
    ncode = nblocks * 128 * bits
    words = msg[:ncode].view(np.uint32).reshape(nblocks, bits, 32)
    scale = msg[ncode: ncode + 4 * nblocks].view(F32)
    return words, scale


def encode_blocks(y: np.ndarray, bits: int, block_idx, tag: int, step: int, seed: int, rank: int = 0,
                  world: int = 1, layout: str = "simt") -> np.ndarray:
    codes, scale = quantize(y, bits, np.asarray(block_idx), tag, step, seed, rank, world, layout)
    return to_message(pack(codes, bits), scale)


def decode_add_blocks(msg: np.ndarray, nblocks: int, bits: int, acc: np.ndarray, layout: str = "simt") -> np.ndarray:
    words, scale = from_message(msg, nblocks, bits)
    return dequantize_add(unpack(words, bits), scale, bits, acc, layout)


def decode_blocks(msg: np.ndarray, nblocks: int, bits: int, layout: str = "simt") -> np.ndarray:
    words, scale = from_message(msg, nblocks, bits)
    return dequantize(unpack(words, bits), scale, bits, layout)


# ---- a width per block ----------------------------------------------------------------------------------
# Message of a shard whose blocks have widths w_0 .. w_{n-1}: the blocks' code bytes back to back (block k
# takes 128 w_k bytes), then the fp32 scales at a fixed offset sized for 8-bit blocks, so that a receiver
# finds a scale without the prefix sum.  The bytes below are the codes then the scales, without the gap.

def encode_blocks_mixed(y: np.ndarray, widths: np.ndarray, block_idx, tag: int, step: int, seed: int, rank: int = 0,
                        world: int = 1, layout: str = "simt") -> np.ndarray:
    widths = np.asarray(widths)
    block_idx = np.asarray(block_idx)
    parts, scales = [None] * len(widths), np.zeros(len(widths), dtype=F32)
    for b in np.unique(widths):
        sel = np.nonzero(widths == b)[0]
        codes, sc = quantize(y[sel], int(b), block_idx[sel], tag, step, seed, rank, world, layout)
        words = pack(codes, int(b))
        for j, k in enumerate(sel):
            parts[k] = words[j].reshape(-1).view(np.uint8)
        scales[sel] = sc
    return np.concatenate(parts + [scales.view(np.uint8)]) if len(widths) else np.zeros(0, np.uint8)


def _split_mixed(msg: np.ndarray, widths: np.ndarray):
    widths = np.asarray(widths, dtype=np.int64)
    offs = np.concatenate([[0], np.cumsum(128 * widths)])
    scale = msg[offs[-1]: offs[-1] + 4 * len(widths)].view(F32)
    return offs, scale


def decode_blocks_mixed(msg: np.ndarray, widths: np.ndarray, layout: str = "simt",
                        acc: np.ndarray = None) -> np.ndarray:
    """Decoded blocks [n, 1024]; with `acc` the hop's fused multiply-add into it."""
    widths = np.asarray(widths)
    offs, scale = _split_mixed(msg, widths)
    out = np.zeros((len(widths), BLOCK), dtype=F32) if acc is None else acc.astype(F32, copy=True)
    for b in np.unique(widths):
        sel = np.nonzero(widths == b)[0]
        words = np.stack([msg[offs[k]: offs[k] + 128 * int(b)].view(np.uint32).reshape(int(b), 32) for k in sel])
        codes = unpack(words, int(b))
        if acc is None:
            out[sel] = dequantize(codes, scale[sel], int(b), layout)
        else:
            out[sel] = dequantize_add(codes, scale[sel], int(b), acc[sel], layout)
    return out


def mixed_payload_bytes(widths) -> int:
    widths = np.asarray(widths, dtype=np.int64)
    return int(128 * widths.sum() + 4 * len(widths))


def nmse(estimate: np.ndarray, exact: np.ndarray) -> float:
    """||estimate - exact||^2 / ||exact||^2 in float64 (the reference's vNMSE,
    simulations_llm/new_comm_hooks/comm_hooks.py:22-50)."""
    e = np.asarray(estimate, dtype=np.float64) - np.asarray(exact, dtype=np.float64)
    d = float(np.sum(np.asarray(exact, dtype=np.float64) ** 2))
    return float(np.sum(e * e)) / d if d > 0 else 0.0
