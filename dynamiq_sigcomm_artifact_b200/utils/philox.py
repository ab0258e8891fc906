"""Counter-based random numbers (Philox-4x32-10) shared by the CPU oracle and the CUDA kernels.

The reference draws its stochastic-rounding uniforms from a pre-generated pool whose
window is moved by an LCG (testbed_evaluation/new_comm_hooks/utils_aggregation.py:384-420),
which makes the codes depend on allocation size and call order.  Here every uniform is a
pure function of (seed, step, bucket, stream tag, block index, position), so a run is
bit-reproducible from its seed on any topology and after a resume.

The same function is implemented for the device in ``csrc/common/philox.cuh``; the two
must stay in lock-step (tests compare them word for word).
"""
from __future__ import annotations

import numpy as np

PHILOX_M0 = np.uint64(0xD2511F53)
PHILOX_M1 = np.uint64(0xCD9E8D57)
PHILOX_W0 = 0x9E3779B9
PHILOX_W1 = 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)

# stream tags (counter word c2): one per use of randomness inside a collective
TAG_SIGN = 0x5349474E  # "SIGN": the Rademacher diagonal
TAG_ENCODE = 0x00000100  # first encode of a shard; hop h uses TAG_ENCODE + h
TAG_FINAL = 0x00000200  # owner's re-encode before the all-gather
TAG_SCALE = 0x00000300  # stochastic scale rounding (superchunk family)


def philox4x32(c0, c1, c2, c3, k0, k1, rounds: int = 10):
    """Vectorised Philox-4x32.  Inputs broadcast; returns four uint32 arrays."""
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) & _MASK32 for c in (c0, c1, c2, c3))
    c0, c1, c2, c3 = np.broadcast_arrays(c0, c1, c2, c3)
    k0 = int(k0) & 0xFFFFFFFF
    k1 = int(k1) & 0xFFFFFFFF
    for _ in range(rounds):
        p0 = PHILOX_M0 * c0
        p1 = PHILOX_M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK32
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK32
        n0 = hi1 ^ c1 ^ np.uint64(k0)
        n2 = hi0 ^ c3 ^ np.uint64(k1)
        c0, c1, c2, c3 = n0, lo1, n2, lo0
        k0 = (k0 + PHILOX_W0) & 0xFFFFFFFF
        k1 = (k1 + PHILOX_W1) & 0xFFFFFFFF
    return tuple(c.astype(np.uint32) for c in (c0, c1, c2, c3))


UNIFORM_ROUNDS = 7  # Philox-4x32-7 (the shortest crush-resistant variant) for the rounding uniforms


def block_uniforms8(block_idx, tag: int, step: int, seed: int) -> np.ndarray:
    """8-bit uniforms for whole 1024-element blocks.

    Returns uint8 array ``[len(block_idx), 32 lanes, 32 values]``.  Lane ``l`` makes two
    Philox-4x32-7 calls (counter word c1 = 2*l + q); call ``q`` yields values ``16q .. 16q+15``
    as the bytes, least significant first, of its four output words.
    """
    block_idx = np.asarray(block_idx, dtype=np.uint64).reshape(-1, 1)
    call = np.arange(64, dtype=np.uint64).reshape(1, -1)
    w = philox4x32(block_idx, call, tag, step, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF, rounds=UNIFORM_ROUNDS)
    words = np.stack(w, axis=-1)  # [nb, 64 calls, 4 words]
    by = np.stack([(words >> np.uint32(8 * k)) & np.uint32(0xFF) for k in range(4)], axis=-1).astype(np.uint8)
    return by.reshape(len(block_idx), 32, 32)


def sign_words(step: int, bucket: int, seed: int) -> np.ndarray:
    """1024 Rademacher sign bits as 32 uint32 words (bit e%32 of word e//32 set => -1)."""
    quad = np.arange(8, dtype=np.uint64)
    w = philox4x32(quad, step, TAG_SIGN, bucket, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    return np.stack(w, axis=-1).reshape(32).astype(np.uint32)


def sign_vector(step: int, bucket: int, seed: int) -> np.ndarray:
    """The diagonal as 1024 float32 values in {+1, -1}."""
    words = sign_words(step, bucket, seed)
    e = np.arange(1024)
    bits = (words[e >> 5] >> (e & 31).astype(np.uint32)) & np.uint32(1)
    return np.where(bits == 1, np.float32(-1.0), np.float32(1.0)).astype(np.float32)
