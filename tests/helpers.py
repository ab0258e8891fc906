"""Shared test inputs."""
import numpy as np


def heavy_tail_grad(n: int, seed: int) -> np.ndarray:
    """N(0,1) with 1% of the entries scaled by 100 (heavy tails), from a seeded generator."""
    rng = np.random.default_rng(seed)
    g = rng.standard_normal(n).astype(np.float32)
    g[rng.random(n) < 0.01] *= 100
    return g


def lognormal_block_grad(n: int, seed: int, sigma: float = 2.0) -> np.ndarray:
    """N(0,1) with a lognormal scale per 1024-element block."""
    rng = np.random.default_rng(seed)
    g = rng.standard_normal(n).astype(np.float32)
    nb = (n + 1023) // 1024
    s = np.exp(sigma * rng.standard_normal(nb)).astype(np.float32)
    return (g * np.repeat(s, 1024)[:n]).astype(np.float32)


def small_int_grad(n: int, seed: int) -> np.ndarray:
    """Integers in [-31, 31] times a power of two per 1024-element block.  A 1024-point Hadamard
    transform of such a block is exact in any arithmetic that keeps 11 significant bits of its inputs
    and of the 32-term partial sums (|partial sum| <= 992), which is what a single-TF32 tensor-core
    rotation provides: on these inputs it must agree with fp32 butterflies bit for bit."""
    rng = np.random.default_rng(seed)
    g = np.clip(np.rint(rng.standard_normal(n) * 8.0), -31, 31)
    g[rng.random(n) < 0.3] = 0
    nb = (n + 1023) // 1024
    e = rng.integers(-6, 7, nb)
    return (g * np.repeat(np.exp2(e), 1024)[:n]).astype(np.float32)
