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
