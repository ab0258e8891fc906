"""Constants of THC's uniform stochastic quantiser, derived instead of read from a table file.

The reference ships an offline solver and generated lookup tables
(simulations_llm/compression/{compression,Gen_lookup_tables,solver}.py, ``new_tables/*``) of which the run
time reads one number: the clipping threshold ``T = 3.2971933456919635`` from ``..._data.txt``
(testbed_evaluation/new_comm_hooks/thc_hooks.py:115-121).  After the randomized Hadamard rotation the
coordinates of a d-vector are close to N(0, |g|^2 / d), so the range ``+-T |g| / sqrt(d)`` clips a
coordinate with probability ``2 (1 - Phi(T))``; T is the two-sided normal quantile of probability 2^-10.
This module restates that derivation and the error model behind the choice of (T, levels): clipping error
plus the variance of stochastic rounding on a uniform grid.
"""
from __future__ import annotations

import math
from typing import Tuple

THC_T = 3.2971933456919635


def _phi(x: float) -> float:
    return 0.5 * math.erfc(-x / math.sqrt(2.0))


def _pdf(x: float) -> float:
    return math.exp(-0.5 * x * x) / math.sqrt(2.0 * math.pi)


def clip_threshold(p_clip: float = 2.0 ** -10) -> float:
    """T with P(|N(0,1)| > T) = p_clip, by bisection on the normal tail (p_clip = 2^-10 gives THC's T)."""
    if not 0.0 < p_clip < 1.0:
        raise ValueError("p_clip must be in (0, 1)")
    lo, hi = 0.0, 40.0
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if 2.0 * (1.0 - _phi(mid)) > p_clip:
            lo = mid
        else:
            hi = mid
    return 0.5 * (lo + hi)


def clipping_error(T: float) -> float:
    """E[(|x| - T)^2 ; |x| > T] for x ~ N(0, 1)."""
    tail = 1.0 - _phi(T)
    return 2.0 * ((1.0 + T * T) * tail - T * _pdf(T))


def rounding_variance(T: float, levels: int, steps: int = 4096) -> float:
    """Variance added by unbiased stochastic rounding of x ~ N(0,1), |x| <= T, onto `levels` uniform points."""
    if levels < 2:
        raise ValueError("need at least two levels")
    delta = 2.0 * T / (levels - 1)
    total, h = 0.0, 2.0 * T / steps
    for i in range(steps):  # midpoint rule; the integrand is smooth inside each cell
        x = -T + (i + 0.5) * h
        r = (x + T) / delta
        frac = r - math.floor(r)
        total += frac * (1.0 - frac) * delta * delta * _pdf(x) * h
    return total


def expected_error(T: float, levels: int) -> float:
    """Mean squared error per coordinate (unit-variance input) of clip + stochastic uniform quantisation."""
    return clipping_error(T) + rounding_variance(T, levels)


def best_threshold(levels: int, lo: float = 0.5, hi: float = 8.0) -> Tuple[float, float]:
    """(T, error) minimising :func:`expected_error` for `levels` points, by golden-section search."""
    g = (math.sqrt(5.0) - 1.0) / 2.0
    a, b = lo, hi
    c, d = b - g * (b - a), a + g * (b - a)
    fc, fd = expected_error(c, levels), expected_error(d, levels)
    for _ in range(80):
        if fc < fd:
            b, d, fd = d, c, fc
            c = b - g * (b - a)
            fc = expected_error(c, levels)
        else:
            a, c, fc = c, d, fd
            d = a + g * (b - a)
            fd = expected_error(d, levels)
    t = 0.5 * (a + b)
    return t, expected_error(t, levels)
