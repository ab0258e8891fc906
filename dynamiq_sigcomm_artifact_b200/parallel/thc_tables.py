"""Constants of THC's uniform stochastic quantiser, derived instead of read from a table file.

The reference ships an offline solver and generated lookup tables
(simulations_llm/compression/{compression,Gen_lookup_tables,solver}.py, ``new_tables/*``) of which the run
time reads one number: the clipping threshold ``T = 3.2971933456919635`` from ``..._data.txt``
(testbed_evaluation/new_comm_hooks/thc_hooks.py:115-121).  After the randomized Hadamard rotation the
coordinates of a d-vector are close to N(0, |g|^2 / d), so the range ``+-T |g| / sqrt(d)`` clips a
coordinate with probability ``2 (1 - Phi(T))``; T is the two-sided normal quantile of probability 2^-10.
This module restates that derivation and the error model behind the choice of (T, levels): clipping error
plus the variance of stochastic rounding on a uniform grid.  Its second half is the offline tool itself:
:func:`solve_levels` finds the non-uniform levels on an integer grid that minimise the rounding variance
(it reproduces the errors and positions of the reference's ``optimal_INCA_*`` result files to 1e-12), and
:func:`sender_table` / :func:`receiver_table` build the lookup tables a table-driven THC would read.
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


# ---- non-uniform levels on an integer grid (the reference's offline table tooling) -----------------------
#
# THC sums integer table VALUES on the way (a switch or a peer can add them without decoding), so the 2^b
# quantisation levels must sit on an integer grid: level = position * T / g with positions in -g..g.  The
# reference searches those positions offline (simulations_llm/compression/solver.py:94-200 for the error
# model, Gen_lookup_tables.py for the sender / receiver tables, results in optimal_INCA_*_bits_*.txt and
# new_tables/*).  The search is restated here as a dynamic programme over closed-form interval costs.


def interval_cost(a: float, b: float) -> float:
    """Variance of unbiased stochastic rounding of x ~ N(0,1) between neighbouring levels a <= b:
    the integral of (x - a)(b - x) pdf(x) over [a, b], from the normal moments in closed form."""
    if b <= a:
        return 0.0
    m0 = _phi(b) - _phi(a)
    m1 = _pdf(a) - _pdf(b)
    m2 = m0 + a * _pdf(a) - b * _pdf(b)
    return -m2 + (a + b) * m1 - a * b * m0


def solve_levels(bits: int, granularity: int, T: float = THC_T) -> Tuple[float, list]:
    """(error, positions): the 2^(bits-1) non-negative grid positions p_1 <= ... <= p_last = granularity
    whose mirrored level set {+-p_i T / granularity} minimises the rounding variance on [-T, T].

    A position may repeat when the grid has fewer points than levels (the repeated level costs nothing and
    buys nothing).  Exact: every candidate is scored, O(granularity^2 * levels)."""
    if bits < 1 or granularity < 1:
        raise ValueError("bits and granularity must be positive")
    half, g = 1 << (bits - 1), int(granularity)
    unit = T / g
    cost = [[interval_cost(i * unit, j * unit) if j > i else 0.0 for j in range(g + 1)] for i in range(g + 1)]
    inf = float("inf")
    # best[k][j]: cheapest way to put k levels on positions <= j with the k-th exactly at j
    best = [[inf] * (g + 1) for _ in range(half + 1)]
    back = [[-1] * (g + 1) for _ in range(half + 1)]
    for j in range(g + 1):
        best[1][j] = interval_cost(-j * unit, j * unit)  # the central interval between -p_1 and +p_1
    for k in range(2, half + 1):
        for j in range(g + 1):
            for i in range(j + 1):
                c = best[k - 1][i] + 2.0 * cost[i][j]
                if c < best[k][j] - 1e-18:
                    best[k][j], back[k][j] = c, i
    positions, j = [], g
    for k in range(half, 0, -1):
        positions.append(j)
        j = back[k][j]
    positions.reverse()
    return best[half][g], positions


def level_values(positions: list, granularity: int, T: float = THC_T) -> list:
    """The full sorted level set of `positions` (as :func:`solve_levels` returns them)."""
    unit = T / granularity
    return [-p * unit for p in reversed(positions)] + [p * unit for p in positions]


def receiver_table(positions: list, granularity: int) -> list:
    """Integer the receiver adds for each level index: the level's grid position shifted to start at 0
    (0 .. 2 * granularity), so that a sum of W table values decodes as (sum - W * granularity) * T / g."""
    return [granularity - p for p in reversed(positions)] + [granularity + p for p in positions]


def sender_table(positions: list, granularity: int, fine_levels: int, T: float = THC_T) -> Tuple[list, list]:
    """(lower level index, probability of rounding up) for each of `fine_levels` equally spaced inputs on
    [-T, T]: what a sender looks up after quantising its clipped coordinate to the fine grid."""
    levels = level_values(positions, granularity, T)
    lower, prob, k = [], [], 0
    for q in range(fine_levels):
        x = -T + 2.0 * T * q / (fine_levels - 1)
        while k + 2 < len(levels) and levels[k + 1] <= x:
            k += 1
        width = levels[k + 1] - levels[k]
        lower.append(k)
        prob.append(0.0 if width <= 0.0 else min(max((x - levels[k]) / width, 0.0), 1.0))
    return lower, prob
