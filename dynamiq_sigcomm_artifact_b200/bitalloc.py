"""Bit-width selection: threshold split, the dynamic-bitrate controller, per-bucket widths.

Restates the reference's policies so that they can be unit-tested on CPU:

* threshold split (testbed_evaluation/new_comm_hooks/comm_hooks.py:713-721): stable descending
  argsort of the per-superchunk energy; the top ``thr[8]`` fraction is sent at 8 bits, the
  bottom ``thr[2]`` at 2, the rest at 4;
* dynamic bitrate (comm_hooks.py:48-139,907-930; spec new_comm_hooks/dynamic_bitrate.md):
  ``q = 2 ** clamp(floor(log2(c * log2 F + u)), 1, 3)`` with ``c = 4 / (512 / 17)``; ``u``
  starts at 60, is bisected on [-10, 60] on the first compressed step and then nudged every
  step so that ``mean(q)`` stays within 0.1 of ``b - 0.625`` (0.625 bit/element is what the
  scales and the mean cost on the wire);
* per-bucket widths for the rotation codec (this framework's addition): whole buckets move
  between b-1, b and b+1 bits by their energy per element, under the same average budget.
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence, Tuple

import torch

HEADROOM = 0.625
U_MIN, U_MAX = -10.0, 60.0
TOL = 0.1
MAX_ITERS = 32
NORM_SCALE = 4.0 / (512.0 / 17.0)


def split_by_thresholds(norms: torch.Tensor, thresholds: Dict[int, float], fixed: bool = False
                        ) -> Dict[int, torch.Tensor]:
    """{8: idx, 4: idx, 2: idx} row indices of the three groups (empty groups included)."""
    n = norms.numel()
    top = int(n * thresholds.get(8, 0.0))
    bottom = int(n * thresholds.get(2, 0.0))
    if top + bottom > n:
        bottom = max(0, n - top)
    order = torch.argsort(norms.float(), descending=True, stable=True)
    groups = {8: order[:top], 4: order[top: n - bottom], 2: order[n - bottom:] if bottom > 0 else order[:0]}
    if fixed:  # only the 4-bit group is communicated (comm_hooks.py:767-771)
        groups[8], groups[2] = order[:0], order[:0]
    return groups


def qbits(norms: torch.Tensor, u: float) -> torch.Tensor:
    """Per-superchunk code width in {2, 4, 8} for controller state `u`."""
    eps = 1e-20
    score = torch.log2(torch.clamp(norms.float(), min=eps)) * NORM_SCALE + float(u)
    z = torch.floor(torch.log2(torch.clamp(score, min=eps))).to(torch.int64).clamp_(1, 3)
    return torch.bitwise_left_shift(torch.ones_like(z), z)


def split_by_bitrate(norms: torch.Tensor, u: float) -> Dict[int, torch.Tensor]:
    q = qbits(norms, u)
    return {b: torch.nonzero(q == b, as_tuple=False).reshape(-1) for b in (8, 4, 2)}


def average_bits(norms_list: Sequence[torch.Tensor], u: float) -> float:
    total, count = 0.0, 0
    for norms in norms_list:
        if norms.numel():
            total += float(qbits(norms, u).sum())
            count += norms.numel()
    return total / count if count else 0.0


class DynamicBitrateController:
    """Keeps ``mean(q)`` at ``target_bits - 0.625`` by moving ``u``."""

    def __init__(self, target_bits: float):
        self.target = float(target_bits) - HEADROOM
        self.u = U_MAX
        self.last_avg = 0.0
        self.last_delta = 0.0
        self.initialised = False
        self._norms: List[torch.Tensor] = []

    def observe(self, norms: torch.Tensor) -> None:
        self._norms.append(norms.detach().float().cpu())

    def _delta(self, u: float) -> Tuple[float, float]:
        avg = average_bits(self._norms, u)
        return avg, self.target - avg

    def _bisect(self) -> Tuple[float, float, float]:
        low, high = U_MIN, U_MAX
        best_u = high
        best_avg, best_delta = self._delta(best_u)
        for _ in range(MAX_ITERS):
            mid = 0.5 * (low + high)
            avg, delta = self._delta(mid)
            if abs(delta) < abs(best_delta):
                best_u, best_avg, best_delta = mid, avg, delta
            if abs(delta) <= TOL:
                return mid, avg, delta
            if delta > 0:
                low = mid
            else:
                high = mid
        return best_u, best_avg, best_delta

    def _adjust(self) -> Tuple[float, float, float]:
        prev = min(U_MAX, max(U_MIN, self.u))
        old_avg, old_delta = self._delta(prev)
        if abs(old_delta) <= TOL:
            return prev, old_avg, old_delta
        step = old_delta
        best = (prev, old_avg, old_delta)
        for _ in range(MAX_ITERS):
            cand = min(U_MAX, max(U_MIN, prev + step))
            avg, delta = self._delta(cand)
            if abs(delta) < abs(best[2]):
                best = (cand, avg, delta)
            if abs(delta) <= TOL or old_delta * delta >= 0:
                return cand, avg, delta
            step *= 0.5
        return best

    def end_of_step(self) -> None:
        """Call after the last bucket of a step: updates ``u`` for the next step."""
        if not self._norms:
            return
        u, avg, delta = self._adjust() if self.initialised else self._bisect()
        self.u, self.last_avg, self.last_delta = float(u), float(avg), float(delta)
        self.initialised = True
        self._norms = []

    def state_dict(self) -> dict:
        return {"u": self.u, "initialised": self.initialised, "target": self.target}

    def load_state_dict(self, d: dict) -> None:
        self.u, self.initialised, self.target = float(d["u"]), bool(d["initialised"]), float(d["target"])


class DeviceBitrateController:
    """The same controller with its state on the GPU: nothing is read back to the host.

    ``state`` is four doubles on the device (u, initialised, last average width, last delta).  Every
    bucket's widths come from ``torch.ops.dq.superchunk_widths`` (which also returns the scores it
    used); after the step's last bucket the scores are sorted once and one small kernel walks the
    bisection / adjustment with binary searches (csrc/kernels/bitalloc_ops.cu).  The update runs on the
    stream it is called on and is published through ``ready`` (an event) for the next step's first bucket.
    Widths come from thresholds on the score (8 from 8 up, 4 from 4 up, else 2), which is
    :func:`qbits` without the round trip through ``log2``.
    """

    def __init__(self, target_bits: float, device, u: float = U_MAX, initialised: bool = False):
        self.target = float(target_bits) - HEADROOM
        self.device = torch.device(device)
        self.state = torch.tensor([float(u), 1.0 if initialised else 0.0, 0.0, 0.0], dtype=torch.float64,
                                  device=self.device)
        self._scores: List[torch.Tensor] = []
        self.ready = None  # torch.cuda.Event of the last update

    def widths(self, stats: torch.Tensor) -> torch.Tensor:
        """stats [nsc, 2] (all-reduced; energy in column 1) -> uint8 widths [nsc]; remembers the scores."""
        from . import ops as _ops

        if self.ready is not None:
            torch.cuda.current_stream(self.device).wait_event(self.ready)
        nsc = stats.shape[0]
        scores = torch.empty(nsc, dtype=torch.float32, device=stats.device)
        widths = torch.empty(nsc, dtype=torch.uint8, device=stats.device)
        _ops.require().superchunk_widths(stats, self.state, scores, widths)
        self._scores.append(scores)
        return widths

    def end_of_step(self) -> None:
        from . import ops as _ops

        if not self._scores:
            return
        s = torch.cat(self._scores) if len(self._scores) > 1 else self._scores[0]
        self._scores = []
        _ops.require().superchunk_bitrate_update(torch.sort(s).values, self.state, self.target)
        self.ready = torch.cuda.Event()
        self.ready.record(torch.cuda.current_stream(self.device))

    def state_dict(self) -> dict:
        u, init, avg, delta = self.state.tolist()  # synchronises; checkpoints only
        return {"u": u, "initialised": bool(init), "target": self.target, "last_avg": avg, "last_delta": delta}

    def load_state_dict(self, d: dict) -> None:
        self.target = float(d.get("target", self.target))
        self.state.copy_(torch.tensor([float(d["u"]), 1.0 if d.get("initialised", True) else 0.0,
                                       float(d.get("last_avg", 0.0)), float(d.get("last_delta", 0.0))],
                                      dtype=torch.float64))


KTH_INIT, KTH_SMALLER_INIT = 1.1562e-4, 2.6375e-06


class MomentumThresholds:
    """Widths from two energy thresholds that follow the step's quantiles with momentum.

    A superchunk is sent at 8 bits if its energy exceeds ``kth``, at 2 bits if it is below
    ``kth_smaller``, else at 4.  After the step's last bucket all energies of the step are sorted once
    (descending) and ``kth <- 0.25 * E[int(n * t8)] + 0.75 * kth``, ``kth_smaller <- 0.25 * E[int(n * (t8 +
    t4))] + 0.75 * kth_smaller`` (simulations_llm/new_comm_hooks/comm_hooks.py:326-370, initial values
    :498-499).  No per-bucket sort and, on CUDA, no value ever read back: the thresholds are a device tensor.
    """

    def __init__(self, thresholds: Dict[int, float], device="cpu", kth: float = KTH_INIT,
                 kth_smaller: float = KTH_SMALLER_INIT):
        self.t8 = float(thresholds.get(8, 0.0))
        self.t4 = float(thresholds.get(4, 0.0))
        self.device = torch.device(device)
        self.state = torch.tensor([kth, kth_smaller], dtype=torch.float32, device=self.device)
        self._energies: List[torch.Tensor] = []
        self.ready = None

    def widths(self, energy: torch.Tensor) -> torch.Tensor:
        if self.ready is not None and energy.is_cuda:
            torch.cuda.current_stream(energy.device).wait_event(self.ready)
        e = energy.float()
        self._energies.append(e)
        w = (e > self.state[0]).to(torch.uint8) * 4 + 4 - (e < self.state[1]).to(torch.uint8) * 2
        return w.to(torch.uint8)

    def groups(self, energy: torch.Tensor) -> Dict[int, torch.Tensor]:
        """Row indices per width (the three-group form used on CPU tensors)."""
        w = self.widths(energy)
        return {b: torch.nonzero(w == b, as_tuple=False).reshape(-1) for b in (8, 4, 2)}

    def end_of_step(self) -> None:
        if not self._energies:
            return
        e = torch.cat(self._energies) if len(self._energies) > 1 else self._energies[0]
        self._energies = []
        n = e.numel()
        srt = torch.sort(e, descending=True).values
        i8 = min(n - 1, int(n * self.t8))
        i4 = min(n - 1, int(n * (self.t8 + self.t4)))
        self.state.mul_(0.75).add_(0.25 * torch.stack([srt[i8], srt[i4]]))
        if e.is_cuda:
            self.ready = torch.cuda.Event()
            self.ready.record(torch.cuda.current_stream(e.device))

    def state_dict(self) -> dict:
        kth, small = self.state.tolist()
        return {"kth": kth, "kth_smaller": small}

    def load_state_dict(self, d: dict) -> None:
        self.state.copy_(torch.tensor([float(d["kth"]), float(d["kth_smaller"])], dtype=torch.float32))


def threshold_widths(energy: torch.Tensor, thresholds: Dict[int, float]) -> torch.Tensor:
    """uint8 width per superchunk for the threshold split, built on the device without reading a size back:
    the group sizes follow from the element count alone (:func:`split_by_thresholds`)."""
    n = energy.numel()
    top = int(n * thresholds.get(8, 0.0))
    bottom = int(n * thresholds.get(2, 0.0))
    if top + bottom > n:
        bottom = max(0, n - top)
    order = torch.argsort(energy.float(), descending=True, stable=True)
    widths = torch.full((n,), 4, dtype=torch.uint8, device=energy.device)
    # index_fill_ takes the value as a scalar argument: no host-to-device copy (and none of its stream syncs)
    if top:
        widths.index_fill_(0, order[:top], 8)
    if bottom:
        widths.index_fill_(0, order[n - bottom:], 2)
    return widths


# ---- rotation codec: a code width per 1024-element block -------------------------------------------------
#
# Reverse water-filling: with a fixed budget of bits, a block whose rotated coefficients are 2^d times
# larger than another's should get d more bits (each bit quarters its error).  So
#     width_k = clamp(round(c + log2(absmax_k)), RHT_MIN_BITS, RHT_MAX_BITS)
# with one offset c per bucket chosen so that the mean width meets the target - the rotation-codec
# counterpart of the reference's 8 / 4 / 2 threshold split and dynamic-bitrate controller
# (testbed_evaluation/new_comm_hooks/comm_hooks.py:48-139,713-721,842-856).  absmax_k is what every rank
# already holds after a collective: the scale of block k in the all-gathered message times R(width), bit
# identical on all ranks, so the widths of the NEXT step need no extra communication and no host read.
# Everything is integer arithmetic on 1/8-bit quantised logarithms (``quantised_log2``), so the device
# kernel (csrc/kernels/bitalloc_ops.cu: rht_widths_update) and this host twin agree exactly.

RHT_MIN_BITS, RHT_MAX_BITS = 2, 8
_LOG2_STEPS = None


def _log2_thresholds():
    """fp32 values of 2^(j/8), j = 1..7, as the device kernel spells them."""
    global _LOG2_STEPS
    if _LOG2_STEPS is None:
        import numpy as np

        _LOG2_STEPS = np.array([1.0905077, 1.1892071, 1.2968396, 1.4142135, 1.5422108, 1.6817929, 1.8340080],
                               dtype=np.float32)
    return _LOG2_STEPS


def quantised_log2(x):
    """floor(8 log2 x) for positive finite fp32 x, from the exponent field and seven comparisons of the
    mantissa; x <= 0, NaN and infinity give the smallest value (-1016 = 8 * -127)."""
    import numpy as np

    x = np.asarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    expo = ((bits >> np.uint32(23)) & np.uint32(0xFF)).astype(np.int32) - 127
    mant = ((bits & np.uint32(0x007FFFFF)) | np.uint32(0x3F800000)).view(np.float32)  # in [1, 2)
    frac = (mant[..., None] >= _log2_thresholds()).sum(axis=-1).astype(np.int32)
    ok = (x > 0) & np.isfinite(x)
    return np.where(ok, 8 * expo + frac, -1016).astype(np.int32)


def rht_block_widths(absmax, target_bits: float):
    """(widths uint8 [nblocks], offset c in 1/8 bit) for per-block magnitudes `absmax`: the largest offset
    whose total width does not exceed round(target_bits * nblocks)."""
    import numpy as np

    lq = quantised_log2(absmax)
    budget = int(round(float(target_bits) * lq.size))

    def widths_at(c8: int):
        return np.clip((lq + c8 + 4) >> 3, RHT_MIN_BITS, RHT_MAX_BITS)

    lo, hi = -2048, 2048  # invariant: total(lo) <= budget (or lo is the floor), total(hi) > budget (or hi is the cap)
    if int(widths_at(hi).sum()) <= budget:
        return widths_at(hi).astype(np.uint8), hi
    while hi - lo > 1:
        mid = (lo + hi) // 2
        if int(widths_at(mid).sum()) <= budget:
            lo = mid
        else:
            hi = mid
    return widths_at(lo).astype(np.uint8), lo


def rht_plan(widths):
    """int32 [2 nblocks + 1]: exclusive prefix sum of the widths (message offset of each block's codes in
    units of 128 bytes), then the widths - the layout the kernel reads."""
    import numpy as np

    w = np.asarray(widths, dtype=np.int64)
    return np.concatenate([[0], np.cumsum(w), w]).astype(np.int32)
