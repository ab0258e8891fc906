"""Typed configuration and the parser for the legacy ``aggregation_method`` strings.

The reference selects hook, codec, bit budget, topology and debug modes by *substring*
tests on one free-form string, in a fixed order
(testbed_evaluation/train_llm_causal.py:294-314; smoke_test_new_comm_hooks.py:200-219), and
configures its transport through environment variables
(testbed_evaluation/new_comm_hooks/ring_rdma.py:399-404, butterfly_rdma.py:40-137,
rdma_comm_compress/ring_allreduce_ext/ring_allreduce_backend.cu:99-115,344-368).
:func:`parse_method` accepts the same strings so reference command lines keep working and
returns a :class:`MethodSpec`; :class:`DynamiqConfig` replaces the env-var layer, reading
``DQ_*`` variables with the old names as aliases where they still mean something.
"""
from __future__ import annotations

import os
import re
from dataclasses import asdict, dataclass, field
from typing import Dict, Optional

HOOK_KINDS = ("dynamiq", "dynamiq_bitrate", "bf16", "fp16", "fp32", "mxfp8", "fpx", "thc", "omnireduce")

# fraction of superchunks sent at 8 / 4 / 2 bits for a nominal average width
# (testbed_evaluation/new_comm_hooks/comm_hooks.py:842-856)
THRESHOLD_TABLE: Dict[str, Dict[int, float]] = {
    "3bit": {8: 1 / 40, 4: 13 / 40, 2: 26 / 40},
    "4bit": {8: 0.05, 4: 0.60, 2: 0.35},
    "4bit_fixed": {8: 0.0, 4: 1.0, 2: 0.0},
    "5bit": {8: 0.35, 4: 0.45, 2: 0.20},
    "6bit": {8: 0.55, 4: 0.35, 2: 0.10},
    "7bit": {8: 0.75, 4: 0.22, 2: 0.03},
}


@dataclass
class MethodSpec:
    """Everything an ``aggregation_method`` string selects."""

    name: str
    hook: str  # one of HOOK_KINDS
    family: str = "rht"  # "rht" | "superchunk" | "sim" (dynamiq hooks only)
    lattice: str = "aee"  # "aee" linear | "mee" logarithmic lattice (superchunk family)
    bits: int = 5  # nominal average code width
    fixed: bool = False  # superchunk: only the 4-bit group is communicated
    dynamic_bitrate: bool = False
    momentum: bool = False  # superchunk: widths from two energy thresholds tracked with momentum across steps
    mixed: bool = False  # rotation codec: a code width per 1024-element block around the `bits` average
    topology: str = "direct"  # ring | butterfly | direct (direct unless the method string or the config names one)
    correlated: bool = False  # stratified uniforms across ranks
    no_compress: bool = False  # run the selection logic but skip the collective (debug)
    compute_only: bool = False  # "coov": kernels run, nothing is transmitted (debug)
    fpx_format: Optional[str] = None  # "fp4" | "fp6" | "zero" for the fpx hook
    shared_scale: bool = False  # fpx / fp8: block maxima MAX-reduced over the ranks, adaptive gain (simulation hook)
    quantization_levels: Optional[int] = None  # thc
    thresholds: Dict[int, float] = field(default_factory=dict)

    def to_dict(self) -> dict:
        return asdict(self)


def _bits_in(name: str, default: int) -> int:
    m = re.search(r"(\d)bit", name)
    return int(m.group(1)) if m else default


def parse_method(name: str, topology: Optional[str] = None) -> MethodSpec:
    """Parse e.g. ``dynamiQ_aee_5bit``, ``dynamiQ_mee_5bit_dynamic_bitrate_butterfly``, ``MXfp8``.

    The substring order is the reference's: thc, omnireduce, bf16, dynamiq(+bitrate), fp8,
    fp4/fp6/zero; then fp16/fp32, which the reference defines but cannot reach.

    Topology: ``_butterfly`` / ``_ring`` / ``_direct`` in the name, or the `topology` argument, select one.
    Without either the collective is ``direct``: on an NVSwitch box every shard goes straight to its owner,
    which is as fast as or faster than the ring at every message size and rounds a value twice instead of
    once per rank (the reference, built for rings of RDMA links, defaults to the ring).

    Codec family of ``dynamiQ_*``: names with ``mee``, ``fixed``, ``bitrate``, ``momentum`` or
    ``superchunk`` select the reference's superchunk records; plain ``dynamiQ_aee_{b}bit`` selects the
    rotation codec (randomised Hadamard rotation of 1024-element blocks, one scale per block, b-bit codes) -
    add ``_superchunk`` to run that name through the reference's AEE superchunk format instead, and
    ``_mixed`` to let the rotation codec choose a width per block around the b-bit average.
    """
    low = name.lower()
    topo = topology or ("butterfly" if "butterfly" in low else "ring" if "ring" in low else "direct")
    common = dict(name=name, topology=topo, compute_only="coov" in low)
    if "thc" in low:
        return MethodSpec(hook="thc", bits=5, quantization_levels=31, **common)
    if "omnireduce" in low or "omni" in low:
        return MethodSpec(hook="omnireduce", bits=16, **common)
    if "bf16" in low:
        return MethodSpec(hook="bf16", bits=16, **common)
    if "dynamiq" in low:
        bits = _bits_in(low, 5)
        family = "superchunk" if ("superchunk" in low or "mee" in low or "bitrate" in low or "fixed" in low
                                  or "momentum" in low) else "rht"
        if "rht" in low or "mixed" in low:
            family = "rht"
        if low.endswith("_sim") or "_sim_" in low:  # the simulation stack's hierarchical compressor (any width)
            family = "sim"
        mixed = family == "rht" and ("mixed" in low or "bitrate" in low)
        lattice = "aee" if "aee" in low else "mee"
        fixed = "fixed" in low
        key = f"{bits}bit_fixed" if (fixed and bits == 4) else f"{bits}bit"
        thresholds = dict(THRESHOLD_TABLE.get(key, THRESHOLD_TABLE["5bit"]))
        return MethodSpec(hook="dynamiq_bitrate" if "bitrate" in low else "dynamiq", family=family,
                          lattice=lattice, bits=bits, fixed=fixed, dynamic_bitrate="bitrate" in low,
                          correlated="correlated" in low, no_compress="no_compress" in low,
                          momentum="momentum" in low, mixed=mixed,
                          thresholds=thresholds, **common)
    shared = "shared" in low or "adaptive" in low
    if "fp8" in low:
        if shared:
            return MethodSpec(hook="fpx", bits=8, fpx_format="fp8", shared_scale=True, **common)
        return MethodSpec(hook="mxfp8", bits=8, **common)
    for fmt, b in (("fp4", 4), ("fp6", 6), ("zero", 0)):
        if fmt in low:
            return MethodSpec(hook="fpx", bits=b, fpx_format=fmt, shared_scale=shared and fmt != "zero", **common)
    if "fp16" in low:
        return MethodSpec(hook="fp16", bits=16, **common)
    if "fp32" in low or low in ("none", "nccl", "allreduce"):
        return MethodSpec(hook="fp32", bits=32, **common)
    raise ValueError(f"unknown aggregation_method {name!r}")


def _env(names, default, cast):
    for n in names:
        v = os.environ.get(n)
        if v is not None and v != "":
            try:
                return cast(v)
            except ValueError as e:
                raise ValueError(f"bad value {v!r} for {n}") from e
    return default


def _bool(v: str) -> bool:
    return v.strip().lower() in ("1", "true", "yes", "on")


@dataclass
class DynamiqConfig:
    """Runtime knobs of the hooks and the NVLink transport."""

    method: str = "dynamiQ_aee_5bit"
    topology: Optional[str] = None  # overrides what the method string says
    seed: int = 0
    warmup_steps: int = 2  # steps served by the plain library all-reduce (reference: batch_idx 0 and 1)
    comm_ctas: int = 64  # CTAs of the persistent collective kernel (SM carve-out against backward)
    comm_threads: int = 256
    tail_ctas: int = 148  # grid of a step's last bucket, which nothing overlaps (0: same as comm_ctas)
    comm_prefetch: bool = True  # bulk-copy staging of the next raw block (4 KiB of shared memory per warp)
    rotation: str = "simt"  # "simt": fp32 butterflies (bit-exact with the CPU oracle); "tc": tcgen05 / TMEM
    wait_timeout_ms: int = 2000  # budget of every device-side wait before it gives up with an error status
    max_bucket_mb: int = 128  # symmetric-buffer capacity (grown on demand between steps)
    overlap: bool = True  # run the collective on a side stream under backward
    use_nvls: bool = False  # uncompressed wires (bf16 method) reduce inside the NVSwitch (multimem) when the box
    #                         exposes a multicast object and there are more than two ranks.  Off by default: on four
    #                         B200s the point-to-point cast wire was faster at every size from 1 MB to 1 GB
    #                         (256 MB fp32 bucket, bf16 wire: 0.47 ms against 0.54 ms), its casts ride in the same
    #                         pass as the transfer while the in-switch path stages through a symmetric buffer
    measure_comm_error: bool = False  # exact all-reduce of a clone + vNMSE accounting
    nvtx: bool = False
    debug: bool = False  # guard zones around the mailbox / flag regions, checked by every status check
    validate_topology: bool = True

    @classmethod
    def from_env(cls, **overrides) -> "DynamiqConfig":
        c = cls(**overrides)
        c.comm_ctas = _env(["DQ_COMM_CTAS"], c.comm_ctas, int)
        c.tail_ctas = _env(["DQ_TAIL_CTAS"], c.tail_ctas, int)
        c.comm_threads = _env(["DQ_COMM_THREADS"], c.comm_threads, int)
        c.comm_prefetch = _env(["DQ_COMM_PREFETCH"], c.comm_prefetch, _bool)
        c.wait_timeout_ms = int(1000 * _env(["DQ_TIMEOUT_SECONDS", "RING_RDMA_TIMEOUT_SECONDS"],
                                             c.wait_timeout_ms / 1000, float))
        c.max_bucket_mb = _env(["DQ_MAX_BUCKET_MB"], c.max_bucket_mb, int)
        c.rotation = _env(["DQ_ROTATION"], c.rotation, str)
        c.overlap = _env(["DQ_OVERLAP", "RING_OVERLAP_LOCAL_P2P"], c.overlap, _bool)
        c.use_nvls = _env(["DQ_USE_NVLS"], c.use_nvls, _bool)
        c.debug = _env(["DQ_DEBUG", "RING_RDMA_DEBUG"], c.debug, _bool)
        c.nvtx = _env(["DQ_NVTX"], c.nvtx, _bool)
        c.validate_topology = _env(["DQ_VALIDATE_NVLINK", "RING_VALIDATE_NVLINK"], c.validate_topology, _bool)
        return c

    def spec(self) -> MethodSpec:
        return parse_method(self.method, self.topology)
