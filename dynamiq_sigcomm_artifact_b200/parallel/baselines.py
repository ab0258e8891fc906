"""Baseline aggregation methods: MXFP8, FP4 / FP6 / zero, THC, OmniReduce.

Numerics follow the reference's *simulation* stack, which is the clean specification; its
testbed copies exist to measure time and are wrong on purpose or by accident (fp4 / fp6 / zero
only truncate the message, testbed_evaluation/new_comm_hooks/comm_hooks.py:214-248; the testbed
MXFP8 scale is inverted, :407-409).  All of them run on the device-agnostic backend.
"""
import math

import torch
import torch.distributed as dist

from .codecs import BlockFloatCodec, CastCodec, IntBinsCodec
from .torch_backend import allreduce_torch, uniform_bytes

THC_T = 3.2971933456919635  # table metadata of the reference (simulations_llm/compression/new_tables/*_data.txt)
THC_MAX_PART = 1 << 23


def _begin(state, bucket):
    state = state[0] if isinstance(state, (list, tuple)) else state
    state._auto_advance(bucket.index())
    if bucket.buffer().numel() > state.get("max_bucket_numel", 0):
        state["max_bucket_numel"] = bucket.buffer().numel()
    return state


def _done(buf):
    fut = torch.futures.Future()
    fut.set_result(buf)
    return fut


def _warmup(state, buf):
    from ..hooks import _library_mean

    return _library_mean(state, buf)


def _block_float_hook(fmt_of):
    def hook(state, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
        state = _begin(state, bucket)
        buf = bucket.buffer()
        if state["batch_idx"] < state["config"].warmup_steps:
            return _warmup(state, buf)
        world = dist.get_world_size(state["group"])
        fmt = fmt_of(state["spec"])
        if world == 1:
            return _done(buf)
        if fmt == "zero":  # traffic-free debug mode: every rank keeps its own share
            buf.div_(world)
            return _done(buf)
        spec = state["spec"]
        if buf.is_cuda and buf.dtype in (torch.float32, torch.bfloat16):
            # fused kernel: native E4M3 / E3M2 / E2M1 conversions, peer stores over NVLink
            from ..hooks import _engine

            eng = _engine(state)
            width = {"fp8": 8, "fp6": 6, "fp4": 4}[fmt]
            eng.allreduce_(buf.reshape(-1), width, spec.topology, state["config"].seed, int(state["batch_idx"]),
                           bucket.index(), no_transmit=spec.compute_only, codec="mx")
            return _done(buf)
        out = allreduce_torch(buf, BlockFloatCodec(fmt), spec.topology, state["group"],
                              transmit=not spec.compute_only)
        buf.copy_(out.to(buf.dtype))
        return _done(buf)

    return hook


mxfp8_hook = _block_float_hook(lambda spec: "fp8")
_local_scale_fpx_hook = _block_float_hook(lambda spec: spec.fpx_format)

SHARED_CHUNK = 32  # values that share one power-of-two scale in the shared-scale variant
SHARED_PROPORTION = 0.01  # saturated share of a bucket above which the gain backs off


def fpx_shared_hook(state, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """``fp4_shared`` / ``fp6_shared`` / ``fp8_shared``: the simulation stack's block-float hook
    (simulations_llm/new_comm_hooks/comm_hooks.py:990-1060).  Every 32-value chunk is divided by a
    power-of-two bound of its magnitude that is MAX-reduced over the ranks first, so all ranks share the
    scales and the hops add bare minifloats; the values are then multiplied by a gain ``mu`` per bucket
    that a feedback rule keeps just below saturation: if more than 1 % of the reduced values sit at the
    format's largest magnitude, mu shrinks by 5 % (not below vmax / (2 W)); otherwise it grows by 2^0.02
    (not above vmax).  FP6 and FP8 keep mu fixed, as in the reference.  The MAX reduction is a library
    collective: this variant reproduces the simulation's numerics, not a fused fast path."""
    from .codecs import _FORMATS, MinifloatCodec

    state = _begin(state, bucket)
    buf = bucket.buffer()
    if state["batch_idx"] < state["config"].warmup_steps:
        return _warmup(state, buf)
    group, spec = state["group"], state["spec"]
    world = dist.get_world_size(group)
    if world == 1:
        return _done(buf)
    fmt = spec.fpx_format
    vmax = _FORMATS[fmt][2]
    index, n = bucket.index(), buf.numel()
    mus = state["params"].setdefault("fpx_mu", {})
    mu = mus.get(index, vmax / world)
    nchunk = (n + SHARED_CHUNK - 1) // SHARED_CHUNK
    x = torch.zeros(nchunk * SHARED_CHUNK, dtype=torch.float32, device=buf.device)
    x[:n] = buf.reshape(-1).float() / world
    x = x.view(nchunk, SHARED_CHUNK)
    bound = x.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    bound = torch.exp2(torch.ceil(torch.log2(bound)))  # round up to a power of two
    dist.all_reduce(bound, op=dist.ReduceOp.MAX, group=group)
    eps = 5e-7 if fmt == "fp4" else 1e-23
    scaled = (x / (bound + eps) * mu).reshape(-1)
    total = allreduce_torch(scaled, MinifloatCodec(fmt), spec.topology, group, transmit=not spec.compute_only) * world
    if fmt == "fp4":  # saturation feedback, decided from the reduced values every rank holds identically
        saturated = int((total.abs() >= vmax - 5e-8).sum())
        if saturated > total.numel() * SHARED_PROPORTION:
            mus[index] = max(mu * 0.95, vmax / world / 2)
        else:
            mus[index] = min(vmax, mu * 2 ** 0.02)
    else:
        mus[index] = mu
    out = (total.view(nchunk, SHARED_CHUNK) / mu * (bound + eps)).reshape(-1)[:n]
    buf.copy_(out.to(buf.dtype).view_as(buf))
    return _done(buf)


def fpx_hook(state, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    st = state[0] if isinstance(state, (list, tuple)) else state
    return (fpx_shared_hook if st["spec"].shared_scale else _local_scale_fpx_hook)(state, bucket)


def fwht_(x: torch.Tensor) -> torch.Tensor:
    """In-place unnormalised Walsh-Hadamard transform of the last dimension (a power of two)."""
    n = x.shape[-1]
    h = 1
    while h < n:
        y = x.view(*x.shape[:-1], n // (2 * h), 2, h)
        a, b = y[..., 0, :].clone(), y[..., 1, :]
        y[..., 0, :] = a + b
        y[..., 1, :] = a - b
        h *= 2
    return x


def _signs(n: int, seed: int, device) -> torch.Tensor:
    bits = uniform_bytes((n + 7) // 8, 0x5448, 0, seed, device)
    b = ((bits.unsqueeze(1) >> torch.arange(8, device=device)) & 1).reshape(-1)[:n]
    return 1.0 - 2.0 * b.float()


def _rotate(x: torch.Tensor) -> torch.Tensor:
    """Orthonormal Walsh-Hadamard transform of a power-of-two vector (native kernels on CUDA)."""
    if x.is_cuda:
        from ..ops.fwht import fwht_pow2

        return fwht_pow2(x, normalize=True)
    return fwht_(x) / math.sqrt(x.numel())


def _p2p_mean(state, x: torch.Tensor, wire_bits: int, spec, step: int, bucket_id: int) -> torch.Tensor:
    """In-place mean of a flat fp32 CUDA tensor over the fused kernel's identity wire (bf16 or fp32)."""
    from ..hooks import _engine

    eng = _engine(state)
    eng.allreduce_(x, wire_bits, spec.topology, state["config"].seed, step, bucket_id,
                   no_transmit=spec.compute_only, codec="cast")
    return x


def thc_hook(state, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """THC: randomized Hadamard transform of power-of-two partitions, uniform stochastic
    quantisation to `quantization_levels` bins over +-T * max||g|| / sqrt(d), bins summed exactly,
    first coordinate sent exactly (thc_hooks.py:124-324; simulation thc_hooks.py:123-339)."""
    state = _begin(state, bucket)
    buf = bucket.buffer()
    if state["batch_idx"] < state["config"].warmup_steps:
        return _warmup(state, buf)
    group, spec, cfg = state["group"], state["spec"], state["config"]
    world = dist.get_world_size(group)
    if world == 1:
        return _done(buf)
    levels = spec.quantization_levels or 31
    step, index = int(state["batch_idx"]), bucket.index()
    rank = dist.get_rank(group)
    flat = buf.reshape(-1)
    pos, part = 0, 0
    while pos < flat.numel():
        m = min(THC_MAX_PART, flat.numel() - pos)
        d = max(64, 1 << (m - 1).bit_length())
        x = torch.zeros(d, dtype=torch.float32, device=buf.device)
        x[:m] = flat[pos: pos + m].float()
        cache = state["params"].setdefault("thc_signs", {})
        s = cache.get((index, part, d))
        if s is None:  # fixed per (bucket, partition): kept as int8
            s = cache[(index, part, d)] = _signs(d, cfg.seed + 7919 * part, buf.device).to(torch.int8)
        y = _rotate(x * s)
        # rounding offsets are private to a rank (independent errors average out) and a pure function of
        # (seed, step, bucket, partition, rank) on both devices
        tag = ((index & 0xFFF) << 20) | ((part & 0xFF) << 12) | (rank & 0xFFF)
        if buf.is_cuda:
            total = _thc_partition_cuda(state, y, x, d, levels, world, rank, tag, step, index, part)
            mean = total  # dequantised in place
        else:
            norm = x.norm().reshape(1)
            dist.all_reduce(norm, op=dist.ReduceOp.MAX, group=group)
            first = y[:1].clone()
            dist.all_reduce(first, group=group)
            rng = (THC_T * norm / math.sqrt(d)).clamp_min(1e-30)
            u = (uniform_bytes(d, tag, step, cfg.seed, buf.device).float() + 0.5) / 256.0
            t = (y.clamp(-rng, rng) + rng) / (2 * rng) * (levels - 1)
            bins = torch.floor(t + u).clamp_(0, levels - 1)
            total = allreduce_torch(bins, IntBinsCodec(), spec.topology, group, transmit=not spec.compute_only) * world
            mean = (total / (levels - 1) * (2 * rng) - world * rng) / world
            mean[0] = first[0] / world
        out = _rotate(mean) * s
        flat[pos: pos + m] = out[:m].to(buf.dtype)
        pos += m
        part += 1
    return _done(buf)


def _thc_partition_cuda(state, y: torch.Tensor, x: torch.Tensor, d: int, levels: int, world: int, rank: int, tag: int,
                        step: int, index: int, part: int) -> torch.Tensor:
    """CUDA body of one THC partition, without a library collective: one small sum all-reduce of
    [||g_0||, .., ||g_{W-1}||, first coordinate] over this package's fp32 point-to-point kernel, the quantise
    kernel, the bins over the identity wire (bf16 carries sums up to 256 exactly), the dequantise kernel."""
    from .. import ops as _ops
    from ..hooks import _engine
    from ..utils import counters

    dq = _ops.require()
    spec, cfg = state["spec"], state["config"]
    eng = _engine(state)
    stats = torch.zeros(world + 1, dtype=torch.float32, device=y.device)
    stats[rank] = x.norm()
    stats[world] = y[0]
    bid = ((index & 0xFFF) << 4) | (part & 0xF)
    eng.allreduce_(stats, 32, "direct", cfg.seed, step, bid ^ 0x8000, codec="cast", post_scale=1.0)
    scale = THC_T / math.sqrt(d)
    dq.thc_quantize_(y, stats, world, scale, levels, tag, step, cfg.seed)
    counters.add("thc_quantize")
    wire = 16 if world * (levels - 1) <= 256 else 32
    eng.allreduce_(y, wire, spec.topology, cfg.seed, step, bid, no_transmit=spec.compute_only, codec="cast",
                   post_scale=1.0)
    dq.thc_dequantize_(y, stats, world, scale, levels)
    counters.add("thc_dequantize")
    return y


def _omni_union_cuda(state, rows: torch.Tensor, bitmap: torch.Tensor, k: int, world: int, index: int, params: dict):
    """CUDA body of OmniReduce without a library collective and without a device-to-host read on the step's
    path.  The bitmap is summed over this package's fp32 point-to-point kernel; the union of the ranks' rows
    (at most world * k rows) is compacted into a buffer of exactly that capacity with a prefix sum, reduced on
    the bf16 identity wire, and scattered back; rows of `rows` outside the union are zeroed in place.  The
    union's density, which steers the next steps' k, is read one step late through pinned memory.  Returns
    the density observed at an EARLIER step of this bucket (None until one has arrived)."""
    from ..hooks import _engine

    spec, cfg = state["spec"], state["config"]
    step = int(state["batch_idx"])
    eng = _engine(state)
    nrows = rows.shape[0]
    eng.allreduce_(bitmap, 32, "direct", cfg.seed, step, ((index & 0xFFF) << 4) | 1, codec="cast", post_scale=1.0)
    mask = bitmap > 0
    cap = min(nrows, world * k)
    pos = torch.cumsum(mask, 0) - 1
    slot = torch.where(mask & (pos < cap), pos, torch.full_like(pos, cap))  # row `cap` collects what is dropped
    dense = torch.zeros(cap + 1, 256, dtype=torch.float32, device=rows.device)
    dense.index_copy_(0, slot, rows)
    eng.allreduce_(dense[:cap].reshape(-1), 16, spec.topology, cfg.seed, step, (index & 0xFFF) << 4,
                   no_transmit=spec.compute_only, codec="cast")
    dense[cap].zero_()
    rows.copy_(dense.index_select(0, slot))
    # density feedback, one step late and without blocking
    pend = params.setdefault("omni_pending", {})
    seen = None
    old = pend.get(index)
    if old is not None and old[1].query():
        seen = float(old[0][0]) / nrows
        pend.pop(index)
    if index not in pend:
        host = torch.zeros(1, dtype=torch.float32).pin_memory()
        host.copy_(mask.sum().float().reshape(1), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        pend[index] = (host, ev)
    return seen


def omnireduce_hook(state, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """OmniReduce-style block sparsification: 256-element rows, local top-k rows by L2 norm, a
    bitmap all-reduce, the union of rows reduced densely in bf16, and a feedback rule that steers
    the union's density to the target (comm_hooks.py:524-678; simulation :833-986)."""
    state = _begin(state, bucket)
    buf = bucket.buffer()
    if state["batch_idx"] < state["config"].warmup_steps:
        return _warmup(state, buf)
    group, spec = state["group"], state["spec"]
    world = dist.get_world_size(group)
    if world == 1:
        return _done(buf)
    params = state["params"]
    target = float(params.get("target_topk", 0.25))
    topks = params.setdefault("local_topks", {})
    index = bucket.index()
    local = topks.get(index, target / world)
    n = buf.numel()
    nrows = (n + 255) // 256
    x = torch.zeros(nrows * 256, dtype=torch.float32, device=buf.device)
    x[:n] = buf.reshape(-1).float()
    rows = x.view(nrows, 256)
    k = max(1, min(nrows, int(round(local * nrows))))
    top = torch.topk(rows.pow(2).sum(dim=1), k).indices
    bitmap = torch.zeros(nrows, dtype=torch.float32, device=buf.device)
    bitmap[top] = 1.0
    if buf.is_cuda:
        real = _omni_union_cuda(state, rows, bitmap, k, world, index, params)
        out = rows  # reduced in place: rows outside the union are zero
    else:
        dist.all_reduce(bitmap, group=group)
        union = torch.nonzero(bitmap > 0, as_tuple=False).reshape(-1)
        out = torch.zeros_like(rows)
        if union.numel():
            dense = rows.index_select(0, union).reshape(-1)
            red = allreduce_torch(dense, CastCodec(torch.bfloat16), spec.topology, group,
                                  transmit=not spec.compute_only)
            out.index_copy_(0, union, red.view(-1, 256))
        real = union.numel() / nrows
    if real is not None:
        ratio = min(max(real / target, 0.6), 1 / 0.6)
        topks[index] = 0.75 * local + 0.25 * local / ratio
        params["last_density"] = real
    buf.copy_(out.reshape(-1)[:n].to(buf.dtype))
    return _done(buf)
