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
fpx_hook = _block_float_hook(lambda spec: spec.fpx_format)


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
        norm = x.norm().reshape(1)
        dist.all_reduce(norm, op=dist.ReduceOp.MAX, group=group)
        first = y[:1].clone()
        dist.all_reduce(first, group=group)
        rng = (THC_T * norm / math.sqrt(d)).clamp_min(1e-30)
        if buf.is_cuda:  # rounding offsets are private to a rank: the device generator is enough
            u = torch.rand(d, device=buf.device)
        else:
            u = (uniform_bytes(d, ((index & 0xFFFF) << 16) | part, step, cfg.seed, buf.device).float() + 0.5) / 256.0
        t = (y.clamp(-rng, rng) + rng) / (2 * rng) * (levels - 1)
        bins = torch.floor(t + u).clamp_(0, levels - 1)
        if bins.is_cuda:
            # integer bins over this package's point-to-point kernel: bf16 carries sums up to 256 exactly
            wire = 16 if world * (levels - 1) <= 256 else 32
            total = _p2p_mean(state, bins, wire, spec, step, ((index & 0xFFF) << 4) | (part & 0xF)) * world
        else:
            total = allreduce_torch(bins, IntBinsCodec(), spec.topology, group, transmit=not spec.compute_only) * world
        mean = (total / (levels - 1) * (2 * rng) - world * rng) / world
        mean[0] = first[0] / world
        out = _rotate(mean) * s
        flat[pos: pos + m] = out[:m].to(buf.dtype)
        pos += m
        part += 1
    return _done(buf)


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
    dist.all_reduce(bitmap, group=group)
    union = torch.nonzero(bitmap > 0, as_tuple=False).reshape(-1)
    out = torch.zeros_like(rows)
    if union.numel():
        dense = rows.index_select(0, union).reshape(-1)
        if dense.is_cuda:
            red = _p2p_mean(state, dense, 16, spec, int(state["batch_idx"]), index)
        else:
            red = allreduce_torch(dense, CastCodec(torch.bfloat16), spec.topology, group,
                                  transmit=not spec.compute_only)
        out.index_copy_(0, union, red.view(-1, 256))
    real = union.numel() / nrows
    ratio = min(max(real / target, 0.6), 1 / 0.6)
    topks[index] = 0.75 * local + 0.25 * local / ratio
    params["last_density"] = real
    buf.copy_(out.reshape(-1)[:n].to(buf.dtype))
    return _done(buf)
