"""The reference-faithful DynamiQ path: mean-centred superchunks in 8 / 4 / 2-bit groups.

Per bucket (testbed_evaluation/new_comm_hooks/comm_hooks.py:681-780, dynamic-bitrate variant
:903-1144):

1. split into 256-element superchunks, subtract each superchunk's mean, keep
   ``stats = (mean / W, sum((x / W)^2))`` (kernel K21, cuda_hadamard.cu:1304-1349);
2. all-reduce the stats (sum) -> mean of means and the summed energies ``F_i``;
3. choose a code width per superchunk from ``F_i``: by the threshold table of the method name,
   or by the dynamic-bitrate controller (``bitalloc.py``);
4. for each non-empty group gather its rows, all-reduce them with the hierarchical AEE / MEE
   codec of that width over the method's topology, scatter them back;
5. add the mean of means back (K22, cuda_hadamard.cu:1351-1369).

On CUDA buckets everything is native and nothing is read back to the host: ``superchunk_center`` /
``superchunk_add_mean`` (csrc/kernels/superchunk_ops.cu), the widths (``superchunk_widths`` for the
dynamic-bitrate controller whose state lives on the device, an ``argsort`` with statically known group
sizes for the threshold table), ``superchunk_plan`` (block offsets of the message), and ONE launch of
the persistent fused collective kernel with the mixed-width superchunk codec
(``FusedAllreduce.allreduce_(codec="scmix_aee" | "scmix_mee", plan=...)``, csrc/common/sc_codec.cuh): the
rows stay in place instead of being gathered into three width groups and scattered back.  The
three-group form remains for the debug variants that drop groups (``fixed`` on a mixed table,
``no_compress``).  On CPU tensors (gloo) the same steps run on the device-agnostic backend
(``torch_backend.py``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import bitalloc
from .codecs import SUPERCHUNK, SuperchunkCodec
from .torch_backend import allreduce_torch


def mean_center(x: torch.Tensor, world: int):
    """x [n] -> (residual [nsc, 256] fp32, stats [nsc, 2] fp32 = (mean / W, sum((x/W)^2)))."""
    n = x.numel()
    nsc = (n + SUPERCHUNK - 1) // SUPERCHUNK
    pad = torch.zeros(nsc * SUPERCHUNK, dtype=torch.float32, device=x.device)
    pad[:n] = torch.nan_to_num(x.float(), nan=0.0, posinf=0.0, neginf=0.0)
    rows = pad.view(nsc, SUPERCHUNK)
    valid = torch.full((nsc,), SUPERCHUNK, dtype=torch.float32, device=x.device)
    if n % SUPERCHUNK:
        valid[-1] = n % SUPERCHUNK
    mean = rows.sum(dim=1) / SUPERCHUNK  # the reference averages over the padded 256 as well
    resid = rows - mean.unsqueeze(1)
    if n % SUPERCHUNK:
        resid[-1, n % SUPERCHUNK:] = 0.0  # zero padded tail (cuda_hadamard.cu:1336-1342)
    stats = torch.stack([mean / world, (rows / world).pow(2).sum(dim=1)], dim=1)
    return resid, stats


def superchunk_allreduce(state, bucket) -> torch.futures.Future:
    spec, cfg = state["spec"], state["config"]
    group = state["group"]
    world = dist.get_world_size(group)
    buf = bucket.buffer()
    n = buf.numel()
    fut = torch.futures.Future()
    if world == 1 or n == 0:
        fut.set_result(buf)
        return fut
    step, index = int(state["batch_idx"]), bucket.index()
    native = buf.is_cuda
    dropped = spec.fixed and (spec.thresholds.get(8, 0.0) > 0 or spec.thresholds.get(2, 0.0) > 0)
    if native and not spec.no_compress and not dropped:
        return _native_mixed(state, bucket)
    if native:
        from .. import ops as _ops
        from ..hooks import _engine
        from ..utils import counters

        dq = _ops.require()
        eng = _engine(state)
        flat, stats = dq.superchunk_center(buf.reshape(-1), world)
        counters.add("superchunk_center")
        resid = flat.view(-1, SUPERCHUNK)
    else:
        resid, stats = mean_center(buf, world)
    dist.all_reduce(stats, group=group)
    mean_of_means, energy = stats[:, 0], stats[:, 1]
    params = state["params"]
    if spec.dynamic_bitrate:
        ctl = params.get("bitrate")
        if ctl is None:
            ctl = params["bitrate"] = bitalloc.DynamicBitrateController(spec.bits)
            if "bitrate_u" in params:
                ctl.u, ctl.initialised = float(params["bitrate_u"]), True
        ctl.observe(energy)
        groups = bitalloc.split_by_bitrate(energy, ctl.u)
    elif spec.momentum and not spec.fixed:
        mom = params.get("momentum")
        if mom is None:
            mom = params["momentum"] = bitalloc.MomentumThresholds(spec.thresholds, energy.device)
        groups = mom.groups(energy)
    else:
        groups = bitalloc.split_by_thresholds(energy, spec.thresholds, fixed=spec.fixed)
    st = state["stats"]
    st["collectives"] += 1
    st["buckets"][index] = {"numel": n, "groups": {b: int(i.numel()) for b, i in groups.items()}}
    done = torch.zeros(resid.shape[0], dtype=torch.bool, device=resid.device)
    for gid, bits in enumerate((8, 4, 2)):
        idx = groups[bits]
        if idx.numel() == 0:
            continue
        done[idx] = True
        rows = resid.index_select(0, idx).reshape(-1)
        if spec.no_compress:
            rows = rows / world
        elif native:
            eng.allreduce_(rows, bits, spec.topology, cfg.seed, step, (index << 2) | gid,
                           no_transmit=spec.compute_only, codec=f"sc_{spec.lattice}")
        else:
            codec = SuperchunkCodec(bits, spec.lattice, cfg.seed, step, (index << 2) | gid)
            rows = allreduce_torch(rows, codec, spec.topology, group, transmit=not spec.compute_only)
        resid.index_copy_(0, idx, rows.view(-1, SUPERCHUNK))
    if not bool(done.all()):  # rows of a dropped group keep their local share, as in the reference
        resid[~done] /= world
    if native:
        dq.superchunk_add_mean(resid.reshape(-1), mean_of_means.contiguous(), buf.reshape(-1))
        counters.add("superchunk_add_mean")
    else:
        out = (resid + mean_of_means.unsqueeze(1)).reshape(-1)[:n]
        buf.copy_(out.to(buf.dtype))
    if spec.dynamic_bitrate and bucket.is_last():
        ctl = params["bitrate"]
        ctl.end_of_step()
        params["bitrate_u"] = ctl.u
        params["bitrate_last_avg_bits"] = ctl.last_avg
    if "momentum" in params and bucket.is_last():
        params["momentum"].end_of_step()
    fut.set_result(buf)
    return fut


def _native_mixed(state, bucket) -> torch.futures.Future:
    """CUDA path: centre -> all-reduce stats -> widths -> plan -> one mixed-width collective -> add mean,
    on the hook's communication stream, without a device-to-host read."""
    from .. import ops as _ops
    from ..hooks import _engine, _grid
    from ..utils import counters

    spec, cfg, group = state["spec"], state["config"], state["group"]
    world = dist.get_world_size(group)
    buf = bucket.buffer()
    step, index = int(state["batch_idx"]), bucket.index()
    dq = _ops.require()
    eng = _engine(state)
    stream = state["comm_stream"]
    stream.wait_stream(torch.cuda.current_stream(buf.device))
    fut = torch.futures.Future(devices=[buf.device])
    params = state["params"]
    with torch.cuda.stream(stream):
        flat, stats = dq.superchunk_center(buf.reshape(-1), world)
        counters.add("superchunk_center")
        # (mean, energy) per superchunk, summed over the ranks by this package's own point-to-point kernel on
        # the fp32 identity wire: no library collective on the hook's path
        eng.allreduce_(stats.view(-1), 32, "direct", cfg.seed, step, (index << 2) | 2, codec="cast", post_scale=1.0)
        if spec.dynamic_bitrate:
            ctl = params.get("bitrate")
            if ctl is None:
                ctl = params["bitrate"] = bitalloc.DeviceBitrateController(
                    spec.bits, buf.device, u=float(params.get("bitrate_u", bitalloc.U_MAX)),
                    initialised="bitrate_u" in params)
            widths = ctl.widths(stats)
            counters.add("superchunk_widths")
        elif spec.momentum and not spec.fixed:
            mom = params.get("momentum")
            if mom is None:
                mom = params["momentum"] = bitalloc.MomentumThresholds(spec.thresholds, buf.device)
            widths = mom.widths(stats[:, 1])
        else:
            widths = bitalloc.threshold_widths(stats[:, 1], spec.thresholds)
        plan = dq.superchunk_plan(widths)
        counters.add("superchunk_plan")
        eng.allreduce_(flat, 8, spec.topology, cfg.seed, step, (index << 2) | 3, no_transmit=spec.compute_only,
                       codec=f"scmix_{spec.lattice}", plan=plan, ctas=_grid(state, bucket),
                       wire_bits=float(spec.bits))  # nominal: the realised mixture depends on the data
        dq.superchunk_add_mean(flat, stats[:, 0].contiguous(), buf.reshape(-1))
        counters.add("superchunk_add_mean")
        st = state["stats"]
        st["collectives"] += 1
        st["buckets"][index] = {"numel": buf.numel(), "mixed_widths": True}
        if spec.dynamic_bitrate and bucket.is_last():
            ctl.end_of_step()
            counters.add("superchunk_bitrate_update")
        if "momentum" in params and bucket.is_last():
            params["momentum"].end_of_step()
        buf.record_stream(stream)
        fut.set_result(buf)
    return fut
