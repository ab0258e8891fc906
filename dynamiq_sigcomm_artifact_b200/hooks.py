"""DDP communication hooks with the reference's contract.

Contract (testbed_evaluation/new_comm_hooks/comm_hooks.py:681-900, smoke_test_new_comm_hooks.py:303-326):
``hook(state, bucket) -> Future[Tensor]`` where ``state`` is a *list holding one dict*, the
future's value is the bucket's flat tensor holding the **mean** gradient, the caller advances
``state["batch_idx"]`` before each backward, and the first steps (``batch_idx`` 0 and 1 in
the reference) are served by the library all-reduce while DDP settles its buckets.

What differs: the custom path is one fused kernel per bucket launched on a side stream
(so bucket k's collective overlaps the backward of bucket k+1) instead of Python-driven
ring steps executed synchronously in the reducer callback (comm_hooks.py:892-900); buckets
can therefore stay at DDP's 25 MB instead of one 4000 MiB bucket (train_llm_causal.py:216,416).
On CPU tensors (gloo) the same programs run through ``parallel/cpu_backend.py``.
"""
import time
from typing import Callable, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from .config import DynamiqConfig, MethodSpec, parse_method
from .utils import tracing


class HookState(dict):
    """The mutable dict the hooks read; ``[state]`` is what ``register_comm_hook`` receives.

    Keys kept from the reference: ``batch_idx``, ``params`` (scratch), ``args``.  New keys:
    ``spec``, ``config``, ``engine``, ``stats``.
    """

    def __init__(self, config: DynamiqConfig, group=None):
        super().__init__()
        self["config"] = config
        self["spec"] = config.spec()
        self["batch_idx"] = 0
        self["params"] = {}
        self["args"] = config
        self["group"] = group
        self["engine"] = None
        self["comm_stream"] = None
        self["auto_step"] = True
        self["stats"] = {"buckets": {}, "collectives": 0, "wire_bytes": 0, "err_sq": 0.0, "ref_sq": 0.0}
        self["_seen_first"] = False

    # -- step accounting -------------------------------------------------------------------
    def begin_step(self, batch_idx: Optional[int] = None) -> None:
        """Call before each backward (the reference's ``state["batch_idx"] += 1``)."""
        self["auto_step"] = False
        self["batch_idx"] = self["batch_idx"] + 1 if batch_idx is None else int(batch_idx)

    def _auto_advance(self, bucket_index: int) -> None:
        if self["auto_step"] and bucket_index == 0:
            if self["_seen_first"]:
                self["batch_idx"] += 1
            self["_seen_first"] = True

    # -- persistence (hook state is never saved by the reference; see checkpoint.py) ---------
    def state_dict(self) -> dict:
        d = {"batch_idx": self["batch_idx"], "method": self["config"].method, "seed": self["config"].seed,
             "stats": {k: v for k, v in self["stats"].items() if k != "buckets"}}
        plans = self["params"].get("rht_plans")
        if plans:  # per-block widths of the rotation codec (mixed methods): needed to resume bit for bit
            d["rht_plans"] = {int(k): (v.cpu() if torch.is_tensor(v) else torch.as_tensor(v)) for k, v in plans.items()}
        ctl = self["params"].get("bitrate")
        if ctl is not None and hasattr(ctl, "state_dict"):
            sd = ctl.state_dict()
            if sd.get("initialised"):
                self["params"]["bitrate_u"] = sd["u"]
        for k in ("bitrate_u",):
            if k in self["params"]:
                d[k] = self["params"][k]
        return d

    def load_state_dict(self, d: dict) -> None:
        self["batch_idx"] = int(d["batch_idx"])
        self["auto_step"] = False
        if "rht_plans" in d:
            self["params"]["rht_plans_restored"] = {int(k): v for k, v in d["rht_plans"].items()}
        for k in ("bitrate_u",):
            if k in d:
                self["params"][k] = d[k]

    def close(self) -> None:
        if self["engine"] is not None:
            self["engine"].close()
            self["engine"] = None
        if self.get("nvls") is not None:
            self["nvls"].close()
            self["nvls"] = None


def _unwrap(state) -> HookState:
    return state[0] if isinstance(state, (list, tuple)) else state


def _world(state: HookState) -> int:
    return dist.get_world_size(state["group"]) if dist.is_initialized() else 1


def _library_mean(state: HookState, buf: torch.Tensor, wire_dtype: Optional[torch.dtype] = None
                  ) -> torch.futures.Future:
    """Mean through the library all-reduce, optionally casting the wire to `wire_dtype`."""
    world = _world(state)
    if world == 1:
        fut = torch.futures.Future()
        fut.set_result(buf)
        return fut
    if wire_dtype is None or wire_dtype == buf.dtype:
        buf.div_(world)
        return dist.all_reduce(buf, group=state["group"], async_op=True).get_future().then(lambda f: f.value()[0])
    wire = buf.to(wire_dtype).div_(world)
    fut = dist.all_reduce(wire, group=state["group"], async_op=True).get_future()

    def back(f):
        buf.copy_(f.value()[0])
        return buf

    return fut.then(back)


def _done(buf: torch.Tensor) -> torch.futures.Future:
    fut = torch.futures.Future()
    fut.set_result(buf)
    return fut


def widest_wire(spec: MethodSpec) -> tuple:
    """(bits, codec) of the largest message per element that `spec` can put on the wire."""
    if spec.hook in ("dynamiq", "dynamiq_bitrate"):
        if spec.family == "rht":
            return (8, "rht_mix") if spec.mixed else (spec.bits, "rht")
        return (8, "scmix_" + spec.lattice)  # records of per-superchunk width: sized for the widest
    if spec.hook == "mxfp8":
        return (8, "mx")
    if spec.hook == "fpx":
        return (max(spec.bits, 4), "mx")
    if spec.hook in ("bf16", "omnireduce"):
        return (16, "cast")
    return (32, "cast")


def note_bucket(state: HookState, buf: torch.Tensor) -> None:
    """Remember the largest bucket seen; the library-served warm-up steps see every bucket of the model, so
    the engine created afterwards is sized once and never re-allocates inside a training step."""
    if buf.numel() > state.get("max_bucket_numel", 0):
        state["max_bucket_numel"] = buf.numel()


def _engine(state: HookState):
    """The NVLink engine, created on first use (a collective call: every rank gets here together).  Its
    mailbox is sized for the largest bucket seen so far (or announced through ``state["max_bucket_numel"]``
    by the bucket reducer) on the widest wire the method can select."""
    if state["engine"] is None:
        from .parallel.fused import FusedAllreduce

        cfg: DynamiqConfig = state["config"]
        numel = int(state.get("max_bucket_numel", 0)) or cfg.max_bucket_mb * (1 << 20) // 4
        state["engine"] = FusedAllreduce(group=state["group"], max_numel=numel,
                                         ctas=cfg.comm_ctas, threads=cfg.comm_threads,
                                         timeout_ms=cfg.wait_timeout_ms, validate=cfg.validate_topology,
                                         rotation=cfg.rotation, max_ctas=max(cfg.comm_ctas, cfg.tail_ctas),
                                         prefetch=cfg.comm_prefetch, widest=widest_wire(state["spec"]),
                                         debug=cfg.debug)
        state["engine"].stats_sink = state["stats"]  # every collective adds the bytes it puts on the wire
        state["comm_stream"] = torch.cuda.Stream(priority=-1)
    return state["engine"]


def _nvls(state: HookState, numel: int, wire_bits: int):
    """The in-switch (NVLS) all-reduce engine for the uncompressed wires, or None: off by configuration
    (``use_nvls``), no multicast support on this box, two ranks only (nothing to reduce inside the switch), or a
    bucket larger than its staging buffer.  Created once, sized for the largest bucket seen."""
    cfg: DynamiqConfig = state["config"]
    if not cfg.use_nvls or _world(state) <= 2:
        return None
    eng = state.get("nvls")
    if eng is None:
        from .parallel.nvls import NvlsAllreduce

        cap = max(int(state.get("max_bucket_numel", 0)), numel)
        eng = state["nvls"] = NvlsAllreduce(group=state["group"], max_numel=cap, wire_bits=32,
                                            timeout_ms=cfg.wait_timeout_ms)
        if not eng.available and dist.get_rank(state["group"]) == 0:
            print(f"[dynamiq] NVLS all-reduce not used: {eng.reason}", flush=True)
    return eng if eng.fits(numel, wire_bits) else None


def _grid(state: HookState, bucket) -> Optional[int]:
    """The step's last bucket has no backward pass left to share the GPU with: give it the wide grid."""
    cfg: DynamiqConfig = state["config"]
    if cfg.tail_ctas > 0 and (bucket.is_last() or getattr(bucket, "exposed", False)):
        return cfg.tail_ctas
    return None


def _mixed_plan(state: HookState, index: int, numel: int, device) -> torch.Tensor:
    """The width plan of bucket `index` (int32 [2 nblocks + 1]: offsets, then widths): what the previous
    collective of this bucket derived, the restored one after a resume, or every block at the nominal width."""
    from .parallel.fused import BLOCK, uniform_plan

    plans = state["params"].setdefault("rht_plans", {})
    nb = (numel + BLOCK - 1) // BLOCK
    plan = plans.get(index)
    if plan is None or plan.numel() != 2 * nb + 1:
        restored = state["params"].get("rht_plans_restored", {}).pop(index, None)
        if restored is not None and restored.numel() == 2 * nb + 1:
            plan = restored.to(device=device, dtype=torch.int32)
        else:
            plan = uniform_plan(numel, state["spec"].bits, device)
        plans[index] = plan
    return plan


def _rht_allreduce(state: HookState, bucket) -> torch.futures.Future:
    spec: MethodSpec = state["spec"]
    cfg: DynamiqConfig = state["config"]
    buf = bucket.buffer()
    index, step = bucket.index(), int(state["batch_idx"])
    world = _world(state)
    if world == 1 or buf.numel() == 0:
        return _done(buf)
    bits = spec.bits
    st = state["stats"]
    st["collectives"] += 1
    st["buckets"][index] = {"numel": buf.numel(), "bits": bits, "mixed": spec.mixed}
    exact = None
    if cfg.measure_comm_error:
        exact = buf.detach().clone().float()
        dist.all_reduce(exact, group=state["group"])
        exact.div_(world)
    if buf.is_cuda:
        eng = _engine(state)
        if spec.mixed and eng.tensor_rotation:
            raise ValueError("a code width per block needs rotation='simt' (DQ_ROTATION)")

        def launch(grid):
            if spec.mixed:  # one collective with a width per block, then the next step's widths from its scales
                plan = _mixed_plan(state, index, buf.numel(), buf.device)
                eng.allreduce_(buf, 8, spec.topology, cfg.seed, step, index, no_transmit=spec.compute_only,
                               correlated=spec.correlated, codec="rht_mix", plan=plan, ctas=grid,
                               wire_bits=float(bits))  # the width policy meets `bits` on average
                if not spec.compute_only:
                    eng.update_widths_(plan, buf.numel(), float(bits))
            else:
                eng.allreduce_(buf, bits, spec.topology, cfg.seed, step, index, no_transmit=spec.compute_only,
                               correlated=spec.correlated, ctas=grid)

        if cfg.overlap:
            stream = state["comm_stream"]
            stream.wait_stream(torch.cuda.current_stream())
            fut = torch.futures.Future(devices=[buf.device])
            with torch.cuda.stream(stream), tracing.nvtx_range(f"bucket{index}.fused_{spec.topology}_{bits}bit"):
                launch(_grid(state, bucket))
                buf.record_stream(stream)
                if exact is not None:
                    _account_error(state, buf, exact)
                fut.set_result(buf)
            return fut
        launch(None)
    else:
        from .parallel import cpu_backend as cb

        factory, made = None, {}
        if spec.mixed:
            nb = (buf.numel() + 1023) // 1024
            widths = state["params"].setdefault("rht_widths", {}).get(index)
            if widths is None or len(widths) != nb:
                widths = np.full(nb, bits, dtype=np.uint8)

            def factory(_bits, seed, step_, bucket_, world_, rank_):
                made["codec"] = cb.RhtMixCodecCPU(widths, seed, step_, bucket_, world_, rank_)
                return made["codec"]

        out = cb.allreduce_gloo(buf.detach().float().numpy(), bits, spec.topology, cfg.seed, step, index,
                                group=state["group"], correlated=spec.correlated, codec_factory=factory)
        from .parallel.fused import wire_bytes_per_rank

        st["wire_bytes"] += wire_bytes_per_rank(buf.numel(), world, float(bits), "rht_mix" if spec.mixed else "rht")
        if spec.mixed:
            from . import bitalloc

            state["params"]["rht_widths"][index] = bitalloc.rht_block_widths(made["codec"].block_absmax(nb), bits)[0]
        buf.copy_(torch.from_numpy(out).to(buf.dtype))
    if exact is not None:
        _account_error(state, buf, exact)
    return _done(buf)


def _account_error(state: HookState, got: torch.Tensor, exact: torch.Tensor) -> None:
    """vNMSE bookkeeping (simulations_llm/new_comm_hooks/comm_hooks.py:1167-1198)."""
    st = state["stats"]
    st["err_sq"] += float((got.float() - exact).pow(2).sum())
    st["ref_sq"] += float(exact.pow(2).sum())


def dynamiq_hook(state, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """`dynamiQ_*` methods: rotation codec (`rht`) or the reference's superchunk codec."""
    state = _unwrap(state)
    state._auto_advance(bucket.index())
    note_bucket(state, bucket.buffer())
    if state["batch_idx"] < state["config"].warmup_steps:
        return _library_mean(state, bucket.buffer())
    if state["spec"].family == "superchunk":
        from .parallel.superchunk import superchunk_allreduce

        return superchunk_allreduce(state, bucket)
    if state["spec"].family == "sim":
        return _sim_allreduce(state, bucket)
    return _rht_allreduce(state, bucket)


def _sim_allreduce(state: HookState, bucket) -> torch.futures.Future:
    """``dynamiQ_{aee,mee}_{b}bit_sim``: the simulation stack's hierarchical compressor over the step programs,
    executed with tensor operators on whatever device the bucket lives on (numerics study, not a fast path)."""
    from .parallel.codecs import SimHierarchicalCodec
    from .parallel.torch_backend import allreduce_torch

    spec, cfg = state["spec"], state["config"]
    buf = bucket.buffer()
    world = _world(state)
    if world == 1 or buf.numel() == 0:
        return _done(buf)
    codec = SimHierarchicalCodec(spec.bits, spec.lattice, seed=cfg.seed, step=int(state["batch_idx"]),
                                 bucket=bucket.index())
    n = buf.numel()
    pad = (-n) % (codec.align * world)
    x = torch.zeros(n + pad, dtype=torch.float32, device=buf.device)
    x[:n] = buf.reshape(-1).float()
    out = allreduce_torch(x, codec, spec.topology, state["group"], transmit=not spec.compute_only)
    buf.copy_(out[:n].to(buf.dtype).view_as(buf))
    state["stats"]["collectives"] += 1
    return _done(buf)


def _cast_hook(dtype: Optional[torch.dtype]) -> Callable:
    def hook(state, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
        state = _unwrap(state)
        state._auto_advance(bucket.index())
        return _library_mean(state, bucket.buffer(), dtype)

    return hook


def bf16_hook(state, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """bf16 wire.  On CUDA: this framework's own point-to-point all-reduce (the fused kernel with the
    identity codec, no library collective), as the reference's bf16 method is its own ring carrying
    bf16 (testbed_evaluation/new_comm_hooks/comm_hooks.py:175-212).  ``DQ_BF16_LIBRARY=1`` or a CPU
    bucket selects the library all-reduce with a bf16 cast instead."""
    import os

    state = _unwrap(state)
    state._auto_advance(bucket.index())
    buf = bucket.buffer()
    note_bucket(state, buf)
    world = _world(state)
    use_p2p = (buf.is_cuda and world > 1 and buf.dtype in (torch.float32, torch.bfloat16)
               and os.environ.get("DQ_BF16_LIBRARY", "0") not in ("1", "true")
               and state["batch_idx"] >= state["config"].warmup_steps)
    if not use_p2p:
        return _library_mean(state, buf, torch.bfloat16)
    spec, cfg = state["spec"], state["config"]
    eng = _engine(state)  # also owns the side stream
    nvls = _nvls(state, buf.numel(), 16) if not spec.compute_only else None
    stream = state["comm_stream"]
    stream.wait_stream(torch.cuda.current_stream())
    fut = torch.futures.Future(devices=[buf.device])
    with torch.cuda.stream(stream), tracing.nvtx_range(f"bucket{bucket.index()}.p2p_bf16_{spec.topology}"):
        if nvls is not None:  # in-switch reduction on the bf16 wire
            nvls.allreduce_(buf.reshape(-1), 16, ctas=_grid(state, bucket) or cfg.comm_ctas)
        else:
            eng.allreduce_(buf.reshape(-1), 16, spec.topology, cfg.seed, int(state["batch_idx"]), bucket.index(),
                           no_transmit=spec.compute_only, codec="cast", ctas=_grid(state, bucket))
        buf.record_stream(stream)
        fut.set_result(buf)
    return fut
fp16_hook = _cast_hook(torch.float16)
fp32_hook = _cast_hook(None)


def select_comm_hook(method: str, topology: Optional[str] = None) -> Callable:
    """Hook function for an ``aggregation_method`` string (train_llm_causal.py:294-314)."""
    spec = parse_method(method, topology)
    if spec.hook in ("dynamiq", "dynamiq_bitrate"):
        return dynamiq_hook
    if spec.hook == "bf16":
        return bf16_hook
    if spec.hook == "fp16":
        return fp16_hook
    if spec.hook == "fp32":
        return fp32_hook
    from .parallel import baselines

    return {"mxfp8": baselines.mxfp8_hook, "fpx": baselines.fpx_hook, "thc": baselines.thc_hook,
            "omnireduce": baselines.omnireduce_hook}[spec.hook]


def build_comm_state(config: DynamiqConfig, group=None) -> List[HookState]:
    """``[state]`` as the reference's ``build_comm_state`` returns it (train_llm_causal.py:242-286)."""
    return [HookState(config, group)]


def register(model, method: str = "dynamiQ_aee_5bit", config: Optional[DynamiqConfig] = None, group=None,
             **overrides) -> HookState:
    """Register the hook for `method` on a DDP model; returns the state (call ``begin_step``)."""
    cfg = config or DynamiqConfig.from_env(method=method, **overrides)
    cfg.method = method
    state_list = build_comm_state(cfg, group)
    model.register_comm_hook(state_list, select_comm_hook(method, cfg.topology))
    return state_list[0]
