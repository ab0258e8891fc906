"""Standalone all-reduce benchmark: library fp32 / bf16 against the fused compressed collectives.

Multi-GPU (one rank per GPU):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m dynamiq_sigcomm_artifact_b200.train.bench_allreduce --sizes-mb 1,16,256 --bits 4,5,8

Single GPU, kernel throughput of the codec stages (the reference's kernel benchmark,
cuda_kernels/tests/benchmark_scaling_quantization.py:41-112):

    python -m dynamiq_sigcomm_artifact_b200.train.bench_allreduce --kernels --numel 268435456

Protocol (rdma_comm_compress/sample_allreduce.py:688-739): warm-up iterations, then timed
iterations of ``work.copy_(base); allreduce_(work)``, MAX over ranks; here timed on the device
with CUDA events and with the copy outside the timed interval.  ``algbw = 2(W-1)/W * input
bytes / t`` as in the reference (:721-727); ``wire_gbs`` counts the bytes that really cross
NVLink per GPU and direction.  Inputs: N(0,1) with a lognormal (sigma 2) scale per 1024-element
block, seeded per rank.  NMSE is against the exact fp64 mean.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..parallel import schedules as sch
from ..parallel.fused import BLOCK, FusedAllreduce, Layout, LocalCluster

NVLINK_NOMINAL_GBS = 900.0  # NVLink 5, per direction per GPU; replaced by --peer-copy's measurement
HBM_GBS_FALLBACK = 6650.0


def measure_peer_copy(eng: FusedAllreduce, nbytes: int = 256 << 20, iters: int = 10) -> float:
    """GB/s of a device-to-device copy out of the NEXT rank's symmetric buffer into local memory, all ranks
    copying at once (every link direction loaded): the link bandwidth a kernel's peer traffic can hope for.
    MAX time over the ranks, CUDA events."""
    from .. import ops as _ops

    dq = _ops.require()
    world, rank = eng.world, eng.rank
    nbytes = min(nbytes, eng.buf.nbytes // 4096 * 4096)
    peer = dq.wrap_ptr(eng.buf.ptrs[(rank + 1) % world], nbytes, eng.device)
    dst = torch.empty(nbytes, dtype=torch.uint8, device=peer.device)
    for _ in range(3):
        dst.copy_(peer)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        dst.copy_(peer)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return nbytes / float(t[0]) / 1e6


def measured_peaks() -> dict:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return json.load(f)
    except OSError:
        return {}


def make_input(numel: int, rank: int, seed: int, device) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    x = torch.randn(numel, generator=g, device=device)
    nb = (numel + BLOCK - 1) // BLOCK
    s = torch.exp(2.0 * torch.randn(nb, generator=g, device=device))
    return x * s.repeat_interleave(BLOCK)[:numel]


def time_op(fn, prepare, iters: int, warmup: int, reps: int = 1) -> float:
    """Mean device milliseconds of fn(); prepare() runs before each timed interval, outside it.
    With reps > 1 an interval holds that many back-to-back calls (the device stays busy, so the
    host's launch latency is not part of the figure) and the result is per call."""
    for _ in range(warmup):
        prepare()
        fn()
    samples = []
    for _ in range(iters):
        prepare()
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        samples.append(e0.elapsed_time(e1) / reps)
    t = torch.tensor(samples, dtype=torch.float64)
    if dist.is_initialized():  # every sample is the slowest rank's
        t = t.cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t = t.cpu()
    global LAST_SPREAD
    LAST_SPREAD = {"median_ms": float(t.median()), "min_ms": float(t.min()), "max_ms": float(t.max()), "iters": iters}
    return float(t.mean())


LAST_SPREAD: dict = {}


def nmse_vs(exact: torch.Tensor, got: torch.Tensor) -> float:
    return float(((got.double() - exact) ** 2).sum() / (exact ** 2).sum())


def run_collectives(args) -> None:
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))))
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    sizes = [int(float(s) * (1 << 20)) // 4 for s in args.sizes_mb.split(",")]
    bits_list = [int(b) for b in args.bits.split(",")]
    topologies = args.topologies.split(",")
    eng = FusedAllreduce(max_numel=max(sizes), ctas=args.ctas, threads=args.threads, timeout_ms=5000,
                         rotation=args.rotation)
    link_gbs, link_kind = NVLINK_NOMINAL_GBS, "nominal"
    if args.peer_copy:
        link_gbs, link_kind = measure_peer_copy(eng), "measured"
        if rank == 0:
            print(json.dumps({"peer_copy_gbs_per_direction": link_gbs, "world": world,
                              "how": "device-to-device copy of 256 MB out of the next rank's buffer, all ranks at once"}),
                  flush=True)
    nvls = None
    if not args.no_nvls and world > 1:
        from ..parallel.nvls import NvlsAllreduce

        nvls = NvlsAllreduce(max_numel=max(sizes), wire_bits=32, ctas=148, timeout_ms=5000)
        if rank == 0 and not nvls.available:
            print(json.dumps({"nvls": "unavailable", "reason": nvls.reason}), flush=True)
    rows = []
    for numel in sizes:
        base = make_input(numel, rank, args.seed, dev)
        exact = base.double().clone()
        dist.all_reduce(exact)
        exact /= world
        work = torch.empty_like(base)
        in_bytes = numel * 4

        def record(name, ms, wire_bytes, err, extra=None):
            row = {"method": name, "world": world, "numel": numel, "input_mb": in_bytes / 2 ** 20, "ms": ms,
                   "algbw_gbs": 2 * (world - 1) / world * in_bytes / ms / 1e6,
                   "input_gbs": in_bytes / ms / 1e6, "wire_gbs": wire_bytes / ms / 1e6,
                   f"link_fraction_of_{link_kind}": wire_bytes / ms / 1e6 / link_gbs, "nmse": err, **LAST_SPREAD}
            row.update(extra or {})
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)

        # library baselines
        def nccl32():
            dist.all_reduce(work)
            work.div_(world)

        ms = time_op(nccl32, lambda: work.copy_(base), args.iters, args.warmup)
        record("nccl_fp32", ms, 2 * (world - 1) / world * in_bytes, nmse_vs(exact, work))
        wb = torch.empty(numel, dtype=torch.bfloat16, device=dev)

        def nccl16():
            wb.copy_(work)
            dist.all_reduce(wb)
            work.copy_(wb)
            work.div_(world)

        ms = time_op(nccl16, lambda: work.copy_(base), args.iters, args.warmup)
        record("nccl_bf16", ms, 2 * (world - 1) / world * numel * 2, nmse_vs(exact, work))
        # this framework's own point-to-point all-reduce of uncompressed values (identity codec)
        for cbits, label in ((16, "p2p_bf16"), (32, "p2p_fp32")):
            it0 = [0]

            def p2p():
                it0[0] += 1
                eng.allreduce_(work, cbits, "direct", seed=args.seed, step=it0[0], bucket_id=0, codec="cast")

            ms = time_op(p2p, lambda: work.copy_(base), args.iters, args.warmup)
            eng.check()
            lay = Layout(numel, world, cbits, "cast")
            record(f"{label}_direct", ms, 2 * (world - 1) * lay.blocks_per_shard * 128 * cbits, nmse_vs(exact, work))
        # in-switch reduction (NVLS) on the same wires, when the box exposes a multicast object
        if nvls is not None and nvls.available:
            for cbits, label in ((16, "nvls_bf16"), (32, "nvls_fp32")):
                ms = time_op(lambda: nvls.allreduce_(work, cbits), lambda: work.copy_(base), args.iters, args.warmup)
                nvls.check()
                record(label, ms, 2 * numel * cbits // 8, nmse_vs(exact, work))
        for topo in topologies:
            if topo == "butterfly" and world & (world - 1):
                continue
            for bits in bits_list:
                lay = Layout(numel, world, bits)
                shard_bytes = lay.blocks_per_shard * (128 * bits + 4)
                wire = 2 * (world - 1) * shard_bytes  # per GPU, each direction
                it = [0]

                def fused():
                    it[0] += 1
                    eng.allreduce_(work, bits, topo, seed=args.seed, step=it[0], bucket_id=0)

                ms = time_op(fused, lambda: work.copy_(base), args.iters, args.warmup)
                eng.check()
                hbm = measured_peaks().get("hbm_gbs", HBM_GBS_FALLBACK)
                t_link = wire / (link_gbs * 1e6)
                t_hbm = (2 * in_bytes + 3 * wire) / (hbm * 1e6)
                record(f"fused_{topo}_{bits}bit" + ("_tc" if args.rotation == "tc" else ""), ms, wire, nmse_vs(exact, work),
                       {"roofline_ms": max(t_link, t_hbm), "roofline_fraction": max(t_link, t_hbm) / ms,
                        "bound": "nvlink" if t_link > t_hbm else "hbm", "link_gbs": link_gbs, "link": link_kind})
        # whole communication hooks by method name on the same tensor (the counterpart of the reference arm's rows):
        # what a training step pays per bucket, statistics passes and width policies included
        for method in [m for m in args.hook_methods.split(",") if m]:
            from .. import hooks as _hooks
            from ..config import DynamiqConfig
            from ..parallel.reducer import FlatBucket

            dcfg = DynamiqConfig.from_env(method=method, seed=args.seed, comm_ctas=args.ctas, comm_threads=args.threads,
                                          tail_ctas=args.ctas)
            state = _hooks.build_comm_state(dcfg)[0]
            hook = _hooks.select_comm_hook(method, dcfg.topology)
            _hooks.note_bucket(state, work)
            bucket = FlatBucket(0, work, [], True)
            step = [dcfg.warmup_steps]

            def run_hook():
                state.begin_step(step[0])  # past the library-served warm-up steps from the first call on
                step[0] += 1
                hook([state], bucket).wait()

            ms = time_op(run_hook, lambda: work.copy_(base), args.iters, max(args.warmup, 3))
            if state["engine"] is not None:
                state["engine"].check()
            spread = dict(LAST_SPREAD)
            err = nmse_vs(exact, work)
            sent = state["stats"]["wire_bytes"]  # bytes of ONE more call (statistics collectives included)
            work.copy_(base)
            run_hook()
            torch.cuda.synchronize()
            sent = state["stats"]["wire_bytes"] - sent
            LAST_SPREAD.update(spread)
            spec = state["spec"]
            record(f"hook_{method}", ms, float(sent), err,
                   {"family": spec.family, "hook": spec.hook, "topology": spec.topology})
            state.close()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    eng.close()
    dist.destroy_process_group()


def run_kernels(args) -> None:
    """Codec stages on one GPU: encode, hop (decode + add + encode), decode; bytes over HBM."""
    dev = torch.device("cuda", 0)
    numel = args.numel
    hbm = measured_peaks().get("hbm_gbs", HBM_GBS_FALLBACK)
    x = make_input(numel, 0, args.seed, dev)
    rows = []
    for bits in [int(b) for b in args.bits.split(",")]:
        cl = LocalCluster(1, numel, ctas=args.ctas, threads=args.threads, device=dev, rotation=args.rotation)
        lay = Layout(numel, 1, bits)
        work = torch.empty_like(x)
        msg = lay.nblocks * (128 * bits + 4)
        progs = {
            "encode": (sch.Step(shard=0, out=sch.OUT_SEND, dst=0, send_slot=0, tag=sch.TAG_ENCODE), 4 * numel + msg),
            "hop": (sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_SEND, dst=0, send_slot=1,
                             tag=sch.TAG_ENCODE + 1), 4 * numel + 2 * msg),
            "decode": (sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_DECODE), 4 * numel + msg),
            "final": (sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_FINAL, tag=sch.TAG_FINAL, send_slot=1),
                      8 * numel + msg),
        }
        for name, (step, nbytes) in progs.items():
            if args.stages and name not in args.stages.split(","):
                continue
            prog = torch.tensor([[step.as_ints()]], dtype=torch.int32)
            ms = time_op(lambda: cl.run([work], prog, bits, seed=args.seed, preset_flags=True),
                         lambda: work.copy_(x), args.iters, args.warmup, args.reps)
            cl.check()
            row = {"kernel": f"rht_{name}", "bits": bits, "numel": numel, "ms": ms, "gbs": nbytes / ms / 1e6,
                   "gelem_s": numel / ms / 1e6, "hbm_fraction_of_measured": nbytes / ms / 1e6 / hbm,
                   "ctas": args.ctas, "threads": args.threads, "rotation": args.rotation, "reps": args.reps}
            rows.append(row)
            print(json.dumps(row), flush=True)
    if args.rht_only:
        if args.out:
            with open(args.out, "w") as f:
                json.dump(rows, f, indent=1)
        return
    from ..ops import require

    dq = require()
    # the other wire codecs of the same kernel: superchunk records with a width per superchunk (the
    # reference's 5-bit threshold mixture), block-float fp8, the bf16 identity wire
    nsc = (numel + 255) // 256
    g = torch.Generator().manual_seed(args.seed)
    wsel = torch.rand(nsc, generator=g)
    widths = torch.where(wsel < 0.35, 8, torch.where(wsel < 0.80, 4, 2)).to(torch.uint8).to(dev)
    plan = dq.superchunk_plan(widths)
    wire_mix = float(plan[(nsc + 3) // 4].item()) * 8.0  # bytes of the whole mixed message
    cl = LocalCluster(1, numel, ctas=args.ctas, threads=args.threads, device=dev)
    work = torch.empty_like(x)
    for codec, cbits, msg, kw in (("scmix_mee", 8, wire_mix, {"plan": plan}), ("mx", 8, numel * 1.03125, {}),
                                  ("cast", 16, numel * 2.0, {})):
        progs = {
            "encode": (sch.Step(shard=0, out=sch.OUT_SEND, dst=0, send_slot=0, tag=sch.TAG_ENCODE), 4 * numel + msg),
            "hop": (sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_SEND, dst=0, send_slot=1,
                             tag=sch.TAG_ENCODE + 1), 4 * numel + 2 * msg),
            "decode": (sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_DECODE), 4 * numel + msg),
        }
        for name, (step, nbytes) in progs.items():
            prog = torch.tensor([[step.as_ints()]], dtype=torch.int32)
            ms = time_op(lambda: cl.run([work], prog, cbits, seed=args.seed, preset_flags=True, codec=codec, **kw),
                         lambda: work.copy_(x), args.iters, args.warmup)
            cl.check()
            row = {"kernel": f"{codec}_{name}", "bits": cbits, "numel": numel, "ms": ms, "gbs": nbytes / ms / 1e6,
                   "gelem_s": numel / ms / 1e6, "hbm_fraction_of_measured": nbytes / ms / 1e6 / hbm,
                   "ctas": args.ctas, "threads": args.threads}
            rows.append(row)
            print(json.dumps(row), flush=True)
    # the tensor-core Hadamard kernel on its own: reads and writes every element once
    n4 = numel // 4096 * 4096
    xin = x[:n4].contiguous()
    ms = time_op(lambda: dq.fwht1024_tcgen05(xin, args.seed, 0, 0, True, 1.0 / 32.0, 0), lambda: None, args.iters,
                 args.warmup)
    row = {"kernel": "fwht1024_tcgen05", "numel": n4, "ms": ms, "gbs": 8 * n4 / ms / 1e6,
           "gelem_s": n4 / ms / 1e6, "hbm_fraction_of_measured": 8 * n4 / ms / 1e6 / hbm,
           "tf32_tflops": 2 * 2 * 2 * 32 * n4 / ms / 1e9}
    rows.append(row)
    print(json.dumps(row), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


def run_reference(args) -> None:
    """The reference arm lives beside the checkout's baseline/ folder, outside the package, and imports
    nothing of it; it prints its own rows (or one ``unavailable`` line).  With ``--kernels`` it is the reference's
    own kernel benchmark, run unmodified (cuda_kernels/tests/benchmark_scaling_quantization.py: 2^28 bf16
    elements, compress / decompress / decompress+compress of its hierarchical codec at 2, 4 and 8 bits)."""
    import importlib.util

    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if args.kernels:
        import runpy

        path = os.path.join(root, "baseline", "_ref", "tests", "benchmark_scaling_quantization.py")
        if not os.path.isfile(path):
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/tests/benchmark_scaling_quantization.py "
                              "is missing: run baseline/install_reference.sh <path of the reference checkout>"}))
            return
        runpy.run_path(path, run_name="__main__")
        return
    path = os.path.join(root, "baseline", "reference_allreduce.py")
    if not os.path.isfile(path):
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": "baseline/reference_allreduce.py not found beside the package"}))
        return
    spec = importlib.util.spec_from_file_location("reference_allreduce", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    argv = ["--sizes-mb", args.sizes_mb, "--methods", args.methods, "--iters", str(args.iters), "--warmup",
            str(args.warmup), "--seed", str(args.seed)]
    if args.out:
        argv += ["--out", args.out]
    mod.main(argv)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernels", action="store_true", help="single-GPU codec kernel throughput")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"],
                    help="reference: the unmodified reference hook (its eden_utils kernels and NCCL point-to-point "
                         "butterfly) on the same tensors, through baseline/reference_allreduce.py")
    ap.add_argument("--methods", default="dynamiQ_aee_5bit", help="--impl reference: comma list of its method names")
    ap.add_argument("--numel", type=int, default=1 << 26)
    ap.add_argument("--sizes-mb", default="1,4,16,64,256")
    ap.add_argument("--bits", default="4,5,8")
    ap.add_argument("--topologies", default="ring,butterfly,direct")
    ap.add_argument("--ctas", type=int, default=148)
    ap.add_argument("--threads", type=int, default=512)
    ap.add_argument("--rotation", default="simt", choices=["simt", "tc"])
    ap.add_argument("--reps", type=int, default=1, help="--kernels: back-to-back launches per timed interval")
    ap.add_argument("--stages", default="", help="--kernels: comma list out of encode,hop,decode,final (default all)")
    ap.add_argument("--rht-only", action="store_true", help="--kernels: only the rotation codec's stages")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-nvls", action="store_true", help="skip the in-switch (NVLS) rows")
    ap.add_argument("--peer-copy", action="store_true",
                    help="measure the peer-copy bandwidth first and use it as the link figure of the roofline fractions")
    ap.add_argument("--hook-methods", default="",
                    help="comma list of aggregation_method names: also time the whole communication hook of each on the "
                         "same tensors (rows hook_<method>)")
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    if args.impl == "reference":
        run_reference(args)
    elif args.kernels:
        run_kernels(args)
    else:
        run_collectives(args)


if __name__ == "__main__":
    main()
