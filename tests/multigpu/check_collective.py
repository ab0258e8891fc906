"""Multi-process oracle check of the fused compressed all-reduce over real peer mappings.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        tests/multigpu/check_collective.py [--rotation simt|tc] [--stress 200] [--quick]

One rank per GPU.  Every rank regenerates ALL ranks' seeded inputs on the CPU, runs the step-program
simulator (``cpu_backend.simulate_allreduce``) and compares what its own GPU produced:

* ``--rotation simt``: the bucket must equal the simulator's with ``torch.equal`` (fp32), or the simulator's
  result rounded to bf16 (bf16 buckets, ring / direct).
* ``--rotation tc``: inputs are small integers times a power of two per block, on which the tensor-core
  rotation is exact, so every message found in this rank's mailbox afterwards (reduce-scatter hops and
  all-gather shards) must equal the simulator's message byte for byte; the bucket must be within TF32
  accuracy of the simulator's and identical on all ranks (checksum exchange).

Then a stress phase: ``--stress`` collectives are launched back to back without a host synchronisation,
alternating two grid sizes (each one pairs with its own flag columns) and both slot sets, with one growth of
the symmetric buffers in the middle; every single result is checked afterwards.

What this covers and the single-GPU tests cannot: ``cudaIpcOpenMemHandle`` mappings, system-scope
release / acquire flags across NVLink, slot-set alternation across hundreds of collectives, re-allocation
of the symmetric buffers, different grids inside one run.  Waits keep their short budgets; a failure is a
Python exception on the rank that saw it, never a device fault.

Reference counterparts: the cross-rank checksum of testbed_evaluation/smoke_test_new_comm_hooks.py:233-250
and the correctness check of rdma_comm_compress/sample_allreduce.py:518-547.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from dynamiq_sigcomm_artifact_b200 import codec_ref as cr  # noqa: E402
from dynamiq_sigcomm_artifact_b200.parallel import cpu_backend as cb  # noqa: E402
from dynamiq_sigcomm_artifact_b200.parallel import schedules as sch  # noqa: E402
from dynamiq_sigcomm_artifact_b200.parallel.fused import FusedAllreduce, Layout  # noqa: E402
from helpers import heavy_tail_grad, small_int_grad  # noqa: E402


def bf16_round(x: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(x)).bfloat16().float().numpy()


def mailbox_messages(eng: FusedAllreduce, lay: Layout) -> dict:
    """{slot: (code bytes, scale bytes)} of the slot set the engine's last collective used."""
    parity = eng.epoch & 1
    raw = eng.buf.local()[parity * eng.set_bytes: (parity + 1) * eng.set_bytes].cpu().numpy()
    out = {}
    for slot in range(eng.nslots):
        base = slot * lay.slot_stride
        out[slot] = raw[base: base + lay.slot_stride]
    return out


def check_one(eng, rank, world, xs, bits, topology, dtype, rotation, seed, step, bucket, ctas, log) -> None:
    layout = "tc" if rotation == "tc" else "simt"
    n = xs[0].size
    want, transport = cb.simulate_allreduce(xs, bits, topology, seed=seed, step=step, bucket=bucket,
                                            return_transport=True, layout=layout)
    buf = torch.from_numpy(xs[rank]).cuda().to(dtype)
    eng.allreduce_(buf, bits, topology, seed=seed, step=step, bucket_id=bucket, ctas=ctas)
    eng.check()
    got = buf.float().cpu().numpy()
    ref = want[rank] if dtype == torch.float32 else bf16_round(want[rank])
    what = f"{topology} {bits}bit {str(dtype)[6:]} n={n} grid={ctas}"
    if rotation == "simt":
        if not np.array_equal(got, ref):
            raise AssertionError(f"rank {rank}: {what}: bucket differs from the simulator, max diff "
                                 f"{np.abs(got - ref).max()}")
    else:
        lay = Layout(n, world, bits, "rht_tc")
        slots = mailbox_messages(eng, lay)
        nmsg = 0
        for (src, dst, slot), msg in transport.log.items():
            if dst != rank:
                continue
            nb = msg.size // (128 * bits + 4)
            raw = slots[slot]
            if not (np.array_equal(raw[: nb * 128 * bits], msg[: nb * 128 * bits]) and
                    np.array_equal(raw[lay.scales_off: lay.scales_off + 4 * nb], msg[nb * 128 * bits:])):
                raise AssertionError(f"rank {rank}: {what}: message from rank {src} in slot {slot} differs from "
                                     f"the simulator's")
            nmsg += 1
        tol = 4e-3 * np.repeat(np.abs(cr.to_blocks(want[rank])).max(axis=1), 1024)[:n] + 1e-30
        if dtype != torch.float32:
            tol = tol + np.abs(ref) * 2.0 ** -7
        if not (np.abs(got - ref) <= tol).all():
            raise AssertionError(f"rank {rank}: {what}: bucket outside TF32 tolerance of the simulator")
        log["messages"] += nmsg
    # all ranks must hold the same bits
    digest = torch.tensor([int(np.frombuffer(buf.cpu().view(torch.uint8).numpy().tobytes(), np.uint8)
                               .astype(np.uint64).sum()), int(buf.float().abs().sum().item() * 1e3)],
                          device="cuda", dtype=torch.int64)
    all_d = [torch.empty_like(digest) for _ in range(world)]
    dist.all_gather(all_d, digest)
    if any(not torch.equal(all_d[0], d) for d in all_d):
        raise AssertionError(f"rank {rank}: {what}: ranks hold different results")
    log["collectives"] += 1
    log["wire_bytes"] += transport.sent_bytes[rank]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rotation", default="tc", choices=["simt", "tc"])
    ap.add_argument("--stress", type=int, default=200)
    ap.add_argument("--quick", action="store_true", help="fewer sizes and widths")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    import datetime

    # a rank that raises leaves the others in a library collective: bound that wait
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))
    rank, world = dist.get_rank(), dist.get_world_size()
    gen = small_int_grad if args.rotation == "tc" else heavy_tail_grad
    t0 = time.time()
    log = {"collectives": 0, "messages": 0, "wire_bytes": 0}
    grids = (64, 148)
    eng = FusedAllreduce(max_numel=64 * 1024, ctas=grids[0], threads=256, timeout_ms=4000,
                         rotation=args.rotation, max_ctas=grids[1])
    sizes = [37 * 1024 + 517] if args.quick else [5 * 1024, 37 * 1024 + 517, 200 * 1024 + 3]
    widths = [5] if args.quick else [4, 5, 8]
    topologies = [t for t in sch.TOPOLOGIES if t != "butterfly" or world & (world - 1) == 0]
    step = 0
    for n in sizes:
        xs = [gen(n, 100 + r) for r in range(world)]
        for topology in topologies:
            for bits in widths:
                for dtype in (torch.float32, torch.bfloat16):
                    if dtype == torch.bfloat16 and (topology == "butterfly" or bits != 5):
                        continue  # butterfly keeps partial sums in the bf16 bucket; the simulator keeps fp32
                    step += 1
                    xin = xs if dtype == torch.float32 else [bf16_round(x) for x in xs]
                    check_one(eng, rank, world, xin, bits, topology, dtype, args.rotation, seed=77, step=step,
                              bucket=step % 5, ctas=grids[step % 2], log=log)
    # ---- stress: back-to-back launches, no host synchronisation in between ----
    n = 24 * 1024 + 100
    xs = [gen(n, 300 + r) for r in range(world)]
    layout = "tc" if args.rotation == "tc" else "simt"
    outs = []
    grow_at = args.stress // 2
    for i in range(args.stress):
        if i == grow_at:  # collective re-allocation of the symmetric buffers in the middle of the run
            torch.cuda.synchronize()
            eng.ensure_capacity(4 * eng.max_numel)
        buf = torch.from_numpy(xs[rank]).cuda()
        eng.allreduce_(buf, 5, topologies[i % len(topologies)], seed=5, step=1000 + i, bucket_id=i % 7,
                       ctas=grids[i % 2])
        outs.append(buf)
    torch.cuda.synchronize()
    eng.check()
    for i, buf in enumerate(outs):
        want = cb.simulate_allreduce(xs, 5, topologies[i % len(topologies)], seed=5, step=1000 + i, bucket=i % 7,
                                     layout=layout)[rank]
        got = buf.cpu().numpy()
        if args.rotation == "simt":
            ok = np.array_equal(got, want)
        else:
            tol = 4e-3 * np.repeat(np.abs(cr.to_blocks(want)).max(axis=1), 1024)[:n] + 1e-30
            ok = bool((np.abs(got - want) <= tol).all())
        if not ok:
            raise AssertionError(f"rank {rank}: stress collective {i} differs from the simulator")
        log["collectives"] += 1
    ok_t = torch.ones(1, device="cuda")
    dist.all_reduce(ok_t)
    summary = {"world": world, "rotation": args.rotation, "bit_exact": args.rotation == "simt",
               "messages_byte_exact": log["messages"], "collectives_checked": log["collectives"],
               "stress": args.stress, "seconds": round(time.time() - t0, 1), "ok": int(ok_t.item()) == world}
    if rank == 0:
        print(json.dumps(summary), flush=True)
        if args.out:
            with open(args.out, "w") as f:
                json.dump(summary, f)
    eng.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
