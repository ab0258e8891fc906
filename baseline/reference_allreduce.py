"""Reference arm of the all-reduce benchmark: the unmodified reference hook on one flat gradient.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        baseline/reference_allreduce.py --sizes-mb 16,256 --methods dynamiQ_aee_5bit,bf16

What runs is the reference's own code from ``baseline/_ref``: ``select_hook`` / ``build_comm_state`` of
testbed_evaluation/smoke_test_new_comm_hooks.py, its compressors and ``eden_utils`` kernels, with the
``_butterfly`` topology over NCCL point-to-point (``BUTTERFLY_RDMA_DISABLE=1``, comm_hooks.py:36-45), the
only one of its topologies that runs on a single host.  The hook is reached the way a user reaches it:
``DistributedDataParallel.register_comm_hook`` around a module.  The module here has ONE bf16 parameter of
the requested size whose backward hands over a prepared gradient without arithmetic, so that the timed
backward is the hook plus the two bucket copies DistributedDataParallel always makes.

Input: the tensor ``train/bench_allreduce.py`` draws for the same rank and seed (rounded to bf16, the dtype
the reference trains in); NMSE is against the exact fp64 mean of the bf16 inputs.  Nothing
of this package's engine or kernels is imported.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_TB = os.path.join(HERE, "_ref", "testbed_evaluation")


def synth(n: int, rank: int, seed: int, device):
    """N(0,1) times a lognormal (sigma 2) scale per 1024-element block, seeded per rank: statement for
    statement what train/bench_allreduce.py feeds its own arm, so that both arms see the same numbers."""
    import torch

    g = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    x = torch.randn(n, generator=g, device=device)
    nb = (n + 1023) // 1024
    s = torch.exp(2.0 * torch.randn(nb, generator=g, device=device))
    return x * s.repeat_interleave(1024)[:n]


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", default="16,256", help="fp32-equivalent megabytes (elements x 4 bytes)")
    ap.add_argument("--methods", default="dynamiQ_aee_5bit")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    def unavailable(why: str) -> None:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)

    if not os.path.isdir(os.path.join(REF_TB, "new_comm_hooks")):
        return unavailable("baseline/_ref is missing: run baseline/install_reference.sh <path of the reference checkout>")
    if world < 2 or world & (world - 1):
        return unavailable("the reference's butterfly needs a power-of-two world size of at least 2")
    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ["BUTTERFLY_RDMA_DISABLE"] = "1"
    dist.init_process_group("nccl", device_id=dev)
    sys.path.insert(0, REF_TB)

    class Handover(torch.autograd.Function):
        """forward: a scalar; backward: the prepared gradient, as is."""

        @staticmethod
        def forward(ctx, p, grad):
            ctx.save_for_backward(grad)
            return p.new_zeros(())

        @staticmethod
        def backward(ctx, _g):
            (grad,) = ctx.saved_tensors
            return grad, None

    class OneTensor(torch.nn.Module):
        def __init__(self, n):
            super().__init__()
            self.w = torch.nn.Parameter(torch.zeros(n, dtype=torch.bfloat16, device=dev))

        def forward(self, grad):
            return Handover.apply(self.w, grad)

    rows = []
    for method in args.methods.split(","):
        name = method if "butterfly" in method.lower() else method + "_butterfly"
        for mb in [float(s) for s in args.sizes_mb.split(",")]:
            n = int(mb * (1 << 20)) // 4
            argv = sys.argv
            sys.argv = ["smoke_test_new_comm_hooks.py", "--aggregation_method", name]
            try:
                import smoke_test_new_comm_hooks as ref_smoke  # the reference's own module, unmodified

                ref_args = ref_smoke.parse_args()
            finally:
                sys.argv = argv
            ref_args.numel = n
            state = ref_smoke.build_comm_state(ref_args, world)
            hook = ref_smoke.select_hook(name)
            dist._DEFAULT_FIRST_BUCKET_BYTES = 8000 * 1024 * 1024
            net = DDP(OneTensor(n), device_ids=[local], bucket_cap_mb=8000)
            net.register_comm_hook([state], hook)
            x0 = synth(n, rank, args.seed, dev).bfloat16()
            exact = x0.double()
            dist.all_reduce(exact)
            exact /= world
            x = torch.empty_like(x0)
            times = []
            for it in range(args.warmup + args.iters):
                state["batch_idx"] = it
                net.module.w.grad = None
                x.copy_(x0)  # autograd may adopt the handed-over tensor as .grad, which the hook then overwrites
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                net(x).backward()
                e1.record()
                torch.cuda.synchronize()
                if it >= args.warmup:
                    times.append(e0.elapsed_time(e1))
            got = net.module.w.grad.double()
            nmse = float(((got - exact) ** 2).sum() / (exact ** 2).sum())
            t = torch.tensor(times, dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            row = {"impl": "reference", "method": name, "hook": hook.__name__, "world": world, "numel": n,
                   "input_mb": mb, "dtype": "bf16 gradient", "ms": float(t.mean()), "median_ms": float(t.median()),
                   "min_ms": float(t.min()), "max_ms": float(t.max()), "iters": args.iters, "nmse": nmse,
                   "how": "backward of a one-parameter DistributedDataParallel module with the reference hook "
                          "registered; includes DistributedDataParallel's copy into and out of its bucket"}
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
            del net, state
            torch.cuda.empty_cache()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
