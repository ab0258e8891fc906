"""Hook smoke test: a one-parameter model under real DDP, any aggregation method.

Same idea as the reference's integration test (testbed_evaluation/smoke_test_new_comm_hooks.py):
``SingleBucketModel`` of ``numel`` elements (:56-64), ``loss = (w * x).sum()`` so that the
gradient of ``w`` is ``x`` (:341-343), no optimizer, a cross-rank gradient checksum
(:233-250) and mean step time from step 3 on (:329,367-371).  Added: the error against the
exact mean (the reference only checks that ranks agree) and a CPU/gloo mode.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m dynamiq_sigcomm_artifact_b200.train.smoke_hooks --aggregation_method dynamiQ_aee_5bit
"""
from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel as DDP

from .. import hooks
from ..codec_ref import nmse
from ..config import DynamiqConfig


class SingleBucketModel(nn.Module):
    def __init__(self, numel: int, dtype=torch.float32):
        super().__init__()
        self.w = nn.Parameter(torch.zeros(numel, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return (self.w * x).sum()


def synthetic_grad(numel: int, rank: int, step: int, seed: int) -> torch.Tensor:
    """N(0,1) with 1% of entries scaled by 100, from a generator seeded by (seed, rank, step)."""
    g = torch.Generator().manual_seed(seed * 1_000_003 + rank * 1009 + step)
    x = torch.randn(numel, generator=g)
    mask = torch.rand(numel, generator=g) < 0.01
    return torch.where(mask, x * 100, x)


def check_grad_sync(grad: torch.Tensor, group=None) -> float:
    """Largest cross-rank difference of (sum, norm) of the gradient."""
    mine = torch.tensor([grad.double().sum().item(), grad.double().norm().item()], dtype=torch.float64,
                        device=grad.device)
    allv = [torch.zeros_like(mine) for _ in range(dist.get_world_size(group))]
    dist.all_gather(allv, mine, group=group)
    return max(float((v - allv[0]).abs().max()) for v in allv)


def run(args) -> dict:
    rank, world = dist.get_rank(), dist.get_world_size()
    use_cuda = args.device == "cuda"
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.dtype]
    model = SingleBucketModel(args.numel, dtype).to(device)
    ddp = DDP(model, device_ids=[device.index] if use_cuda else None, bucket_cap_mb=args.bucket_cap_mb)
    cfg = DynamiqConfig.from_env(method=args.aggregation_method, seed=args.seed, warmup_steps=args.warmup_steps,
                                 topology=args.topology)
    state = hooks.register(ddp, args.aggregation_method, config=cfg)
    times, errs, deltas, digest = [], [], [], []
    for step in range(args.steps):
        state.begin_step(step)
        x = synthetic_grad(args.numel, rank, step, args.seed).to(device=device, dtype=dtype)
        model.w.grad = None
        if use_cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        ddp(x).backward()
        if use_cuda:
            torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
        exact = x.double().clone()
        dist.all_reduce(exact)
        exact /= world
        g = model.w.grad
        errs.append(nmse(g.double().cpu().numpy(), exact.cpu().numpy()))
        deltas.append(check_grad_sync(g))
        digest.append(float(g.double().sum().item()))
    if state["engine"] is not None:
        state["engine"].check()
    out = {"method": args.aggregation_method, "world": world, "numel": args.numel, "nmse": errs,
           "checksum_delta": deltas, "grad_sum": digest, "wire_bytes": int(state["stats"]["wire_bytes"]),
           "collectives": int(state["stats"]["collectives"]),
           "mean_step_s": float(np.mean(times[3:])) if len(times) > 3 else None}
    state.close()
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--aggregation_method", default="dynamiQ_aee_5bit")
    ap.add_argument("--topology", default=None, choices=[None, "ring", "butterfly", "direct"])
    ap.add_argument("--numel", type=int, default=1 << 20)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup_steps", type=int, default=2)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--bucket_cap_mb", type=int, default=4000)
    ap.add_argument("--checksum_atol", type=float, default=0.0)
    args = ap.parse_args(argv)
    dist.init_process_group("nccl" if args.device == "cuda" else "gloo")
    if args.device == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    res = run(args)
    bad = [d for d in res["checksum_delta"][args.warmup_steps:] if d > args.checksum_atol]
    if dist.get_rank() == 0:
        print(json.dumps(res))
    dist.destroy_process_group()
    if bad:
        raise SystemExit(f"gradient checksum differs across ranks: {bad}")


if __name__ == "__main__":
    main()
