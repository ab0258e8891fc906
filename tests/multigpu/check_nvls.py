"""Multi-process check of the in-switch (NVLS) all-reduce against a float64 mean.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        tests/multigpu/check_nvls.py

Skips (exit 0, says so) when the box exposes no multicast object.  No rank leaves and no wait is made to
expire here: both are exercised elsewhere without NVLS."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from dynamiq_sigcomm_artifact_b200.parallel.nvls import NvlsAllreduce  # noqa: E402


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    eng = NvlsAllreduce(max_numel=(1 << 22) + 64, wire_bits=32, ctas=32)
    out = {"world": world, "available": eng.available, "reason": eng.reason, "cases": 0}
    if eng.available:
        for n in (7, 1000, 1 << 20, (1 << 22) + 13):
            for wire, dtype, tol in ((32, torch.float32, 1e-12), (16, torch.float32, 5e-5), (16, torch.bfloat16, 5e-5)):
                for rep in range(3):  # back to back: the flags and the staging buffer are reused
                    g = torch.Generator(device="cuda").manual_seed(rank * 7 + n + rep)
                    x = torch.randn(n, device="cuda", generator=g).to(dtype)
                    exact = x.double().clone()
                    dist.all_reduce(exact)
                    exact /= world
                    eng.allreduce_(x, wire)
                    eng.check()
                    err = float(((x.double() - exact) ** 2).sum() / (exact ** 2).sum())
                    assert err < tol, (n, wire, dtype, err)
                    ys = [torch.empty_like(x) for _ in range(world)]
                    dist.all_gather(ys, x)
                    assert all(torch.equal(ys[0], t) for t in ys), "ranks disagree"
                    out["cases"] += 1
    if rank == 0:
        print(json.dumps(out), flush=True)
    eng.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
