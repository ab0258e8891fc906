"""Multi-process check of the two gradient reducers of the trainer against each other.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        tests/multigpu/check_trainers.py

``reducer="flat"`` (this package's bucket reducer with in-place gradients) and ``reducer="ddp"``
(``DistributedDataParallel`` with the same hook registered through ``register_comm_hook``, the way the
reference attaches its hooks, testbed_evaluation/train_llm_causal.py:416-431) train the same tiny model on the
same per-rank batches.  With the uncompressed method both must produce the same losses; with the 5-bit
rotation codec the losses stay close (the two reducers cut the gradient into different buckets, so the
rounding noise differs).  After every run all ranks must hold identical parameters."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from dynamiq_sigcomm_artifact_b200.train.engine import TrainConfig, Trainer  # noqa: E402


def run(method: str, reducer: str, steps: int, tail: int = 0):
    tr = Trainer(TrainConfig(model="gpt2-tiny", method=method, reducer=reducer, micro_batch=2, seq_len=128, lr=1e-3,
                             weight_decay=0.01, bucket_cap_mb=1, tail_pipeline_mb=tail, seed=3))
    losses = []
    for _ in range(steps):
        losses.append(float(tr.train_step(tr.synthetic_batch())))
    tr.check()
    flat = torch.cat([p.detach().float().reshape(-1) for p in tr.model.parameters()])
    every = [torch.empty_like(flat) for _ in range(dist.get_world_size())]
    dist.all_gather(every, flat)
    assert all(torch.equal(every[0], t) for t in every), f"{method} / {reducer}: ranks hold different parameters"
    tr.close()
    return losses, flat


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", 0))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:  # the same comparison on CPU ranks (host twin of the codec)
        dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    out = {"world": world, "cases": 0}
    for method, loss_tol, par_tol in (("none", 2e-3, 2e-5), ("dynamiQ_aee_5bit", 5e-2, 1e-3)):
        la, pa = run(method, "flat", 6)
        lb, pb = run(method, "ddp", 6)
        lc, pc = run(method, "flat", 6, tail=1)  # buckets sent after backward, optimizer steps on a second stream
        # same buckets and the same collectives; only library kernels whose backward accumulates with atomics keep
        # the two runs from being identical to the last bit
        assert all(abs(a - c) <= 1e-5 * max(1.0, abs(a)) for a, c in zip(la, lc)), (method, la, lc)
        assert float((pa - pc).abs().mean()) <= 1e-6, (method, float((pa - pc).abs().mean()))
        for s, (a, b) in enumerate(zip(la, lb)):
            assert abs(a - b) <= loss_tol * max(1.0, abs(b)), (method, s, a, b)
        diff = float((pa - pb).abs().mean())
        assert diff <= par_tol, (method, diff)
        out[method] = {"flat": la, "ddp": lb, "mean_abs_param_diff": diff}
        out["cases"] += 1
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
