"""Bucket reducer on CPU: layout, readiness order, equivalence with a plain optimizer step, gloo ranks."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dynamiq_sigcomm_artifact_b200.models import build_model
from dynamiq_sigcomm_artifact_b200.ops.layers import FusedAdamW
from dynamiq_sigcomm_artifact_b200.parallel.reducer import BucketReducer, FlatBucket
from dynamiq_sigcomm_artifact_b200.train.engine import TrainConfig, Trainer


def _ids(model, seed, batch=2, seq=32):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, model.config.vocab, (batch, seq), generator=g)


def test_layout_groups_follow_backward_order():
    torch.manual_seed(0)
    m = build_model("gpt2-tiny")
    r = BucketReducer(m, bucket_cap_mb=1e-6)  # every group its own bucket
    names = {id(p): n for n, p in m.named_parameters()}
    first = [names[id(p)] for p in r.groups[0]]
    last = [names[id(p)] for p in r.groups[-1]]
    assert any(n.startswith("ln_f") for n in first) and any(n.startswith("blocks.1.") for n in first)
    assert last == ["wte.weight", "wpe.weight"]
    assert len(r.buckets) == len(r.groups) == 3
    # gradients are views of the arena, contiguous per bucket, 16-byte aligned
    for b in r.buckets:
        lo, hi = b.buffer().data_ptr(), b.buffer().data_ptr() + 4 * b.buffer().numel()
        for p in b.parameters():
            assert lo <= p.grad.data_ptr() < hi and p.grad.data_ptr() % 16 == 0
    assert sum(b.buffer().numel() for b in r.buckets) == r.arena.numel() >= sum(p.numel() for p in m.parameters())
    r.detach()


def test_buckets_fire_in_order_during_backward_and_match_autograd():
    torch.manual_seed(0)
    m = build_model("llama-tiny")
    ref = build_model("llama-tiny")
    ref.load_state_dict(m.state_dict())
    order = []
    r = BucketReducer(m, bucket_cap_mb=1e-6, on_reduced=None)
    r.on_reduced = None
    seen = {}

    def hook(state, bucket: FlatBucket):
        order.append(bucket.index())
        seen[bucket.index()] = bucket.buffer().clone()
        f = torch.futures.Future()
        f.set_result(bucket.buffer())
        return f

    r.hook, r.hook_state = hook, None
    ids = _ids(m, 1)
    r.begin_step()
    m(ids, ids).backward()
    assert order == list(range(len(r.buckets) - 1)), "all but the embedding bucket fire inside backward"
    r.finish()
    assert order == list(range(len(r.buckets)))
    ref(ids, ids).backward()
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p.grad, q.grad, rtol=1e-5, atol=1e-7), n
    # the buffer a hook saw was already complete for that bucket
    for bi, b in enumerate(r.buckets):
        assert torch.equal(seen[bi], b.buffer())
    r.detach()


def test_flat_trainer_matches_plain_adamw_over_steps():
    cfg = dict(model="gpt2-tiny", micro_batch=2, seq_len=32, lr=1e-3, dtype="fp32", weight_decay=0.01)
    a = Trainer(TrainConfig(reducer="flat", **cfg), device=torch.device("cpu"))
    b = Trainer(TrainConfig(reducer="ddp", **cfg), device=torch.device("cpu"))  # world 1: plain step
    b.model.load_state_dict(a.model.state_dict())
    for s in range(4):
        ids = _ids(a.model, 10 + s)
        la, lb = a.train_step(ids), b.train_step(ids)
        assert abs(la - lb) < 1e-5, (s, la, lb)
    for (n, p), (_, q) in zip(a.model.named_parameters(), b.model.named_parameters()):
        assert torch.allclose(p, q, rtol=1e-5, atol=1e-6), n


def _rank_main(rank, world, port, method, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = dict(model="gpt2-tiny", method=method, micro_batch=2, seq_len=32, lr=1e-3, dtype="fp32",
                   bucket_cap_mb=0.05, warmup_steps=1)
        tr = Trainer(TrainConfig(reducer="flat", **cfg), device=torch.device("cpu"))
        losses = []
        for s in range(4):
            g = torch.Generator().manual_seed(100 + 7 * s + rank)
            ids = torch.randint(0, tr.model.config.vocab, (2, 32), generator=g)
            losses.append(tr.train_step(ids))
        flat = torch.cat([p.detach().reshape(-1) for p in tr.model.parameters()])
        gathered = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(gathered, flat)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        q.put((rank, losses, same, len(tr.reducer.buckets), float(flat.double().norm())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("method", ["fp32", "dynamiQ_aee_5bit"])
def test_flat_reducer_over_gloo_keeps_ranks_identical(method):
    world, port = 2, 29400 + (os.getpid() % 500)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, method, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert all(r[2] for r in res), "parameters diverged between ranks"
    assert all(r[3] > 1 for r in res)
    assert all(all(l == l and l < 12 for l in r[1]) for r in res)


def test_flat_and_ddp_reducers_train_alike_on_gloo_ranks():
    """The multi-process comparison of the two reducers (tests/multigpu/check_trainers.py) on two CPU ranks."""
    import json
    import os
    import socket
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(root, "tests", "multigpu", "check_trainers.py")]
    res = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("{")][-1]
    assert json.loads(line)["cases"] == 2
