"""DDP hook plumbing on CPU: gloo, world_size 2, one 1 Mi-element fp32 bucket, dynamiQ_aee_5bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dynamiq_sigcomm_artifact_b200.config import parse_method


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, method, numel, steps, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    from argparse import Namespace

    from dynamiq_sigcomm_artifact_b200.train import smoke_hooks

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        out = []
        for m in (method if isinstance(method, (list, tuple)) else [method]):
            args = Namespace(aggregation_method=m, topology=None, numel=numel, steps=steps, warmup_steps=2,
                             seed=1234, dtype="float32", device="cpu", bucket_cap_mb=4000)
            out.append(smoke_hooks.run(args))
        if rank == 0:
            q.put(out if isinstance(method, (list, tuple)) else out[0])
    finally:
        dist.destroy_process_group()


def _run(method, numel=1 << 20, steps=4, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, method, numel, steps, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    return q.get()


def test_method_grammar():
    s = parse_method("dynamiQ_aee_5bit")
    assert (s.hook, s.family, s.bits, s.topology) == ("dynamiq", "rht", 5, "direct")
    assert parse_method("dynamiQ_aee_5bit_ring").topology == "ring"
    s = parse_method("dynamiQ_mee_5bit_dynamic_bitrate_butterfly")
    assert (s.hook, s.family, s.lattice, s.topology, s.dynamic_bitrate) == ("dynamiq_bitrate", "superchunk", "mee",
                                                                            "butterfly", True)
    assert parse_method("dynamiQ_aee_4bit_fixed").thresholds == {8: 0.0, 4: 1.0, 2: 0.0}
    assert parse_method("dynamiQ_mee_4bit").thresholds == {8: 0.05, 4: 0.60, 2: 0.35}
    assert parse_method("MXfp8").hook == "mxfp8" and parse_method("bf16").hook == "bf16"
    assert parse_method("fp4").fpx_format == "fp4" and parse_method("zero").bits == 0
    assert parse_method("thc").quantization_levels == 31 and parse_method("omnireduce").hook == "omnireduce"
    assert parse_method("dynamiQ_aee_5bit_coov").compute_only
    with pytest.raises(ValueError):
        parse_method("nonsense")


def test_dynamiq_aee_5bit_ring_world2():
    a = _run("dynamiQ_aee_5bit")
    # steps 0,1 are the library all-reduce (exact up to fp32 rounding); 2,3 the compressed ring
    assert max(a["nmse"][:2]) < 1e-12
    assert all(1e-4 < e < 3e-2 for e in a["nmse"][2:]), a["nmse"]
    assert max(a["checksum_delta"]) == 0.0
    # two compressed steps of 2^20 elements on 2 ranks: 2 (W - 1) shards of 512 blocks x (640 code + 4 scale bytes)
    assert a["wire_bytes"] == 2 * 2 * 512 * 644 and a["collectives"] == 2
    b = _run("dynamiQ_aee_5bit")
    assert a["grad_sum"] == b["grad_sum"], "not bit-reproducible from the seed"


def test_bf16_and_fp32_baselines_world2():
    r = _run("fp32", numel=1 << 16, steps=3)
    assert max(r["nmse"]) < 1e-12
    r = _run("bf16", numel=1 << 16, steps=3)
    assert 0 < max(r["nmse"]) < 1e-4


def test_every_method_family_world2():
    """One pass over the reference's default evaluation matrix (plus fixed / butterfly / direct
    variants) under gloo: every hook returns the same gradient on both ranks, within the error
    its format allows."""
    bounds = {
        "dynamiQ_mee_5bit": 4e-2, "dynamiQ_aee_5bit_superchunk": 4e-2, "dynamiQ_aee_4bit_fixed": 5e-2,
        "dynamiQ_mee_5bit_dynamic_bitrate": 4e-2, "dynamiQ_mee_4bit_butterfly": 0.1,
        "dynamiQ_aee_8bit_direct": 5e-4, "MXfp8": 5e-3, "fp6": 1e-2, "fp4": 5e-2, "thc": 5e-2,
        "omnireduce": 1.0, "fp16": 1e-6, "fp4_shared": 0.2, "fp8_shared": 5e-3, "dynamiQ_aee_5bit_mixed": 3e-2,
        "dynamiQ_mee_5bit_sim": 5e-2,
    }
    res = _run(list(bounds), numel=1 << 16, steps=4, world=2)
    for r in res:
        m = r["method"]
        assert max(r["checksum_delta"]) < 1e-3, (m, r["checksum_delta"])
        assert max(r["nmse"][:2]) < 1e-6, m
        assert all(e <= bounds[m] for e in r["nmse"][2:]), (m, r["nmse"])
        if m != "fp16":
            assert all(e > 0 for e in r["nmse"][2:]), (m, r["nmse"])
    zero = _run("zero", numel=1 << 12, steps=3, world=2)
    assert zero["nmse"][2] > 0.1  # the traffic-free debug mode is wrong on purpose
