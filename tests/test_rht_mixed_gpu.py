"""Rotation codec with a code width per block inside the fused kernel, and the device-side width policy,
against the CPU twins (all ranks emulated on one GPU)."""
import numpy as np
import pytest
import torch

from dynamiq_sigcomm_artifact_b200 import bitalloc, codec_ref as cr
from dynamiq_sigcomm_artifact_b200.parallel import cpu_backend as cb
from dynamiq_sigcomm_artifact_b200.parallel import schedules as sch

from helpers import heavy_tail_grad, lognormal_block_grad

pytestmark = pytest.mark.gpu


def _simulate(xs, widths, topology, seed, step, bucket):
    codecs = {}

    def factory(bits, seed_, step_, bucket_, world_, rank):
        codecs[rank] = cb.RhtMixCodecCPU(widths, seed_, step_, bucket_, world_, rank)
        return codecs[rank]

    return cb.simulate_allreduce(xs, 8, topology, seed=seed, step=step, bucket=bucket, codec_factory=factory), codecs


@pytest.mark.parametrize("topology", sch.TOPOLOGIES)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_mixed_width_collective_matches_the_simulator_bit_for_bit(world, topology):
    from dynamiq_sigcomm_artifact_b200.parallel.fused import LocalCluster

    n, seed, step, bucket = 37 * 1024 + 517, 1234, 7, 2
    nb = (n + 1023) // 1024
    xs = [lognormal_block_grad(n, 10 + r) for r in range(world)]
    widths = np.random.default_rng(world).integers(2, 9, nb).astype(np.uint8)
    want, _ = _simulate(xs, widths, topology, seed, step, bucket)
    plan = torch.from_numpy(bitalloc.rht_plan(widths)).cuda()
    cl = LocalCluster(world, n, ctas=5, threads=128)
    bufs = [torch.from_numpy(x).cuda() for x in xs]
    cl.allreduce_(bufs, 8, topology, seed=seed, step=step, bucket_id=bucket, codec="rht_mix", plan=plan)
    cl.check()
    for r in range(world):
        assert np.array_equal(bufs[r].cpu().numpy(), want[r]), f"rank {r}"


def test_uniform_plan_equals_the_fixed_width_codec():
    from dynamiq_sigcomm_artifact_b200.parallel.fused import LocalCluster, uniform_plan

    world, n = 4, 21 * 1024 + 9
    xs = [heavy_tail_grad(n, r) for r in range(world)]
    cl = LocalCluster(world, n, ctas=4)
    a = [torch.from_numpy(x).cuda() for x in xs]
    b = [torch.from_numpy(x).cuda() for x in xs]
    cl.allreduce_(a, 5, "direct", seed=3, step=1)
    cl.allreduce_(b, 8, "direct", seed=3, step=1, codec="rht_mix", plan=uniform_plan(n, 5, "cuda"))
    cl.check()
    assert torch.equal(a[0], b[0])


@pytest.mark.parametrize("world,target", [(4, 5.0), (8, 4.0), (2, 6.5)])
def test_device_width_policy_equals_the_host_twin(world, target):
    """After a collective every rank's mailbox holds the same block scales; the kernel that turns them into
    the next plan gives, on every rank, exactly what the NumPy policy gives from the simulator's scales."""
    from dynamiq_sigcomm_artifact_b200.parallel.fused import LocalCluster, uniform_plan

    n, seed, step = 203 * 1024 + 77, 5, 3
    nb = (n + 1023) // 1024
    xs = [lognormal_block_grad(n, 40 + r) for r in range(world)]
    xs[0][: 2048] = 0  # two all-zero blocks on one rank keep their data from the others
    for x in xs:
        x[4096: 5120] = 0  # a block that is zero everywhere: absmax 0, smallest width
    start = np.full(nb, 5, np.uint8)
    _, codecs = _simulate(xs, start, "direct", seed, step, 0)
    want_w, _ = bitalloc.rht_block_widths(codecs[0].block_absmax(nb), target)
    want = bitalloc.rht_plan(want_w)
    cl = LocalCluster(world, n, ctas=6, threads=256)
    bufs = [torch.from_numpy(x).cuda() for x in xs]
    base = uniform_plan(n, 5, "cuda")
    cl.allreduce_(bufs, 8, "direct", seed=seed, step=step, codec="rht_mix", plan=base)
    cl.check()
    for r in range(world):
        plan = base.clone()
        cl.update_widths_(plan, n, target, rank=r)
        assert np.array_equal(plan.cpu().numpy(), want), f"rank {r}"
    assert want_w[4] == 2 and abs(want_w.mean() - target) <= 0.1


def test_two_steps_with_learned_widths_cut_the_error():
    from dynamiq_sigcomm_artifact_b200.parallel.fused import LocalCluster, uniform_plan

    world, n = 8, 128 * 1024
    xs = [lognormal_block_grad(n, 10 + r) for r in range(world)]
    exact = np.mean(np.stack(xs).astype(np.float64), 0)
    cl = LocalCluster(world, n, ctas=8, threads=256)
    plan = uniform_plan(n, 5, "cuda")
    errs = []
    for step in (1, 2):
        bufs = [torch.from_numpy(x).cuda() for x in xs]
        cl.allreduce_(bufs, 8, "direct", seed=5, step=step, codec="rht_mix", plan=plan)
        cl.check()
        errs.append(cr.nmse(bufs[0].cpu().numpy(), exact))
        cl.update_widths_(plan, n, 5.0, rank=0)
    w = plan.cpu().numpy()[n // 1024 + 1:]
    assert 4.9 <= w.mean() <= 5.0
    assert errs[1] < errs[0] / 3, errs
