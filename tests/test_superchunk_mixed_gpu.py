"""Mixed-width superchunk codec, device-side plan and dynamic-bitrate controller on the GPU."""
import numpy as np
import pytest
import torch

from dynamiq_sigcomm_artifact_b200 import bitalloc
from dynamiq_sigcomm_artifact_b200.parallel import schedules as sch
from dynamiq_sigcomm_artifact_b200.parallel.codecs import superchunk_bytes

from helpers import heavy_tail_grad

pytestmark = pytest.mark.gpu


def _widths(nsc, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.tensor([2, 4, 8], dtype=torch.uint8)[torch.randint(0, 3, (nsc,), generator=g)]


def _one_step(cl, buf, step_obj, codec, **kw):
    prog = torch.tensor([[step_obj.as_ints()]], dtype=torch.int32)
    cl.run([buf], prog, 8, codec=codec, **kw)
    cl.check()


def test_plan_kernel_matches_host_arithmetic():
    from dynamiq_sigcomm_artifact_b200 import ops

    dq = ops.require()
    nsc = 4 * 37 + 3  # a partial last block: missing superchunks count as 2-bit
    w = _widths(nsc, 1)
    plan = dq.superchunk_plan(w.cuda()).cpu()
    nb = (nsc + 3) // 4
    assert plan.numel() == 2 * nb + 1
    wp = torch.cat([w, torch.full((4 * nb - nsc,), 2, dtype=torch.uint8)]).view(nb, 4).long()
    sizes = (16 * (2 * wp + 1) + 2).sum(1)
    assert (sizes % 8 == 0).all()
    offs = torch.cat([torch.zeros(1, dtype=torch.long), torch.cumsum(sizes // 8, 0)])
    assert torch.equal(plan[: nb + 1].long(), offs)
    pack = wp[:, 0] | (wp[:, 1] << 8) | (wp[:, 2] << 16) | (wp[:, 3] << 24)
    assert torch.equal(plan[nb + 1:].long(), pack)


@pytest.mark.parametrize("lattice", ["aee", "mee"])
def test_mixed_records_equal_fixed_width_records(lattice):
    """Every superchunk's record in a mixed message is the record the fixed-width kernel writes for it."""
    from dynamiq_sigcomm_artifact_b200 import ops
    from dynamiq_sigcomm_artifact_b200.parallel.fused import Layout, LocalCluster

    dq = ops.require()
    n, seed, step, bucket, tag = 9 * 1024, 5, 3, 2, sch.TAG_ENCODE
    nsc, nb = n // 256, n // 1024
    x = torch.from_numpy(heavy_tail_grad(n, 17))
    w = _widths(nsc, 4)
    plan = dq.superchunk_plan(w.cuda())
    cl = LocalCluster(1, n, ctas=3, threads=128)
    send = sch.Step(shard=0, out=sch.OUT_SEND, dst=0, send_slot=0, tag=tag)
    fixed = {}
    for b in (2, 4, 8):
        prog = torch.tensor([[send.as_ints()]], dtype=torch.int32)
        cl.run([x.clone().cuda()], prog, b, codec=f"sc_{lattice}", seed=seed, step=step, bucket_id=bucket)
        cl.check()
        lay = Layout(n, 1, b, f"sc_{lattice}")
        fixed[b] = cl.slot_bytes(0, 0, lay, nb).cpu().clone().view(nsc, superchunk_bytes(b))
    _one_step(cl, x.clone().cuda(), send, f"scmix_{lattice}", seed=seed, step=step, bucket_id=bucket, plan=plan)
    offs = plan[: nb + 1].cpu().long() * 8
    total = int(offs[-1])
    lay = Layout(n, 1, 8, f"scmix_{lattice}")
    got = cl.slot_bytes(0, 0, lay, nb).cpu()[:total]
    pos = 0
    for i in range(nsc):
        b = int(w[i])
        rec = superchunk_bytes(b)
        if i % 4 == 0:
            assert pos == int(offs[i // 4])
        assert torch.equal(got[pos: pos + rec], fixed[b][i]), (i, b)
        pos += rec
    assert pos == total
    # decode of the mixed message = decode of each fixed-width message on its superchunks
    out = torch.zeros(n, device="cuda")
    _one_step(cl, out, sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_DECODE), f"scmix_{lattice}",
              seed=seed, step=step, bucket_id=bucket, preset_flags=True, plan=plan)
    err = float(((out.cpu().double() - x.double()) ** 2).sum() / (x.double() ** 2).sum())
    assert err < 0.2
    for b in (2, 4, 8):
        lay_b = Layout(n, 1, b, f"sc_{lattice}")
        cl.slot_bytes(0, 0, lay_b, nb).copy_(fixed[b].reshape(-1).cuda())
        ref = torch.zeros(n, device="cuda")
        prog = torch.tensor([[sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_DECODE).as_ints()]], dtype=torch.int32)
        cl.run([ref], prog, b, codec=f"sc_{lattice}", seed=seed, step=step, bucket_id=bucket, preset_flags=True)
        cl.check()
        rows = (w == b).nonzero().reshape(-1)
        assert torch.equal(out.cpu().view(nsc, 256)[rows], ref.cpu().view(nsc, 256)[rows]), b


@pytest.mark.parametrize("topology", sch.TOPOLOGIES)
def test_mixed_collective(topology):
    from dynamiq_sigcomm_artifact_b200 import ops
    from dynamiq_sigcomm_artifact_b200.parallel.fused import LocalCluster

    dq = ops.require()
    world, n = 4, 50 * 1024 + 256 * 3 + 11  # partial last block and superchunk
    nsc = (n + 255) // 256
    xs = [heavy_tail_grad(n, 60 + r) for r in range(world)]
    exact = torch.from_numpy(np.mean(np.stack(xs).astype(np.float64), 0))
    cl = LocalCluster(world, nsc * 256, ctas=4, threads=128)
    errs = {}
    for name, w in (("all8", torch.full((nsc,), 8, dtype=torch.uint8)), ("mixed", _widths(nsc, 9)),
                    ("all2", torch.full((nsc,), 2, dtype=torch.uint8))):
        plan = dq.superchunk_plan(w.cuda())
        bufs = [torch.zeros(nsc * 256, device="cuda") for _ in xs]
        for b, x in zip(bufs, xs):
            b[:n] = torch.from_numpy(x).cuda()
        cl.allreduce_(bufs, 8, topology, seed=6, codec="scmix_mee", plan=plan)
        cl.check()
        assert all(torch.equal(bufs[0], b) for b in bufs)
        errs[name] = float(((bufs[0][:n].cpu().double() - exact) ** 2).sum() / (exact ** 2).sum())
    assert errs["all8"] < 2e-3 and errs["all8"] < errs["mixed"] < errs["all2"] < 1.5, errs


def test_device_controller_follows_host_controller():
    from dynamiq_sigcomm_artifact_b200 import ops

    dq = ops.require()
    g = torch.Generator().manual_seed(3)
    host = bitalloc.DynamicBitrateController(5)
    dev = bitalloc.DeviceBitrateController(5, "cuda")
    for step in range(4):
        # two "buckets" per step; energies drift from step to step
        es = [torch.exp(torch.randn(3000, generator=g) * 3 - 8 + 0.5 * step),
              torch.exp(torch.randn(5000, generator=g) * 2 - 10 + 0.5 * step)]
        for e in es:
            stats = torch.stack([torch.zeros_like(e), e], 1).cuda().contiguous()
            w = dev.widths(stats).cpu()
            u = float(dev.state[0])
            # widths follow the thresholds on the score
            score = (torch.log2(e.clamp_min(1e-20)) * bitalloc.NORM_SCALE).cuda() + torch.tensor(u, device="cuda").float()
            want = torch.where(score >= 8, 8, torch.where(score >= 4, 4, 2)).to(torch.uint8).cpu()
            assert float((w != want).float().mean()) < 1e-3
            host.observe(e)
        host.end_of_step()
        dev.end_of_step()
        torch.cuda.synchronize()
        sd = dev.state_dict()
        assert sd["initialised"]
        assert abs(sd["last_avg"] - (5 - bitalloc.HEADROOM)) <= 0.1 + 1e-6 or abs(sd["u"]) in (10.0, 60.0)
        assert abs(sd["u"] - host.u) < 0.05 and abs(sd["last_avg"] - host.last_avg) < 0.02, (step, sd, host.u, host.last_avg)
