"""Guard zones of the symmetric buffer (debug net against out-of-region stores)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_guard_zones_are_checked_and_name_the_region(monkeypatch):
    import torch.distributed as dist

    from dynamiq_sigcomm_artifact_b200.parallel.fused import CANARY_VALUE, FusedAllreduce, MailboxOverrun

    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29641", rank=0, world_size=1)
    try:
        eng = FusedAllreduce(max_numel=8 * 1024, ctas=4, max_ctas=8, debug=True, validate=False)
        assert all(bool((g == CANARY_VALUE).all()) for g in eng._guards)
        eng.check()  # clean
        x = torch.randn(8 * 1024, device="cuda")
        eng.allreduce_(x, 5, "direct")  # world 1: returns at once, nothing is written
        eng.check()
        eng._guards[1][17] = 0  # what a store past the end of slot set 1 would do
        with pytest.raises(MailboxOverrun, match="slot set 1.*byte 17"):
            eng.check()
        eng.close()
    finally:
        dist.destroy_process_group()


def test_debug_mode_refuses_a_plan_that_leaves_its_slot():
    """Offsets of the plan-driven codecs live in device memory, out of the host checks' sight.  In debug mode a
    plan whose block would start beyond the slot's code region ends the collective with a status and no access.
    (The bad offset still lies inside the mailbox allocation, which is sized for the fp32 identity wire.)"""
    import numpy as np

    from dynamiq_sigcomm_artifact_b200 import bitalloc
    from dynamiq_sigcomm_artifact_b200.parallel.fused import CollectiveTimeout, LocalCluster

    n = 16 * 1024
    widths = np.full(16, 5, np.uint8)
    good = torch.from_numpy(bitalloc.rht_plan(widths)).cuda()
    cl = LocalCluster(1, n, ctas=2, threads=128, debug=True)
    try:
        x = torch.randn(n, device="cuda")
        before = x.clone()
        cl.allreduce_([x], 8, "ring", seed=1, step=1, codec="rht_mix", plan=good)
        cl.check()  # a sound plan passes the checks
        assert not torch.equal(x, before) and float((x - before).abs().mean()) < 0.2
        bad = good.clone()
        bad[9:17] += 2 * 8 * 16  # blocks 9.. start two full-width shards further than the slot's code region holds
        y = before.clone()
        cl.allreduce_([y], 8, "ring", seed=1, step=2, codec="rht_mix", plan=bad)
        with pytest.raises(CollectiveTimeout, match="debug mode"):
            cl.check()
        bad_w = good.clone()
        bad_w[17 + 3] = 11  # a width outside 2..8
        cl.allreduce_([before.clone()], 8, "ring", seed=1, step=3, codec="rht_mix", plan=bad_w)
        with pytest.raises(CollectiveTimeout, match="debug mode"):
            cl.check()
    finally:
        cl.ops.set_debug(False)


@pytest.mark.parametrize("codec,bits", [(None, 5), ("sc_mee", 4), ("mx", 8), ("cast", 16)])
def test_debug_mode_does_not_change_results(codec, bits):
    from dynamiq_sigcomm_artifact_b200.parallel.fused import LocalCluster

    world, n = 4, 13 * 1024 + 77
    xs = [torch.randn(n, device="cuda") * (r + 1) for r in range(world)]
    outs = []
    for debug in (False, True):
        cl = LocalCluster(world, n, ctas=3, threads=128, debug=debug)
        bufs = [x.clone() for x in xs]
        cl.allreduce_(bufs, bits, "direct", seed=5, step=9, codec=codec)
        cl.check()
        outs.append(bufs)
    cl.ops.set_debug(False)
    for a, b in zip(*outs):
        assert torch.equal(a, b)
