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
