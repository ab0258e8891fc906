"""Fused-kernel superchunk (AEE / MEE) codec against the PyTorch-op codec run on CPU."""
import numpy as np
import pytest
import torch

from dynamiq_sigcomm_artifact_b200.parallel import schedules as sch
from dynamiq_sigcomm_artifact_b200.parallel.codecs import SuperchunkCodec, superchunk_bytes

from helpers import heavy_tail_grad

pytestmark = pytest.mark.gpu


def _one_step(cl, buf, step_obj, bits, codec, **kw):
    prog = torch.tensor([[step_obj.as_ints()]], dtype=torch.int32)
    cl.run([buf], prog, bits, codec=codec, **kw)
    cl.check()


@pytest.mark.parametrize("lattice", ["aee", "mee"])
@pytest.mark.parametrize("bits", [2, 4, 8])
def test_encode_decode_hop_match_cpu_codec(bits, lattice):
    from dynamiq_sigcomm_artifact_b200.parallel.fused import Layout, LocalCluster

    codec_name = f"sc_{lattice}"
    n, seed, step, bucket, tag = 6 * 1024 + 512, 21, 4, 3, sch.TAG_ENCODE
    x = torch.from_numpy(heavy_tail_grad(n, 7))
    x[9] = float("inf")
    ref = SuperchunkCodec(bits, lattice, seed=seed, step=step, bucket=bucket)
    want = ref.encode(x, 0, tag)
    cl = LocalCluster(1, n, ctas=3, threads=128)
    lay = Layout(n, 1, bits, codec_name)
    buf = x.clone().cuda()
    _one_step(cl, buf, sch.Step(shard=0, out=sch.OUT_SEND, dst=0, send_slot=0, tag=tag), bits, codec_name,
              seed=seed, step=step, bucket_id=bucket)
    got = cl.slot_bytes(0, 0, lay, lay.nblocks).cpu()[: want.numel()]
    if lattice == "aee":
        assert torch.equal(got, want), f"{int((got != want).sum())} bytes differ"
    else:  # log2 differs in the last place between the CPU and the GPU: a few codes move by one level
        assert float((got != want).float().mean()) < 0.01
    # decode what the CPU codec wrote
    rec = superchunk_bytes(bits)
    cl.slot_bytes(0, 0, lay, lay.nblocks)[: want.numel()].copy_(want.cuda())
    out = torch.zeros(n, device="cuda")
    _one_step(cl, out, sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_DECODE), bits, codec_name,
              seed=seed, step=step, bucket_id=bucket, preset_flags=True)
    dec = ref.decode(want, n)
    assert torch.equal(out.cpu(), dec)
    # one hop: local + decoded, re-encoded into slot 1
    x2 = torch.from_numpy(heavy_tail_grad(n, 8))
    buf2 = x2.clone().cuda()
    _one_step(cl, buf2, sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_SEND, dst=0, send_slot=1, tag=tag + 1),
              bits, codec_name, seed=seed, step=step, bucket_id=bucket, preset_flags=True)
    want2 = ref.encode(x2 + dec, 0, tag + 1)
    got2 = cl.slot_bytes(0, 1, lay, lay.nblocks).cpu()[: want2.numel()]
    if lattice == "aee":
        assert torch.equal(got2, want2)
    else:
        assert float((got2 != want2).float().mean()) < 0.01
    assert want.numel() == n // 256 * rec


@pytest.mark.parametrize("topology", sch.TOPOLOGIES)
def test_superchunk_collective(topology):
    from dynamiq_sigcomm_artifact_b200.parallel.fused import LocalCluster

    world, n = 4, 50 * 1024
    xs = [heavy_tail_grad(n, 40 + r) for r in range(world)]
    exact = torch.from_numpy(np.mean(np.stack(xs).astype(np.float64), 0))
    cl = LocalCluster(world, n, ctas=4, threads=128)
    for codec_name, bits, bound in (("sc_aee", 4, 0.12), ("sc_mee", 8, 2e-3), ("sc_aee", 2, 1.0)):
        bufs = [torch.from_numpy(x).cuda() for x in xs]
        cl.allreduce_(bufs, bits, topology, seed=6, codec=codec_name)
        cl.check()
        assert all(torch.equal(bufs[0], b) for b in bufs)
        err = float(((bufs[0].cpu().double() - exact) ** 2).sum() / (exact ** 2).sum())
        assert err < bound, (codec_name, bits, err)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mean_centre_kernels_match_torch(dtype):
    from dynamiq_sigcomm_artifact_b200 import ops
    from dynamiq_sigcomm_artifact_b200.parallel.superchunk import mean_center

    dq = ops.require()
    n, world = 5 * 256 + 77, 4
    x = torch.from_numpy(heavy_tail_grad(n, 2)).to(dtype)
    resid, stats = dq.superchunk_center(x.cuda(), world)
    r_ref, s_ref = mean_center(x, world)
    assert torch.allclose(resid.cpu().view(-1, 256), r_ref, atol=1e-4, rtol=1e-5)
    assert torch.allclose(stats.cpu(), s_ref, atol=1e-5, rtol=1e-4)
    out = torch.empty(n, dtype=dtype, device="cuda")
    dq.superchunk_add_mean(resid, (stats[:, 0] * world).contiguous(), out)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert torch.allclose(out.cpu().float(), torch.nan_to_num(x.float()), atol=tol, rtol=tol)


@pytest.mark.parametrize("fmt,bits", [("fp8", 8), ("fp6", 6), ("fp4", 4)])
def test_block_float_kernel_matches_cpu_codec(fmt, bits):
    """Native cvt (E4M3 / E3M2 / E2M1) inside the fused kernel against the PyTorch-op codec on CPU."""
    from dynamiq_sigcomm_artifact_b200.parallel.codecs import BlockFloatCodec
    from dynamiq_sigcomm_artifact_b200.parallel.fused import Layout, LocalCluster

    n = 5 * 1024
    x = torch.from_numpy(heavy_tail_grad(n, 12))
    x[3], x[40:72] = float("nan"), 0.0  # a sanitised value and an all-zero scaling block
    ref = BlockFloatCodec(fmt)
    want = ref.encode(x, 0, 0)
    cl = LocalCluster(1, n, ctas=2, threads=128)
    lay = Layout(n, 1, bits, "mx")
    buf = x.clone().cuda()
    _one_step(cl, buf, sch.Step(shard=0, out=sch.OUT_SEND, dst=0, send_slot=0, tag=sch.TAG_ENCODE), bits, "mx")
    got = cl.slot_bytes(0, 0, lay, lay.nblocks).cpu()
    assert got.numel() == want.numel() == ref.message_bytes(n)
    assert torch.equal(got, want), f"{int((got != want).sum())} of {want.numel()} bytes differ"
    out = torch.zeros(n, device="cuda")
    _one_step(cl, out, sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_DECODE), bits, "mx", preset_flags=True)
    assert torch.equal(out.cpu(), ref.decode(want, n))
    # collective
    world = 4
    xs = [heavy_tail_grad(20 * 1024, 60 + r) for r in range(world)]
    exact = torch.from_numpy(np.mean(np.stack(xs).astype(np.float64), 0))
    cl4 = LocalCluster(world, 20 * 1024, ctas=3, threads=128)
    bufs = [torch.from_numpy(a).cuda() for a in xs]
    cl4.allreduce_(bufs, bits, "ring", codec="mx")
    cl4.check()
    assert all(torch.equal(bufs[0], b) for b in bufs)
    err = float(((bufs[0].cpu().double() - exact) ** 2).sum() / (exact ** 2).sum())
    assert err < {"fp8": 5e-3, "fp6": 2e-2, "fp4": 0.15}[fmt], err


@pytest.mark.parametrize("bits,tol", [(16, 2e-5), (32, 1e-13)])
def test_identity_wire_collective(bits, tol):
    """Uncompressed point-to-point all-reduce through the fused kernel (bf16 or fp32 on the wire)."""
    from dynamiq_sigcomm_artifact_b200.parallel.fused import LocalCluster

    world, n = 4, 30 * 1024 + 40
    xs = [heavy_tail_grad(n, 70 + r) for r in range(world)]
    exact = torch.from_numpy(np.mean(np.stack(xs).astype(np.float64), 0))
    cl = LocalCluster(world, n, ctas=3, threads=128)
    for topology in sch.TOPOLOGIES:
        bufs = [torch.from_numpy(a).cuda() for a in xs]
        cl.allreduce_(bufs, bits, topology, codec="cast")
        cl.check()
        assert all(torch.equal(bufs[0], b) for b in bufs)
        err = float(((bufs[0].cpu().double() - exact) ** 2).sum() / (exact ** 2).sum())
        assert err < tol, (topology, err)
