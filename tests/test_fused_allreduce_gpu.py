"""Fused compressed all-reduce kernel against the CPU oracle (all ranks emulated on one GPU)."""
import numpy as np
import pytest
import torch

from dynamiq_sigcomm_artifact_b200 import codec_ref as cr
from dynamiq_sigcomm_artifact_b200.parallel import cpu_backend as cb
from dynamiq_sigcomm_artifact_b200.parallel import schedules as sch
from dynamiq_sigcomm_artifact_b200.utils import philox

from helpers import heavy_tail_grad, small_int_grad

pytestmark = pytest.mark.gpu


def _cluster(world, n, **kw):
    from dynamiq_sigcomm_artifact_b200.parallel.fused import LocalCluster

    return LocalCluster(world, n, **kw)


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 7, 8])
def test_standalone_ops_match_oracle_bytes(bits):
    from dynamiq_sigcomm_artifact_b200.parallel.fused import RhtCodec

    n, seed, step, bucket = 7 * 1024 + 333, 99, 5, 3
    x = heavy_tail_grad(n, 1)
    x[5] = np.inf
    x[6] = np.nan
    codec = RhtCodec(bits, n, seed=seed, ctas=4)
    words, scales = codec.compress(torch.from_numpy(x).cuda(), step=step, bucket_id=bucket)
    ref = cb.RhtCodecCPU(bits, seed, step, bucket, world=1)
    y = ref.rotate(cr.to_blocks(x))
    codes, rscale = cr.quantize(y, bits, np.arange(y.shape[0]), ref._tag_base | sch.TAG_ENCODE, step, seed)
    rwords = cr.pack(codes, bits)
    assert np.array_equal(words.cpu().numpy().view(np.uint32), rwords)
    assert np.array_equal(scales.cpu().numpy(), rscale)
    # decode -> inverse rotation
    out = codec.decompress((words, scales), n, step=step, bucket_id=bucket, post_scale=0.25)
    rout = cr.rotate_inv(cr.dequantize(codes, rscale, bits), ref.signs, 0.25).reshape(-1)[:n]
    assert np.array_equal(out.cpu().numpy(), rout)
    # one hop: decode + add rotated local + re-encode
    x2 = heavy_tail_grad(n, 2)
    w2, s2 = codec.dec_comp((words, scales), torch.from_numpy(x2).cuda(), step=step, bucket_id=bucket)
    v = cr.dequantize_add(codes, rscale, bits, ref.rotate(cr.to_blocks(x2)))
    c2, rs2 = cr.quantize(v, bits, np.arange(v.shape[0]), ref._tag_base | (sch.TAG_ENCODE + 1), step, seed)
    assert np.array_equal(w2.cpu().numpy().view(np.uint32), cr.pack(c2, bits))
    assert np.array_equal(s2.cpu().numpy(), rs2)


@pytest.mark.parametrize("topology", sch.TOPOLOGIES)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_collective_matches_simulator_bit_for_bit(world, topology):
    n, bits, seed, step, bucket = 37 * 1024 + 517, 5, 1234, 7, 2
    xs = [heavy_tail_grad(n, 10 + r) for r in range(world)]
    want = cb.simulate_allreduce(xs, bits, topology, seed=seed, step=step, bucket=bucket)
    cl = _cluster(world, n, ctas=6, threads=128)
    bufs = [torch.from_numpy(x).cuda() for x in xs]
    cl.allreduce_(bufs, bits, topology, seed=seed, step=step, bucket_id=bucket)
    cl.check()
    for r in range(world):
        got = bufs[r].cpu().numpy()
        assert np.array_equal(got, want[r]), f"rank {r}: max diff {np.abs(got - want[r]).max()}"
    exact = np.mean(np.stack(xs).astype(np.float64), 0)
    assert cr.nmse(bufs[0].cpu().numpy(), exact) < 0.08


def test_collective_is_reusable_and_deterministic():
    world, n = 4, 20 * 1024
    cl = _cluster(world, n, ctas=4)
    outs = []
    for rep in range(3):
        bufs = [torch.from_numpy(heavy_tail_grad(n, r)).cuda() for r in range(world)]
        cl.allreduce_(bufs, 4, "butterfly", seed=5, step=1)
        outs.append(bufs[0].clone())
    cl.check()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


def test_bf16_bucket():
    world, n = 4, 16 * 1024 + 64
    xs = [torch.from_numpy(heavy_tail_grad(n, r)).cuda().bfloat16() for r in range(world)]
    exact = torch.stack([x.float() for x in xs]).mean(0)
    cl = _cluster(world, n, ctas=4)
    cl.allreduce_(xs, 8, "ring", seed=3)
    cl.check()
    assert all(torch.equal(xs[0], x) for x in xs)
    err = float((xs[0].float() - exact).pow(2).sum() / exact.pow(2).sum())
    assert err < 2e-3


def test_wait_budget_expiry_returns_an_error_status():
    """A receive whose flag nobody sets: the kernel gives up after its budget and reports it."""
    from dynamiq_sigcomm_artifact_b200.parallel.fused import CollectiveTimeout

    n = 4 * 1024
    cl = _cluster(1, n, ctas=2, timeout_ms=20)
    out = torch.zeros(n, device="cuda")
    prog = torch.tensor([[sch.Step(shard=0, recv_slot=0, nrecv=1, out=sch.OUT_DECODE).as_ints()]], dtype=torch.int32)
    cl.run([out], prog, 4)  # flags stay at 0, epoch is 1
    with pytest.raises(CollectiveTimeout, match="timed out"):
        cl.check()
    # the context is still usable and the cluster works afterwards
    x = torch.randn(n, device="cuda")
    cl2 = _cluster(2, n, ctas=2)
    bufs = [x.clone(), x.clone()]
    cl2.allreduce_(bufs, 8, "ring")
    cl2.check()
    assert float((bufs[0] - x).abs().max()) < 0.2


@pytest.mark.parametrize("topology,world", [("direct", 8), ("ring", 4), ("butterfly", 4), ("direct", 3)])
def test_correlated_rounding_matches_simulator_and_lowers_error(topology, world):
    n, bits, seed = 24 * 1024 + 100, 5, 77
    xs = [heavy_tail_grad(n, 50 + r) for r in range(world)]
    want = cb.simulate_allreduce(xs, bits, topology, seed=seed, step=2, bucket=1, correlated=True)
    cl = _cluster(world, n, ctas=4, threads=128)
    bufs = [torch.from_numpy(x).cuda() for x in xs]
    cl.allreduce_(bufs, bits, topology, correlated=True, seed=seed, step=2, bucket_id=1)
    cl.check()
    for r in range(world):
        assert np.array_equal(bufs[r].cpu().numpy(), want[r]), f"rank {r}"
    exact = np.mean(np.stack(xs).astype(np.float64), 0)
    plain = cb.simulate_allreduce(xs, bits, topology, seed=seed, step=2, bucket=1)
    assert cr.nmse(want[0], exact) < cr.nmse(plain[0], exact)


def _store_program():
    return torch.tensor([[sch.Step(shard=0, out=sch.OUT_STORE).as_ints()]], dtype=torch.int32)


def _stored_to_coeff(buf: np.ndarray) -> np.ndarray:
    """Bucket written by a STORE step of the tensor-core body -> [nb, 1024] in coefficient order.
    The step keeps register t = 4 j + k of lane l at element 128 j + 4 l + k, and that register holds
    coefficient 32 t + l."""
    got = buf.reshape(-1, 8, 32, 4)  # [block, j, lane, k]
    t = 4 * np.arange(8)[:, None, None] + np.arange(4)[None, None, :]
    coeff = (32 * t + np.arange(32)[None, :, None]).reshape(-1)
    out = np.empty((got.shape[0], 1024), np.float32)
    out[:, coeff] = got.reshape(got.shape[0], -1)
    return out


@pytest.mark.parametrize("threads", [128, 256, 384, 512])
def test_tensor_core_rotation_inside_the_fused_kernel(threads):
    """STORE program = rotate and keep.  Exact on inputs whose sums fit TF32; within 2^-9 of the
    largest coefficient against a float64 Hadamard product otherwise."""
    n, seed, step, bucket = 41 * 1024, 11, 2, 5
    signs = philox.sign_vector(step, bucket, seed)
    cl = _cluster(1, n, ctas=3, threads=threads, rotation="tc")
    x = small_int_grad(n, 3)
    buf = torch.from_numpy(x).cuda()
    cl.run([buf], _store_program(), 8, seed=seed, step=step, bucket_id=bucket)
    cl.check()
    assert np.array_equal(_stored_to_coeff(buf.cpu().numpy()), cr.rotate_fwd(cr.to_blocks(x), signs))
    x = heavy_tail_grad(n, 3)
    buf = torch.from_numpy(x).cuda()
    cl.run([buf], _store_program(), 8, seed=seed, step=step, bucket_id=bucket)
    cl.check()
    h = np.array([[1.0]])
    for _ in range(10):
        h = np.block([[h, h], [h, -h]])
    want = (cr.to_blocks(x).astype(np.float64) * signs) @ h.T  # unnormalised
    got = _stored_to_coeff(buf.cpu().numpy())
    err = np.abs(got - want).max(axis=1) / np.abs(want).max(axis=1)
    assert err.max() < 2e-3, err.max()


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 7, 8])
def test_tensor_core_standalone_ops_match_oracle_bytes(bits):
    """compress / hop bytes equal the oracle's on TF32-exact inputs; on arbitrary inputs they equal the
    oracle fed with the kernel's own rotated coefficients (taken from a STORE step)."""
    from dynamiq_sigcomm_artifact_b200.parallel.fused import RhtCodec

    n, seed, step, bucket = 9 * 1024 + 333, 99, 5, 3
    codec = RhtCodec(bits, n, seed=seed, ctas=2, threads=256, rotation="tc")
    ref = cb.RhtCodecCPU(bits, seed, step, bucket, world=1, layout="tc")
    tagbase = ref._tag_base
    for exact in (True, False):
        x = small_int_grad(n, 1) if exact else heavy_tail_grad(n, 1)
        if not exact:
            x[5] = np.inf  # its whole block is sent as zeros
        xg = torch.from_numpy(x).cuda()
        if exact:
            y = ref.rotate(cr.to_blocks(x))
        else:
            buf = xg.clone()
            codec.cluster.run([buf], _store_program(), bits, seed=seed, step=step, bucket_id=bucket)
            y = _stored_to_coeff(np.concatenate([buf.cpu().numpy(), np.zeros(-n % 1024, np.float32)]))
            # the partial last block is stored in a side buffer, not in the bucket
            y[-1] = _stored_to_coeff(codec.cluster.tail_ws[0].cpu().numpy())[0]
        words, scales = codec.compress(xg, step=step, bucket_id=bucket)
        codes, rscale = cr.quantize(y, bits, np.arange(y.shape[0]), tagbase | sch.TAG_ENCODE, step, seed, layout="tc")
        assert np.array_equal(words.cpu().numpy().view(np.uint32), cr.pack(codes, bits))
        assert np.array_equal(scales.cpu().numpy(), rscale)
        if not exact:
            assert rscale[0] == 0 and (codes[0] == cr.qmax(bits)).all()
        # decode -> inverse rotation: TF32 accuracy against the oracle's fp32 butterflies
        out = codec.decompress((words, scales), n, step=step, bucket_id=bucket, post_scale=0.25).cpu().numpy()
        rout = cr.rotate_inv(cr.dequantize(codes, rscale, bits, "tc"), ref.signs, 0.25).reshape(-1)[:n]
        tol = 4e-3 * np.repeat(np.abs(cr.to_blocks(rout)).max(axis=1), 1024)[:n] + 1e-30
        assert (np.abs(out - rout) <= tol).all()
        # one hop: decode + add rotated local + re-encode (the local operand is TF32-exact)
        x2 = small_int_grad(n, 2)
        w2, s2 = codec.dec_comp((words, scales), torch.from_numpy(x2).cuda(), step=step, bucket_id=bucket)
        v = cr.dequantize_add(codes, rscale, bits, ref.rotate(cr.to_blocks(x2)), "tc")
        c2, rs2 = cr.quantize(v, bits, np.arange(v.shape[0]), tagbase | (sch.TAG_ENCODE + 1), step, seed, layout="tc")
        assert np.array_equal(w2.cpu().numpy().view(np.uint32), cr.pack(c2, bits))
        assert np.array_equal(s2.cpu().numpy(), rs2)


@pytest.mark.parametrize("topology", sch.TOPOLOGIES)
@pytest.mark.parametrize("world,threads", [(2, 384), (4, 256), (8, 128)])
def test_tensor_core_collective_messages_match_the_simulator(world, threads, topology):
    """Every message of the collective (reduce-scatter hops and all-gather shards, as found in the
    mailboxes afterwards) equals the simulator's byte for byte on TF32-exact inputs; the result is the
    simulator's within TF32 accuracy of the inverse rotation, and identical on all ranks."""
    from dynamiq_sigcomm_artifact_b200.parallel.fused import Layout

    n, bits, seed, step, bucket = 53 * 1024 + 517, 5, 1234, 7, 2
    xs = [small_int_grad(n, 10 + r) for r in range(world)]
    want, transport = cb.simulate_allreduce(xs, bits, topology, seed=seed, step=step, bucket=bucket,
                                            return_transport=True, layout="tc")
    cl = _cluster(world, n, ctas=3, threads=threads, rotation="tc")
    for rep in range(2):  # twice: TMEM columns, barriers and slots are reused across launches
        bufs = [torch.from_numpy(x).cuda() for x in xs]
        cl.allreduce_(bufs, bits, topology, seed=seed, step=step, bucket_id=bucket)
        cl.check()
        lay = Layout(n, world, bits, "rht_tc")
        assert transport.log, "the simulator recorded no message"
        for (src, dst, slot), msg in transport.log.items():
            nb = msg.size // (128 * bits + 4)
            codes, scales = cl.slot(dst, slot, lay, nb)
            assert np.array_equal(codes.cpu().numpy().reshape(-1).view(np.uint8), msg[: nb * 128 * bits]), (src, dst, slot)
            assert np.array_equal(scales.cpu().numpy().view(np.uint8), msg[nb * 128 * bits:]), (src, dst, slot)
        assert all(torch.equal(bufs[0], b) for b in bufs), "ranks disagree"
        got = bufs[0].cpu().numpy()
        tol = 4e-3 * np.repeat(np.abs(cr.to_blocks(want[0])).max(axis=1), 1024)[:n] + 1e-30
        assert (np.abs(got - want[0]) <= tol).all()


@pytest.mark.parametrize("topology", sch.TOPOLOGIES)
def test_collective_with_tensor_core_rotation(topology):
    world, n, bits = 4, 45 * 1024 + 77, 5
    xs = [heavy_tail_grad(n, 20 + r) for r in range(world)]
    exact = np.mean(np.stack(xs).astype(np.float64), 0)
    ref_nmse = cr.nmse(cb.simulate_allreduce(xs, bits, topology, seed=4)[0], exact)
    cl = _cluster(world, n, ctas=3, threads=256, rotation="tc")
    for rep in range(2):
        bufs = [torch.from_numpy(x).cuda() for x in xs]
        cl.allreduce_(bufs, bits, topology, seed=4)
        cl.check()
        assert all(torch.equal(bufs[0], b) for b in bufs), "ranks disagree"
        got = cr.nmse(bufs[0].cpu().numpy(), exact)
        assert abs(got - ref_nmse) < 0.15 * ref_nmse, (got, ref_nmse)
    # 8-bit round trip through the standalone operators
    from dynamiq_sigcomm_artifact_b200.parallel.fused import RhtCodec

    codec = RhtCodec(8, n, seed=1, ctas=4, threads=128, rotation="tc")
    x = torch.from_numpy(xs[0]).cuda()
    back = codec.decompress(codec.compress(x), n)
    assert float((back - x).pow(2).sum() / x.pow(2).sum()) < 3e-4
    xb = x.bfloat16()
    back16 = codec.decompress(codec.compress(xb), n, dtype=torch.bfloat16)
    assert float((back16.float() - xb.float()).pow(2).sum() / xb.float().pow(2).sum()) < 1e-3


def test_tensor_core_collective_correlated_rounding_and_bf16():
    world, n = 4, 24 * 1024 + 100
    xs = [small_int_grad(n, 50 + r) for r in range(world)]
    want = cb.simulate_allreduce(xs, 5, "direct", seed=77, step=2, bucket=1, correlated=True, layout="tc")
    cl = _cluster(world, n, ctas=4, threads=128, rotation="tc")
    bufs = [torch.from_numpy(x).cuda() for x in xs]
    cl.allreduce_(bufs, 5, "direct", correlated=True, seed=77, step=2, bucket_id=1)
    cl.check()
    tol = 4e-3 * np.repeat(np.abs(cr.to_blocks(want[0])).max(axis=1), 1024)[:n] + 1e-30
    assert (np.abs(bufs[0].cpu().numpy() - want[0]) <= tol).all()
    xb = [torch.from_numpy(heavy_tail_grad(n, r)).cuda().bfloat16() for r in range(world)]
    exact = torch.stack([x.float() for x in xb]).mean(0)
    cl.allreduce_(xb, 8, "ring", seed=3)
    cl.check()
    assert all(torch.equal(xb[0], x) for x in xb)
    assert float((xb[0].float() - exact).pow(2).sum() / exact.pow(2).sum()) < 2e-3


@pytest.mark.parametrize("topology", ["ring", "direct"])
def test_collective_without_staging_buffer_is_bit_identical(topology):
    """prefetch=False halves the shared memory of a CTA and must not change a single bit."""
    from dynamiq_sigcomm_artifact_b200.parallel.fused import LocalCluster

    world, n = 4, 37 * 1024 + 5
    xs = [heavy_tail_grad(n, 90 + r) for r in range(world)]
    outs = []
    for prefetch in (True, False):
        cl = LocalCluster(world, n, ctas=5, threads=128, prefetch=prefetch)
        bufs = [torch.from_numpy(x).cuda() for x in xs]
        cl.allreduce_(bufs, 5, topology, seed=3, step=2, bucket_id=1)
        cl.check()
        outs.append(bufs[0].clone())
    assert torch.equal(outs[0], outs[1])
