"""Torch codecs and bit allocation (CPU): wire sizes, round trips, statistics, controller."""
import numpy as np
import pytest
import torch

from dynamiq_sigcomm_artifact_b200 import bitalloc
from dynamiq_sigcomm_artifact_b200.parallel import codecs
from dynamiq_sigcomm_artifact_b200.parallel.torch_backend import philox4x32_torch, plan_rounds, uniform_bytes
from dynamiq_sigcomm_artifact_b200.utils import philox


def test_torch_philox_matches_numpy():
    c = torch.arange(100, dtype=torch.int64)
    got = philox4x32_torch(c, c * 3 + 1, torch.tensor([7]), torch.tensor([0xFFFFFFFF]), 0xDEADBEEF, 0x12345678)
    want = philox.philox4x32(np.arange(100), np.arange(100) * 3 + 1, 7, 0xFFFFFFFF, 0xDEADBEEF, 0x12345678)
    for g, w in zip(got, want):
        assert np.array_equal(g.numpy().astype(np.uint32), w)
    u = uniform_bytes(100000, 3, 4, 5, "cpu").float()
    assert abs(float(u.mean()) - 127.5) < 1.0


@pytest.mark.parametrize("bits,nbytes", [(2, 82), (4, 146), (8, 274)])
def test_superchunk_wire_size_matches_reference(bits, nbytes):
    assert codecs.superchunk_bytes(bits) == nbytes
    assert codecs.SuperchunkCodec(bits).message_bytes(256 * 7) == 7 * nbytes
    assert abs(nbytes * 8 / 256 - (bits + 0.5625)) < 1e-12


@pytest.mark.parametrize("lattice", ["aee", "mee"])
@pytest.mark.parametrize("bits", [2, 4, 8])
def test_superchunk_roundtrip_error_and_unbiasedness(bits, lattice):
    torch.manual_seed(0)
    x = torch.randn(256 * 40) * torch.exp(torch.randn(256 * 40 // 16).repeat_interleave(16))
    acc = torch.zeros_like(x)
    reps = 64
    for step in range(reps):
        c = codecs.SuperchunkCodec(bits, lattice, seed=3, step=step)
        msg = c.encode(x, 0, 0x100)
        assert msg.numel() == c.message_bytes(x.numel()) and msg.dtype == torch.uint8
        acc += c.decode(msg, x.numel())
    one = c.decode(msg, x.numel())
    rel = float((one - x).pow(2).sum() / x.pow(2).sum())
    assert rel < {2: 0.6, 4: 0.05, 8: 5e-4}[bits] * (3 if lattice == "mee" and bits == 8 else 1.5)
    bias = float(((acc / reps) - x).pow(2).sum() / x.pow(2).sum())
    assert bias < rel / 8  # averaging independent draws removes most of the error: rounding is unbiased
    # zeros and a non-finite input survive
    z = torch.zeros(256)
    assert float(c.decode(c.encode(z, 0, 0), 256).abs().max()) == 0.0
    y = x[:256].clone()
    y[3] = float("inf")
    assert torch.isfinite(c.decode(c.encode(y, 0, 0), 256)).all()


def test_superchunk_scale_rounds_up_so_codes_never_clip():
    torch.manual_seed(1)
    x = torch.randn(256 * 16) * 10
    c = codecs.SuperchunkCodec(4, "aee")
    out = c.decode(c.encode(x, 0, 1), x.numel())
    # round-up chunk scales: |decoded| can exceed |x| by at most one quantisation step of its chunk
    step = x.view(-1, 16).abs().amax(1, keepdim=True) / 7 * 1.02 + 1e-6
    assert bool(((out - x).view(-1, 16).abs() <= step * 1.01).all())


@pytest.mark.parametrize("fmt,bits", [("fp8", 8.25), ("fp6", 6.25), ("fp4", 4.25)])
def test_block_float_formats(fmt, bits):
    torch.manual_seed(2)
    c = codecs.BlockFloatCodec(fmt)
    x = torch.randn(1024 * 5)
    msg = c.encode(x, 0, 0)
    assert msg.numel() * 8 / x.numel() == bits
    y = c.decode(msg, x.numel())
    rel = float((y - x).pow(2).sum() / x.pow(2).sum())
    assert rel < {"fp8": 2e-3, "fp6": 2e-2, "fp4": 8e-2}[fmt]
    assert torch.equal(c.decode(c.encode(y, 0, 0), x.numel()), y)  # values on the grid are fixed points
    assert c.table.numel() == {"fp8": 127, "fp6": 32, "fp4": 8}[fmt]


def test_cast_and_bins_codecs():
    x = torch.randn(1000)
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        c = codecs.CastCodec(dt)
        assert torch.equal(c.decode(c.encode(x, 0, 0), 1000), x.to(dt).float())
    b = torch.randint(-100, 100, (77,)).float()
    c = codecs.IntBinsCodec()
    assert torch.equal(c.decode(c.encode(b, 0, 0), 77), b)


def test_threshold_split_matches_reference_rule():
    norms = torch.tensor([5.0, 1.0, 9.0, 3.0, 7.0, 2.0, 8.0, 4.0, 6.0, 0.5])
    g = bitalloc.split_by_thresholds(norms, {8: 0.2, 4: 0.5, 2: 0.3})
    assert sorted(g[8].tolist()) == [2, 6] and sorted(g[2].tolist()) == [1, 5, 9] and g[4].numel() == 5
    g = bitalloc.split_by_thresholds(norms, {8: 0.0, 4: 1.0, 2: 0.0})
    assert g[4].numel() == 10 and g[8].numel() == 0 and g[2].numel() == 0


def test_dynamic_bitrate_controller_converges_to_budget():
    torch.manual_seed(3)
    ctl = bitalloc.DynamicBitrateController(5)
    assert ctl.u == 60.0
    for step in range(6):
        norms = torch.exp(torch.randn(20000) * 3 + step * 0.2)
        ctl.observe(norms)
        ctl.end_of_step()
        avg = bitalloc.average_bits([norms], ctl.u)
        assert abs(avg - (5 - 0.625)) <= 0.1 + 1e-6 or step == 0 and abs(avg - 4.375) < 0.2
    q = bitalloc.qbits(norms, ctl.u)
    assert set(q.tolist()) <= {2, 4, 8}
    d = ctl.state_dict()
    c2 = bitalloc.DynamicBitrateController(5)
    c2.load_state_dict(d)
    assert c2.u == ctl.u and c2.initialised


@pytest.mark.parametrize("topology", ["ring", "butterfly", "direct"])
def test_round_plan_covers_program(topology):
    from dynamiq_sigcomm_artifact_b200.parallel import schedules as sch

    rounds = plan_rounds(4, topology)
    for r in range(4):
        flat = [st for rnd in rounds for st in rnd[r]]
        assert flat == sch.build_program(r, 4, topology)
    assert len(rounds) <= 6


def test_minifloat_codec_rounds_to_the_grid_and_saturates():
    from dynamiq_sigcomm_artifact_b200.parallel.codecs import MinifloatCodec

    c = MinifloatCodec("fp4")
    v = torch.tensor([0.0, 0.2, 0.26, 0.8, 1.2, 2.4, 3.4, 5.1, 7.0, -9.0, 0.74])
    back = c.decode(c.encode(v, 0, 0), v.numel())
    assert back.tolist() == [0.0, 0.0, 0.5, 1.0, 1.0, 2.0, 3.0, 6.0, 6.0, -6.0, 0.5]
    from dynamiq_sigcomm_artifact_b200.config import parse_method

    s = parse_method("fp4_shared")
    assert s.hook == "fpx" and s.shared_scale and s.fpx_format == "fp4" and not parse_method("fp4").shared_scale


@pytest.mark.parametrize("bits,lattice", [(4, "mee"), (5, "mee"), (8, "aee"), (2, "mee")])
def test_simulation_hierarchical_codec_is_unbiased_and_bounded(bits, lattice):
    from dynamiq_sigcomm_artifact_b200.parallel.codecs import SIM_EPS, SimHierarchicalCodec

    torch.manual_seed(bits)
    n = 16 * 16 * 8
    x = torch.randn(n) * torch.exp(torch.randn(n // 16)).repeat_interleave(16)
    acc = torch.zeros(n)
    reps = 200
    for rep in range(reps):
        c = SimHierarchicalCodec(bits, lattice, seed=3, step=rep, bucket=1)
        msg = c.encode(x, 0, 0x100)
        assert msg.numel() == c.message_bytes(n)
        y = c.decode(msg, n)
        acc += y
    mean = acc / reps
    # unbiased: the error of the mean of many independent roundings (codes and chunk scales both round
    # stochastically) falls like 1 / reps; one rounding stays within the width's error level
    nm = lambda a: float((a - x).pow(2).sum() / x.pow(2).sum())
    single, averaged = nm(y), nm(mean)
    assert single < {2: 0.5, 4: 0.05, 5: 0.02, 8: 3e-4}[bits], single
    assert averaged < single / (reps / 4), (single, averaged)
    assert SIM_EPS[5] == 0.18
    with pytest.raises(ValueError):
        SimHierarchicalCodec(3)
