"""THC quantise / dequantise kernels against the plain PyTorch chain they replace (fp32, same rounding
offsets from the counter-based generator)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d,levels,world", [(1 << 12, 31, 8), ((1 << 14) + 0, 15, 2), (64, 31, 4)])
def test_thc_kernels_match_the_torch_chain(d, levels, world):
    from dynamiq_sigcomm_artifact_b200 import ops
    from dynamiq_sigcomm_artifact_b200.parallel.baselines import THC_T
    from dynamiq_sigcomm_artifact_b200.parallel.torch_backend import uniform_bytes

    dq = ops.require()
    torch.manual_seed(d)
    y = torch.randn(d, device="cuda") * 3
    y[7] = 1e6  # clipped
    stats = torch.rand(world + 1, device="cuda") * 50 + 1
    stats[world] = -3.25
    scale = THC_T / math.sqrt(d)
    rng = (torch.tensor(scale, device="cuda", dtype=torch.float32) * stats[:world].max()).clamp_min(1e-30)
    tag, step, seed = 0x00123045, 9, (5 << 32) | 77
    u = (uniform_bytes(d, tag, step, seed, "cuda").float() + 0.5) / 256.0
    t = (y.clamp(-rng, rng) + rng) / (2 * rng) * (levels - 1)
    want = torch.floor(t + u).clamp_(0, levels - 1)
    got = y.clone()
    dq.thc_quantize_(got, stats, world, scale, levels, tag, step, seed)
    assert torch.equal(got, want)
    again = y.clone()
    dq.thc_quantize_(again, stats, world, scale, levels, tag, step, seed)
    assert torch.equal(again, got)  # reproducible from the seed
    other = y.clone()
    dq.thc_quantize_(other, stats, world, scale, levels, tag + 1, step, seed)
    assert not torch.equal(other, got)
    total = want * world  # as if every rank had sent the same bins
    # a tensor divisor makes PyTorch divide (a Python scalar would become a multiplication by its reciprocal)
    top = torch.full((), float(levels - 1), device="cuda")
    ref = (total / top * (2 * rng) - world * rng) / world
    ref[0] = stats[world] / world
    out = total.clone()
    dq.thc_dequantize_(out, stats, world, scale, levels)
    assert torch.equal(out, ref)
    assert float((out[1:] - y.clamp(-rng, rng)[1:]).abs().max()) <= float(2 * rng / (levels - 1)) * 1.01
