"""EDEN codec and bit-plane packing (CPU path; the GPU kernels are compared with it in the GPU test)."""
import pytest
import torch

from dynamiq_sigcomm_artifact_b200.parallel import eden


def test_lloyd_max_levels_are_the_known_optimum():
    c1, _ = eden.lloyd_max_normal(1)
    assert torch.allclose(c1, torch.tensor([-0.7979, 0.7979]), atol=1e-3)
    c2, b2 = eden.lloyd_max_normal(2)
    assert torch.allclose(c2, torch.tensor([-1.510, -0.4528, 0.4528, 1.510]), atol=2e-3)
    assert torch.allclose(b2, torch.tensor([-0.9816, 0.0, 0.9816]), atol=2e-3)
    assert eden.lloyd_max_normal(8)[0].numel() == 256


@pytest.mark.parametrize("bits", [1, 3, 8])
def test_bitplane_pack_roundtrip_cpu(bits):
    bins = torch.randint(0, 1 << bits, (1000,), dtype=torch.uint8)
    w = eden.pack_bins(bins, bits)
    assert w.shape == (bits, 32) and w.dtype == torch.int32
    assert torch.equal(eden.unpack_bins(w, bits, 1000), bins)


@pytest.mark.parametrize("bits,bound", [(1, 0.60), (2, 0.15), (4, 0.013), (8, 1e-4)])
def test_eden_nmse_matches_lloyd_max_distortion(bits, bound):
    torch.manual_seed(0)
    x = torch.randn(16 * 1024) * torch.exp(torch.randn(16).repeat_interleave(1024))
    codec = eden.Eden(bits, seed=5)
    y = codec.decompress(codec.compress(x))
    nmse = float((y - x).pow(2).sum() / x.pow(2).sum())
    assert nmse < bound, nmse
    assert abs(codec.wire_bits_per_element() - (bits + 0.03125)) < 1e-9


@pytest.mark.gpu
def test_eden_gpu_matches_cpu():
    torch.manual_seed(1)
    x = torch.randn(8 * 1024 + 100)
    for bits in (2, 5):
        cpu = eden.Eden(bits, seed=3)
        words_c, scale_c, n = cpu.compress(x)
        gpu = eden.Eden(bits, seed=3)
        words_g, scale_g, _ = gpu.compress(x.cuda())
        same = (words_g.cpu() == words_c).float().mean()
        assert same > 0.98  # the two rotations differ in the last bits, which moves few bins
        assert torch.allclose(scale_g.cpu(), scale_c, rtol=1e-3)
        back = gpu.decompress((words_g, scale_g, n)).cpu()
        ref = cpu.decompress((words_c, scale_c, n))
        assert float((back - ref).pow(2).sum() / ref.pow(2).sum()) < 5e-3
        bins = torch.randint(0, 1 << bits, (5000,), dtype=torch.uint8)
        assert torch.equal(eden.pack_bins(bins.cuda(), bits).cpu(), eden.pack_bins(bins, bits))
        assert torch.equal(eden.unpack_bins(eden.pack_bins(bins.cuda(), bits), bits, 5000).cpu(), bins)
