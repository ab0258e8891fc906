"""tcgen05 / TMEM Hadamard kernel against a float64 dense Hadamard product."""
import numpy as np
import pytest
import torch

from dynamiq_sigcomm_artifact_b200.utils import philox

pytestmark = pytest.mark.gpu


def _dense(x: np.ndarray, signs: np.ndarray) -> np.ndarray:
    h = np.array([[1.0]])
    for _ in range(10):
        h = np.block([[h, h], [h, -h]])
    return (x.astype(np.float64) * signs) @ h.T / 32.0


@pytest.mark.parametrize("nblocks", [4, 12, 1000])
def test_fwht_matches_dense_hadamard(nblocks):
    from dynamiq_sigcomm_artifact_b200.ops.fwht import fwht1024

    rng = np.random.default_rng(nblocks)
    x = (rng.standard_normal((nblocks, 1024)) * np.exp(rng.standard_normal((nblocks, 1)))).astype(np.float32)
    x[0, 7] = np.inf  # sanitised to 0
    seed, step, bucket = 77, 3, 2
    y = fwht1024(torch.from_numpy(x).cuda(), seed, step, bucket).cpu().numpy()
    xs = np.where(np.isfinite(x), x, 0.0)
    want = _dense(xs, philox.sign_vector(step, bucket, seed))
    err = np.abs(y - want).max(axis=1) / np.abs(want).max(axis=1)
    assert err.max() < 2e-5, err.max()
    # orthonormal: energy preserved
    assert np.allclose((y.astype(np.float64) ** 2).sum(1), (xs.astype(np.float64) ** 2).sum(1), rtol=1e-4)


def test_fwht_roundtrip_and_padding():
    from dynamiq_sigcomm_artifact_b200.ops.fwht import fwht1024, ifwht1024

    x = torch.randn(5000, device="cuda")  # not a multiple of 4096: padded internally
    y = fwht1024(x, seed=5)
    back = ifwht1024(torch.cat([y, y.new_zeros(0)]), seed=5)
    # the padded tail is part of the transform, so invert on the padded vector
    full = torch.zeros(8192, device="cuda")
    full[:5000] = x
    yf = fwht1024(full, seed=5)
    assert torch.allclose(ifwht1024(yf, seed=5), full, atol=2e-5)
    assert y.shape == x.shape and back.shape == x.shape
    cpu = fwht1024(full.cpu(), seed=5)
    assert torch.allclose(yf.cpu(), cpu, atol=2e-4)


@pytest.mark.parametrize("log2d", [6, 9, 10, 12, 13, 17, 20])
def test_whole_vector_transform_matches_butterflies(log2d):
    """Tensor-core 1024-blocks + strided upper levels = the plain butterfly transform of the whole vector."""
    from dynamiq_sigcomm_artifact_b200.ops.fwht import fwht_pow2

    d = 1 << log2d
    g = torch.Generator().manual_seed(log2d)
    x = torch.randn(d, generator=g)
    want = fwht_pow2(x.double().float(), normalize=True)  # CPU butterflies
    got = fwht_pow2(x.cuda(), normalize=True).cpu()
    assert float((got - want).abs().max()) < 2e-5 * max(1.0, float(want.abs().max()))
    # orthonormal and an involution
    back = fwht_pow2(got.cuda(), normalize=True).cpu()
    assert float((back - x).abs().max()) < 5e-5
