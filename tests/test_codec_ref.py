"""CPU oracle: packing, rotation, quantiser statistics, determinism."""
import numpy as np
import pytest

from dynamiq_sigcomm_artifact_b200 import codec_ref as cr
from dynamiq_sigcomm_artifact_b200.utils import philox

from helpers import heavy_tail_grad


def test_philox_known_answer():
    # Random123 known-answer vectors for philox4x32-10
    assert [int(x) for x in philox.philox4x32(0, 0, 0, 0, 0, 0)] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    out = philox.philox4x32(0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF)
    assert [int(x) for x in out] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]


@pytest.mark.parametrize("bits", range(2, 9))
def test_pack_roundtrip(bits):
    rng = np.random.default_rng(bits)
    codes = rng.integers(0, 1 << bits, size=(5, 32, 32)).astype(np.uint8)
    words = cr.pack(codes, bits)
    assert words.shape == (5, bits, 32) and words.dtype == np.uint32
    assert np.array_equal(cr.unpack(words, bits), codes)


def test_pack_is_dense():
    assert cr.payload_bytes(1, 5) == 640 + 4
    assert abs(cr.wire_bits_per_element(5) - 5.03125) < 1e-12


def test_rotation_is_orthonormal_and_matches_dense_hadamard():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 1024)).astype(np.float32)
    s = philox.sign_vector(3, 1, 42)
    assert set(np.unique(s)) == {-1.0, 1.0}
    y = cr.rotate_fwd(x, s)
    h = np.array([[1.0]])
    for _ in range(10):
        h = np.block([[h, h], [h, -h]])
    dense = (x.astype(np.float64) * s) @ h.T
    assert np.allclose(y, dense, atol=2e-3)
    assert np.allclose(np.sum(y.astype(np.float64) ** 2, 1), 1024 * np.sum(x.astype(np.float64) ** 2, 1), rtol=1e-5)
    assert np.allclose(cr.rotate_inv(y, s), x, atol=1e-5)


@pytest.mark.parametrize("bits", [2, 4, 5, 8])
def test_quantiser_is_unbiased_and_bounded(bits):
    rng = np.random.default_rng(1)
    y = np.tile(rng.standard_normal((1, 1024)).astype(np.float32), (400, 1))
    codes, scale = cr.quantize(y, bits, np.arange(400), 0x100, 0, 7)
    R = cr.qmax(bits)
    assert codes.max() <= 2 * R and codes.min() >= 0
    deq = cr.dequantize(codes, scale, bits)
    assert np.max(np.abs(deq - y)) <= scale[0] * (1 + 1e-5)
    bias = np.abs(deq.mean(0) - y[0])
    assert bias.max() < 6 * scale[0] / np.sqrt(400)  # mean of 400 draws is within a few sigma


def test_encode_is_deterministic_and_stream_dependent():
    y = cr.rotate_fwd(cr.to_blocks(heavy_tail_grad(4096, 0)), philox.sign_vector(0, 0, 9))
    a = cr.encode_blocks(y, 5, np.arange(4), 0x100, 3, 9)
    b = cr.encode_blocks(y, 5, np.arange(4), 0x100, 3, 9)
    c = cr.encode_blocks(y, 5, np.arange(4), 0x101, 3, 9)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    assert a.size == cr.payload_bytes(4, 5)


def test_a_block_with_nonfinite_values_is_sent_as_zeros():
    """NaN / Inf reach every coefficient of their block; the quantiser then sends scale 0 and the
    zero code everywhere, and the neighbouring blocks are untouched."""
    x = np.ones(2048, dtype=np.float32)
    x[3], x[77] = np.inf, np.nan
    signs = philox.sign_vector(0, 0, 1)
    y = cr.rotate_fwd(cr.to_blocks(x), signs)
    assert not np.isfinite(y[0]).any() and np.isfinite(y[1]).all()
    codes, scale = cr.quantize(y, 4, np.arange(2), 0, 0, 0)
    assert scale[0] == 0 and (codes[0] == cr.qmax(4)).all() and scale[1] > 0
    back = cr.rotate_inv(cr.dequantize(codes, scale, 4), signs)
    assert (back[0] == 0).all() and cr.nmse(back[1], np.ones(1024)) < 0.2
    codes, scale = cr.quantize(np.zeros((1, 1024), np.float32), 4, np.arange(1), 0, 0, 0)
    assert scale[0] == 0 and (codes == cr.qmax(4)).all()


def test_tensor_core_layout_is_a_permutation_of_the_same_codec():
    """The two wire layouts carry the same codes in a different lane / register order."""
    y = cr.rotate_fwd(cr.to_blocks(heavy_tail_grad(4096, 4)), philox.sign_vector(0, 0, 9))
    for layout in ("simt", "tc"):
        msg = cr.encode_blocks(y, 5, np.arange(4), 0x100, 3, 9, layout=layout)
        back = cr.decode_blocks(msg, 4, 5, layout=layout)
        assert cr.nmse(back, y) < 0.02
        acc = cr.decode_add_blocks(msg, 4, 5, y, layout=layout)
        assert np.allclose(acc, back + y, rtol=1e-6, atol=1e-6)
    assert sorted(cr.RHO_TC.reshape(-1)) == list(range(1024))
