"""CPU tests of the quantizer oracle: algebraic properties of both quantizer flavours and packing."""
import numpy as np
import pytest

from oracle import quant


def _w(n, k, seed=0, std=0.02):
    return (np.random.default_rng(seed).standard_normal((n, k)) * std).astype(np.float32)


@pytest.mark.parametrize("bits", [3, 4, 5, 6, 8])
@pytest.mark.parametrize("mode", ["mlx", "doc"])
def test_shapes_and_ranges(bits, mode):
    w = _w(16, 256)
    packed, s, b = quant.quantize_affine(w, 64, bits, mode)
    assert packed.dtype == np.uint32 and packed.shape == (16, 256 * bits // 32)
    assert s.shape == b.shape == (16, 4)
    q = quant.unpack_codes(packed, bits)
    assert q.min() >= 0 and q.max() <= (1 << bits) - 1


@pytest.mark.parametrize("bits", [3, 4, 5, 6, 8])
def test_doc_mode_matches_formula(bits):
    w = _w(8, 128, seed=1)
    packed, s, b = quant.quantize_affine(w, 64, bits, "doc")
    g = w.reshape(8, 2, 64)
    np.testing.assert_array_equal(b, g.min(-1))
    np.testing.assert_array_equal(s, ((g.max(-1) - g.min(-1)) / np.float32((1 << bits) - 1)).astype(np.float32))
    q = quant.unpack_codes(packed, bits).reshape(8, 2, 64)
    # extremes map to the end codes
    assert (q.min(-1) == 0).all() and (q.max(-1) == (1 << bits) - 1).all()


@pytest.mark.parametrize("bits", [3, 4, 5, 6, 8])
def test_mlx_mode_zero_is_representable_and_error_bounded(bits):
    w = _w(32, 512, seed=2)
    packed, s, b = quant.quantize_affine(w, 64, bits, "mlx")
    # 0.0 must sit exactly on the grid: -bias/scale is an integer code
    code0 = -b / s
    np.testing.assert_allclose(code0, np.rint(code0), atol=1e-3)
    w_hat = quant.dequantize_affine(packed, s, b, 64, bits)
    err = np.abs(w_hat - w).reshape(32, 8, 64).max(-1)
    # snapping the scale to edge/rint(edge/scale) can shrink it by up to 1/15, which clips the far
    # extreme by up to one step; everything else rounds to the nearest code
    assert (err <= np.abs(s) * 1.01 + 1e-9).all()
    assert np.median(err / np.abs(s)) <= 0.51


def test_packing_is_little_end_first():
    w = np.tile(np.linspace(-1, 1, 64, dtype=np.float32), (1, 1))
    packed, s, b = quant.quantize_affine(w, 64, 4, "doc")
    q = np.clip(np.rint((w[0] - b[0, 0]) / s[0, 0]), 0, 15).astype(np.uint32)
    word0 = sum(int(q[j]) << (4 * j) for j in range(8))
    assert int(packed[0, 0]) == word0
    packed8, s8, b8 = quant.quantize_affine(w, 64, 8, "doc")
    q8 = np.clip(np.rint((w[0] - b8[0, 0]) / s8[0, 0]), 0, 255).astype(np.uint32)
    assert int(packed8[0, 0]) == sum(int(q8[j]) << (8 * j) for j in range(4))


def test_constant_and_zero_groups():
    w = np.zeros((2, 64), np.float32)
    w[1] = 0.25
    for mode in ("mlx", "doc"):
        packed, s, b = quant.quantize_affine(w, 64, 4, mode)
        w_hat = quant.dequantize_affine(packed, s, b, 64, 4)
        assert np.isfinite(w_hat).all()
        np.testing.assert_allclose(w_hat, w, atol=1e-6)


def test_row_concatenation_is_bit_identical():
    """Quantizing row-stacked matrices equals stacking their quantizations (fused q|k|v layout)."""
    a, b_ = _w(8, 128, 3), _w(8, 128, 4)
    pa = quant.quantize_affine(a, 64, 4)
    pb = quant.quantize_affine(b_, 64, 4)
    pc = quant.quantize_affine(np.concatenate([a, b_]), 64, 4)
    for x, y, z in zip(pa, pb, pc):
        np.testing.assert_array_equal(np.concatenate([x, y]), z)


def test_bf16_storage_rounding():
    w = quant.round_to_dtype(_w(4, 64, 5), "bf16")
    _, s, b = quant.quantize_affine(w, 64, 4, "mlx", dtype="bf16")
    np.testing.assert_array_equal(s, quant.round_to_dtype(s, "bf16"))
    import torch

    t = torch.from_numpy(_w(4, 64, 6))
    np.testing.assert_array_equal(quant.round_to_dtype(t.numpy(), "bf16"), t.to(torch.bfloat16).float().numpy())


def test_qlinear_matches_dense():
    w = _w(32, 128, 7)
    x = np.random.default_rng(8).standard_normal((5, 128)).astype(np.float32)
    bias = _w(1, 32, 9)[0]
    packed, s, b = quant.quantize_affine(w, 64, 8)
    y = quant.qlinear(x, packed, s, b, bias, 64, 8)
    assert quant.rel_l2(y, x @ w.T + bias) < 2e-2


def test_bad_arguments():
    with pytest.raises(ValueError):
        quant.quantize_affine(_w(4, 96), 64, 4)
    with pytest.raises(ValueError):
        quant.quantize_affine(_w(4, 64), 64, 7)


@pytest.mark.parametrize("bits", [3, 5, 6])
def test_odd_widths_pack_as_mlx_byte_groups(bits):
    """MLX packs 3- and 5-bit codes eight at a time into 3 / 5 bytes and 6-bit codes four at a time into 3 bytes,
    each group a little-endian integer with code i at bits [i*bits, (i+1)*bits): the bytes of the packed words must
    read that way, and the packed row has K*bits/32 words."""
    rng = np.random.default_rng(bits)
    q = rng.integers(0, 1 << bits, size=(3, 64)).astype(np.uint32)
    packed = quant.pack_codes(q, bits)
    assert packed.shape == (3, 64 * bits // 32)
    per, nbytes = (8, bits) if bits in (3, 5) else (4, 3)
    raw = packed.view(np.uint8).reshape(3, -1)
    for row in range(3):
        for grp in range(64 // per):
            v = sum(int(q[row, grp * per + i]) << (bits * i) for i in range(per))
            want = [(v >> (8 * j)) & 0xFF for j in range(nbytes)]
            assert list(raw[row, grp * nbytes:(grp + 1) * nbytes]) == want
    np.testing.assert_array_equal(quant.unpack_codes(packed, bits), q)
