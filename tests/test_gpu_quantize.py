"""GPU parity of the quantizer/dequantizer kernels through the C ABI: bit-exact against the oracle."""
import numpy as np
import pytest
import torch

from oracle import quant

pytestmark = pytest.mark.gpu


def _weights(n, k, seed, dtype):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02).to(dtype)


_NAMES = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}


@pytest.mark.parametrize("mode", ["mlx", "doc"])
@pytest.mark.parametrize("bits", [3, 4, 5, 6, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_quantize_bit_exact(lib_built, mode, bits, dtype):
    from mflux_b200 import ops

    w = _weights(384, 1024, 11, dtype)
    wq, s, b = ops.quantize_affine(w.cuda(), 64, bits, mode)
    torch.cuda.synchronize()
    pq, ps, pb = quant.quantize_affine(w, 64, bits, mode, dtype=_NAMES[dtype])
    np.testing.assert_array_equal(wq.cpu().numpy(), pq)
    np.testing.assert_array_equal(s.float().cpu().numpy(), ps)
    np.testing.assert_array_equal(b.float().cpu().numpy(), pb)
    assert s.dtype == dtype and b.dtype == dtype and wq.dtype == torch.uint32


def test_quantize_config1_full_size_bit_exact(lib_built):
    """W fp32 [12288, 3072] ~ N(0, 0.02), bits 4, group 64, seed 0 (the single-linear configuration)."""
    from mflux_b200 import ops

    w = _weights(12288, 3072, 0, torch.float32)
    wq, s, b = ops.quantize_affine(w.cuda(), 64, 4)
    pq, ps, pb = quant.quantize_affine(w, 64, 4)
    assert wq.shape == (12288, 384) and s.shape == (12288, 48)
    np.testing.assert_array_equal(wq.cpu().numpy(), pq)
    np.testing.assert_array_equal(s.cpu().numpy(), ps)
    np.testing.assert_array_equal(b.cpu().numpy(), pb)


def test_quantize_edge_groups(lib_built):
    """Constant groups, all-zero groups, a single outlier, and values that tie at .5 codes."""
    from mflux_b200 import ops

    w = torch.zeros(8, 128)
    w[1] = 0.25
    w[2, :64] = torch.linspace(-1, 1, 64)
    w[3, 5] = 100.0
    w[4] = torch.arange(128) % 16 * 0.5 - 3.75  # exact half-way points for scale 1
    w[5] = -torch.arange(128, dtype=torch.float32)
    for mode in ("mlx", "doc"):
        for bits in (3, 4, 5, 6, 8):
            wq, s, b = ops.quantize_affine(w.cuda(), 64, bits, mode)
            pq, ps, pb = quant.quantize_affine(w, 64, bits, mode)
            np.testing.assert_array_equal(wq.cpu().numpy(), pq)
            np.testing.assert_array_equal(s.cpu().numpy(), ps)
            np.testing.assert_array_equal(b.cpu().numpy(), pb)


@pytest.mark.parametrize("bits", [3, 4, 5, 6, 8])
@pytest.mark.parametrize("sb_dtype", [torch.float32, torch.bfloat16])
def test_dequantize_bit_exact_and_round_trip(lib_built, bits, sb_dtype):
    from mflux_b200 import ops

    w = _weights(256, 512, 3, sb_dtype)
    wq, s, b = ops.quantize_affine(w.cuda(), 64, bits)
    w_hat = ops.dequantize_affine(wq, s, b, 64, bits, dtype=torch.float32)
    ref = quant.dequantize_affine(wq.cpu().numpy(), s.float().cpu().numpy(), b.float().cpu().numpy(), 64, bits)
    np.testing.assert_array_equal(w_hat.cpu().numpy(), ref)
    # round trip: every value lands within one quantization step of where it started
    err = (w_hat.cpu() - w.float()).abs().reshape(256, 8, 64).amax(-1)
    # (scales/biases stored in bf16 move every code by their own rounding error as well)
    sf, bf = s.float().cpu().abs(), b.float().cpu().abs()
    slack = 0.0 if sb_dtype == torch.float32 else 2.0 ** -8
    assert (err <= sf * (1.01 + slack * ((1 << bits) - 1)) + bf * slack + 1e-9).all()


def test_quantize_rejects_bad_arguments(lib_built):
    from mflux_b200 import ops

    with pytest.raises(ValueError):
        ops.quantize_affine(torch.zeros(4, 96, device="cuda"), 64, 4)
    with pytest.raises(ValueError):
        ops.quantize_affine(torch.zeros(4, 64, device="cuda"), 64, 7)
    with pytest.raises(RuntimeError):
        ops.quantize_affine(torch.zeros(4, 64), 64, 4)
