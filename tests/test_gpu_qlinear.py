"""GPU parity of the quantized linear layer (tcgen05 kernel) through the C ABI.

Tolerance: rel-L2 <= 1e-2 against the float32 oracle (dequantize, then X @ W^T + b in float32),
the bound for bf16 layer outputs against the float32 result.
"""
import numpy as np
import pytest
import torch

from oracle import quant

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _case(m, n, k, bits, seed, w_dtype=torch.float32, bias=True):
    g = torch.Generator(device="cpu").manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * 0.02).to(w_dtype)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    b = (torch.randn(n, generator=g) * 0.02).to(w_dtype) if bias else None
    return w, x, b


def _oracle(w, x, b, bits, w_dtype_name):
    pq, ps, pb = quant.quantize_affine(w, 64, bits, dtype=w_dtype_name)
    return pq, ps, pb, quant.qlinear(x, pq, ps, pb, b, 64, bits)


def _run(w, x, b, bits, **kw):
    from mflux_b200 import ops

    wq, s, bi = ops.quantize_affine(w.cuda(), 64, bits)
    y = ops.qlinear(x.cuda(), wq, s, bi, None if b is None else b.cuda(), bits=bits, **kw)
    torch.cuda.synchronize()
    assert ops.poll_device_status() == 0
    return wq, s, bi, y


def test_config1_single_linear(lib_built):
    """M=4096, N=12288, K=3072, W4 g64, fp32 weights, seed 0."""
    w, x, b = _case(4096, 12288, 3072, 4, 0)
    pq, ps, pb, ref = _oracle(w, x, b, 4, "f32")
    wq, s, bi, y = _run(w, x, b, 4)
    np.testing.assert_array_equal(wq.cpu().numpy(), pq)
    assert y.dtype == torch.bfloat16 and y.shape == (4096, 12288)
    err = quant.rel_l2(y, ref)
    assert err <= TOL, err


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("nk", [(3072, 3072), (9216, 3072), (3072, 12288)])
@pytest.mark.parametrize("m", [256, 1024])
def test_sweep_shapes(lib_built, bits, nk, m):
    n, k = nk
    w, x, b = _case(m, n, k, bits, hash((bits, n, k, m)) % (2**31), torch.bfloat16)
    _, _, _, ref = _oracle(w, x, b, bits, "bf16")
    _, _, _, y = _run(w, x, b, bits)
    err = quant.rel_l2(y, ref)
    assert err <= TOL, err


@pytest.mark.parametrize("bits", [3, 5, 6])
@pytest.mark.parametrize("mnk", [(300, 520, 320), (16, 1032, 192), (1, 264, 256), (4096, 3072, 3072)])
def test_odd_code_widths(lib_built, bits, mnk):
    """3-, 5- and 6-bit weights (the other choices of the reference's -q flag, cli/defaults/defaults.py:63): codes
    packed as MLX packs them (bit stream, codes straddling words), widened when the weight is prepared; both the
    tensor-core kernel and the small-M kernel against the float32 oracle, rel-L2 <= 1e-2."""
    m, n, k = mnk
    w, x, b = _case(m, n, k, bits, 300 + bits + m, torch.bfloat16)
    pq, _, _, ref = _oracle(w, x, b, bits, "bf16")
    wq, _, _, y = _run(w, x, b, bits)
    assert wq.shape == (n, k * bits // 32)
    np.testing.assert_array_equal(wq.cpu().numpy(), pq)
    err = quant.rel_l2(y, ref)
    assert err <= TOL, err


def test_odd_width_model_step(lib_built):
    """A FLUX-shaped step quantized to 6 and to 3 bits (Flux1(quantize=6 | 3)) against the oracle."""
    from mflux_b200.flux import FluxConfig, Transformer
    from oracle import flux as oflux

    cfg = FluxConfig(hidden=256, heads=2, num_joint=1, num_single=1, context_dim=128, pooled_dim=64)
    g = torch.Generator(device="cpu").manual_seed(17)
    lat = torch.randn(1, 64, cfg.in_channels, generator=g)
    ctx = torch.randn(1, 24, cfg.context_dim, generator=g).to(torch.bfloat16)
    pooled = torch.randn(1, cfg.pooled_dim, generator=g).to(torch.bfloat16)
    ts, gd = torch.full((1,), 400.0), torch.full((1,), 3500.0)
    for bits in (6, 3):
        model = Transformer(cfg, bits=bits, device="cuda", seed=bits)
        out = model(lat.cuda(), ctx.cuda(), pooled.cuda(), ts.cuda(), gd.cuda(), 128, 128)
        ref = oflux.forward(model, lat.to(torch.bfloat16), ctx, pooled, ts, gd, 128, 128)
        assert quant.rel_l2(out, ref.numpy()) <= TOL


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("w_dtype,name", [(torch.float16, "f16"), (torch.float32, "f32")])
def test_scales_wider_than_bf16_are_rounded_within_tolerance(lib_built, bits, w_dtype, name):
    """The matmul kernels carry scale and bias of every group as bf16 (8 mantissa bits) whatever dtype the
    checkpoint stores them in; MLX keeps f16 / f32 scales as they are. The rounding moves every dequantized weight
    by at most 2^-9 relative to scale and bias, which stays far inside the 1e-2 bound against an oracle that uses
    the unrounded f16 / f32 values."""
    w, x, b = _case(700, 1024, 1024, bits, 77 + bits, w_dtype)
    _, _, _, ref = _oracle(w, x, b, bits, name)
    _, s, _, y = _run(w, x, b, bits)
    assert s.dtype == w_dtype
    err = quant.rel_l2(y, ref)
    assert err <= TOL, err
    w1, x1, b1 = _case(8, 1024, 1024, bits, 78 + bits, w_dtype)      # small-M kernel, same blob format
    _, _, _, ref1 = _oracle(w1, x1, b1, bits, name)
    _, _, _, y1 = _run(w1, x1, b1, bits)
    assert quant.rel_l2(y1, ref1) <= TOL


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("mnk", [(1, 64, 64), (7, 8, 128), (129, 264, 192), (300, 1000, 320), (128, 256, 64),
                                 (513, 520, 3840)])
def test_ragged_edges(lib_built, bits, mnk):
    """Row, column and depth tails: M not a multiple of 128, N not a multiple of 256, one k-block."""
    m, n, k = mnk
    w, x, b = _case(m, n, k, bits, 100 + m + n + k, torch.bfloat16)
    _, _, _, ref = _oracle(w, x, b, bits, "bf16")
    _, _, _, y = _run(w, x, b, bits)
    err = quant.rel_l2(y, ref)
    assert err <= TOL, err
    # fp32 output leaves only the operand rounding
    _, _, _, y32 = _run(w, x, b, bits, out_dtype=torch.float32)
    assert quant.rel_l2(y32, ref) <= TOL


def test_no_bias_and_canary(lib_built):
    """Rows/columns beyond the problem must not be written: output padded with a canary."""
    from mflux_b200 import ops

    m, n, k = 200, 328, 256
    w, x, _ = _case(m, n, k, 4, 5, torch.bfloat16, bias=False)
    wq, s, bi = ops.quantize_affine(w.cuda(), 64, 4)
    buf = torch.full((m + 64, n + 64), 7.0, dtype=torch.bfloat16, device="cuda")
    out = buf[:m, :n]
    ops.qlinear(x.cuda(), wq, s, bi, None, bits=4, out=out)
    torch.cuda.synchronize()
    assert (buf[m:] == 7.0).all() and (buf[:, n:] == 7.0).all()
    ref = quant.qlinear(x, wq.cpu().numpy(), s.float().cpu().numpy(), bi.float().cpu().numpy(), None, 64, 4)
    assert quant.rel_l2(out, ref) <= TOL


def test_batched_strided_views(lib_built):
    """[batch, rows, K] slices of a larger sequence buffer in, slices of another buffer out."""
    from mflux_b200 import ops

    bsz, s_all, off, rows, k, n = 3, 640, 128, 500, 256, 512
    g = torch.Generator(device="cpu").manual_seed(9)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    seq = torch.randn(bsz, s_all, k, generator=g).to(torch.bfloat16)
    wq, s, bi = ops.quantize_affine(w.cuda(), 64, 4)
    seq_d = seq.cuda()
    out_buf = torch.zeros(bsz, s_all, 2 * n, dtype=torch.bfloat16, device="cuda")
    ops.qlinear(seq_d[:, off:off + rows], wq, s, bi, None, bits=4, out=out_buf[:, off:off + rows, n:])
    torch.cuda.synchronize()
    ref = quant.qlinear(seq[:, off:off + rows], wq.cpu().numpy(), s.float().cpu().numpy(),
                        bi.float().cpu().numpy(), None, 64, 4)
    assert quant.rel_l2(out_buf[:, off:off + rows, n:], ref) <= TOL
    assert (out_buf[:, :off] == 0).all() and (out_buf[:, off + rows:] == 0).all() and (out_buf[..., :n] == 0).all()


@pytest.mark.parametrize("epi", ["gelu", "gelu_approx", "silu"])
def test_activation_epilogues(lib_built, epi):
    m, n, k = 256, 512, 256
    w, x, b = _case(m, n, k, 4, 21, torch.bfloat16)
    _, _, _, ref = _oracle(w, x, b, 4, "bf16")
    t = torch.from_numpy(ref) * 8  # spread the values over the non-linear range
    _, _, _, y = _run(w * 8, x, b * 8, 4, epilogue=epi, out_dtype=torch.float32)
    _, _, _, ref8 = _oracle(w * 8, x, b * 8, 4, "bf16")
    t = torch.from_numpy(ref8)
    act = {"gelu": torch.nn.functional.gelu(t), "gelu_approx": torch.nn.functional.gelu(t, approximate="tanh"),
           "silu": torch.nn.functional.silu(t)}[epi]
    assert quant.rel_l2(y, act.numpy()) <= TOL


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gate_residual_epilogue(lib_built, dtype):
    from mflux_b200 import ops

    bsz, rows, k, n = 2, 300, 256, 512
    g = torch.Generator(device="cpu").manual_seed(33)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    bias = (torch.randn(n, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(bsz, rows, k, generator=g).to(torch.bfloat16)
    gate = torch.randn(bsz, n, generator=g).to(torch.bfloat16)
    res = torch.randn(bsz, rows, n, generator=g).to(dtype)
    wq, s, bi = ops.quantize_affine(w.cuda(), 64, 4)
    y = ops.qlinear(x.cuda(), wq, s, bi, bias.cuda(), bits=4, epilogue="gate_residual", gate=gate.cuda(),
                    residual=res.cuda())
    torch.cuda.synchronize()
    lin = quant.qlinear(x, wq.cpu().numpy(), s.float().cpu().numpy(), bi.float().cpu().numpy(), bias, 64, 4)
    ref = res.float().numpy() + gate.float().numpy()[:, None, :] * lin
    assert y.dtype == dtype
    assert quant.rel_l2(y, ref) <= TOL


def test_deterministic_run_to_run(lib_built):
    w, x, b = _case(512, 768, 512, 4, 77, torch.bfloat16)
    _, _, _, y1 = _run(w, x, b, 4)
    _, _, _, y2 = _run(w, x, b, 4)
    assert torch.equal(y1, y2)


def test_rejects_bad_arguments(lib_built):
    from mflux_b200 import ops

    w, x, b = _case(64, 64, 128, 4, 1, torch.bfloat16)
    wq, s, bi = ops.quantize_affine(w.cuda(), 64, 4)
    with pytest.raises(ValueError):
        ops.qlinear(x.cuda()[:, :64], wq, s, bi, None, bits=4)  # K mismatch
    with pytest.raises(RuntimeError):
        ops.qlinear(x, wq, s, bi, None, bits=4)  # CPU tensor


# ---------------------------------------------------------------- at most 16 rows: the weight-streaming kernel
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m", [1, 3, 16])
@pytest.mark.parametrize("nk", [(3072, 3072), (18432, 3072), (15360, 256), (1032, 192), (3072, 12288)])
def test_small_m_streaming_kernel(lib_built, bits, m, nk):
    """AdaLN / embedder shapes: narrow and wide N, K = 256 (Z-Image modulation), K = 192 (ragged last 128-wide
    slice of 4-bit rows), N = 1032 (a last block of 8 rows that is only partly used in the 32-row variant)."""
    n, k = nk
    w, x, b = _case(m, n, k, bits, hash((bits, n, k, m, 7)) % (2**31), torch.bfloat16)
    _, _, _, ref = _oracle(w, x, b, bits, "bf16")
    _, _, _, y = _run(w, x, b, bits)
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    err = quant.rel_l2(y, ref)
    assert err <= TOL, err


@pytest.mark.parametrize("bits", [4, 8])
def test_small_m_matches_large_m_kernel_and_epilogues(lib_built, bits):
    """The same 16 rows through the streaming kernel and (as part of 17 rows) through the tcgen05 kernel; SiLU
    epilogue, float32 output, strided input rows and an output view."""
    from mflux_b200 import ops

    n, k = 6144, 3072
    w, x17, b = _case(17, n, k, bits, 99 + bits, torch.bfloat16)
    wq, s, bi = ops.quantize_affine(w.cuda(), 64, bits)
    big = ops.qlinear(x17.cuda(), wq, s, bi, b.cuda(), bits=bits, epilogue="silu", out_dtype=torch.float32)
    xs = torch.zeros(16, 2 * k, dtype=torch.bfloat16, device="cuda")
    xs[:, :k] = x17[:16].cuda()
    out = torch.full((16, n + 64), 7.0, dtype=torch.float32, device="cuda")
    ops.qlinear(xs[:, :k], wq, s, bi, b.cuda(), bits=bits, epilogue="silu", out=out[:, :n])
    torch.cuda.synchronize()
    assert ops.poll_device_status() == 0
    assert quant.rel_l2(out[:, :n], big[:16].cpu().numpy()) <= 2e-3
    assert torch.all(out[:, n:] == 7.0)
    ref = quant.qlinear(x17[:16], *quant.quantize_affine(w, 64, bits, dtype="bf16"), b, 64, bits)
    ref = ref / (1 + np.exp(-ref))
    assert quant.rel_l2(out[:, :n], ref) <= TOL
