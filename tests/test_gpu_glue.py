"""GPU parity of the glue and attention kernels against the float32 oracle (rel-L2 <= 1e-2, the
bound for bf16 layer outputs against the float32 result)."""
import pytest
import torch

from oracle import blocks
from oracle.quant import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _g(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [256, 3072, 3840])
def test_layer_norm_modulate(lib_built, dtype, d):
    from mflux_b200 import ops

    g = _g(d)
    x = (torch.randn(3, 37, d, generator=g) * 3 + 0.5).to(dtype)
    shift = torch.randn(3, d, generator=g).to(torch.bfloat16)
    scale = torch.randn(3, d, generator=g).to(torch.bfloat16)
    y = ops.norm_modulate(x.cuda(), shift.cuda(), scale.cuda(), eps=1e-6)
    ref = blocks.modulate(x, shift, scale)
    assert y.dtype == torch.bfloat16
    assert rel_l2(y, ref.numpy()) <= TOL
    # no modulation: plain LayerNorm
    y0 = ops.norm_modulate(x.cuda())
    assert rel_l2(y0, blocks.layer_norm(x).numpy()) <= TOL


def test_norm_modulate_strided_views_and_chunks(lib_built):
    """Slices of a joint sequence buffer in and out; shift/scale as chunks of one [B, 6D] tensor."""
    from mflux_b200 import ops

    g = _g(7)
    d = 512
    seq = torch.randn(2, 96, d, generator=g)
    mod = torch.randn(2, 6 * d, generator=g)
    x = seq.cuda()
    modc = mod.cuda()
    out = torch.zeros(2, 96, d, dtype=torch.bfloat16, device="cuda")
    ops.norm_modulate(x[:, 32:], modc[:, 0:d], modc[:, d:2 * d], out=out[:, 32:])
    ref = blocks.modulate(seq[:, 32:], mod[:, 0:d], mod[:, d:2 * d])
    assert rel_l2(out[:, 32:], ref.numpy()) <= TOL
    assert (out[:, :32] == 0).all()


def test_rms_norm_weight(lib_built):
    from mflux_b200 import ops

    g = _g(11)
    x = torch.randn(5, 3584, generator=g).to(torch.bfloat16)
    w = torch.rand(3584, generator=g).to(torch.bfloat16)
    y = ops.norm_modulate(x.cuda(), weight=w.cuda(), eps=1e-6, rms=True)
    assert rel_l2(y, blocks.rms_norm(x, w, 1e-6).numpy()) <= TOL


def test_qknorm_rope(lib_built):
    from mflux_b200 import ops

    g = _g(3)
    b, txt, hgt, wid, heads = 2, 24, 64, 96, 3
    s = txt + (hgt // 16) * (wid // 16)
    qkv = torch.randn(b, s, 3 * heads * 128, generator=g).to(torch.bfloat16)
    ws = [(torch.rand(128, generator=g) + 0.5).to(torch.bfloat16) for _ in range(4)]
    cs = blocks.rope_table(blocks.flux_ids(hgt, wid, txt))
    out = ops.qknorm_rope(qkv.cuda().clone(), heads, ws[0].cuda(), ws[1].cuda(), ws[2].cuda(), ws[3].cuda(), txt,
                          cs.cuda())
    hd = heads * 128
    for which, (wa, wb) in enumerate([(ws[0], ws[2]), (ws[1], ws[3])]):
        x = blocks.heads_first(qkv[..., which * hd:(which + 1) * hd], heads)  # [B, H, S, 128]
        n = torch.cat([blocks.rms_norm(x[:, :, :txt], wa), blocks.rms_norm(x[:, :, txt:], wb)], dim=2)
        ref = blocks.heads_last(blocks.apply_rope(n, cs[None, None]))
        assert rel_l2(out[..., which * hd:(which + 1) * hd], ref.numpy()) <= TOL
    assert torch.equal(out[..., 2 * hd:].cpu(), qkv[..., 2 * hd:])  # V untouched


@pytest.mark.parametrize("shape", [(1, 128, 1), (2, 256, 2), (1, 384, 3), (2, 200, 2), (1, 1000, 1), (1, 17, 1), (2, 97, 2),
                                   (1, 161, 1), (1, 1300, 2)])
@pytest.mark.parametrize("kernel", ["pair", "pingpong"])
def test_fmha(lib_built, shape, kernel, monkeypatch):
    """Both attention kernels on every shape: `pair` (one 128-query tile per CTA, two CTAs per SM) and `pingpong`
    (two query tiles per CTA); the library picks by sequence length and grid size when the variable is unset."""
    from mflux_b200 import ops

    monkeypatch.setenv("MFX_FMHA_KERNEL", kernel)
    b, s, heads = shape
    g = _g(s)
    qkv = torch.randn(b, s, 3 * heads * 128, generator=g).to(torch.bfloat16)
    out = ops.fmha(qkv.cuda(), heads)
    torch.cuda.synchronize()
    assert ops.poll_device_status() == 0
    hd = heads * 128
    q, k, v = (blocks.heads_first(qkv[..., i * hd:(i + 1) * hd], heads) for i in range(3))
    ref = blocks.heads_last(blocks.sdpa(q, k, v))
    err = rel_l2(out, ref.numpy())
    assert err <= TOL, err


@pytest.mark.parametrize("kernel", ["pair", "pingpong"])
def test_fmha_peaked_scores_and_strided_output(lib_built, kernel, monkeypatch):
    """Large score ranges exercise the running-max rescale; output written into a wider buffer."""
    from mflux_b200 import ops

    monkeypatch.setenv("MFX_FMHA_KERNEL", kernel)
    b, s, heads = 1, 512, 2
    g = _g(99)
    qkv = torch.randn(b, s, 3 * heads * 128, generator=g)
    qkv[..., :2 * heads * 128] *= 3.0  # scores with std ~ 9 * sqrt(128) / sqrt(128)
    qkv[:, 300:, :heads * 128] *= 2.0
    qkv = qkv.to(torch.bfloat16)
    buf = torch.zeros(b, s, 5 * heads * 128, dtype=torch.bfloat16, device="cuda")
    ops.fmha(qkv.cuda(), heads, out=buf[..., :heads * 128])
    hd = heads * 128
    q, k, v = (blocks.heads_first(qkv[..., i * hd:(i + 1) * hd], heads) for i in range(3))
    ref = blocks.heads_last(blocks.sdpa(q, k, v))
    assert rel_l2(buf[..., :hd], ref.numpy()) <= TOL
    assert (buf[..., hd:] == 0).all()


def test_vec_ops_and_euler(lib_built):
    from mflux_b200 import ops

    g = _g(5)
    a, b_, c = (torch.randn(4, 3072, generator=g) for _ in range(3))
    y = ops.vec_sum_act(a.cuda(), b_.cuda(), c.cuda(), act="silu", out_dtype=torch.float32)
    torch.testing.assert_close(y.cpu(), torch.nn.functional.silu(a + b_ + c), rtol=1e-5, atol=1e-5)
    lat = torch.randn(2, 4096, 64, generator=g)
    noise = torch.randn(2, 4096, 64, generator=g).to(torch.bfloat16)
    out = ops.euler_step(lat.cuda(), noise.cuda(), -0.03125)
    torch.testing.assert_close(out.cpu(), lat + noise.float() * -0.03125, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("y_dtype", [torch.bfloat16, torch.float32])
def test_gate_residual_dense_and_row_range(lib_built, y_dtype):
    """out = residual + gate * (y + bias) on the whole stream and on a row range of it (a chunk of a linear
    evaluated in pieces), in place."""
    from mflux_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(21)
    b, s, d = 3, 50, 256
    stream = torch.randn(b, s, d, device="cuda", generator=g)
    gate = torch.randn(b, 3 * d, device="cuda", generator=g).to(torch.bfloat16)[:, d:2 * d]   # strided gate rows
    bias = torch.randn(d, device="cuda", generator=g).to(torch.bfloat16)
    for lo, hi in ((0, s), (7, 31)):
        y = torch.randn(b, hi - lo, d, device="cuda", generator=g).to(y_dtype)
        before = stream.clone()
        ops.gate_residual(y, gate, stream[:, lo:hi], bias)
        torch.cuda.synchronize()
        ref = before[:, lo:hi] + gate.float()[:, None] * (y.float() + bias.float())
        torch.testing.assert_close(stream[:, lo:hi], ref, rtol=1e-6, atol=1e-6)
        assert torch.equal(stream[:, :lo], before[:, :lo]) and torch.equal(stream[:, hi:], before[:, hi:])


@pytest.mark.parametrize("shape", [(2, 256, 2, 40), (1, 200, 1, 70), (2, 1000, 1, 130), (1, 97, 2, 5)])
@pytest.mark.parametrize("kernel", ["pair", "pingpong"])
def test_fmha_key_padding_bias(lib_built, shape, kernel, monkeypatch):
    """Additive per-key bias as AttentionUtils.convert_key_padding_mask_to_additive_mask builds it
    (attention_utils.py:55-72): the first `pad` keys of sample 0 (text keys come first) carry -1e9, which may
    cover whole 64-key tiles at the start of the sequence; sample 1 keeps every key. rel-L2 <= 1e-2 against the
    float32 oracle, the tolerance north_star states for layer outputs."""
    from mflux_b200 import ops

    monkeypatch.setenv("MFX_FMHA_KERNEL", kernel)
    b, s, heads, pad = shape
    g = _g(s + pad)
    qkv = torch.randn(b, s, 3 * heads * 128, generator=g).to(torch.bfloat16)
    keep = torch.ones(b, s)
    keep[0, :pad] = 0.0
    if b > 1:
        keep[1, 3] = 0.0       # a single masked key in the middle of a tile
    bias = (1.0 - keep) * -1e9
    out = ops.fmha(qkv.cuda(), heads, key_bias=bias.cuda())
    torch.cuda.synchronize()
    assert ops.poll_device_status() == 0
    hd = heads * 128
    q, k, v = (blocks.heads_first(qkv[..., i * hd:(i + 1) * hd], heads) for i in range(3))
    ref = blocks.heads_last(blocks.sdpa(q, k, v, mask=bias))
    assert rel_l2(out, ref.numpy()) <= TOL
    # masked keys do not contribute: dropping them from the sequence gives the same rows for the kept queries
    if b == 1:
        kept = ops.fmha(qkv[:, pad:].contiguous().cuda(), heads)
        assert rel_l2(out[:, pad:], kept.float().cpu().numpy()) <= 3e-3
    # an all-zero bias reproduces the plain kernel
    plain = ops.fmha(qkv.cuda(), heads)
    zero = ops.fmha(qkv.cuda(), heads, key_bias=torch.zeros(b, s, device="cuda"))
    assert rel_l2(zero, plain.float().cpu().numpy()) <= 1e-3


def test_fmha_bias_argument_validation(lib_built):
    from mflux_b200 import ops

    qkv = torch.zeros(2, 64, 3 * 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        ops.fmha(qkv, 1, key_bias=torch.zeros(2, 63, device="cuda"))
    with pytest.raises(ValueError):
        ops.fmha(qkv, 1, key_bias=torch.zeros(2, 64, device="cuda", dtype=torch.bfloat16))
    # rows of 66 floats: the second sample's bias would not start on a 16-byte boundary; the wrapper re-pads it
    out = ops.fmha(qkv, 1, key_bias=torch.zeros(2, 66, device="cuda")[:, :64])
    assert torch.isfinite(out.float()).all()


def test_fmha_default_kernel_choice_matches_both(lib_built, monkeypatch):
    """With the variable unset the library chooses by shape (here a grid that fills whole waves of CTAs, so the
    two-query-tile kernel); either way the result is the oracle's."""
    from mflux_b200 import ops

    monkeypatch.delenv("MFX_FMHA_KERNEL", raising=False)
    b, s, heads = 37, 1024, 4   # 4 x 4 x 37 = 592 CTAs of two query tiles = exactly 4 waves of 148
    g = _g(5)
    qkv = torch.randn(b, s, 3 * heads * 128, generator=g).to(torch.bfloat16).cuda()
    out = ops.fmha(qkv, heads)
    torch.cuda.synchronize()
    assert ops.poll_device_status() == 0
    hd = heads * 128
    sample = qkv[3:4].cpu()
    q, k, v = (blocks.heads_first(sample[..., i * hd:(i + 1) * hd], heads) for i in range(3))
    ref = blocks.heads_last(blocks.sdpa(q, k, v))
    assert rel_l2(out[3:4], ref.numpy()) <= TOL
    for kernel in ("pair", "pingpong"):
        monkeypatch.setenv("MFX_FMHA_KERNEL", kernel)
        assert rel_l2(ops.fmha(qkv, heads), out.float().cpu().numpy()) <= 3e-3


@pytest.mark.parametrize("kernel", ["pair", "pingpong"])
@pytest.mark.parametrize("shape", [(2, 200, 200, 8, 2), (1, 300, 429, 4, 4), (2, 130, 1200, 6, 3), (1, 97, 33, 2, 1)])
def test_fmha_grouped_heads_and_longer_keys(lib_built, shape, kernel, monkeypatch):
    """mfx_fmha_ex: fewer key/value heads than query heads (the reference repeats K and V,
    krea2_transformer/attention.py:33-38) and key/value sequences longer or shorter than the query sequence (cached
    reference tokens appended to K and V, flux2_kv_cache.py:51-61), with and without a key bias. rel-L2 <= 1e-2
    against the float32 oracle."""
    from mflux_b200 import ops

    monkeypatch.setenv("MFX_FMHA_KERNEL", kernel)
    b, sq, skv, heads, kvh = shape
    g = _g(sq + skv)
    q = torch.randn(b, sq, heads * 128, generator=g).to(torch.bfloat16)
    kv = torch.randn(b, skv, 2 * kvh * 128, generator=g).to(torch.bfloat16)   # k | v of one fused projection
    kv_d = kv.cuda()
    k_d, v_d = kv_d[..., :kvh * 128], kv_d[..., kvh * 128:]
    bias = torch.zeros(b, skv)
    bias[0, 1::5] = -1e9
    rep = heads // kvh
    qh = blocks.heads_first(q, heads)
    kh = blocks.heads_first(kv[..., :kvh * 128], kvh).repeat_interleave(rep, dim=1)
    vh = blocks.heads_first(kv[..., kvh * 128:], kvh).repeat_interleave(rep, dim=1)
    for mask in (None, bias):
        out = ops.fmha_ex(q.cuda(), k_d, v_d, heads, kvh, key_bias=None if mask is None else mask.cuda())
        torch.cuda.synchronize()
        assert ops.poll_device_status() == 0
        ref = blocks.heads_last(blocks.sdpa(qh, kh, vh, mask=mask))
        err = rel_l2(out, ref.numpy())
        assert err <= TOL, (err, mask is None)
