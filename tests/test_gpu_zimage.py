"""GPU parity of the Z-Image-shaped denoising step (reduced configuration) and of the kernels only it uses
(SwiGLU matmul epilogue, post-norm gated residual, tanh) against the float32 oracle / plain torch.
Tolerance: rel-L2 <= 1e-2 on step outputs and matmul outputs; 2e-3 on the float32 residual update."""
import pytest
import torch

from oracle import zimage as oz
from oracle.quant import dequantize_affine, rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _small_cfg(**kw):
    from mflux_b200.zimage import ZImageConfig

    base = dict(dim=256, n_layers=2, n_refiner_layers=1, n_heads=2, cap_feat_dim=128, ffn_hidden=704)
    base.update(kw)
    return ZImageConfig(**base)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_swiglu_epilogue_matches_separate_projections(lib_built, bits, out_dtype):
    from mflux_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(11)
    m, k, h = 300, 256, 1104          # ragged rows; 2h = 2208 is not a multiple of the 256-wide tile
    x = torch.randn(2, m, k, device="cuda", generator=g).to(torch.bfloat16)
    w1 = (torch.randn(h, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    w3 = (torch.randn(h, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    q1, q3 = ops.quantize_affine(w1, 64, bits), ops.quantize_affine(w3, 64, bits)
    inter = lambda a, b: torch.stack([a, b], dim=1).reshape(2 * h, -1).contiguous()  # noqa: E731
    wq = inter(q1[0].view(torch.int32), q3[0].view(torch.int32)).view(torch.uint32)
    y = ops.qlinear(x, wq, inter(q1[1], q3[1]), inter(q1[2], q3[2]), bits=bits, epilogue="swiglu", out_dtype=out_dtype)
    torch.cuda.synchronize()
    assert y.shape == (2, m, h) and y.dtype == out_dtype
    d = [torch.from_numpy(dequantize_affine(q[0].cpu().numpy(), q[1].float().cpu().numpy(),
                                            q[2].float().cpu().numpy(), 64, bits)) for q in (q1, q3)]
    xf = x.float().cpu()
    ref = torch.nn.functional.silu(xf @ d[0].T) * (xf @ d[1].T)
    assert rel_l2(y, ref.numpy()) <= TOL


def test_swiglu_rejects_odd_pair_count(lib_built):
    from mflux_b200 import ops

    x = torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(24, 64, device="cuda").to(torch.bfloat16)   # N = 24: multiple of 8 but not of 16
    wq, s, b = ops.quantize_affine(w, 64, 4)
    with pytest.raises(Exception):
        ops.qlinear(x, wq, s, b, bits=4, epilogue="swiglu")


@pytest.mark.parametrize("y_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("gated", [True, False])
@pytest.mark.parametrize("d", [256, 3840])
def test_norm_gate_residual(lib_built, y_dtype, gated, d):
    from mflux_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(5)
    b, s, lo, hi = 2, 70, 3, 64        # a strided view of a larger stream, as the refiners use it
    y_full = (torch.randn(b, s, d, device="cuda", generator=g) * 3).to(y_dtype)
    res_full = torch.randn(b, s, d, device="cuda", generator=g)
    weight = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).to(torch.bfloat16)
    gate = torch.tanh(torch.randn(b, d, device="cuda", generator=g)).to(torch.bfloat16) if gated else None
    before = res_full.clone()
    ops.norm_gate_residual(y_full[:, lo:hi], weight, res_full[:, lo:hi], gate, eps=1e-5)
    torch.cuda.synchronize()
    yf = y_full[:, lo:hi].float()
    normed = yf * torch.rsqrt((yf * yf).mean(-1, keepdim=True) + 1e-5) * weight.float()
    ref = before[:, lo:hi] + (gate.float()[:, None] if gated else 1.0) * normed
    assert rel_l2(res_full[:, lo:hi], ref.cpu().numpy()) <= 2e-3
    # rows outside the view are untouched
    assert torch.equal(res_full[:, :lo], before[:, :lo]) and torch.equal(res_full[:, hi:], before[:, hi:])


def test_tanh_activation(lib_built):
    from mflux_b200 import ops

    a = torch.linspace(-6, 6, 1000, device="cuda").to(torch.bfloat16)
    out = ops.vec_sum_act(a, act="tanh", out_dtype=torch.float32)
    torch.testing.assert_close(out, torch.tanh(a.float()), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("bits", [4, 8])
def test_step_matches_oracle(lib_built, bits):
    from mflux_b200.zimage import ZImageTransformer

    cfg = _small_cfg()
    model = ZImageTransformer(cfg, bits=bits, device="cuda", seed=3)
    g = torch.Generator(device="cpu").manual_seed(9)
    with torch.no_grad():   # the reference initialises the pad tokens to zero; trained ones are not
        model.x_pad_token.copy_(torch.randn(1, cfg.dim, generator=g) * 0.5)
        model.cap_pad_token.copy_(torch.randn(1, cfg.dim, generator=g) * 0.5)
        for blk in list(model.layers) + list(model.noise_refiner) + list(model.context_refiner):
            for n in (blk.attention_norm1, blk.attention_norm2, blk.ffn_norm1, blk.ffn_norm2):
                n.weight.copy_(1 + 0.1 * torch.randn(cfg.dim, generator=g))
    b = 2
    lat = torch.randn(b, cfg.in_channels, 1, 18, 14, generator=g).to(torch.bfloat16)   # 9 x 7 = 63 tokens -> padded to 64
    cap = torch.randn(b, 20, cfg.cap_feat_dim, generator=g).to(torch.bfloat16)         # 20 -> padded to 32
    t = torch.tensor([0.17, 0.59])
    out = model(lat.cuda(), t.cuda(), cap.cuda())
    torch.cuda.synchronize()
    ref = oz.forward(model, lat, t, cap)
    assert out.shape == lat.shape
    err = rel_l2(out, ref.numpy())
    assert err <= TOL, err


def test_unpadded_shapes_and_dense_model(lib_built):
    from mflux_b200.zimage import ZImageTransformer

    cfg = _small_cfg(n_layers=1)
    model = ZImageTransformer(cfg, bits=None, device="cuda", seed=1)
    g = torch.Generator(device="cpu").manual_seed(2)
    lat = torch.randn(1, cfg.in_channels, 1, 16, 16, generator=g).to(torch.bfloat16)   # 64 tokens, no padding
    cap = torch.randn(1, 32, cfg.cap_feat_dim, generator=g).to(torch.bfloat16)
    t = torch.tensor([0.4])
    out = model(lat.cuda(), t.cuda(), cap.cuda())
    ref = oz.forward(model, lat, t, cap)
    assert rel_l2(out, ref.numpy()) <= TOL


def test_rope_table_matches_reference_construction(lib_built):
    from mflux_b200.zimage import ZImageTransformer

    cfg = _small_cfg(n_layers=0, n_refiner_layers=0)
    model = ZImageTransformer(cfg, bits=None, device="cuda")
    full, img, cap = model.rope_table((1, 9, 7), 20, "cuda")
    lat = torch.zeros(cfg.in_channels, 1, 18, 14)
    _, _, _, x_ids, cap_ids, _, _ = oz.patchify(lat, torch.zeros(20, 4))
    tables = oz.rope_tables(cfg.axes_dims, cfg.axes_lens, cfg.rope_theta)
    torch.testing.assert_close(img.cpu(), oz.rope_lookup(tables, x_ids), rtol=0, atol=0)
    torch.testing.assert_close(cap.cpu(), oz.rope_lookup(tables, cap_ids), rtol=0, atol=0)
    assert full.shape == (64 + 32, 64, 2)


def test_denoise_loop_with_and_without_guidance(lib_built):
    from mflux_b200.zimage import ZImage

    # guidance needs the base model (supports_guidance); the Turbo configuration forces it to 0
    zi = ZImage(quantize=8, model_config=_small_cfg(n_layers=1, supports_guidance=True), seed=2)
    g = torch.Generator(device="cuda").manual_seed(0)
    cap = torch.randn(2, 32, 128, device="cuda", generator=g).to(torch.bfloat16)
    neg = torch.randn(2, 32, 128, device="cuda", generator=g).to(torch.bfloat16)
    plain = zi.generate_image(1, cap, num_inference_steps=2, height=128, width=128)
    guided = zi.generate_image(1, cap, neg, num_inference_steps=2, height=128, width=128, guidance=3.0)
    assert plain.shape == guided.shape == (2, 16, 1, 16, 16)
    assert torch.isfinite(plain).all() and torch.isfinite(guided).all()
    assert not torch.allclose(plain, guided)
    turbo = ZImage(quantize=8, model_config=_small_cfg(n_layers=1), seed=2)
    t_plain = turbo.generate_image(1, cap, num_inference_steps=2, height=128, width=128)
    t_guided = turbo.generate_image(1, cap, neg, num_inference_steps=2, height=128, width=128, guidance=3.0)
    assert torch.equal(t_plain, t_guided)   # variants/z_image.py:60-62: no guidance support, guidance = 0
    # one guided step equals the hand-combined two evaluations
    lat = torch.randn(2, 16, 1, 16, 16, device="cuda", generator=g)
    t = torch.full((2,), 0.3, device="cuda")
    n_pos = zi.transformer(lat, t, cap).clone()
    n_neg = zi.transformer(lat, t, neg).clone()
    step = zi.denoise_step(lat, cap, neg, 0.7, -0.1, 3.0)
    ref = lat + (n_pos + 3.0 * (n_pos - n_neg)) * -0.1
    torch.testing.assert_close(step, ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("scaled", [True, False])
def test_norm_gate_residual_with_following_pre_norm(lib_built, scaled):
    """The fused second stage equals norm_modulate(rms) applied to the updated stream."""
    from mflux_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(17)
    b, s, d, lo, hi = 2, 40, 3840, 4, 36
    y = (torch.randn(b, s, d, device="cuda", generator=g) * 2).to(torch.bfloat16)
    res = torch.randn(b, s, d, device="cuda", generator=g)
    w1 = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).to(torch.bfloat16)
    w2 = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).to(torch.bfloat16)
    gate = torch.tanh(torch.randn(b, d, device="cuda", generator=g)).to(torch.bfloat16)
    scale = (0.3 * torch.randn(b, 4 * d, device="cuda", generator=g)).to(torch.bfloat16)[:, 2 * d:3 * d] if scaled else None
    res_a, res_b = res.clone(), res.clone()
    nb = torch.zeros(b, s, d, device="cuda", dtype=torch.bfloat16)
    ops.norm_gate_residual(y[:, lo:hi], w1, res_a[:, lo:hi], gate, 1e-5, next_weight=w2, next_scale=scale,
                           next_out=nb[:, lo:hi])
    ops.norm_gate_residual(y[:, lo:hi], w1, res_b[:, lo:hi], gate, 1e-5)
    ref = ops.norm_modulate(res_b[:, lo:hi], None, scale, weight=w2, eps=1e-5, rms=True)
    torch.cuda.synchronize()
    assert torch.equal(res_a, res_b)
    assert rel_l2(nb[:, lo:hi], ref.float().cpu().numpy()) <= 1e-3
    assert (nb[:, :lo] == 0).all() and (nb[:, hi:] == 0).all()


def test_step_with_adapters_on_fused_projections(lib_built):
    """Adapters on q / v (row-fused projection), on the gate and up projections (interleaved SwiGLU matmul) and on
    the down projection: the step matches the oracle, which adds every adapter's term layer by layer, and the
    fused paths are the ones that ran."""
    from mflux_b200.flux import FusedRows
    from mflux_b200.lora import apply_lora
    from mflux_b200.zimage import FusedSwiGLU, ZImageTransformer

    cfg = _small_cfg(n_layers=1, n_refiner_layers=0)
    model = ZImageTransformer(cfg, bits=4, device="cuda", seed=5)
    g = torch.Generator(device="cpu").manual_seed(12)

    def ad(i, o, r, scale):
        return ((torch.randn(i, r, generator=g) * i ** -0.5).cuda(), (torch.randn(r, o, generator=g) * 0.1).cuda(), scale)

    d, h = cfg.dim, cfg.ffn_hidden
    apply_lora(model, {
        "layers.0.attention.to_q": [ad(d, d, 8, 1.0)],
        "layers.0.attention.to_v": [ad(d, d, 4, -0.8), ad(d, d, 16, 0.6)],
        "layers.0.feed_forward.w1": [ad(d, h, 8, 1.2)],
        "layers.0.feed_forward.w3": [ad(d, h, 24, -0.9)],
        "layers.0.feed_forward.w2": [ad(h, d, 8, 1.0)],
    })
    lat = torch.randn(2, cfg.in_channels, 1, 16, 16, generator=g).to(torch.bfloat16)
    cap = torch.randn(2, 32, cfg.cap_feat_dim, generator=g).to(torch.bfloat16)
    t = torch.tensor([0.3, 0.8])
    out = model(lat.cuda(), t.cuda(), cap.cuda())
    torch.cuda.synchronize()
    ref = oz.forward(model, lat, t, cap)
    assert rel_l2(out, ref.numpy()) <= TOL
    fused = list(model._fused.values())
    assert any(isinstance(f, FusedRows) and f.terms is not None for f in fused)
    assert any(isinstance(f, FusedSwiGLU) and f.terms is not None for f in fused)
    # and the adapters matter: the bare model gives something else
    bare = ZImageTransformer(cfg, bits=4, device="cuda", seed=5)
    assert rel_l2(bare(lat.cuda(), t.cuda(), cap.cuda()), ref.numpy()) > 2 * TOL


def test_cuda_graph_replay_equals_launch_by_launch(lib_built):
    from mflux_b200.zimage import ZImage

    eager = ZImage(quantize=8, model_config=_small_cfg(n_layers=2), seed=4)
    graphed = ZImage(quantize=8, model_config=_small_cfg(n_layers=2), seed=4, cuda_graph=True)
    g = torch.Generator(device="cuda").manual_seed(1)
    cap = torch.randn(1, 32, 128, device="cuda", generator=g).to(torch.bfloat16)
    a = eager.generate_image(2, cap, num_inference_steps=3, height=128, width=128)
    b = graphed.generate_image(2, cap, num_inference_steps=3, height=128, width=128)
    assert torch.equal(a, b)
    graphed.release_graphs()
