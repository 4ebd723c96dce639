"""Parity against the float32 oracle at the sizes of the benchmark configurations themselves.

  * one block of every kind at the real width: FLUX joint + single block (hidden 3072, 24 heads, 4096 image + 512
    text tokens, W4), Z-Image refiners + main block (hidden 3840, 30 heads, SwiGLU 10240, 4096 + 512 tokens, W8),
    Qwen-Image block (hidden 3072, 6889 image + 256 text tokens, W4), batch 1 as the reference runs them;
  * the real depth at reduced width (hidden 512): 19 + 38 FLUX blocks, 2 + 2 + 30 Z-Image blocks, 60 Qwen blocks,
    with the error of the residual stream after every block recorded, so that the growth of bf16 rounding over the
    depth is measured rather than assumed;
  * every point of the quantized-linear sweep (bits 4/8 x four (N, K) x five M); beyond 1024 rows a seeded subset
    of 512 output rows is compared (the oracle's float32 GEMM over all 16384 rows would take minutes).

Tolerance everywhere: rel-L2 <= 1e-2 of the float32 result, the bound stated for layer and step outputs.
With MFX_PARITY_REPORT=<file> every measured error is appended to that file as one JSON line.
"""
import json
import os

import numpy as np
import pytest
import torch

from oracle import flux as oflux
from oracle import quant
from oracle import qwen as oq
from oracle import zimage as oz
from oracle.quant import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _report(name, **values):
    path = os.environ.get("MFX_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"case": name, **values}) + "\n")


def _cpu_gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


# --------------------------------------------------------------------------- FLUX
def _flux_case(cfg, bits, height, width, txt, seed):
    from mflux_b200.flux import Transformer

    model = Transformer(cfg, bits=bits, device="cuda", seed=seed)
    g = _cpu_gen(seed + 1)
    si = (height // 16) * (width // 16)
    lat = torch.randn(1, si, cfg.in_channels, generator=g)
    ctx = torch.randn(1, txt, cfg.context_dim, generator=g).to(torch.bfloat16)
    pooled = torch.randn(1, cfg.pooled_dim, generator=g).to(torch.bfloat16)
    ts, gd = torch.full((1,), 650.0), torch.full((1,), 3500.0)
    model.trace = {}
    out = model(lat.cuda(), ctx.cuda(), pooled.cuda(), ts.cuda(), gd.cuda(), height, width)
    torch.cuda.synchronize()
    got = {k: v.float().cpu() for k, v in model.trace.items()}
    model.trace = None
    want = {}
    ref = oflux.forward(model, lat.to(torch.bfloat16), ctx, pooled, ts, gd, height, width, collect=want)
    curve = {k: rel_l2(got[k], want[k].numpy()) for k in want}
    return rel_l2(out, ref.numpy()), curve


def test_flux_blocks_at_full_width(lib_built):
    from mflux_b200.flux import FluxConfig

    err, curve = _flux_case(FluxConfig(num_joint=1, num_single=1), 4, 1024, 1024, 512, 21)
    _report("flux full width 1+1 blocks W4, 4096+512 tokens", output=err, streams=curve)
    assert err <= TOL and max(curve.values()) <= TOL, (err, curve)


def test_flux_full_depth_at_reduced_width(lib_built):
    from mflux_b200.flux import FluxConfig

    cfg = FluxConfig(hidden=512, heads=4, num_joint=19, num_single=38, context_dim=256, pooled_dim=128)
    err, curve = _flux_case(cfg, 4, 256, 256, 64, 22)
    _report("flux 19+38 blocks at hidden 512 W4, 256+64 tokens", output=err, streams=curve)
    assert len(curve) == 57
    assert err <= TOL and max(curve.values()) <= TOL, (err, max(curve.values()))


# --------------------------------------------------------------------------- Z-Image
def _zimage_case(cfg, bits, lat_hw, cap_len, seed):
    from mflux_b200.zimage import ZImageTransformer

    model = ZImageTransformer(cfg, bits=bits, device="cuda", seed=seed)
    g = _cpu_gen(seed + 1)
    lat = torch.randn(1, cfg.in_channels, 1, lat_hw, lat_hw, generator=g).to(torch.bfloat16)
    cap = torch.randn(1, cap_len, cfg.cap_feat_dim, generator=g).to(torch.bfloat16)
    t = torch.tensor([0.37])
    model.trace = {}
    out = model(lat.cuda(), t.cuda(), cap.cuda())
    torch.cuda.synchronize()
    got = {k: v.float().cpu() for k, v in model.trace.items()}
    model.trace = None
    want = {}
    ref = oz.forward(model, lat, t, cap, collect=want)
    curve = {k: rel_l2(got[k][0], want[k][0].numpy()) for k in want}
    return rel_l2(out, ref.numpy()), curve


def test_zimage_blocks_at_full_width(lib_built):
    from mflux_b200.zimage import ZImageConfig

    cfg = ZImageConfig(n_layers=1, n_refiner_layers=1)       # hidden 3840, 30 heads, SwiGLU 10240
    err, curve = _zimage_case(cfg, 8, 128, 512, 31)            # 1024 x 1024 px: 4096 image tokens + 512 caption tokens
    _report("zimage full width 1+1 refiners + 1 block W8, 4096+512 tokens", output=err, streams=curve)
    assert err <= TOL and max(curve.values()) <= TOL, (err, curve)


def test_zimage_full_depth_at_reduced_width(lib_built):
    from mflux_b200.zimage import ZImageConfig

    cfg = ZImageConfig(dim=512, n_heads=4, n_layers=30, n_refiner_layers=2, cap_feat_dim=256, ffn_hidden=1408)
    err, curve = _zimage_case(cfg, 8, 32, 64, 32)              # 256 image tokens + 64 caption tokens
    _report("zimage 2+2+30 blocks at hidden 512 W8, 256+64 tokens", output=err, streams=curve)
    assert sum(k.startswith("layer") for k in curve) == 30 and len(curve) == 34   # + 2 + 2 refiner blocks
    assert err <= TOL and max(curve.values()) <= TOL, (err, max(curve.values()))


# --------------------------------------------------------------------------- Qwen-Image
def _qwen_case(cfg, bits, height, width, txt, seed):
    from mflux_b200.qwen import QwenTransformer

    model = QwenTransformer(cfg, bits=bits, device="cuda", seed=seed)
    g = _cpu_gen(seed + 1)
    si = (height // 16) * (width // 16)
    lat = torch.randn(1, si, cfg.in_channels, generator=g)
    ctx = torch.randn(1, txt, cfg.joint_attention_dim, generator=g).to(torch.bfloat16)
    sigma = torch.tensor([0.58])
    model.trace = {}
    out = model(lat.cuda(), ctx.cuda(), sigma.cuda(), height, width)
    torch.cuda.synchronize()
    got = {k: tuple(t.float().cpu() for t in v) for k, v in model.trace.items()}
    model.trace = None
    want = {}
    ref = oq.forward(model, lat.to(torch.bfloat16), ctx, sigma, height, width, collect=want)
    curve = {k: rel_l2(torch.cat(got[k], dim=1), torch.cat(want[k], dim=1).numpy()) for k in want}
    return rel_l2(out, ref.numpy()), curve


def test_qwen_block_at_full_width(lib_built):
    from mflux_b200.qwen import QwenConfig

    err, curve = _qwen_case(QwenConfig(num_layers=1), 4, 1328, 1328, 256, 41)   # 6889 image + 256 text tokens
    _report("qwen full width 1 block W4, 6889+256 tokens", output=err, streams=curve)
    assert err <= TOL and max(curve.values()) <= TOL, (err, curve)


def test_qwen_full_depth_at_reduced_width(lib_built):
    from mflux_b200.qwen import QwenConfig

    cfg = QwenConfig(hidden=512, heads=4, num_layers=60, joint_attention_dim=256)
    err, curve = _qwen_case(cfg, 4, 240, 272, 48, 42)         # 15 x 17 = 255 image tokens + 48 text tokens
    _report("qwen 60 blocks at hidden 512 W4, 255+48 tokens", output=err, streams=curve)
    assert len(curve) == 60
    assert err <= TOL and max(curve.values()) <= TOL, (err, max(curve.values()))


# --------------------------------------------------------------------------- quantized-linear sweep
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("n,k", [(3072, 3072), (9216, 3072), (12288, 3072), (3072, 12288)])
def test_qlinear_sweep_point(lib_built, bits, n, k):
    from mflux_b200 import ops

    seed = bits * 1_000_003 + n * 31 + k
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(n, k, device="cuda", generator=g) * 0.02
    wq, s, b = ops.quantize_affine(w, 64, bits)
    del w
    bias = (torch.randn(n, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w_hat = quant.dequantize_affine(wq.cpu().numpy(), s.cpu().numpy(), b.cpu().numpy(), 64, bits)
    prepared = ops.prepare_qlinear(wq, s, b, bits, 64)
    errs = {}
    for m in (256, 1024, 4096, 4608, 16384):
        x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
        y = ops.qlinear(x, wq, s, b, bias, bits=bits, prepared=prepared)
        torch.cuda.synchronize()
        rows = np.arange(m) if m <= 1024 else np.sort(np.random.default_rng(seed + m).choice(m, 512, replace=False))
        idx = torch.from_numpy(rows).cuda()
        ref = x[idx].float().cpu().numpy() @ w_hat.T + bias.float().cpu().numpy()[None, :]
        errs[m] = rel_l2(y[idx], ref)
        assert torch.isfinite(y.float()).all()
        del x, y
    assert ops.poll_device_status() == 0
    _report(f"qlinear sweep W{bits} N={n} K={k}", errors=errs)
    assert max(errs.values()) <= TOL, errs
