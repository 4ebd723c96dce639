"""GPU parity of the LoRA wrappers over the quantized linear and of a FLUX-shaped step with adapters on fused and
epilogue-carrying linears, against the float32 oracle. Tolerance: rel-L2 <= 1e-2."""
import pytest
import torch

from oracle import flux as oflux
from oracle.quant import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _adapter(g, i, o, r, dev="cuda"):
    return ((torch.randn(i, r, generator=g) * i ** -0.5).to(dev), (torch.randn(r, o, generator=g) * 0.05).to(dev))


@pytest.mark.parametrize("bits", [4, 8])
def test_lora_linear_matches_oracle(lib_built, bits):
    from mflux_b200 import nn
    from mflux_b200.lora import FusedLoRALinear, LoRALinear

    g = torch.Generator(device="cpu").manual_seed(3)
    lin = nn.Linear(512, 768, bias=True, device="cuda")
    with torch.no_grad():
        lin.weight.copy_(torch.randn(768, 512, generator=g) * 0.05)
        lin.bias.copy_(torch.randn(768, generator=g) * 0.05)
    q = lin.to_quantized(bits=bits)
    one = LoRALinear.from_linear(q, r=16, scale=0.7)
    assert one.lora_A.shape == (512, 16) and one.lora_B.shape == (16, 768) and one.linear is q
    a, b = _adapter(g, 512, 768, 16)
    one.lora_A.data, one.lora_B.data = a.to(torch.bfloat16), b.to(torch.bfloat16)
    two = LoRALinear.from_linear(q, r=8, scale=-1.3)
    a2, b2 = _adapter(g, 512, 768, 8)
    two.lora_A.data, two.lora_B.data = a2.to(torch.bfloat16), b2.to(torch.bfloat16)
    fused = FusedLoRALinear(q, [one, two])
    for shape in ((300, 512), (2, 150, 512)):
        x = torch.randn(*shape, generator=g).to(torch.bfloat16)
        y1, y2 = one(x.cuda()), fused(x.cuda())
        assert rel_l2(y1, oflux.lin(one, x).numpy()) <= TOL
        assert rel_l2(y2, oflux.lin(fused, x).numpy()) <= TOL
        # the adapter is not a no-op at this scale
        assert rel_l2(y1, oflux.lin(q, x).numpy()) > 5 * TOL


def test_flux_step_with_adapters(lib_built):
    from mflux_b200.flux import FluxConfig, Transformer
    from mflux_b200.lora import FusedLoRALinear, LoRALinear, apply_lora

    cfg = FluxConfig(hidden=256, heads=2, num_joint=1, num_single=1, context_dim=128, pooled_dim=64)
    model = Transformer(cfg, bits=4, device="cuda", seed=6)
    g = torch.Generator(device="cpu").manual_seed(12)
    d = cfg.hidden
    adapters = {
        "transformer_blocks.0.attn.to_q": [(*_adapter(g, d, d, 8), 6.0)],                 # one of a fused q|k|v
        "transformer_blocks.0.attn.to_out.0": [(*_adapter(g, d, d, 8), 5.0)],             # gate * y + residual
        "transformer_blocks.0.ff.linear1": [(*_adapter(g, d, 4 * d, 4), 4.0), (*_adapter(g, d, 4 * d, 16), 3.0)],
        "single_transformer_blocks.0.proj_out": [(*_adapter(g, 5 * d, d, 8), 6.0)],
    }
    b, height, width, txt = 2, 64, 96, 20
    lat = torch.randn(b, (height // 16) * (width // 16), cfg.in_channels, generator=g)
    ctx = torch.randn(b, txt, cfg.context_dim, generator=g).to(torch.bfloat16)
    pooled = torch.randn(b, cfg.pooled_dim, generator=g).to(torch.bfloat16)
    ts, gd = torch.tensor([250.0, 750.0]), torch.full((b,), 3500.0)
    args = (ts.cuda(), gd.cuda(), height, width)
    plain = model(lat.cuda(), ctx.cuda(), pooled.cuda(), *args).clone()
    apply_lora(model, adapters)
    assert isinstance(model.transformer_blocks[0].attn.to_q, LoRALinear)
    assert isinstance(model.transformer_blocks[0].ff.linear1, FusedLoRALinear)
    out = model(lat.cuda(), ctx.cuda(), pooled.cuda(), *args)
    ref = oflux.forward(model, lat.to(torch.bfloat16), ctx, pooled, ts, gd, height, width)
    assert rel_l2(out, ref.numpy()) <= TOL
    assert rel_l2(out, plain.float().cpu().numpy()) > 2 * TOL
    # a second adapter on an already wrapped layer turns it into the fused form and still matches
    apply_lora(model, {"transformer_blocks.0.attn.to_q": [(*_adapter(g, d, d, 4), 0.6)]})
    assert isinstance(model.transformer_blocks[0].attn.to_q, FusedLoRALinear)
    out2 = model(lat.cuda(), ctx.cuda(), pooled.cuda(), *args)
    ref2 = oflux.forward(model, lat.to(torch.bfloat16), ctx, pooled, ts, gd, height, width)
    assert rel_l2(out2, ref2.numpy()) <= TOL
