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


def _dense_ref(x, q, bits, t, b_rows, bias):
    from oracle.quant import dequantize_affine

    w = torch.from_numpy(dequantize_affine(q[0].cpu().numpy(), q[1].float().cpu().numpy(), q[2].float().cpu().numpy(),
                                           64, bits))
    y = x.float().cpu() @ w.T + t.float().cpu() @ b_rows.float().cpu().T
    return y if bias is None else y + bias.float().cpu()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("rank", [4, 16, 40, 64, 100, 256])
def test_low_rank_term_inside_the_kernel(lib_built, bits, rank):
    """y = x . W^T + t . lb^T + bias with t, lb as extra K columns of the tensor-core accumulation: ragged rows,
    N off the 256-wide tile, an odd number of quantization groups (the last quantized stage is half empty)."""
    from mflux_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(100 * bits + rank)
    m, k, n = 333, 448, 328
    ld = -(-rank // 64) * 64
    x = torch.randn(2, m, k, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    q = ops.quantize_affine(w, 64, bits)
    bias = (torch.randn(n, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    t = torch.zeros(2, m, ld, device="cuda", dtype=torch.bfloat16)
    lb = torch.zeros(n, ld, device="cuda", dtype=torch.bfloat16)
    t[..., :rank] = torch.randn(2, m, rank, device="cuda", generator=g).to(torch.bfloat16)
    lb[:, :rank] = (torch.randn(n, rank, device="cuda", generator=g) * 0.2).to(torch.bfloat16)
    y = ops.qlinear(x, *q, bias, bits=bits, lora_t=t, lora_b=lb, lora_r=rank, out_dtype=torch.float32)
    plain = ops.qlinear(x, *q, bias, bits=bits, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert ops.poll_device_status() == 0
    ref = _dense_ref(x, q, bits, t, lb, bias)
    assert rel_l2(y, ref.numpy()) <= 2e-3
    assert rel_l2(plain, ref.numpy()) > 0.05          # the term matters at these scales
    # the low-rank part alone, isolated by subtraction, is itself right to bf16-product accuracy
    low = (t.float() @ lb.float().T).cpu()
    assert rel_l2((y - plain).cpu(), low.numpy()) <= 1e-2


@pytest.mark.parametrize("bits", [4, 8])
def test_low_rank_term_small_m_and_epilogues(lib_built, bits):
    from mflux_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(7 + bits)
    k, n, rank, ld = 64, 256, 24, 64                   # one quantization group, then one extension stage
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    q = ops.quantize_affine(w, 64, bits)
    lb = torch.zeros(n, ld, device="cuda", dtype=torch.bfloat16)
    lb[:, :rank] = (torch.randn(n, rank, device="cuda", generator=g) * 0.2).to(torch.bfloat16)
    for m in (1, 9, 16, 130):                          # at most 16 rows would otherwise take the small-M kernel
        x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
        t = torch.zeros(m, ld, device="cuda", dtype=torch.bfloat16)
        t[:, :rank] = torch.randn(m, rank, device="cuda", generator=g).to(torch.bfloat16)
        y = ops.qlinear(x, *q, None, bits=bits, lora_t=t, lora_b=lb, lora_r=rank, out_dtype=torch.float32)
        ref = _dense_ref(x, q, bits, t, lb, None)
        assert rel_l2(y, ref.numpy()) <= 2e-3, m
        # gelu and gate * y + residual see the sum, not the base product alone
        ge = ops.qlinear(x, *q, None, bits=bits, lora_t=t, lora_b=lb, lora_r=rank, epilogue="gelu_approx")
        assert rel_l2(ge, torch.nn.functional.gelu(ref, approximate="tanh").numpy()) <= 1e-2
        res = torch.randn(1, m, n, device="cuda", generator=g)
        gate = torch.randn(1, n, device="cuda", generator=g).to(torch.bfloat16)
        before = res.clone()
        ops.qlinear(x.unsqueeze(0), *q, None, bits=bits, lora_t=t.unsqueeze(0), lora_b=lb, lora_r=rank,
                    epilogue="gate_residual", gate=gate, residual=res, out=res)
        want = before.cpu() + gate.float().cpu()[:, None] * ref
        assert rel_l2(res, want.numpy()) <= 2e-3
    assert ops.poll_device_status() == 0


def test_low_rank_arguments_are_validated(lib_built):
    from mflux_b200 import ops

    x = torch.zeros(32, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(64, 64, device="cuda").to(torch.bfloat16)
    q = ops.quantize_affine(w, 64, 4)
    t = torch.zeros(32, 48, device="cuda", dtype=torch.bfloat16)       # row length not a multiple of 64
    lb = torch.zeros(64, 48, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(Exception):
        ops.qlinear(x, *q, None, bits=4, lora_t=t, lora_b=lb, lora_r=16)
    t, lb = torch.zeros(32, 64, device="cuda", dtype=torch.bfloat16), torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(Exception):
        ops.qlinear(x, *q, None, bits=4, lora_t=t, lora_b=lb, lora_r=65)    # rank beyond the row length
    with pytest.raises(Exception):
        ops.qlinear(x, *q, None, bits=4, lora_t=t[:16], lora_b=lb, lora_r=8)   # rows differ from x
    with pytest.raises(Exception):
        ops.qlinear(x, *q, None, bits=4, lora_t=t.float(), lora_b=lb, lora_r=8)


def test_wrappers_take_the_fused_path_and_match_the_library_path(lib_built):
    """Over a quantized base the wrapper's output (low-rank term inside the kernel) agrees with base output plus
    library GEMMs, and it accepts the quantized layer's epilogues."""
    from mflux_b200 import nn
    from mflux_b200.lora import FusedLoRALinear, LoRALinear, _low_rank_add

    g = torch.Generator(device="cpu").manual_seed(21)
    lin = nn.Linear(256, 512, bias=True, device="cuda")
    q = lin.to_quantized(bits=4)
    one = LoRALinear.from_linear(q, r=16, scale=0.9)
    two = LoRALinear.from_linear(q, r=72, scale=-0.4)
    for l, r in ((one, 16), (two, 72)):
        a, b = _adapter(g, 256, 512, r)
        l.lora_A.data, l.lora_B.data = a.to(torch.bfloat16), b.to(torch.bfloat16)
    fused = FusedLoRALinear(q, [one, two])
    assert one.fuses_epilogue and fused.fuses_epilogue
    x = torch.randn(3, 200, 256, generator=g).to(torch.bfloat16).cuda()
    y = fused(x, out_dtype=torch.float32)
    lib = q(x, out_dtype=torch.float32)
    for l in (one, two):
        _low_rank_add(lib, x, l.lora_A.data, l.lora_B.data, l.scale)
    assert rel_l2(y, lib.cpu().numpy()) <= 5e-3
    act = fused(x, epilogue="gelu_approx")
    assert rel_l2(act, torch.nn.functional.gelu(lib, approximate="tanh").cpu().numpy()) <= 1e-2
    # changing a scale rebuilds the cached operands
    one.scale = 0.0
    y0 = one(x, out_dtype=torch.float32)
    assert rel_l2(y0, q(x, out_dtype=torch.float32).cpu().numpy()) <= 1e-6
    dense = LoRALinear.from_linear(lin, r=8)
    assert not dense.fuses_epilogue


@pytest.mark.parametrize("bits", [4, 8])
def test_row_fused_layers_keep_their_adapters(lib_built, bits):
    """q/k/v run as one matmul: a wrapped q, a bare k and a doubly wrapped v give what the three layers give one
    by one, and changing an adapter's scale afterwards is picked up."""
    from mflux_b200 import nn
    from mflux_b200.flux import FusedRows
    from mflux_b200.lora import FusedLoRALinear, LoRALinear

    g = torch.Generator(device="cpu").manual_seed(33 + bits)
    d = 256
    base = []
    for _ in range(3):
        lin = nn.Linear(d, d, bias=True, device="cuda")
        with torch.no_grad():
            lin.weight.copy_(torch.randn(d, d, generator=g) * 0.05)
            lin.bias.copy_(torch.randn(d, generator=g) * 0.05)
        base.append(lin.to_quantized(bits=bits))

    def wrap(q, r, scale):
        l = LoRALinear.from_linear(q, r=r, scale=scale)
        a, b = _adapter(g, d, d, r)
        l.lora_A.data, l.lora_B.data = a.to(torch.bfloat16), b.to(torch.bfloat16)
        return l

    wq = wrap(base[0], 8, 0.9)
    wv = FusedLoRALinear(base[2], [wrap(base[2], 16, -0.7), wrap(base[2], 4, 1.5)])
    layers = [wq, base[1], wv]
    assert FusedRows.accepts(layers) and not FusedRows.accepts([wq, torch.nn.Linear(d, d)])
    fused = FusedRows(layers)
    x = torch.randn(2, 90, d, generator=g).to(torch.bfloat16).cuda()
    out = torch.empty(2, 90, 3 * d, device="cuda", dtype=torch.bfloat16)
    fused(x, out)
    want = torch.cat([l(x) for l in layers], dim=-1)
    torch.cuda.synchronize()
    assert rel_l2(out, want.float().cpu().numpy()) <= 2e-3
    ref = torch.cat([oflux.lin(l, x.cpu()) for l in layers], dim=-1)
    assert rel_l2(out, ref.numpy()) <= TOL
    # k carries no adapter: its block equals the bare layer bit for bit; q's differs from its bare layer
    assert torch.equal(out[..., d:2 * d], base[1](x))
    assert rel_l2(out[..., :d], base[0](x).float().cpu().numpy()) > 0.02
    wq.scale = 0.0
    fused(x, out)
    assert rel_l2(out[..., :d], base[0](x).float().cpu().numpy()) <= 1e-6
