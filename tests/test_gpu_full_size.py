"""Size-independent properties at the full widths of the benchmark configurations (the oracle is too slow there):
linearity of the quantized linear in x, agreement of the large-M and small-M kernels, batch invariance and
run-to-run determinism of a full-width block stack, softmax normalisation of attention at 4608 tokens."""
import pytest
import torch

from oracle.quant import rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits,n,k", [(4, 12288, 3072), (4, 3072, 15360), (8, 20480, 3840)])
def test_qlinear_is_linear_in_x_at_full_width(lib_built, bits, n, k):
    from mflux_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(bits + n)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    wq, s, b = ops.quantize_affine(w, 64, bits)
    m = 4608
    x1 = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    x2 = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    xs = (x1.float() + x2.float()).to(torch.bfloat16)       # exact sums would need more bits: compare to its own split
    x3 = (xs.float() - x1.float()).to(torch.bfloat16)
    y = lambda x: ops.qlinear(x, wq, s, b, bits=bits, out_dtype=torch.float32)  # noqa: E731
    lhs, rhs = y(xs), y(x1) + y(x3)
    # xs == x1 + x3 holds exactly where the subtraction was exact; elsewhere it is off by one bf16 ulp of x
    assert rel_l2(lhs, rhs.cpu().numpy()) <= 5e-3
    # rows are independent: the first 16 rows alone (small-M kernel) equal the same rows of the big call
    small = y(x1[:16].contiguous())
    assert rel_l2(small, y(x1)[:16].cpu().numpy()) <= 3e-3
    # scaling x by 2 (exact in bf16) scales y by 2 exactly, bias-free
    assert torch.equal(y((x1.float() * 2).to(torch.bfloat16)), 2 * y(x1))


def test_full_width_flux_blocks_batch_invariance_and_determinism(lib_built):
    from mflux_b200.flux import FluxConfig, Transformer

    cfg = FluxConfig(num_joint=1, num_single=2)          # hidden 3072, 24 heads, 4096 + 512 tokens
    model = Transformer(cfg, bits=4, device="cuda", seed=3)
    g = torch.Generator(device="cuda").manual_seed(4)
    b = 2
    lat = torch.randn(b, 4096, 64, device="cuda", generator=g)
    ctx = torch.randn(b, 512, 4096, device="cuda", generator=g).to(torch.bfloat16)
    pooled = torch.randn(b, 768, device="cuda", generator=g).to(torch.bfloat16)
    ts = torch.tensor([200.0, 800.0], device="cuda")
    gd = torch.full((b,), 3500.0, device="cuda")
    full = model(lat, ctx, pooled, ts, gd, 1024, 1024).clone()
    assert full.shape == (b, 4096, 64) and torch.isfinite(full).all()
    again = model(lat, ctx, pooled, ts, gd, 1024, 1024)
    assert torch.equal(full, again)
    for i in range(b):
        one = model(lat[i:i + 1], ctx[i:i + 1], pooled[i:i + 1], ts[i:i + 1], gd[i:i + 1], 1024, 1024)
        assert torch.equal(one[0], full[i])              # every linear has more than 16 rows: same kernels
    # swapping the samples swaps the outputs
    sw = model(lat.flip(0), ctx.flip(0), pooled.flip(0), ts.flip(0), gd.flip(0), 1024, 1024)
    assert torch.equal(sw.flip(0), full)


def test_attention_rows_are_convex_combinations_at_4608_tokens(lib_built):
    """With V = const along the sequence the output equals that constant; with V one-hot in d the outputs of a
    row sum to the softmax mass 1 (both independent of the scores)."""
    from mflux_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(8)
    b, s, h = 1, 4608, 24
    qkv = torch.randn(b, s, 3 * h * 128, device="cuda", generator=g).to(torch.bfloat16)
    const = torch.randn(h * 128, device="cuda", generator=g).to(torch.bfloat16)
    qkv[..., 2 * h * 128:] = const
    out = ops.fmha(qkv, h)
    assert rel_l2(out, const.float().expand(b, s, -1).cpu().numpy()) <= 4e-3
    # V[key, :] = e_(key mod 128): every output row then holds the softmax mass per residue class, summing to 1
    v = torch.zeros(s, 128, device="cuda")
    v[torch.arange(s), torch.arange(s) % 128] = 1.0
    qkv[..., 2 * h * 128:] = v.to(torch.bfloat16).repeat(1, h)[None]
    out = ops.fmha(qkv, h).float().reshape(b, s, h, 128)
    assert (out >= 0).all()
    torch.testing.assert_close(out.sum(-1), torch.ones(b, s, h, device="cuda"), rtol=0, atol=2e-2)
