"""GPU parity of the Krea-2-shaped single-stream blocks (grouped-query attention with an output gate, SwiGLU, shared
modulation) against the float32 oracle. Tolerance: rel-L2 <= 1e-2 of the float32 result."""
import pytest
import torch

from oracle import krea2 as ok2
from oracle.quant import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _inputs(dim, b, s, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(b, s, dim, generator=g)
    vec = (torch.randn(b, 6 * dim, generator=g) * 0.3).to(torch.bfloat16)
    ids = torch.zeros(s, 3)
    ids[:, 0] = (torch.arange(s) % 3).float()
    ids[:, 1] = torch.arange(s) // 11
    ids[:, 2] = torch.arange(s) % 11
    return x, vec, ids


@pytest.mark.parametrize("bits,heads,kvheads", [(4, 4, 2), (8, 4, 1), (4, 2, 2), (None, 4, 2)])
def test_krea2_blocks_match_oracle(lib_built, bits, heads, kvheads):
    from mflux_b200.krea2 import Krea2SingleStream

    dim = heads * 128
    model = Krea2SingleStream(features=dim, heads=heads, kvheads=kvheads, multiplier=2, num_layers=2, bits=bits,
                              device="cuda", seed=3)
    x, vec, ids = _inputs(dim, 2, 170, 5)
    cos_sin = model.rope_table(ids)
    torch.testing.assert_close(cos_sin, ok2.rope_table(ids), rtol=0, atol=0)
    model.trace = {}
    out = model(x.cuda().clone(), vec.cuda(), cos_sin.cuda())
    torch.cuda.synchronize()
    from mflux_b200 import ops
    assert ops.poll_device_status() == 0
    want = {}
    ref = ok2.forward(model, x, vec, cos_sin, collect=want)
    assert rel_l2(out, ref.numpy()) <= TOL
    for k, v in want.items():
        assert rel_l2(model.trace[k], v.numpy()) <= TOL, k


def test_qknorm_rope_with_fewer_key_heads_and_act_mul(lib_built):
    """The two glue kernels the block adds: q/k RMSNorm + RoPE on a q (4 heads) | k (2) | v (2) buffer, V and the
    columns behind it untouched; y *= sigmoid(gate) on strided views."""
    from mflux_b200 import ops
    from oracle import blocks

    g = torch.Generator(device="cpu").manual_seed(2)
    b, s, h, hk = 2, 77, 4, 2
    buf = torch.randn(b, s, (h + 2 * hk) * 128 + 64, generator=g).to(torch.bfloat16)
    qw, kw = 1 + 0.1 * torch.randn(128, generator=g), 1 + 0.1 * torch.randn(128, generator=g)
    ang = torch.rand(s, 64, generator=g) * 6.28
    cs = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
    dev = buf.cuda()
    ops.qknorm_rope(dev[..., :(h + 2 * hk) * 128], h, qw.cuda(), kw.cuda(), qw.cuda(), kw.cuda(), 0, cs.cuda(), 1e-5,
                    kv_heads=hk)
    torch.cuda.synchronize()
    q = blocks.apply_rope(blocks.rms_norm(blocks.heads_first(buf[..., :h * 128], h), qw, 1e-5), cs[None, None])
    k = blocks.apply_rope(blocks.rms_norm(blocks.heads_first(buf[..., h * 128:(h + hk) * 128], hk), kw, 1e-5),
                          cs[None, None])
    assert rel_l2(dev[..., :h * 128], blocks.heads_last(q).numpy()) <= TOL
    assert rel_l2(dev[..., h * 128:(h + hk) * 128], blocks.heads_last(k).numpy()) <= TOL
    assert torch.equal(dev[..., (h + hk) * 128:].cpu(), buf[..., (h + hk) * 128:])
    y = torch.randn(b, s, 256, generator=g).to(torch.bfloat16)
    gate = torch.randn(b, s, 512, generator=g).to(torch.bfloat16)
    yd = y.cuda()
    ops.act_mul(yd, gate.cuda()[..., 256:], "sigmoid")
    assert rel_l2(yd, (y.float() * torch.sigmoid(gate[..., 256:].float())).numpy()) <= 5e-3
