"""GPU parity of the ERNIE-Image-shaped transformer blocks (shared modulation, RMSNorm + modulation, half-split rotary
embedding, masked attention, GeGLU) against the float32 oracle. Tolerance: rel-L2 <= 1e-2 of the float32 result."""
import pytest
import torch

from oracle import ernie as oe
from oracle.quant import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _inputs(dim, b, n_img, t, text_len, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    s = n_img + t
    x = torch.randn(b, s, dim, generator=g)
    c = torch.randn(b, dim, generator=g).to(torch.bfloat16)
    w = 9
    ids = torch.zeros(s, 3)   # transformer.py:92-109: image (text_len, y, x), then text (position, 0, 0)
    ids[:n_img, 0] = text_len
    ids[:n_img, 1] = torch.arange(n_img) // w
    ids[:n_img, 2] = torch.arange(n_img) % w
    ids[n_img:, 0] = torch.arange(t).float()
    bias = torch.zeros(b, s)
    bias[:, n_img + text_len:] = -1e9   # padded text keys
    return x, c, ids, bias


@pytest.mark.parametrize("bits", [4, 8, None])
def test_ernie_blocks_match_oracle(lib_built, bits):
    from mflux_b200 import ops
    from mflux_b200.ernie import ErnieBlocks

    model = ErnieBlocks(hidden_size=256, num_attention_heads=2, num_layers=2, ffn_hidden_size=512, bits=bits,
                        device="cuda", seed=3)
    x, c, ids, bias = _inputs(256, 2, 99, 40, 27, 5)
    cos_sin = model.rope_table(ids)
    cos, sin = oe.rope_cos_sin(ids)
    torch.testing.assert_close(cos_sin[..., 0], cos[:, 0::2], rtol=0, atol=0)   # every angle is stored twice
    torch.testing.assert_close(cos_sin[..., 1], sin[:, 1::2], rtol=0, atol=0)
    model.trace = {}
    out = model(x.cuda().clone(), c.cuda(), cos_sin.cuda(), key_bias=bias.cuda())
    torch.cuda.synchronize()
    assert ops.poll_device_status() == 0
    want = {}
    ref = oe.forward(model, x, c, ids, key_bias=bias, collect=want)
    assert rel_l2(out, ref.numpy()) <= TOL
    for k, v in want.items():
        assert rel_l2(model.trace[k], v.numpy()) <= TOL, k


def test_half_split_rope_and_gelu_gate(lib_built):
    """qknorm_rope(rope_mode="halves") against apply_rotary_emb on its own, and act_mul(..., "gelu")."""
    from mflux_b200 import ops
    from oracle import blocks

    g = torch.Generator(device="cpu").manual_seed(4)
    b, s, h = 2, 61, 3
    buf = torch.randn(b, s, 3 * h * 128, generator=g).to(torch.bfloat16)
    qw, kw = 1 + 0.1 * torch.randn(128, generator=g), 1 + 0.1 * torch.randn(128, generator=g)
    ids = torch.stack([torch.arange(s) % 7, torch.arange(s) // 5, torch.arange(s) % 5], dim=1).float()
    cos, sin = oe.rope_cos_sin(ids)
    cs = torch.stack([cos[:, 0::2], sin[:, 0::2]], dim=-1).contiguous()
    dev = buf.cuda()
    ops.qknorm_rope(dev, h, qw.cuda(), kw.cuda(), qw.cuda(), kw.cuda(), 0, cs.cuda(), 1e-6, rope_mode="halves")
    torch.cuda.synchronize()
    for j, w in ((0, qw), (1, kw)):
        t = blocks.rms_norm(buf[..., j * h * 128:(j + 1) * h * 128].reshape(b, s, h, 128), w, 1e-6)
        ref = oe.apply_rotary_emb(t, cos, sin).reshape(b, s, h * 128)
        assert rel_l2(dev[..., j * h * 128:(j + 1) * h * 128], ref.numpy()) <= TOL
    assert torch.equal(dev[..., 2 * h * 128:].cpu(), buf[..., 2 * h * 128:])
    gu = torch.randn(b, s, 512, generator=g).to(torch.bfloat16)
    d = gu.cuda()
    ops.act_mul(d[..., 256:], d[..., :256], "gelu")
    ref = gu[..., 256:].float() * torch.nn.functional.gelu(gu[..., :256].float())
    assert rel_l2(d[..., 256:], ref.numpy()) <= 5e-3
    assert torch.equal(d[..., :256].cpu(), gu[..., :256])
