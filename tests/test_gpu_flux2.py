"""GPU parity of the FLUX.2-shaped single-stream blocks (fused to_qkv_mlp_proj + SwiGLU beside the attention)
against the float32 oracle. Tolerance: rel-L2 <= 1e-2 of the float32 result."""
import pytest
import torch

from oracle import flux2 as of2
from oracle.quant import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _inputs(dim, b, s, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(b, s, dim, generator=g)
    temb = torch.randn(b, dim, generator=g).to(torch.bfloat16)
    ids = torch.zeros(s, 4)
    ids[:, 1] = torch.arange(s) // 9
    ids[:, 2] = torch.arange(s) % 9
    ids[:, 3] = (torch.arange(s) % 5).float()
    return x, temb, ids


@pytest.mark.parametrize("bits", [4, 8, 6, None])
def test_single_stream_blocks_match_oracle(lib_built, bits):
    from mflux_b200.flux2 import Flux2SingleStream

    model = Flux2SingleStream(dim=256, heads=2, num_single_layers=3, bits=bits, device="cuda", seed=3)
    x, temb, ids = _inputs(256, 2, 150, 5)
    cos_sin = model.rope_table(ids)
    torch.testing.assert_close(cos_sin, of2.rope_table(ids), rtol=0, atol=0)
    model.trace = {}
    out = model(x.cuda().clone(), temb.cuda(), cos_sin.cuda())
    torch.cuda.synchronize()
    want = {}
    ref = of2.forward(model, x, temb, cos_sin, collect=want)
    assert rel_l2(out, ref.numpy()) <= TOL
    for k, v in want.items():
        assert rel_l2(model.trace[k], v.numpy()) <= TOL, k


def test_split_projection_equals_the_single_projection(lib_built):
    """The two row-subset launches (q|k|v rows; interleaved MLP rows with the SwiGLU epilogue) reproduce what one
    matmul over the whole to_qkv_mlp_proj followed by the split and silu(x1) * x2 gives."""
    from mflux_b200 import ops
    from mflux_b200.flux2 import Flux2SingleStream, _SplitProjection

    model = Flux2SingleStream(dim=256, heads=2, num_single_layers=1, bits=4, device="cuda", seed=9)
    a = model.single_transformer_blocks[0].attn
    inner, mlp = a.inner_dim, a.mlp_hidden_dim
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(2, 200, 256, device="cuda", generator=g).to(torch.bfloat16)
    whole = a.to_qkv_mlp_proj(x, out_dtype=torch.float32)
    qkv = torch.empty(2, 200, 3 * inner, dtype=torch.bfloat16, device="cuda")
    act = torch.empty(2, 200, mlp, dtype=torch.bfloat16, device="cuda")
    _SplitProjection(a.to_qkv_mlp_proj, inner, mlp)(x, qkv, act)
    torch.cuda.synchronize()
    assert ops.poll_device_status() == 0
    assert torch.equal(qkv, whole[..., :3 * inner].to(torch.bfloat16))
    x1, x2 = whole[..., 3 * inner:3 * inner + mlp], whole[..., 3 * inner + mlp:]
    assert rel_l2(act, (torch.nn.functional.silu(x1) * x2).cpu().numpy()) <= 3e-3


def test_full_width_block(lib_built):
    """One block at the FLUX.2 width (3072, 24 heads, mlp ratio 3: a 27648-row projection, to_out with K = 12288)
    on 4096 + 512 tokens."""
    from mflux_b200.flux2 import Flux2SingleStream

    model = Flux2SingleStream(num_single_layers=1, bits=4, device="cuda", seed=4)
    g = torch.Generator(device="cpu").manual_seed(8)
    s = 4608
    x = torch.randn(1, s, 3072, generator=g)
    temb = torch.randn(1, 3072, generator=g).to(torch.bfloat16)
    ids = torch.zeros(s, 4)
    ids[512:, 1] = (torch.arange(4096) // 64).float()
    ids[512:, 2] = (torch.arange(4096) % 64).float()
    cos_sin = model.rope_table(ids)
    out = model(x.cuda().clone(), temb.cuda(), cos_sin.cuda())
    torch.cuda.synchronize()
    ref = of2.forward(model, x, temb, cos_sin)
    assert rel_l2(out, ref.numpy()) <= TOL
