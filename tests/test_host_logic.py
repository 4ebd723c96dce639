"""CPU tests of the host-side mirror: quantization resolution rules and sigma schedules against the
reference's own golden vectors (tests/schedulers/test_linear_scheduler.py:41-73,
tests/resolution/test_quantization_resolution.py:7-70)."""
import io
import json
from pathlib import Path

import numpy as np
import pytest

from mflux_b200 import resolution
from mflux_b200.schedulers import LinearScheduler

GOLDEN = Path(__file__).parent / "golden" / "linear_scheduler_sigmas.json"


def _vec(hexstr):
    return np.load(io.BytesIO(bytes.fromhex(hexstr)))


def test_sigmas_dev_match_reference_golden():
    g = json.loads(GOLDEN.read_text())
    s = LinearScheduler(14, 1024, 1024, requires_sigma_shift=True)
    want = _vec(g["dev_requires_sigma_shift_true"])
    assert s.sigmas.shape == (15,) and s.sigmas.dtype == np.float32
    np.testing.assert_allclose(s.sigmas, want, rtol=1e-5, atol=1e-8)  # mx.allclose defaults


def test_sigmas_schnell_match_reference_golden():
    g = json.loads(GOLDEN.read_text())
    s = LinearScheduler(14, 1024, 1024, requires_sigma_shift=False)
    np.testing.assert_allclose(s.sigmas, _vec(g["schnell_requires_sigma_shift_false"]), rtol=1e-5, atol=1e-8)


def test_euler_step():
    import torch

    s = LinearScheduler(4, 1024, 1024, requires_sigma_shift=False)
    lat = torch.ones(2, 3)
    out = s.step(torch.full((2, 3), 2.0), 0, lat)
    np.testing.assert_allclose(out.numpy(), 1.0 + 2.0 * (0.75 - 1.0))


LEVELS = [None, 3, 4, 5, 6, 8]


@pytest.mark.parametrize("stored", LEVELS)
@pytest.mark.parametrize("requested", LEVELS)
def test_resolution_rules(stored, requested):
    bits, warning = resolution.resolve(stored, requested)
    if stored is None:
        assert bits == requested and warning is None
    else:
        assert bits == stored
        if requested is not None and requested != stored:
            assert warning == f"Model is pre-quantized at {stored}-bit. Ignoring -q {requested} flag."
        else:
            assert warning is None


def test_supported_bits_are_the_reference_cli_choices():
    """src/mflux/cli/defaults/defaults.py:63 offers 3, 4, 5, 6 and 8."""
    for b in (2, 7, 16):
        with pytest.raises(ValueError):
            resolution.check_supported(b)
    for b in (None, 3, 4, 5, 6, 8):
        resolution.check_supported(b)


def test_zimage_token_layout_matches_oracle():
    """Patch order, padding to multiples of 32 and position ids of the Z-Image path (host logic, no GPU)."""
    import numpy as np
    import torch

    from mflux_b200.zimage import ZImageConfig, ZImageTransformer
    from oracle import zimage as oz

    cfg = ZImageConfig(dim=256, n_layers=0, n_refiner_layers=0, n_heads=2, cap_feat_dim=64, ffn_hidden=704)
    model = ZImageTransformer(cfg, bits=None, device="cpu")
    g = torch.Generator().manual_seed(0)
    lat = torch.randn(2, 16, 1, 18, 14, generator=g)
    cap = torch.randn(20, 64, generator=g)
    tokens = model.patchify(lat)
    img, cap_p, size, x_ids, cap_ids, x_mask, cap_mask = oz.patchify(lat[1], cap)
    assert torch.equal(tokens[1], img[:63]) and img.shape[0] == 64 and torch.equal(img[63], img[62])
    assert cap_p.shape[0] == 32 and int(cap_mask.sum()) == 12 and int(x_mask.sum()) == 1
    # caption ids count from 1 on axis 0; image ids start one past the padded caption, pad tokens sit at 0
    assert cap_ids[0].tolist() == [1, 0, 0] and cap_ids[-1].tolist() == [32, 0, 0]
    assert x_ids[0].tolist() == [33, 0, 0] and x_ids[8].tolist() == [33, 1, 1] and x_ids[63].tolist() == [0, 0, 0]
    mine_img, mine_cap = model.position_ids((1, 9, 7), 20)
    assert np.array_equal(mine_img, x_ids) and np.array_equal(mine_cap, cap_ids)
    out = model.unpatchify(torch.cat([tokens, tokens[:, -1:]], dim=1), (1, 18, 14))
    assert torch.equal(out, lat)
    assert torch.equal(oz.unpatchify(img, size, 16), lat[1])


def test_checkpoint_format_round_trip(tmp_path):
    """Shard naming, metadata, index file and key layout of the reference's saved-model format; packed uint32
    weights survive bit for bit (host logic, no GPU)."""
    import json

    import torch
    from safetensors import safe_open

    from mflux_b200 import checkpoint, nn

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.to_q = nn.QuantizedLinear(128, 64, bias=True, bits=4)
            self.to_out = torch.nn.ModuleList([nn.QuantizedLinear(128, 64, bias=False, bits=4)])

    class Tiny(nn.Module):
        def __init__(self):
            super().__init__()
            self.bits = 4
            self.transformer_blocks = torch.nn.ModuleList([Block(), Block()])
            self.norm = torch.nn.Parameter(torch.ones(8, dtype=torch.bfloat16), requires_grad=False)

    g = torch.Generator().manual_seed(1)
    src = Tiny()
    for p in src.parameters():
        if p.dtype == torch.uint32:
            p.data = torch.randint(0, 2**31 - 1, p.shape, generator=g, dtype=torch.int64).to(torch.uint32)
        else:
            p.data = torch.randn(p.shape, generator=g).to(p.dtype)
    names = checkpoint.save_weights(tmp_path, 4, src, max_file_size_bytes=6000)
    assert names == [f"{i}.safetensors" for i in range(len(names))] and len(names) > 1
    index = json.loads((tmp_path / "transformer" / "model.safetensors.index.json").read_text())
    assert index["metadata"]["quantization_level"] == "4"
    assert index["weight_map"]["transformer_blocks.1.to_out.0.scales"] in names
    assert set(index["weight_map"]) == set(dict(src.named_parameters()))
    with safe_open(str(tmp_path / "transformer" / "0.safetensors"), framework="pt") as f:
        assert f.metadata()["quantization_level"] == "4" and "mflux_version" in f.metadata()
        k = "transformer_blocks.0.to_q.weight"
        assert f.get_tensor(k).dtype == torch.uint32 and tuple(f.get_tensor(k).shape) == (64, 16)
    dst = Tiny()
    assert checkpoint.load_into(dst, tmp_path, requested_bits=8) == 4      # the stored level wins
    for (k, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(a.view(torch.uint8) if a.dtype == torch.uint32 else a,
                           b.view(torch.uint8) if b.dtype == torch.uint32 else b), k
    # a directory of plain safetensors without the metadata is not this format
    other = tmp_path / "plain"
    other.mkdir()
    from safetensors.torch import save_file
    save_file({"x": torch.zeros(2)}, str(other / "0.safetensors"))
    assert checkpoint.load_weights(other) == (None, None, None)
    dst.bits = 8
    import pytest
    with pytest.raises(ValueError):
        checkpoint.load_into(dst, tmp_path)


def test_flow_match_euler_discrete_scheduler():
    """Default schedule: starts at 1, ends at the terminal 0.02 before the appended 0, strictly decreasing;
    empirical mu follows the two published lines; set_mu equals the linear scheduler's shift for the same mu."""
    import math

    import numpy as np

    from mflux_b200.schedulers import FlowMatchEulerDiscreteScheduler as FM, LinearScheduler

    s = FM(20)
    assert s.sigmas.shape == (21,) and s.timesteps.shape == (20,)
    assert abs(s.sigmas[0] - 1.0) < 1e-6 and abs(s.sigmas[19] - 0.02) < 1e-6 and s.sigmas[20] == 0.0
    assert np.all(np.diff(s.sigmas) < 0)
    # second sigma by hand: t = 1000 - 999/19, sigma = t/1000 shifted with mu = 1, then stretched
    sig1 = (1000 - 999 / 19) / 1000
    shifted = math.e / (math.e + (1 / sig1 - 1))
    last = math.e / (math.e + (1 / 0.001 - 1))
    expect = 1 - (1 - shifted) / ((1 - last) / 0.98)
    assert abs(s.sigmas[1] - expect) < 1e-6
    assert abs(FM.compute_empirical_mu(5000, 20) - (0.00016927 * 5000 + 0.45666666)) < 1e-9
    m200, m10 = 0.00016927 * 4096 + 0.45666666, 8.73809524e-05 * 4096 + 1.89833333
    a = (m200 - m10) / 190
    assert abs(FM.compute_empirical_mu(4096, 20) - (a * 20 + m200 - 200 * a)) < 1e-9
    assert abs(FM.compute_linear_mu(4096) - 1.15) < 1e-12 and abs(FM.compute_linear_mu(256) - 0.5) < 1e-12
    s.set_mu(1.15)
    lin = LinearScheduler(20, 1024, 1024, True)   # 4096 image tokens -> mu = 1.15
    np.testing.assert_allclose(s.sigmas, lin.sigmas, rtol=1e-6)
    np.testing.assert_allclose(s.timesteps, lin.sigmas[:-1] * 1000, rtol=1e-6)
    import torch
    lat, noise = torch.ones(4), torch.full((4,), 2.0)
    assert torch.allclose(s.step(noise, 3, lat), lat + 2.0 * float(s.sigmas[4] - s.sigmas[3]))


def test_tensor_parallel_shards_are_slices_of_the_full_quantization():
    """Quantizing a shard equals slicing the quantized full weight: output-row shards trivially, input-column
    shards because groups of 64 run along K and K / tp stays a multiple of 64 (the rule QwenTransformer enforces)."""
    import numpy as np

    from oracle import quant

    rng = np.random.default_rng(5)
    n, k, tp = 48, 512, 4
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    for bits in (4, 8):
        full_q, full_s, full_b = quant.quantize_affine(w, 64, bits)
        words = k * bits // 32
        for r in range(tp):
            rows = slice(r * n // tp, (r + 1) * n // tp)
            q, s, b = quant.quantize_affine(w[rows], 64, bits)
            assert np.array_equal(q, full_q[rows]) and np.array_equal(s, full_s[rows]) and np.array_equal(b, full_b[rows])
            cols = slice(r * k // tp, (r + 1) * k // tp)
            q, s, b = quant.quantize_affine(np.ascontiguousarray(w[:, cols]), 64, bits)
            assert np.array_equal(q, full_q[:, r * words // tp:(r + 1) * words // tp])
            assert np.array_equal(s, full_s[:, r * (k // 64) // tp:(r + 1) * (k // 64) // tp])
            assert np.array_equal(b, full_b[:, r * (k // 64) // tp:(r + 1) * (k // 64) // tp])
        # and the row-split products add up to the full product
        x = rng.standard_normal((5, k)).astype(np.float32)
        y_full = quant.qlinear(x, full_q, full_s, full_b, None, 64, bits)
        y_sum = sum(quant.qlinear(x[:, r * k // tp:(r + 1) * k // tp],
                                  full_q[:, r * words // tp:(r + 1) * words // tp],
                                  full_s[:, r * (k // 64) // tp:(r + 1) * (k // 64) // tp],
                                  full_b[:, r * (k // 64) // tp:(r + 1) * (k // 64) // tp], None, 64, bits)
                    for r in range(tp))
        np.testing.assert_allclose(y_sum, y_full, rtol=1e-4, atol=1e-4)


def test_low_rank_operands_of_row_fused_layers():
    """The two dense operands handed to the matmul kernel for adapters on row-concatenated layers: every adapter
    gets its own columns, acts only on its layer's block of output rows, scales are folded into the second
    operand, columns are padded with zeros to a multiple of 64, and a change of scale rebuilds them."""
    import torch

    from mflux_b200.lora import LoRALinear, _FusedTerms

    g = torch.Generator().manual_seed(4)
    k, n = 96, 40

    def adapter(r, scale):
        l = LoRALinear(k, n, r=r, scale=scale, device="cpu")
        l.lora_A.data = torch.randn(k, r, generator=g).to(torch.bfloat16)
        l.lora_B.data = torch.randn(r, n, generator=g).to(torch.bfloat16)
        return l

    q1, v1, v2 = adapter(8, 0.5), adapter(16, -1.25), adapter(4, 2.0)
    terms = _FusedTerms()
    groups = [(0, [q1]), (2 * n, [v1, v2])]            # rows: q | k (bare) | v | one more bare layer
    a_cat, b_rows, rank = terms.get(None, groups, 4 * n)
    assert rank == 28 and a_cat.shape == (k, 64) and b_rows.shape == (4 * n, 64)
    assert (a_cat[:, 28:] == 0).all() and (b_rows[:, 28:] == 0).all()
    assert (b_rows[n:2 * n] == 0).all() and (b_rows[3 * n:] == 0).all()      # bare layers: no term
    assert (b_rows[:n, 8:] == 0).all() and (b_rows[2 * n:3 * n, :8] == 0).all()   # blocks do not leak
    x = torch.randn(7, k, generator=g).to(torch.bfloat16)
    got = (x.float() @ a_cat.float()) @ b_rows.float().T
    want = torch.zeros(7, 4 * n)
    want[:, :n] = 0.5 * (x.float() @ q1.lora_A.float()) @ q1.lora_B.float()
    for l in (v1, v2):
        want[:, 2 * n:3 * n] += l.scale * (x.float() @ l.lora_A.float()) @ l.lora_B.float()
    # scale * B is rounded to bf16 (2^-9 relative per element): compare in relative L2, not element by element
    assert float((got - want).norm() / want.norm()) <= 5e-3
    same = terms.get(None, groups, 4 * n)
    assert same[1] is b_rows                                              # cached
    v2.scale = 0.0
    _, b2, _ = terms.get(None, groups, 4 * n)
    assert b2 is not b_rows and (b2[2 * n:3 * n, 24:28] == 0).all()
    # two layers whose rows are interleaved (gate / up of a fused SwiGLU): step 2 from row 0 and from row 1
    _, bi, ri = _FusedTerms().get(None, [(0, 2, [q1]), (1, 2, [v1])], 2 * n)
    assert ri == 24 and bi.shape == (2 * n, 64)
    assert (bi[0::2, 8:] == 0).all() and (bi[1::2, :8] == 0).all()
    torch.testing.assert_close(bi[0::2, :8].float(), (0.5 * q1.lora_B.float()).T.to(torch.bfloat16).float())
    torch.testing.assert_close(bi[1::2, 8:24].float(), (-1.25 * v1.lora_B.float()).T.to(torch.bfloat16).float())
    # a single wrapped layer is one block from row 0
    a1, b1, r1 = _FusedTerms().get([q1])
    assert r1 == 8 and b1.shape == (n, 64)
    torch.testing.assert_close(b1[:, :8].float(), (0.5 * q1.lora_B.float()).T.to(torch.bfloat16).float())


def test_captured_step_refuses_host_tensors():
    """Graph replay is a device feature: a step called with host tensors fails before anything is recorded."""
    import pytest
    import torch

    from mflux_b200.graphs import CapturedStep

    step = CapturedStep(lambda a: a + 1)
    with pytest.raises(ValueError):
        step(torch.zeros(4))
    with pytest.raises(ValueError):
        step()
    assert step.captured_shapes == []
    step.release()   # nothing recorded: a no-op


def test_qwen_sigma_schedule_uses_the_qwen_image_config():
    """The reference's "qwen-image" ModelConfig (models/common/config/model_config.py:505-520) shifts with
    max_shift 0.9 over max_seq_len 8192 and stretches the last sigma to 0.02; LinearScheduler._get_sigmas
    (linear_scheduler.py:25-48) applies all three. Values below are that formula evaluated in float64."""
    from mflux_b200.qwen import QwenConfig

    n, w, h = 20, 1328, 1328
    s = QwenConfig().scheduler(n, w, h)
    m = (0.9 - 0.5) / (8192 - 256)
    mu = m * w * h / 256 + (0.5 - m * 256)
    lin = np.linspace(1.0, 1.0 / n, n)
    shifted = np.exp(mu) / (np.exp(mu) + (1.0 / lin - 1.0))
    one_minus = 1.0 - shifted
    want = 1.0 - one_minus / (one_minus[-1] / (1.0 - 0.02))
    assert s.sigmas.shape == (n + 1,) and s.sigmas[-1] == 0.0
    np.testing.assert_allclose(s.sigmas[:-1], want, rtol=2e-5)
    assert abs(float(s.sigmas[-2]) - 0.02) < 1e-6          # terminal stretch
    assert abs(mu - 0.8343) < 1e-3                           # not the FLUX shift (about 1.6 at this size)
    flux_like = LinearScheduler(n, w, h, True)
    assert not np.allclose(flux_like.sigmas, s.sigmas, atol=1e-3)


def test_zimage_scheduler_choice_follows_guidance_support():
    """variants/z_image.py:60-66: guidance support picks flow_match_euler_discrete, Turbo (no guidance) linear;
    Config.scheduler (config.py:146-164) hands the flow-match schedule the image sequence length."""
    from mflux_b200.schedulers import FlowMatchEulerDiscreteScheduler
    from mflux_b200.zimage import ZImage, ZImageConfig

    pick = ZImage.make_scheduler
    turbo = type("P", (), {"model_config": ZImageConfig(supports_guidance=False)})()
    base = type("P", (), {"model_config": ZImageConfig(supports_guidance=True)})()
    assert isinstance(pick(turbo, 9, 1024, 1024), LinearScheduler)
    fm = pick(base, 9, 1024, 1024)
    assert isinstance(fm, FlowMatchEulerDiscreteScheduler)
    want = FlowMatchEulerDiscreteScheduler(9)
    want.set_image_seq_len(64 * 64)
    np.testing.assert_array_equal(fm.sigmas, want.sigmas)
    assert isinstance(pick(base, 9, 1024, 1024, "linear"), LinearScheduler)
    assert isinstance(pick(turbo, 9, 1024, 1024, "flow_match_euler_discrete"), FlowMatchEulerDiscreteScheduler)
    with pytest.raises(NotImplementedError):
        pick(base, 9, 1024, 1024, "ddim")


def test_weight_updates_invalidate_derived_caches():
    """Module.update and nn.quantize move the weights epoch, which empties every cache built from several layers'
    weights (row-fused blobs) the next time it is consulted."""
    import torch

    from mflux_b200 import nn

    class Owner:
        pass

    o = Owner()
    nn.fused_cache(o)["k"] = "blob"
    assert nn.fused_cache(o) == {"k": "blob"}
    m = nn.Module()
    m.lin = torch.nn.Linear(2, 2)
    m.update({"lin": {"weight": torch.zeros(2, 2)}}, strict=False)
    assert nn.fused_cache(o) == {}
    nn.fused_cache(o)["k"] = "blob"
    nn.quantize(torch.nn.Sequential(), class_predicate=lambda p, mod: False)
    assert nn.fused_cache(o) == {}


def test_flux2_kv_cache_modes_and_slots():
    """Flux2KVCache (flux2_kv_cache.py:13-61): only an extracting cache with reference tokens stores; the stored
    rows are the trailing num_ref_tokens of the layer's keys / values; an empty slot raises when it is read."""
    import pytest
    import torch

    from mflux_b200.flux2 import Flux2KVCache

    cache = Flux2KVCache(num_double_layers=2, num_single_layers=3)
    assert not cache.has_reference_tokens and not cache.is_extracting and not cache.is_cached
    k, v = torch.arange(2 * 10 * 4.0).reshape(2, 10, 4), -torch.arange(2 * 10 * 4.0).reshape(2, 10, 4)
    cache.store_reference("single", 1, k, v)           # not configured: nothing is kept
    with pytest.raises(RuntimeError):
        cache.load("single", 1)
    cache.configure(mode="extract", num_ref_tokens=0)   # extracting needs reference tokens
    assert not cache.is_extracting
    cache.configure(mode="extract", num_ref_tokens=3)
    assert cache.is_extracting and not cache.is_cached
    cache.store_reference("single", 1, k, v)
    cache.store_reference("double", 0, k, v)
    rk, rv = cache.load("single", 1)
    assert torch.equal(rk, k[:, -3:]) and torch.equal(rv, v[:, -3:])
    k += 1.0                                            # the cache holds copies
    assert torch.equal(rk, (k - 1.0)[:, -3:])
    cache.configure(mode="cached", num_ref_tokens=3)
    assert cache.is_cached and not cache.is_extracting
    cache.store_reference("single", 2, k, v)            # cached mode does not store
    with pytest.raises(RuntimeError):
        cache.load("single", 2)
    with pytest.raises(ValueError):
        cache.load("triple", 0)
    with pytest.raises(ValueError):
        cache.configure(mode="other", num_ref_tokens=1)


def test_oracle_rotary_layouts_agree_on_what_they_share():
    """The two rotary layouts of the q/k norm + RoPE kernel, restated: rotating (even, odd) pairs (FLUX, Krea-2) and
    x * cos + rotate_half(x) * sin with every angle stored twice (ERNIE). Both preserve the norm of a pair they
    rotate by one angle; the ERNIE layout pairs element j with j + 64 and reads angle j // 2 for either."""
    import torch

    from oracle import blocks
    from oracle import ernie as oe

    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 5, 2, 128, generator=g)
    ids = torch.stack([torch.arange(5.0), torch.arange(5.0) * 2, torch.arange(5.0) % 3], dim=1)
    cos, sin = oe.rope_cos_sin(ids)
    assert cos.shape == (5, 128) and torch.equal(cos[:, 0::2], cos[:, 1::2])     # every angle twice
    y = oe.apply_rotary_emb(x, cos, sin)
    j = 10
    want_lo = x[..., j] * cos[:, j][None, :, None] - x[..., j + 64] * sin[:, j][None, :, None]
    want_hi = x[..., j + 64] * cos[:, j + 64][None, :, None] + x[..., j] * sin[:, j + 64][None, :, None]
    torch.testing.assert_close(y[..., j], want_lo)
    torch.testing.assert_close(y[..., j + 64], want_hi)
    # position 0 has angle 0 everywhere: both layouts leave the row unchanged there
    torch.testing.assert_close(y[:, 0], x[:, 0])
    cs = torch.stack([cos[:, 0::2], sin[:, 0::2]], dim=-1)
    z = blocks.apply_rope(x.permute(0, 2, 1, 3), cs[None, None])
    torch.testing.assert_close(z[:, :, 0], x.permute(0, 2, 1, 3)[:, :, 0])
    # the pair layout is a true rotation: it keeps the norm of every (even, odd) pair (up to the bf16 rounding of the table)
    n_in = (x.permute(0, 2, 1, 3)[..., 0::2] ** 2 + x.permute(0, 2, 1, 3)[..., 1::2] ** 2)
    n_out = (z[..., 0::2] ** 2 + z[..., 1::2] ** 2)
    torch.testing.assert_close(n_out, n_in, rtol=2e-2, atol=1e-3)
