"""Krea-2-shaped single-stream blocks on the B200 kernels: grouped-query attention with an output gate, SwiGLU,
one shared modulation vector.

Module tree, attribute names and arithmetic follow the reference's
src/mflux/models/krea2/model/krea2_transformer/transformer_block.py:10-24, attention.py:9-42, feed_forward.py:5-17,
modulation.py:5-13, common.py:5-28 and rope_embedder.py:26-37 (no biases; RMSNorm weights stored as offsets from 1;
`vec` is the transformer's 6 * features conditioning vector, to which every block adds its own learned offset).
What runs where:
  * prenorm / postnorm + modulation: `norm_modulate` (RMSNorm with weight scale + 1, then * (1 + scale) + shift);
  * wq | wk | wv | gate: ONE quantized matmul over the four layers' rows into a [q | k | v | gate] buffer;
  * q/k RMSNorm + RoPE: `qknorm_rope` with fewer key heads than query heads, in place;
  * attention: `fmha_ex`, query head h reading key/value head h // (heads // kvheads): the reference's
    mx.repeat of K and V (attention.py:36-39) never happens;
  * `out * sigmoid(gate)`: `act_mul` in place;
  * wo and mlp.down: quantized matmuls with the gated residual as their epilogue (x + gate * y);
  * mlp.gate | mlp.up: one quantized matmul with the SwiGLU epilogue.
"""
from __future__ import annotations

import torch

from . import nn, ops
from .flux import FusedRows, _call, _Ctx
from .zimage import FusedSwiGLU


class Krea2RMSNorm(nn.Module):
    """common.py:5-16: the stored `scale` is the weight's offset from 1."""

    def __init__(self, dim: int, eps: float = 1e-5, device="cuda"):
        super().__init__()
        self.scale = torch.nn.Parameter(torch.zeros(dim, dtype=torch.float32, device=device), requires_grad=False)
        self.eps = eps

    def weight(self) -> torch.Tensor:
        return self.scale.data.float() + 1.0


class Krea2QKNorm(nn.Module):
    def __init__(self, head_dim: int, eps: float = 1e-5, device="cuda"):
        super().__init__()
        self.qnorm, self.knorm = Krea2RMSNorm(head_dim, eps, device), Krea2RMSNorm(head_dim, eps, device)


class DoubleSharedModulation(nn.Module):
    """modulation.py:5-13: vec + lin, split in six."""

    def __init__(self, dim: int, device="cuda"):
        super().__init__()
        self.lin = torch.nn.Parameter(torch.zeros(6 * dim, dtype=torch.float32, device=device), requires_grad=False)


class Krea2Attention(nn.Module):
    def __init__(self, ctx, dim: int, heads: int, kvheads: int | None = None):
        super().__init__()
        self.heads, self.kvheads = heads, heads if kvheads is None else kvheads
        if dim != heads * 128:
            raise ValueError("dim must equal heads * 128 (head dimension 128)")
        if self.heads % self.kvheads != 0:
            raise ValueError("heads must be a multiple of kvheads")
        self.wq = ctx.linear(dim, 128 * self.heads, bias=False)
        self.wk = ctx.linear(dim, 128 * self.kvheads, bias=False)
        self.wv = ctx.linear(dim, 128 * self.kvheads, bias=False)
        self.gate = ctx.linear(dim, dim, bias=False)
        self.qknorm = Krea2QKNorm(128, device=ctx.device)
        self.wo = ctx.linear(dim, dim, bias=False)


class Krea2SwiGLU(nn.Module):
    def __init__(self, ctx, features: int, multiplier: int, multiple: int = 128):
        super().__init__()
        mlpdim = int(2 * features / 3) * multiplier
        self.mlpdim = multiple * ((mlpdim + multiple - 1) // multiple)
        self.gate = ctx.linear(features, self.mlpdim, bias=False)
        self.up = ctx.linear(features, self.mlpdim, bias=False)
        self.down = ctx.linear(self.mlpdim, features, bias=False)


class SingleStreamBlock(nn.Module):
    def __init__(self, ctx, features: int, heads: int, multiplier: int, kvheads: int | None = None):
        super().__init__()
        self.mod = DoubleSharedModulation(features, ctx.device)
        self.prenorm, self.postnorm = Krea2RMSNorm(features, device=ctx.device), Krea2RMSNorm(features, device=ctx.device)
        self.attn = Krea2Attention(ctx, features, heads, kvheads)
        self.mlp = Krea2SwiGLU(ctx, features, multiplier)


class Krea2SingleStream(nn.Module):
    """A run of SingleStreamBlocks on one [B, S, features] stream (transformer.py's block loop)."""

    def __init__(self, features: int = 3072, heads: int = 24, kvheads: int | None = 8, multiplier: int = 4,
                 num_layers: int = 4, bits: int | None = 4, device="cuda", std: float = 0.02, seed: int = 0,
                 theta: float = 1000.0, axes_dim=(32, 48, 48)):
        super().__init__()
        if sum(axes_dim) != 128:
            raise ValueError("the rotary axes must add up to the head dimension 128")
        self.features, self.heads, self.kvheads = features, heads, heads if kvheads is None else kvheads
        self.theta, self.axes_dim = theta, tuple(axes_dim)
        ctx = _Ctx(device, bits, std, seed, "mlx")
        self.blocks = torch.nn.ModuleList([SingleStreamBlock(ctx, features, heads, multiplier, kvheads)
                                           for _ in range(num_layers)])
        g = torch.Generator(device=device).manual_seed(seed + 1)
        for blk in self.blocks:   # non-trivial norm weights and modulation offsets (a checkpoint would bring them)
            for prm in (blk.mod.lin, blk.prenorm.scale, blk.postnorm.scale, blk.attn.qknorm.qnorm.scale,
                        blk.attn.qknorm.knorm.scale):
                prm.data.copy_(torch.randn(prm.shape, device=device, generator=g) * 0.1)
        self._buffers_for = None
        self.trace = None

    def rope_table(self, ids: torch.Tensor) -> torch.Tensor:
        """Krea2RopeEmbedder (rope_embedder.py:13-29): position ids [S, 3] -> (cos, sin) [S, 64, 2] per rotated pair."""
        outs = []
        pos = ids.float().cpu()
        for i, dim in enumerate(self.axes_dim):
            omega = 1.0 / (self.theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
            ang = pos[:, i:i + 1] * omega[None, :]
            outs.append(torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1))
        return torch.cat(outs, dim=1).contiguous()

    def forward(self, x: torch.Tensor, vec: torch.Tensor, cos_sin: torch.Tensor) -> torch.Tensor:
        """x [B, S, features] (float32 residual stream, updated in place and returned), vec [B, 6 * features],
        cos_sin [S, 64, 2] on the device."""
        b, s, d = x.shape
        dev = x.device
        h, hk = self.heads, self.kvheads
        wq, wkv = h * 128, hk * 128
        mlpdim = self.blocks[0].mlp.mlpdim
        key = (b, s, str(dev))
        if self._buffers_for != key:
            self.nbuf = torch.empty(b, s, d, dtype=torch.bfloat16, device=dev)
            self.proj = torch.empty(b, s, wq + 2 * wkv + d, dtype=torch.bfloat16, device=dev)   # q | k | v | gate
            self.abuf = torch.empty(b, s, d, dtype=torch.bfloat16, device=dev)
            self.hbuf = torch.empty(b, s, mlpdim, dtype=torch.bfloat16, device=dev)
            self._buffers_for = key
        xs = x if x.dtype == torch.float32 else x.float()
        fused = nn.fused_cache(self)
        for i, blk in enumerate(self.blocks):
            a, mlp = blk.attn, blk.mlp
            m = (vec.float() + blk.mod.lin.data[None]).to(torch.bfloat16)   # [B, 6D]
            prescale, preshift, pregate, postscale, postshift, postgate = (m[:, j * d:(j + 1) * d] for j in range(6))
            ops.norm_modulate(xs, preshift, prescale, weight=blk.prenorm.weight(), eps=blk.prenorm.eps, rms=True,
                              out=self.nbuf)
            f = fused.get(("proj", i))
            if f is None:
                layers = [a.wq, a.wk, a.wv, a.gate]
                f = FusedRows(layers) if FusedRows.accepts(layers) else \
                    (lambda t, out, ls=layers: out.copy_(torch.cat([l(t) for l in ls], dim=-1)))
                fused[("proj", i)] = f
            f(self.nbuf, self.proj)
            qkv = self.proj[..., :wq + 2 * wkv]
            qw, kw = a.qknorm.qnorm.weight(), a.qknorm.knorm.weight()
            ops.qknorm_rope(qkv, h, qw, kw, qw, kw, 0, cos_sin, a.qknorm.qnorm.eps, kv_heads=hk)
            ops.fmha_ex(qkv[..., :wq], qkv[..., wq:wq + wkv], qkv[..., wq + wkv:], h, hk, out=self.abuf)
            ops.act_mul(self.abuf, self.proj[..., wq + 2 * wkv:], "sigmoid")
            _call(a.wo, self.abuf, epilogue="gate_residual", gate=pregate, residual=xs, out=xs)
            ops.norm_modulate(xs, postshift, postscale, weight=blk.postnorm.weight(), eps=blk.postnorm.eps, rms=True,
                              out=self.nbuf)
            g = fused.get(("mlp", i))
            if g is None:
                g = FusedSwiGLU(mlp.gate, mlp.up) if FusedSwiGLU.accepts(mlp.gate, mlp.up) else \
                    (lambda t, out, mm=mlp: out.copy_(torch.nn.functional.silu(mm.gate(t).float()) * mm.up(t).float()))
                fused[("mlp", i)] = g
            g(self.nbuf, self.hbuf)
            _call(mlp.down, self.hbuf, epilogue="gate_residual", gate=postgate, residual=xs, out=xs)
            if self.trace is not None:
                self.trace[f"block{i}"] = xs.clone()
        return xs
