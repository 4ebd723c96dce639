"""Float32 CPU restatement of the reference's Krea-2 single-stream blocks, driven by the parameters of a
`mflux_b200.krea2.Krea2SingleStream` (quantized layers are dequantized with the oracle's own dequantizer).

Test infrastructure (see oracle/__init__.py); parity unpinned (the reference executes on MLX). Follows
src/mflux/models/krea2/model/krea2_transformer/transformer_block.py:20-24, attention.py:24-42 (K and V repeated
heads // kvheads times along the head axis), feed_forward.py:16-17, modulation.py:10-13, common.py:11-16,26-28 and
rope_embedder.py:31-37.
"""
from __future__ import annotations

import torch

from . import blocks
from .flux import bf16, lin, silu


def rope_table(ids, axes_dim=(32, 48, 48), theta=1000.0):
    """Krea2RopeEmbedder: ids [S, 3] -> (cos, sin) as [S, 64, 2] (the rotation [[cos, -sin], [sin, cos]] per pair)."""
    outs = []
    for i, dim in enumerate(axes_dim):
        scale = torch.arange(0, dim, 2, dtype=torch.float32) / dim
        omega = 1.0 / (theta ** scale)
        ang = ids[:, i].float()[:, None] * omega[None, :]
        outs.append(torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1))
    return torch.cat(outs, dim=1)


def forward(model, x, vec, cos_sin, collect=None):
    """Stream [B, S, features] after all blocks, float32."""
    x = x.float().cpu()
    d, heads, kvheads = model.features, model.heads, model.kvheads
    cs = cos_sin.float().cpu()
    for i, blk in enumerate(model.blocks):
        a, mlp = blk.attn, blk.mlp
        m = bf16(vec.float().cpu() + blk.mod.lin.detach().float().cpu()[None])[:, None]
        prescale, preshift, pregate, postscale, postshift, postgate = (m[..., j * d:(j + 1) * d] for j in range(6))
        n = (1 + prescale) * blocks.rms_norm(x, blk.prenorm.scale.detach().float().cpu() + 1.0, blk.prenorm.eps) + preshift
        q = blocks.heads_first(lin(a.wq, n), heads)
        k = blocks.heads_first(lin(a.wk, n), kvheads)
        v = blocks.heads_first(lin(a.wv, n), kvheads)
        gate = lin(a.gate, n)
        q = blocks.rms_norm(q, a.qknorm.qnorm.scale.detach().float().cpu() + 1.0, a.qknorm.qnorm.eps)
        k = blocks.rms_norm(k, a.qknorm.knorm.scale.detach().float().cpu() + 1.0, a.qknorm.knorm.eps)
        q, k = blocks.apply_rope(q, cs[None, None]), blocks.apply_rope(k, cs[None, None])
        rep = heads // kvheads
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        o = blocks.heads_last(blocks.sdpa(q, k, v))
        x = x + pregate * lin(a.wo, o * torch.sigmoid(gate))
        n = (1 + postscale) * blocks.rms_norm(x, blk.postnorm.scale.detach().float().cpu() + 1.0, blk.postnorm.eps) + postshift
        x = x + postgate * lin(mlp.down, silu(lin(mlp.gate, n)) * lin(mlp.up, n))
        if collect is not None:
            collect[f"block{i}"] = x
    return x
