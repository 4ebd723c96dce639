"""Float32 CPU restatement of the reference's ERNIE-Image transformer blocks, driven by the parameters of a
`mflux_b200.ernie.ErnieBlocks` (quantized layers are dequantized with the oracle's own dequantizer).

Test infrastructure (see oracle/__init__.py); parity unpinned (the reference executes on MLX). Follows
src/mflux/models/ernie_image/model/ernie_transformer/transformer_block.py:24-36, attention.py:34-54,
feed_forward.py:12-13, rope_embedder.py:5-37 and transformer.py:147-153, executed as the reference writes it: every
angle stored twice, x * cos + rotate_half(x) * sin over the full head dimension.
"""
from __future__ import annotations

import torch

from . import blocks
from .flux import lin, silu


def rope_cos_sin(ids, axes_dim=(32, 48, 48), theta=256.0):
    """ErnieRopeEmbedder.__call__ + transformer.py:113-114: ids [S, 3] -> cos, sin [S, 128] (bf16-rounded)."""
    parts = []
    for i, dim in enumerate(axes_dim):
        scale = torch.arange(0, dim, 2, dtype=torch.float32) / dim
        omega = 1.0 / (theta ** scale)
        parts.append(ids[:, i].float()[:, None] * omega[None, :])
    emb = torch.cat(parts, dim=-1)                                   # [S, 64]
    emb = torch.stack([emb, emb], dim=-1).reshape(emb.shape[0], -1)  # [S, 128]: every angle twice
    return torch.cos(emb).to(torch.bfloat16).float(), torch.sin(emb).to(torch.bfloat16).float()


def apply_rotary_emb(x, cos, sin):
    """rope_embedder.py:31-37 on x [B, S, H, 128]."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    rot = torch.cat([-x2, x1], dim=-1)
    return x * cos[None, :, None, :] + rot * sin[None, :, None, :]


def forward(model, x, c, ids, key_bias=None, collect=None):
    """Stream [B, S, hidden] after all layers, float32."""
    x = x.float().cpu()
    d, heads = model.hidden_size, model.num_heads
    mod = lin(model.adaln_modulation, silu(c.float().cpu()))[:, None]
    shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = (mod[..., j * d:(j + 1) * d] for j in range(6))
    cos, sin = rope_cos_sin(ids, model.rope_axes_dim, model.rope_theta)
    b, s, _ = x.shape
    for i, blk in enumerate(model.layers):
        a, mlp = blk.self_attention, blk.mlp
        n = blocks.rms_norm(x, blk.adaLN_sa_ln.weight.detach().float().cpu(), model.eps) * (1 + scale_msa) + shift_msa
        q = lin(a.to_q, n).reshape(b, s, heads, 128)
        k = lin(a.to_k, n).reshape(b, s, heads, 128)
        v = lin(a.to_v, n).reshape(b, s, heads, 128)
        if a.norm_q is not None:
            q = blocks.rms_norm(q, a.norm_q.weight.detach().float().cpu(), model.eps)
            k = blocks.rms_norm(k, a.norm_k.weight.detach().float().cpu(), model.eps)
        q, k = apply_rotary_emb(q, cos, sin), apply_rotary_emb(k, cos, sin)
        o = blocks.sdpa(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), mask=key_bias)
        o = o.permute(0, 2, 1, 3).reshape(b, s, d)
        x = x + gate_msa * lin(a.to_out[0], o)
        n = blocks.rms_norm(x, blk.adaLN_mlp_ln.weight.detach().float().cpu(), model.eps) * (1 + scale_mlp) + shift_mlp
        gate = lin(mlp.gate_proj, n)
        x = x + gate_mlp * lin(mlp.linear_fc2, lin(mlp.up_proj, n) * torch.nn.functional.gelu(gate))
        if collect is not None:
            collect[f"layer{i}"] = x
    return x
