"""Float32 CPU restatement of the reference's FLUX.2 single-stream blocks, driven by the parameters of a
`mflux_b200.flux2.Flux2SingleStream` (quantized layers are dequantized with the oracle's own dequantizer).

Test infrastructure (see oracle/__init__.py); parity unpinned (the reference executes on MLX). Follows
src/mflux/models/flux2/model/flux2_transformer/single_transformer_block.py:19-40,
parallel_self_attention.py:22-78, feed_forward.py:10-12, modulation.py:11-19, pos_embed.py:11-31 and
src/mflux/models/flux/model/flux_transformer/common/attention_utils.py:83-99 (apply_rope_bshd), executed as the
reference does it: ONE projection, split into q, k, v and the two MLP halves, explicit concatenation.
"""
from __future__ import annotations

import torch

from . import blocks
from .flux import lin, silu


def rope_table(ids, axes_dim=(32, 32, 32, 32), theta=2000.0):
    """Flux2PosEmbed: ids [S, 4] -> (cos, sin) as [S, 64, 2]."""
    outs = []
    for i, dim in enumerate(axes_dim):
        scale = torch.arange(0, dim, 2, dtype=torch.float32) / dim
        omega = 1.0 / (theta ** scale)
        ang = ids[:, i].float()[:, None] * omega[None, :]
        outs.append(torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1))
    return torch.cat(outs, dim=1)


def forward(model, hidden_states, temb, cos_sin, collect=None, kv_cache=None):
    """Joint hidden states [B, S, D] after all single blocks, float32. `kv_cache` is a dict {"mode", "num_ref",
    "store": {layer: (k, v)}} restating Flux2KVCache (flux2_kv_cache.py): "extract" keeps the keys / values of the
    trailing num_ref tokens per layer, lets those tokens attend to themselves only and the others to everything
    (:63-99); "cached" appends the kept keys / values to the sequence's own (:51-61)."""
    x = hidden_states.float().cpu()
    d, heads = model.dim, model.heads
    mod = lin(model.single_stream_modulation.linear, silu(temb.float().cpu()))
    shift, scale, gate = mod[:, None, 0:d], mod[:, None, d:2 * d], mod[:, None, 2 * d:3 * d]
    cs = cos_sin.float().cpu()
    for i, blk in enumerate(model.single_transformer_blocks):
        a = blk.attn
        inner, mlp = a.inner_dim, a.mlp_hidden_dim
        n = (1 + scale) * blocks.layer_norm(x) + shift
        proj = lin(a.to_qkv_mlp_proj, n)
        q, k, v = (blocks.heads_first(proj[..., j * inner:(j + 1) * inner], heads) for j in range(3))
        q = blocks.rms_norm(q, a.norm_q.weight.detach().float().cpu(), a.norm_q.eps)
        k = blocks.rms_norm(k, a.norm_k.weight.detach().float().cpu(), a.norm_k.eps)
        q, k = blocks.apply_rope(q, cs[None, None]), blocks.apply_rope(k, cs[None, None])
        if kv_cache is not None and kv_cache["mode"] == "extract" and kv_cache["num_ref"] > 0:
            r = kv_cache["num_ref"]
            kv_cache["store"][i] = (k[:, :, -r:], v[:, :, -r:])
            o = torch.cat([blocks.sdpa(q[:, :, :-r], k, v), blocks.sdpa(q[:, :, -r:], k[:, :, -r:], v[:, :, -r:])],
                          dim=2)
            o = blocks.heads_last(o)
        elif kv_cache is not None and kv_cache["mode"] == "cached":
            rk, rv = kv_cache["store"][i]
            o = blocks.heads_last(blocks.sdpa(q, torch.cat([k, rk], dim=2), torch.cat([v, rv], dim=2)))
        else:
            o = blocks.heads_last(blocks.sdpa(q, k, v))
        x1, x2 = proj[..., 3 * inner:3 * inner + mlp], proj[..., 3 * inner + mlp:]
        out = lin(a.to_out, torch.cat([o, silu(x1) * x2], dim=-1))
        x = x + gate * out
        if collect is not None:
            collect[f"single{i}"] = x
    return x
