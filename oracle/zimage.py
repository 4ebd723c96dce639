"""Float32 CPU restatement of the reference's Z-Image transformer forward pass, driven by the parameters of a
`mflux_b200.zimage.ZImageTransformer` (quantized layers are dequantized with the oracle's own dequantizer).

Test infrastructure (see oracle/__init__.py); parity unpinned (the reference executes on MLX, which cannot run
here). Follows src/mflux/models/z_image/model/z_image_transformer/transformer.py:53-143 (forward),
:146-182 (_patchify), :184-199 (_unpatchify), transformer_block.py:19-38, context_block.py:17-24,
attention.py:37-98, feed_forward.py:13-14, final_layer.py:12-17, rope_embedder.py:20-41,
timestep_embedder.py:21-38 -- executed as the reference does it: one sample at a time, separate q/k/v and
w1/w3 projections, explicit concatenation of image and caption tokens.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import blocks
from .flux import lin, silu


def coord_grid(size, start):
    """_create_coord_grid (transformer.py:201-206)."""
    axes = [np.arange(x0, x0 + span, dtype=np.int32) for x0, span in zip(start, size)]
    return np.stack(np.meshgrid(*axes, indexing="ij"), axis=-1)


def patchify(image, cap_feats, p=2, pf=1):
    """_patchify for one sample: image [C, F, H, W], cap_feats [L, Dc]."""
    cap_len = cap_feats.shape[0]
    cap_pad = (-cap_len) % 32
    cap_ids = coord_grid((cap_len + cap_pad, 1, 1), (1, 0, 0)).reshape(-1, 3)
    cap_mask = np.concatenate([np.zeros(cap_len, dtype=bool), np.ones(cap_pad, dtype=bool)])
    cap = torch.cat([cap_feats, cap_feats[-1:].repeat(cap_pad, 1)], dim=0) if cap_pad > 0 else cap_feats
    c, f, h, w = image.shape
    ft, ht, wt = f // pf, h // p, w // p
    img = image.reshape(c, ft, pf, ht, p, wt, p).permute(1, 3, 5, 2, 4, 6, 0).reshape(ft * ht * wt, pf * p * p * c)
    n = img.shape[0]
    pad = (-n) % 32
    ids = coord_grid((ft, ht, wt), (cap_len + cap_pad + 1, 0, 0)).reshape(-1, 3)
    if pad > 0:
        ids = np.concatenate([ids, np.zeros((pad, 3), dtype=np.int32)], axis=0)
        img = torch.cat([img, img[-1:].repeat(pad, 1)], dim=0)
    mask = np.concatenate([np.zeros(n, dtype=bool), np.ones(pad, dtype=bool)])
    return img, cap, (f, h, w), ids, cap_ids, mask, cap_mask


def unpatchify(x, size, c, p=2, pf=1):
    f, h, w = size
    n = (f // pf) * (h // p) * (w // p)
    x = x[:n].reshape(f // pf, h // p, w // p, pf, p, p, c).permute(6, 0, 3, 1, 4, 2, 5)
    return x.reshape(c, f, h, w)


def rope_tables(axes_dims, axes_lens, theta):
    """RopeEmbedder._precompute_freqs_cis: per axis [len, d/2, 2] of (cos, sin)."""
    out = []
    for d, e in zip(axes_dims, axes_lens):
        freqs = 1.0 / (np.float32(theta) ** (np.arange(0, d, 2, dtype=np.float32) / np.float32(d)))
        ang = np.outer(np.arange(e, dtype=np.float32), freqs.astype(np.float32)).astype(np.float32)
        out.append(np.stack([np.cos(ang), np.sin(ang)], axis=-1))
    return out


def rope_lookup(tables, ids):
    """RopeEmbedder.__call__: gather every axis' table at the position ids and concatenate -> [S, 64, 2]."""
    return torch.from_numpy(np.concatenate([tables[i][ids[:, i].astype(np.int64)] for i in range(len(tables))],
                                           axis=1).astype(np.float32))


def apply_rotary(x, freqs):
    """_apply_rotary_emb on [1, S, H, 128] with freqs [S, 64, 2]: (real, imag) = consecutive element pairs."""
    b, s, h, d = x.shape
    x = x.float().reshape(b, s, h, d // 2, 2)
    fr = freqs[None, :, None]
    xr, xi = x[..., 0], x[..., 1]
    c, sn = fr[..., 0], fr[..., 1]
    return torch.stack([xr * c - xi * sn, xr * sn + xi * c], dim=-1).reshape(b, s, h, d)


def timestep_embedding(t, dim=256, max_period=10000.0):
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


def rms(x, norm):
    return blocks.rms_norm(x, norm.weight.detach().cpu(), norm.eps)


def attention(a, x, freqs, heads):
    b, s, d = x.shape
    sp = lambda t: t.reshape(b, s, heads, d // heads)  # noqa: E731
    q, k, v = sp(lin(a.to_q, x)), sp(lin(a.to_k, x)), sp(lin(a.to_v, x))
    q, k = rms(q, a.norm_q), rms(k, a.norm_k)
    q, k = apply_rotary(q, freqs), apply_rotary(k, freqs)
    o = blocks.sdpa(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), scale=(d // heads) ** -0.5)
    return lin(a.to_out[0], o.permute(0, 2, 1, 3).reshape(b, s, d))


def feed_forward(ff, x):
    return lin(ff.w2, silu(lin(ff.w1, x)) * lin(ff.w3, x))


def block(blk, x, freqs, t_emb, heads):
    """ZImageTransformerBlock.__call__ (t_emb given) or ZImageContextBlock.__call__ (t_emb None)."""
    if t_emb is not None:
        mod = lin(blk.adaLN_modulation[0], t_emb)[:, None]
        scale_msa, gate_msa, scale_mlp, gate_mlp = torch.chunk(mod, 4, dim=2)
        scale_msa, scale_mlp = 1.0 + scale_msa, 1.0 + scale_mlp
        gate_msa, gate_mlp = torch.tanh(gate_msa), torch.tanh(gate_mlp)
    else:
        scale_msa = gate_msa = scale_mlp = gate_mlp = 1.0
    attn_out = attention(blk.attention, rms(x, blk.attention_norm1) * scale_msa, freqs, heads)
    x = x + gate_msa * rms(attn_out, blk.attention_norm2)
    ffn_out = feed_forward(blk.feed_forward, rms(x, blk.ffn_norm1) * scale_mlp)
    return x + gate_mlp * rms(ffn_out, blk.ffn_norm2)


def forward_one(model, image, timestep, cap_feats, collect=None):
    """ZImageTransformer.__call__ for one sample: image [C, F, H, W], timestep scalar tensor, cap_feats [L, Dc]."""
    cfg = model.cfg
    heads = cfg.n_heads
    tables = rope_tables(cfg.axes_dims, cfg.axes_lens, cfg.rope_theta)
    te = model.t_embedder
    t_emb = lin(te.linear2, silu(lin(te.linear1, timestep_embedding(timestep.reshape(1).float() * cfg.t_scale))))
    x_emb, cap_emb, size, x_ids, cap_ids, x_mask, cap_mask = patchify(image.float(), cap_feats.float(),
                                                                      cfg.patch_size, cfg.f_patch_size)
    x_emb = lin(model.all_x_embedder[cfg.key], x_emb)
    x_emb = torch.where(torch.from_numpy(x_mask)[:, None], model.x_pad_token.detach().float().cpu(), x_emb)
    x_freqs = rope_lookup(tables, x_ids)
    x_emb = x_emb[None]
    for i, layer in enumerate(model.noise_refiner):
        x_emb = block(layer, x_emb, x_freqs, t_emb, heads)
        if collect is not None:
            collect.setdefault(f"noise{i}", []).append(x_emb[0])
    cap_emb = lin(model.cap_embedder[1], rms(cap_emb, model.cap_embedder[0]))
    cap_emb = torch.where(torch.from_numpy(cap_mask)[:, None], model.cap_pad_token.detach().float().cpu(), cap_emb)
    cap_freqs = rope_lookup(tables, cap_ids)
    cap_emb = cap_emb[None]
    for i, layer in enumerate(model.context_refiner):
        cap_emb = block(layer, cap_emb, cap_freqs, None, heads)
        if collect is not None:
            collect.setdefault(f"context{i}", []).append(cap_emb[0])
    x_len = x_emb.shape[1]
    unified = torch.cat([x_emb, cap_emb], dim=1)
    freqs = torch.cat([x_freqs, cap_freqs], dim=0)
    for i, layer in enumerate(model.layers):
        unified = block(layer, unified, freqs, t_emb, heads)
        if collect is not None:
            collect.setdefault(f"layer{i}", []).append(unified[0])
    fl = model.all_final_layer[cfg.key]
    scale = 1.0 + lin(fl.adaLN_modulation[0], silu(t_emb))
    unified = lin(fl.linear, blocks.layer_norm(unified, 1e-6) * scale[:, None])
    return -unpatchify(unified[0, :x_len], size, cfg.in_channels, cfg.patch_size, cfg.f_patch_size)


def forward(model, images, timesteps, cap_feats, collect=None):
    """All samples, one at a time as the reference runs them. `collect` (a dict) receives, per main layer, the list
    of the samples' unified streams [image tokens, then caption tokens] after that layer ("layer{i}"), and the image
    / caption streams after every refiner block ("noise{i}", "context{i}")."""
    return torch.stack([forward_one(model, images[i], timesteps[i], cap_feats[i], collect)
                        for i in range(images.shape[0])])
