"""Float32 CPU restatement of the reference's Qwen-Image transformer forward pass and guidance combine,
driven by the parameters of a (tensor-parallel size 1) `mflux_b200.qwen.QwenTransformer`.

Test infrastructure (see oracle/__init__.py). Follows src/mflux/models/qwen/model/qwen_transformer/
qwen_transformer.py:37-72, qwen_transformer_block.py:27-76, qwen_attention.py:27-158, qwen_feed_forward.py:11-15,
qwen_rope.py:35-113, qwen_timesteps.py:15-34, qwen_transformer_rms_norm.py:11-23 and
variants/txt2img/qwen_image.py:165-174.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import blocks
from .flux import bf16, lin, silu


def rope_params(index, dim, theta=10000.0):
    scales = np.arange(0, dim, 2, dtype=np.float32) / dim
    omega = 1.0 / (theta ** scales)
    f = np.outer(np.asarray(index, dtype=np.float32), omega)
    return np.stack([np.cos(f), np.sin(f)], axis=-1)


def rope_tables(lh, lw, txt_len, axes=(16, 56, 56)):
    """QwenEmbedRopeMLX.__call__ with scale_rope=True for one (1, lh, lw) image: ((img cos,sin), (txt cos,sin))."""
    pos = np.arange(4096, dtype=np.int32)
    neg = (np.arange(4096, dtype=np.int32)[::-1] * -1) - 1
    pos_f = [rope_params(pos, a) for a in axes]
    neg_f = [rope_params(neg, a) for a in axes]
    fr = np.broadcast_to(pos_f[0][0:1].reshape(1, 1, 1, -1, 2), (1, lh, lw, axes[0] // 2, 2))
    fh = np.concatenate([neg_f[1][-(lh - lh // 2):], pos_f[1][: lh // 2]], axis=0).reshape(1, lh, 1, -1, 2)
    fw = np.concatenate([neg_f[2][-(lw - lw // 2):], pos_f[2][: lw // 2]], axis=0).reshape(1, 1, lw, -1, 2)
    fh = np.broadcast_to(fh, (1, lh, lw, axes[1] // 2, 2))
    fw = np.broadcast_to(fw, (1, lh, lw, axes[2] // 2, 2))
    img = np.concatenate([fr, fh, fw], axis=-2).reshape(lh * lw, -1, 2)
    start = max(lh // 2, lw // 2)
    txt = np.concatenate([f[start:start + txt_len] for f in pos_f], axis=1)
    return torch.from_numpy(img.astype(np.float32)), torch.from_numpy(txt.astype(np.float32))


def time_proj(timestep):
    half = 128
    exponent = -math.log(10000) * torch.arange(half, dtype=torch.float32) / half
    emb = bf16(torch.exp(exponent))                      # .astype(timesteps_dtype), the activation dtype
    emb = 1000.0 * (bf16(timestep.float())[:, None] * emb[None, :])
    emb = torch.cat([torch.sin(emb), torch.cos(emb)], dim=-1)
    return torch.cat([emb[:, half:], emb[:, :half]], dim=-1)


def rms(x, weight, eps):
    x = x.float()
    y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    return y * weight.detach().float().cpu()


def rope(x, cs):
    """_apply_rope_qwen on [B, S, H, 128] with cs [S, 64, 2]."""
    x = x.float()
    xr, xi = x[..., 0::2], x[..., 1::2]
    c, s = cs[None, :, None, :, 0], cs[None, :, None, :, 1]
    return torch.stack([xr * c - xi * s, xr * s + xi * c], dim=-1).reshape(x.shape)


def forward(model, hidden_states, encoder_hidden_states, timestep, height, width, collect=None, mask=None):
    """Predicted noise [B, Si, C] in float32. `mask` [B, St] (1 = real token, 0 = padding) is the reference's
    encoder_hidden_states_mask; `collect` (a dict) receives the two streams after every block."""
    cfg = model.cfg
    d, heads = cfg.hidden, cfg.heads
    hs = lin(model.img_in, hidden_states.float().cpu())
    enc = lin(model.txt_in, rms(encoder_hidden_states.float().cpu(), model.txt_norm.weight, model.txt_norm.eps))
    te = model.time_text_embed.timestep_embedder
    temb = lin(te.linear_2, silu(lin(te.linear_1, time_proj(timestep.float().cpu()))))
    sv = silu(temb)
    b, st = enc.shape[0], enc.shape[1]
    img_cs, txt_cs = rope_tables(height // 16, width // 16, st)
    key_bias = None
    if mask is not None and not bool((mask.float() >= 0.999).all()):   # qwen_attention.py:131-132
        key_bias = blocks.additive_key_mask(mask.cpu(), st + hs.shape[1], st)
    for i, blk in enumerate(model.transformer_blocks):
        a = blk.attn
        mi, mt = lin(blk.img_mod_linear, sv), lin(blk.txt_mod_linear, sv)
        ch = lambda m, j: m[:, j * d:(j + 1) * d]  # noqa: E731
        n_i = blocks.modulate(hs, ch(mi, 0), ch(mi, 1))
        n_t = blocks.modulate(enc, ch(mt, 0), ch(mt, 1))
        sp = lambda t: t.reshape(t.shape[0], t.shape[1], heads, 128)  # noqa: E731
        iq, ik, iv = sp(lin(a.to_q, n_i)), sp(lin(a.to_k, n_i)), sp(lin(a.to_v, n_i))
        tq, tk, tv = sp(lin(a.add_q_proj, n_t)), sp(lin(a.add_k_proj, n_t)), sp(lin(a.add_v_proj, n_t))
        iq, ik = rms(iq, a.norm_q.weight, a.norm_q.eps), rms(ik, a.norm_k.weight, a.norm_k.eps)
        tq, tk = rms(tq, a.norm_added_q.weight, a.norm_added_q.eps), rms(tk, a.norm_added_k.weight, a.norm_added_k.eps)
        iq, ik, tq, tk = rope(iq, img_cs), rope(ik, img_cs), rope(tq, txt_cs), rope(tk, txt_cs)
        q, k, v = torch.cat([tq, iq], 1), torch.cat([tk, ik], 1), torch.cat([tv, iv], 1)
        o = blocks.sdpa(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), mask=key_bias)
        o = o.permute(0, 2, 1, 3).reshape(b, -1, d)
        hs = hs + ch(mi, 2)[:, None] * lin(a.attn_to_out[0], o[:, st:])
        enc = enc + ch(mt, 2)[:, None] * lin(a.to_add_out, o[:, :st])
        hs = hs + ch(mi, 5)[:, None] * lin(blk.img_ff.mlp_out, blocks.gelu(
            lin(blk.img_ff.mlp_in, blocks.modulate(hs, ch(mi, 3), ch(mi, 4))), approx=True))
        enc = enc + ch(mt, 5)[:, None] * lin(blk.txt_ff.mlp_out, blocks.gelu(
            lin(blk.txt_ff.mlp_in, blocks.modulate(enc, ch(mt, 3), ch(mt, 4))), approx=True))
        if collect is not None:
            collect[f"block{i}"] = (enc, hs)
    m = lin(model.norm_out.linear, sv)
    x = blocks.layer_norm(hs) * (1 + m[:, :d])[:, None] + m[:, d:2 * d][:, None]
    return lin(model.proj_out, x)


def guided_noise(noise, noise_negative, guidance):
    n, nn = noise.float(), noise_negative.float()
    comb = nn + guidance * (n - nn)
    cond = torch.sqrt((n * n).sum(-1, keepdim=True) + 1e-12)
    cn = torch.sqrt((comb * comb).sum(-1, keepdim=True) + 1e-12)
    return comb * (cond / cn)
