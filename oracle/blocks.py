"""Float32 restatement (torch on CPU) of the per-block arithmetic of the reference's FLUX transformer.

Test infrastructure (see oracle/__init__.py); parity unpinned for everything that MLX executes.
Every function names the reference lines it follows (paths under src/mflux/models/flux/model/flux_transformer/).
"""
from __future__ import annotations

import math

import torch


def layer_norm(x, eps=1e-6):
    """nn.LayerNorm(affine=False): biased variance over the last dim (ada_layer_norm_zero.py:9)."""
    x = x.float()
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) * torch.rsqrt(var + eps)


def rms_norm(x, weight=None, eps=1e-5):
    """nn.RMSNorm: x * rsqrt(mean(x^2) + eps) * weight (joint_attention.py:22-25)."""
    x = x.float()
    y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight.float()


def modulate(x, shift, scale, eps=1e-6):
    """norm(x) * (1 + scale[:, None]) + shift[:, None] (ada_layer_norm_zero.py:20)."""
    return layer_norm(x, eps) * (1 + scale.float()[:, None]) + shift.float()[:, None]


def rope_table(ids, axes_dim=(16, 56, 56), theta=10000.0):
    """EmbedND (embed_nd.py:12-31): ids [S, 3] -> (cos, sin) [S, 64, 2] for the rotated pairs."""
    outs = []
    for i, dim in enumerate(axes_dim):
        scale = torch.arange(0, dim, 2, dtype=torch.float32) / dim
        omega = 1.0 / (theta ** scale)
        ang = ids[:, i].float()[:, None] * omega[None, :]
        outs.append(torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1))
    return torch.cat(outs, dim=1)


def flux_ids(height, width, txt_len):
    """transformer.py:159-172: text ids are zero; image ids are (0, row, col) of the latent grid."""
    lh, lw = height // 16, width // 16
    img = torch.zeros(lh, lw, 3)
    img[:, :, 1] += torch.arange(lh)[:, None]
    img[:, :, 2] += torch.arange(lw)[None, :]
    return torch.cat([torch.zeros(txt_len, 3), img.reshape(lh * lw, 3)], dim=0)


def apply_rope(x, cos_sin):
    """attention_utils.py:75-80 on x [B, H, S, 128]: rotate (even, odd) pairs by [[cos,-sin],[sin,cos]]."""
    x = x.float()
    x0, x1 = x[..., 0::2], x[..., 1::2]
    c, s = cos_sin[..., 0], cos_sin[..., 1]
    o0 = c * x0 - s * x1
    o1 = s * x0 + c * x1
    return torch.stack([o0, o1], dim=-1).reshape(x.shape)


def additive_key_mask(mask, joint_seq_len, txt_seq_len):
    """AttentionUtils.convert_key_padding_mask_to_additive_mask (attention_utils.py:55-72) and
    QwenAttention._convert_mask_for_qwen (qwen_attention.py:117-135): a [B, St] keep-mask over the text keys
    becomes a [B, S] additive bias, 0 on kept and image keys and -1e9 on padded text keys (text keys first)."""
    m = mask.float()
    joint = torch.cat([m, torch.ones(m.shape[0], joint_seq_len - txt_seq_len)], dim=1)
    return (1.0 - joint) * (-1e9)


def sdpa(q, k, v, scale=None, mask=None):
    """mx.fast.scaled_dot_product_attention (attention_utils.py:48-52), float32, on [B, H, S, 128]; `mask` is an
    additive bias per key, [B, S], broadcast over heads and queries as the reference's [B, 1, 1, S] mask is.
    Large problems go head by head so that the score matrix of one head is all that is ever held."""
    q, k, v = q.float(), k.float(), v.float()
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    bias = None if mask is None else mask.float()[:, None, None, :]
    if q.shape[0] * q.shape[1] * q.shape[2] * k.shape[2] <= (1 << 27):
        s = q @ k.transpose(-1, -2) * scale
        return torch.softmax(s if bias is None else s + bias, dim=-1) @ v
    out = torch.empty(q.shape[:-1] + (v.shape[-1],), dtype=torch.float32)
    for b in range(q.shape[0]):
        for h in range(q.shape[1]):
            s = q[b, h] @ k[b, h].T * scale
            if bias is not None:
                s = s + bias[b, 0]
            out[b, h] = torch.softmax(s, dim=-1) @ v[b, h]
    return out


def heads_first(x, heads):
    """[B, S, H*128] -> [B, H, S, 128] (attention_utils.py:25-28)."""
    b, s, _ = x.shape
    return x.reshape(b, s, heads, -1).permute(0, 2, 1, 3)


def heads_last(x):
    """[B, H, S, 128] -> [B, S, H*128] (attention_utils.py:50-51)."""
    b, h, s, d = x.shape
    return x.permute(0, 2, 1, 3).reshape(b, s, h * d)


def gelu(x, approx=False):
    """nn.gelu (erf) / nn.gelu_approx (tanh) (joint_transformer_block.py:18-19)."""
    return torch.nn.functional.gelu(x.float(), approximate="tanh" if approx else "none")


def time_proj(t):
    """TimeTextEmbed._time_proj (time_text_embed.py:33-43): 256-wide sinusoid, cos half first."""
    half = 128
    exponent = -math.log(10000) * torch.arange(half, dtype=torch.float32) / half
    emb = t.float()[:, None] * torch.exp(exponent)[None, :]
    emb = torch.cat([torch.sin(emb), torch.cos(emb)], dim=-1)
    return torch.cat([emb[:, half:], emb[:, :half]], dim=-1)
