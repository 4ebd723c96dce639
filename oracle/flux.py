"""Float32 CPU restatement of the reference's FLUX transformer forward pass, driven by the parameters of a
`mflux_b200.flux.Transformer` (quantized layers are dequantized with the oracle's own dequantizer).

Test infrastructure (see oracle/__init__.py). Follows, function by function,
src/mflux/models/flux/model/flux_transformer/transformer.py:32-80, joint_transformer_block.py:21-91,
joint_attention.py:27-84, single_transformer_block.py:17-58, single_block_attention.py:20-44,
ada_layer_norm_zero.py:11-21, ada_layer_norm_zero_single.py:11-18, ada_layer_norm_continuous.py:14-20,
feed_forward.py:12-16, time_text_embed.py:19-43 -- executed as the reference does it: separate q/k/v
projections, explicit concatenations, one sample at a time semantics (batched here, which is equivalent).
"""
from __future__ import annotations

import numpy as np
import torch

from . import blocks
from .quant import dequantize_affine


def dense(layer):
    """(W float32 [N, K], bias float32 or None) of a Linear or QuantizedLinear."""
    if hasattr(layer, "scales"):
        w = dequantize_affine(layer.weight.detach().cpu().numpy(), layer.scales.detach().float().cpu().numpy(),
                              layer.biases.detach().float().cpu().numpy(), layer.group_size, layer.bits)
        w = torch.from_numpy(w)
    else:
        w = layer.weight.detach().float().cpu()
    b = None if layer.bias is None else layer.bias.detach().float().cpu()
    return w, b


def lin(layer, x):
    """Linear / QuantizedLinear, or a LoRA wrapper around one: LoRALinear.__call__
    (src/mflux/models/common/lora/layer/linear_lora_layer.py:50-53) and FusedLoRALinear.__call__
    (fused_linear_lora_layer.py:13-20)."""
    if hasattr(layer, "loras"):
        y = lin(layer.base_linear, x)
        for lo in layer.loras:
            y = y + lo.scale * (x.float() @ lo.lora_A.detach().float().cpu()) @ lo.lora_B.detach().float().cpu()
        return y
    if hasattr(layer, "lora_A"):
        return lin(layer.linear, x) + layer.scale * (x.float() @ layer.lora_A.detach().float().cpu()) \
            @ layer.lora_B.detach().float().cpu()
    w, b = dense(layer)
    y = x.float() @ w.T
    return y if b is None else y + b


def silu(x):
    return torch.nn.functional.silu(x.float())


def bf16(x):
    """Values the reference holds in bf16 (its compute dtype) at this point."""
    return x.to(torch.bfloat16).float()


def conditioning(model, timestep, pooled, guidance):
    tte = model.time_text_embed
    ts = bf16(timestep.float().cpu())
    e = lin(tte.timestep_embedder.linear_2, silu(lin(tte.timestep_embedder.linear_1, blocks.time_proj(ts))))
    if tte.guidance_embedder is not None:
        g = bf16(guidance.float().cpu())
        e = e + lin(tte.guidance_embedder.linear_2, silu(lin(tte.guidance_embedder.linear_1, blocks.time_proj(g))))
    p = lin(tte.text_embedder.linear_2, silu(lin(tte.text_embedder.linear_1, pooled.float().cpu())))
    return e + p


def attention(q, k, v, heads, cos_sin, nq, nk, split=None, nq_a=None, nk_a=None):
    """process_qkv + apply_rope + compute_attention on [B, S, D] projections."""
    q, k, v = (blocks.heads_first(t, heads) for t in (q, k, v))
    if split is None:
        q, k = blocks.rms_norm(q, nq.weight.detach().float().cpu()), blocks.rms_norm(k, nk.weight.detach().float().cpu())
    else:
        q = torch.cat([blocks.rms_norm(q[:, :, :split], nq_a.weight.detach().float().cpu()),
                       blocks.rms_norm(q[:, :, split:], nq.weight.detach().float().cpu())], dim=2)
        k = torch.cat([blocks.rms_norm(k[:, :, :split], nk_a.weight.detach().float().cpu()),
                       blocks.rms_norm(k[:, :, split:], nk.weight.detach().float().cpu())], dim=2)
    q, k = blocks.apply_rope(q, cos_sin[None, None]), blocks.apply_rope(k, cos_sin[None, None])
    return blocks.heads_last(blocks.sdpa(q, k, v))


def forward(model, hidden_states, prompt_embeds, pooled, timestep, guidance, height, width, collect=None):
    """Predicted noise [B, Si, C] in float32; `collect` (a dict) receives the streams after every block."""
    cfg = model.cfg
    d, heads = cfg.hidden, cfg.heads
    hs = lin(model.x_embedder, hidden_states.float().cpu())
    enc = lin(model.context_embedder, prompt_embeds.float().cpu())
    st = enc.shape[1]
    vec = conditioning(model, timestep, pooled, guidance)
    sv = silu(vec)
    cos_sin = blocks.rope_table(blocks.flux_ids(height, width, st))
    for i, blk in enumerate(model.transformer_blocks):
        a = blk.attn
        mi = lin(blk.norm1.linear, sv)
        mt = lin(blk.norm1_context.linear, sv)
        ch = lambda m, j: m[:, j * d:(j + 1) * d]  # noqa: E731
        n_i = blocks.modulate(hs, ch(mi, 0), ch(mi, 1))
        n_t = blocks.modulate(enc, ch(mt, 0), ch(mt, 1))
        q = torch.cat([lin(a.add_q_proj, n_t), lin(a.to_q, n_i)], dim=1)
        k = torch.cat([lin(a.add_k_proj, n_t), lin(a.to_k, n_i)], dim=1)
        v = torch.cat([lin(a.add_v_proj, n_t), lin(a.to_v, n_i)], dim=1)
        o = attention(q, k, v, heads, cos_sin, a.norm_q, a.norm_k, st, a.norm_added_q, a.norm_added_k)
        o_t, o_i = o[:, :st], o[:, st:]
        hs = hs + ch(mi, 2)[:, None] * lin(a.to_out[0], o_i)
        enc = enc + ch(mt, 2)[:, None] * lin(a.to_add_out, o_t)
        hs = hs + ch(mi, 5)[:, None] * lin(blk.ff.linear2,
                                           blocks.gelu(lin(blk.ff.linear1, blocks.modulate(hs, ch(mi, 3), ch(mi, 4)))))
        enc = enc + ch(mt, 5)[:, None] * lin(
            blk.ff_context.linear2,
            blocks.gelu(lin(blk.ff_context.linear1, blocks.modulate(enc, ch(mt, 3), ch(mt, 4))), approx=True))
        if collect is not None:
            collect[f"joint{i}"] = torch.cat([enc, hs], dim=1)
    x = torch.cat([enc, hs], dim=1)
    for i, blk in enumerate(model.single_transformer_blocks):
        a = blk.attn
        m = lin(blk.norm.linear, sv)
        n = blocks.modulate(x, m[:, :d], m[:, d:2 * d])
        o = attention(lin(a.to_q, n), lin(a.to_k, n), lin(a.to_v, n), heads, cos_sin, a.norm_q, a.norm_k)
        mlp = blocks.gelu(lin(blk.proj_mlp, n), approx=True)
        x = x + m[:, 2 * d:3 * d][:, None] * lin(blk.proj_out, torch.cat([o, mlp], dim=2))
        if collect is not None:
            collect[f"single{i}"] = x
    x = x[:, st:]
    m = lin(model.norm_out.linear, sv)
    x = blocks.layer_norm(x) * (1 + m[:, :d])[:, None] + m[:, d:2 * d][:, None]
    return lin(model.proj_out, x)
