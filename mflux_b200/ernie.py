"""ERNIE-Image-shaped transformer blocks on the B200 kernels: one modulation shared by all blocks, RMSNorm with
weights before each sub-layer, rotary embedding over half-split pairs, GeGLU feed-forward.

Module tree, attribute names and arithmetic follow the reference's
src/mflux/models/ernie_image/model/ernie_transformer/transformer_block.py:8-36, attention.py:8-54,
feed_forward.py:5-13, rope_embedder.py:5-37 and transformer.py:65,147-156 (no biases in the blocks; the six
modulation vectors come from ONE adaln_modulation linear and are the same for every block). What runs where:
  * adaLN_sa_ln / adaLN_mlp_ln + modulation: `norm_modulate` (RMSNorm with weight, then * (1 + scale) + shift);
  * to_q | to_k | to_v: one quantized matmul; norm_q / norm_k + rotary embedding: `qknorm_rope(rope_mode="halves")`;
  * attention with the text-padding mask as a per-key bias: `fmha`;
  * to_out and linear_fc2: quantized matmuls with the gated residual as their epilogue;
  * gate_proj | up_proj: one quantized matmul into a [gate | up] buffer, `act_mul(up, gate, "gelu")` in place,
    linear_fc2 reads the up half of that buffer.
"""
from __future__ import annotations

import torch

from . import nn, ops
from .flux import FusedRows, RMSNorm, _call, _Ctx


class ErnieAttention(nn.Module):
    def __init__(self, ctx, hidden_size: int, num_heads: int, eps: float, qk_layernorm: bool):
        super().__init__()
        if hidden_size != num_heads * 128:
            raise ValueError("hidden_size must equal num_heads * 128 (head dimension 128)")
        self.num_heads = num_heads
        self.to_q, self.to_k, self.to_v = (ctx.linear(hidden_size, hidden_size, bias=False) for _ in range(3))
        self.to_out = torch.nn.ModuleList([ctx.linear(hidden_size, hidden_size, bias=False)])
        self.norm_q = RMSNorm(128, eps, ctx.device) if qk_layernorm else None
        self.norm_k = RMSNorm(128, eps, ctx.device) if qk_layernorm else None


class ErnieFeedForward(nn.Module):
    def __init__(self, ctx, hidden_size: int, ffn_hidden_size: int):
        super().__init__()
        self.gate_proj = ctx.linear(hidden_size, ffn_hidden_size, bias=False)
        self.up_proj = ctx.linear(hidden_size, ffn_hidden_size, bias=False)
        self.linear_fc2 = ctx.linear(ffn_hidden_size, hidden_size, bias=False)


class ErnieTransformerBlock(nn.Module):
    def __init__(self, ctx, hidden_size: int, num_heads: int, ffn_hidden_size: int, eps: float, qk_layernorm: bool):
        super().__init__()
        self.adaLN_sa_ln = RMSNorm(hidden_size, eps, ctx.device)
        self.self_attention = ErnieAttention(ctx, hidden_size, num_heads, eps, qk_layernorm)
        self.adaLN_mlp_ln = RMSNorm(hidden_size, eps, ctx.device)
        self.mlp = ErnieFeedForward(ctx, hidden_size, ffn_hidden_size)


class ErnieBlocks(nn.Module):
    """`adaln_modulation` + `layers` of ErnieTransformer (transformer.py:65,68-71,147-156) on the joint
    [image, text] sequence."""

    def __init__(self, hidden_size: int = 4096, num_attention_heads: int = 32, num_layers: int = 36,
                 ffn_hidden_size: int = 12288, rope_theta: float = 256.0, rope_axes_dim=(32, 48, 48),
                 eps: float = 1e-6, qk_layernorm: bool = True, bits: int | None = 4, device="cuda",
                 std: float = 0.02, seed: int = 0):
        super().__init__()
        if sum(rope_axes_dim) != 128:
            raise ValueError("the rotary axes must add up to the head dimension 128")
        self.hidden_size, self.num_heads, self.ffn = hidden_size, num_attention_heads, ffn_hidden_size
        self.rope_theta, self.rope_axes_dim, self.eps = rope_theta, tuple(rope_axes_dim), eps
        ctx = _Ctx(device, bits, std, seed, "mlx")
        self.adaln_modulation = ctx.linear(hidden_size, 6 * hidden_size)
        self.layers = torch.nn.ModuleList([ErnieTransformerBlock(ctx, hidden_size, num_attention_heads,
                                                                 ffn_hidden_size, eps, qk_layernorm)
                                           for _ in range(num_layers)])
        g = torch.Generator(device=device).manual_seed(seed + 1)
        for blk in self.layers:   # non-trivial norm weights (a checkpoint would bring them)
            a = blk.self_attention
            for nrm in (blk.adaLN_sa_ln, blk.adaLN_mlp_ln, a.norm_q, a.norm_k):
                if nrm is not None:
                    nrm.weight.data.copy_(1.0 + 0.1 * torch.randn(nrm.weight.shape, device=device, generator=g))
        self._buffers_for = None
        self.trace = None

    def rope_table(self, ids: torch.Tensor) -> torch.Tensor:
        """ErnieRopeEmbedder (rope_embedder.py:5-28) + the bf16 cast of transformer.py:113-114: position ids [S, 3]
        -> (cos, sin) of the 64 angles per token, [S, 64, 2] float32 holding bf16-rounded values."""
        outs = []
        pos = ids.float().cpu()
        for i, dim in enumerate(self.rope_axes_dim):
            omega = 1.0 / (self.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
            ang = pos[:, i:i + 1] * omega[None, :]
            outs.append(torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1))
        return torch.cat(outs, dim=1).to(torch.bfloat16).float().contiguous()

    def forward(self, x: torch.Tensor, c: torch.Tensor, cos_sin: torch.Tensor,
                key_bias: torch.Tensor | None = None) -> torch.Tensor:
        """x [B, S, hidden] (float32 residual stream, updated in place and returned), c [B, hidden] (the time
        embedding), cos_sin [S, 64, 2] on the device (one table for the batch: samples with different text lengths
        have different image positions and go one by one), key_bias float32 [B, S] (0 on real keys, a large
        negative number on padded text keys; transformer.py:116-120 uses -inf)."""
        b, s, d = x.shape
        dev = x.device
        h, ffn = self.num_heads, self.ffn
        key = (b, s, str(dev))
        if self._buffers_for != key:
            self.nbuf = torch.empty(b, s, d, dtype=torch.bfloat16, device=dev)
            self.qkv = torch.empty(b, s, 3 * d, dtype=torch.bfloat16, device=dev)
            self.abuf = torch.empty(b, s, d, dtype=torch.bfloat16, device=dev)
            self.gu = torch.empty(b, s, 2 * ffn, dtype=torch.bfloat16, device=dev)   # gate | up
            self._buffers_for = key
        xs = x if x.dtype == torch.float32 else x.float()
        mod = _call(self.adaln_modulation, ops.vec_sum_act(c.to(torch.bfloat16), act="silu"))
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = (mod[:, j * d:(j + 1) * d] for j in range(6))
        ones = torch.ones(128, dtype=torch.float32, device=dev)
        fused = nn.fused_cache(self)
        for i, blk in enumerate(self.layers):
            a, mlp = blk.self_attention, blk.mlp
            ops.norm_modulate(xs, shift_msa, scale_msa, weight=blk.adaLN_sa_ln.weight.data, eps=self.eps, rms=True,
                              out=self.nbuf)
            f = fused.get(("qkv", i))
            if f is None:
                layers = [a.to_q, a.to_k, a.to_v]
                f = FusedRows(layers) if FusedRows.accepts(layers) else \
                    (lambda t, out, ls=layers: out.copy_(torch.cat([l(t) for l in ls], dim=-1)))
                fused[("qkv", i)] = f
            f(self.nbuf, self.qkv)
            qw = a.norm_q.weight.data if a.norm_q is not None else ones
            kw = a.norm_k.weight.data if a.norm_k is not None else ones
            if a.norm_q is None:
                raise NotImplementedError("qk_layernorm=False: the fused kernel always normalises q and k")
            ops.qknorm_rope(self.qkv, h, qw, kw, qw, kw, 0, cos_sin, self.eps, rope_mode="halves")
            ops.fmha(self.qkv, h, out=self.abuf, key_bias=key_bias)
            _call(a.to_out[0], self.abuf, epilogue="gate_residual", gate=gate_msa, residual=xs, out=xs)
            ops.norm_modulate(xs, shift_mlp, scale_mlp, weight=blk.adaLN_mlp_ln.weight.data, eps=self.eps, rms=True,
                              out=self.nbuf)
            g = fused.get(("gu", i))
            if g is None:
                layers = [mlp.gate_proj, mlp.up_proj]
                g = FusedRows(layers) if FusedRows.accepts(layers) else \
                    (lambda t, out, ls=layers: out.copy_(torch.cat([l(t) for l in ls], dim=-1)))
                fused[("gu", i)] = g
            g(self.nbuf, self.gu)
            up = self.gu[..., ffn:]
            ops.act_mul(up, self.gu[..., :ffn], "gelu")
            _call(mlp.linear_fc2, up, epilogue="gate_residual", gate=gate_mlp, residual=xs, out=xs)
            if self.trace is not None:
                self.trace[f"layer{i}"] = xs.clone()
        return xs
