"""FLUX.2-shaped single-stream blocks on the B200 kernels: the fused `to_qkv_mlp_proj` projection with a SwiGLU
MLP running beside the attention.

Module tree, attribute names and arithmetic follow the reference's
src/mflux/models/flux2/model/flux2_transformer/single_transformer_block.py:8-40,
parallel_self_attention.py:10-78, feed_forward.py:5-14, modulation.py:5-19 and pos_embed.py:5-31 (one shared
modulation for all single blocks, LayerNorm without affine, q/k RMSNorm, rotary pairs, no biases). No kernel is new:
  * `to_qkv_mlp_proj` is ONE quantized weight of 3*inner + 2*mlp rows. It runs as two launches over row subsets of
    that weight: rows [0, 3*inner) into the q|k|v buffer, and the 2*mlp MLP rows with the gate row j and the up row
    j interleaved, so that the matmul's SwiGLU epilogue returns silu(x1) * x2 (Flux2SwiGLU splits the projection in
    halves, feed_forward.py:10-12) straight into the second part of the [attention | mlp] buffer. Rows of a
    quantized weight are independent (groups run along the input dimension), so both launches reproduce the
    single projection bit for bit;
  * `to_out` reads that buffer, so the reference's concatenate (parallel_self_attention.py:75) never happens, and
    applies the gated residual as its epilogue.
The reference's KV cache for reference-image tokens (flux2_kv_cache.py) is `Flux2KVCache` below: nothing is
concatenated for it, the attention kernels take keys / values longer than the queries (`ops.fmha_ex`).
"""
from __future__ import annotations

import torch

from . import nn, ops
from .flux import RMSNorm, _Ctx


class Flux2Modulation(nn.Module):
    """modulation.py: linear(silu(temb)) split into (shift, scale, gate) per parameter set."""

    def __init__(self, ctx, dim: int, mod_param_sets: int = 1):
        super().__init__()
        self.mod_param_sets = mod_param_sets
        self.linear = ctx.linear(dim, dim * 3 * mod_param_sets, bias=False)


class Flux2ParallelSelfAttention(nn.Module):
    def __init__(self, ctx, dim: int, heads: int, mlp_ratio: float = 3.0):
        super().__init__()
        self.heads, self.inner_dim, self.mlp_hidden_dim = heads, heads * 128, int(dim * mlp_ratio)
        self.to_qkv_mlp_proj = ctx.linear(dim, self.inner_dim * 3 + self.mlp_hidden_dim * 2, bias=False)
        self.norm_q, self.norm_k = RMSNorm(128, 1e-5, ctx.device), RMSNorm(128, 1e-5, ctx.device)
        self.to_out = ctx.linear(self.inner_dim + self.mlp_hidden_dim, dim, bias=False)


class Flux2SingleTransformerBlock(nn.Module):
    def __init__(self, ctx, dim: int, heads: int, mlp_ratio: float = 3.0):
        super().__init__()
        self.attn = Flux2ParallelSelfAttention(ctx, dim, heads, mlp_ratio)


class Flux2KVCache:
    """Keys and values of the reference-image tokens, per layer (flux2_kv_cache.py:13-61 with the reference's method
    and attribute names). One pass runs with the reference tokens at the end of the sequence ([text, target,
    reference]) in mode "extract" and keeps their keys and values (after q/k norm and RoPE) for every layer; later
    passes over [text, target] alone run in mode "cached" and attend to those keys and values as well."""

    def __init__(self, num_double_layers: int, num_single_layers: int) -> None:
        self._double = [None] * num_double_layers
        self._single = [None] * num_single_layers
        self.mode = None
        self.num_ref_tokens = 0

    def configure(self, *, mode: str, num_ref_tokens: int) -> None:
        if mode not in ("extract", "cached"):
            raise ValueError("mode is 'extract' or 'cached'")
        self.mode, self.num_ref_tokens = mode, int(num_ref_tokens)

    @property
    def has_reference_tokens(self) -> bool:
        return self.num_ref_tokens > 0

    @property
    def is_extracting(self) -> bool:
        return self.mode == "extract" and self.has_reference_tokens

    @property
    def is_cached(self) -> bool:
        return self.mode == "cached"

    def _slots(self, stream: str):
        if stream == "double":
            return self._double
        if stream == "single":
            return self._single
        raise ValueError(f"Unknown stream {stream!r}")

    def store_reference(self, stream: str, layer_idx: int, key: torch.Tensor, value: torch.Tensor) -> None:
        """key / value: [B, S, heads*128] views; the trailing num_ref_tokens rows are kept (copied)."""
        if self.is_extracting:
            r = self.num_ref_tokens
            self._slots(stream)[layer_idx] = (key[:, -r:].clone(), value[:, -r:].clone())

    def load(self, stream: str, layer_idx: int):
        slot = self._slots(stream)[layer_idx]
        if slot is None:
            raise RuntimeError(f"KV cache slot for {stream} layer {layer_idx} is empty")
        return slot


class _SplitProjection:
    """The two row subsets of one quantized `to_qkv_mlp_proj` as prepared blobs (built on first use, rebuilt when
    any weight of the process changes)."""

    def __init__(self, layer, inner: int, mlp: int):
        w, s, b = layer.weight.data, layer.scales.data, layer.biases.data
        self.bits, self.group = layer.bits, layer.group_size

        def inter(t):   # gate row j -> 2j, up row j -> 2j + 1
            g, u = t[3 * inner:3 * inner + mlp], t[3 * inner + mlp:]
            return torch.stack([g, u], dim=1).reshape(2 * mlp, *t.shape[1:]).contiguous()

        wi = inter(w.view(torch.int32)).view(torch.uint32)
        self.qkv = ops.prepare_qlinear(w[:3 * inner].contiguous(), s[:3 * inner].contiguous(),
                                       b[:3 * inner].contiguous(), self.bits, self.group)
        self.mlp = ops.prepare_qlinear(wi, inter(s), inter(b), self.bits, self.group)
        words = w.shape[1]
        self.qkv_stub = torch.empty((3 * inner, words), dtype=torch.uint32, device="meta")
        self.mlp_stub = torch.empty((2 * mlp, words), dtype=torch.uint32, device="meta")

    def __call__(self, x, qkv_out, mlp_out):
        ops.qlinear(x, self.qkv_stub, None, None, None, bits=self.bits, group_size=self.group, out=qkv_out,
                    prepared=self.qkv)
        ops.qlinear(x, self.mlp_stub, None, None, None, bits=self.bits, group_size=self.group, epilogue="swiglu",
                    out=mlp_out, prepared=self.mlp)


class Flux2SingleStream(nn.Module):
    """`single_stream_modulation` + the single blocks of Flux2Transformer (transformer.py:42,58-66,144-160),
    run on the joint [text, image] hidden states."""

    def __init__(self, dim: int = 3072, heads: int = 24, num_single_layers: int = 20, mlp_ratio: float = 3.0,
                 bits: int | None = 4, device="cuda", std: float = 0.02, seed: int = 0, rope_theta: float = 2000.0,
                 axes_dims_rope=(32, 32, 32, 32)):
        super().__init__()
        if dim != heads * 128:
            raise ValueError("dim must equal heads * 128 (head dimension 128)")
        if sum(axes_dims_rope) != 128:
            raise ValueError("the rotary axes must add up to the head dimension 128")
        self.dim, self.heads, self.mlp_ratio, self.bits = dim, heads, mlp_ratio, bits
        self.rope_theta, self.axes_dims_rope = rope_theta, tuple(axes_dims_rope)
        ctx = _Ctx(device, bits, std, seed, "mlx")
        self.single_stream_modulation = Flux2Modulation(ctx, dim, 1)
        self.single_transformer_blocks = torch.nn.ModuleList(
            [Flux2SingleTransformerBlock(ctx, dim, heads, mlp_ratio) for _ in range(num_single_layers)])
        self._fused, self._buffers_for = {}, None
        self.trace = None

    def rope_table(self, ids: torch.Tensor) -> torch.Tensor:
        """Flux2PosEmbed (pos_embed.py:11-31): position ids [S, 4] -> (cos, sin) [S, 64, 2] of the rotated pairs."""
        outs = []
        pos = ids.float().cpu()
        for i, dim in enumerate(self.axes_dims_rope):
            omega = 1.0 / (self.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
            ang = pos[:, i:i + 1] * omega[None, :]
            outs.append(torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1))
        return torch.cat(outs, dim=1).contiguous()

    def forward(self, hidden_states: torch.Tensor, temb: torch.Tensor, cos_sin: torch.Tensor,
                kv_cache: Flux2KVCache | None = None) -> torch.Tensor:
        """hidden_states [B, S, D] (float32 residual stream, updated in place and returned), temb [B, D],
        cos_sin [S, 64, 2] on the device. With a `kv_cache` in mode "extract" the last num_ref_tokens rows are
        reference-image tokens: their keys and values are kept per layer, they attend to themselves only and the
        other rows to everything (Flux2KVCache.compute_extract_attention, flux2_kv_cache.py:63-99); in mode
        "cached" the kept keys and values follow the sequence's own (append_reference, :51-61)."""
        b, s, d = hidden_states.shape
        dev = hidden_states.device
        a0 = self.single_transformer_blocks[0].attn
        inner, mlp = a0.inner_dim, a0.mlp_hidden_dim
        extra = kv_cache.num_ref_tokens if kv_cache is not None and kv_cache.is_cached else 0
        key = (b, s, extra, str(dev))
        if self._buffers_for != key:
            self.nbuf = torch.empty(b, s, d, dtype=torch.bfloat16, device=dev)
            # q | k | v of the sequence; in cached mode `extra` more rows whose k and v columns take the kept tokens
            self.qkv = torch.empty(b, s + extra, 3 * inner, dtype=torch.bfloat16, device=dev)
            self.cat = torch.empty(b, s, inner + mlp, dtype=torch.bfloat16, device=dev)   # [attention | mlp]
            self._buffers_for = key
        xs = hidden_states if hidden_states.dtype == torch.float32 else hidden_states.float()
        mod = self.single_stream_modulation.linear(ops.vec_sum_act(temb.to(torch.bfloat16), act="silu"))
        shift, scale, gate = mod[:, 0:d], mod[:, d:2 * d], mod[:, 2 * d:3 * d]
        fused = nn.fused_cache(self)
        for i, blk in enumerate(self.single_transformer_blocks):
            a = blk.attn
            ops.norm_modulate(xs, shift, scale, out=self.nbuf)
            proj = fused.get(i)
            if proj is None:
                if isinstance(a.to_qkv_mlp_proj, nn.QuantizedLinear):
                    proj = _SplitProjection(a.to_qkv_mlp_proj, inner, mlp)
                else:   # dense model: the projection as the reference writes it
                    def proj(x, qkv_out, mlp_out, lin=a.to_qkv_mlp_proj):
                        y = lin(x)
                        qkv_out.copy_(y[..., :3 * inner])
                        x1, x2 = y[..., 3 * inner:3 * inner + mlp], y[..., 3 * inner + mlp:]
                        mlp_out.copy_(torch.nn.functional.silu(x1.float()) * x2.float())
                fused[i] = proj
            qkv = self.qkv[:, :s]
            proj(self.nbuf, qkv, self.cat[..., inner:])
            ops.qknorm_rope(qkv, self.heads, a.norm_q.weight.data, a.norm_k.weight.data, a.norm_q.weight.data,
                            a.norm_k.weight.data, 0, cos_sin, a.norm_q.eps)
            q_all, k_all, v_all = qkv[..., :inner], qkv[..., inner:2 * inner], qkv[..., 2 * inner:]
            if kv_cache is not None and kv_cache.is_extracting:
                r = kv_cache.num_ref_tokens
                kv_cache.store_reference("single", i, k_all, v_all)
                ops.fmha_ex(q_all[:, :s - r], k_all, v_all, self.heads, out=self.cat[:, :s - r, :inner])
                ops.fmha_ex(q_all[:, s - r:], k_all[:, s - r:], v_all[:, s - r:], self.heads,
                            out=self.cat[:, s - r:, :inner])
            elif extra:
                ref_k, ref_v = kv_cache.load("single", i)
                self.qkv[:, s:, inner:2 * inner].copy_(ref_k)
                self.qkv[:, s:, 2 * inner:].copy_(ref_v)
                ops.fmha_ex(q_all, self.qkv[..., inner:2 * inner], self.qkv[..., 2 * inner:], self.heads,
                            out=self.cat[..., :inner])
            else:
                ops.fmha(qkv, self.heads, out=self.cat[..., :inner])
            if isinstance(a.to_out, nn.QuantizedLinear):
                a.to_out(self.cat, epilogue="gate_residual", gate=gate, residual=xs, out=xs)
            else:
                xs += gate[:, None].float() * a.to_out(self.cat).float()
            if self.trace is not None:
                self.trace[f"single{i}"] = xs.clone()
        return xs
