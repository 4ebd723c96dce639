"""FLUX.1-shaped MMDiT denoising step on the B200 kernels.

Module tree, attribute names and arithmetic follow the reference's transformer
(src/mflux/models/flux/model/flux_transformer/transformer.py:15-80 and the block files next to it),
so parameter paths such as `transformer_blocks.3.attn.to_q.weight` or
`single_transformer_blocks.7.proj_mlp.scales` match an mflux checkpoint. What differs is the execution:
  * text and image tokens live in one sequence buffer [B, St + Si, D] from the start (text first, the
    order the reference concatenates in joint_attention.py:58-60 and transformer.py:62), so no
    concatenation or slicing copies exist; linears read and write strided slices of it;
  * to_q/to_k/to_v (and add_*_proj) run as one matmul over row-concatenated packed weights, which is
    bit-identical to three separate quantized matmuls because groups run along the input dim;
  * gate * y + residual, GELU and the concatenation [attn, mlp] of the single blocks are epilogues /
    output views of the quantized matmul; the residual stream is kept in float32.
The text encoders and the VAE of the reference are outside this path: callers pass prompt embeddings
and receive latents.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import nn, ops, resolution
from .schedulers import LinearScheduler


@dataclass
class FluxConfig:
    hidden: int = 3072
    heads: int = 24
    mlp_ratio: int = 4
    num_joint: int = 19
    num_single: int = 38
    in_channels: int = 64
    context_dim: int = 4096
    pooled_dim: int = 768
    supports_guidance: bool = True   # FLUX.1-dev; schnell has no guidance embedder
    requires_sigma_shift: bool = True
    num_train_steps: int = 1000

    def __post_init__(self):
        if self.hidden != self.heads * 128:
            raise ValueError("hidden must equal heads * 128 (head dimension 128)")


class RMSNorm(nn.Module):
    """mlx.nn.RMSNorm(dims): holds `weight` [dims]; applied inside the fused qk-norm + RoPE kernel."""

    def __init__(self, dims: int, eps: float = 1e-5, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(dims, device=device, dtype=dtype), requires_grad=False)


def _linear(i, o, bias, device, std, gen):
    lin = nn.Linear(i, o, bias=bias, device=device)
    with torch.no_grad():
        lin.weight.copy_((torch.randn(o, i, device=device, generator=gen) * std).to(lin.weight.dtype))
        if bias:
            lin.bias.copy_((torch.randn(o, device=device, generator=gen) * std).to(lin.bias.dtype))
    return lin


class _Ctx:
    """Construction context: every nn.Linear is created with N(0, std) weights and, when `bits` is set,
    quantized at once so that the dense copy of a 12B-parameter model never exists."""

    def __init__(self, device, bits, std, seed, mode):
        self.device, self.bits, self.std, self.mode = device, bits, std, mode
        self.gen = torch.Generator(device=device).manual_seed(seed)

    def linear(self, i, o, bias=True):
        lin = _linear(i, o, bias, self.device, self.std, self.gen)
        if self.bits is not None and hasattr(lin, "to_quantized") and i % 64 == 0:
            return lin.to_quantized(group_size=64, bits=self.bits, mode=self.mode)
        return lin


class MLPEmbedder(nn.Module):
    """TimestepEmbedder / TextEmbedder / GuidanceEmbedder: linear_1 -> silu -> linear_2."""

    def __init__(self, ctx, i, o):
        super().__init__()
        self.linear_1 = ctx.linear(i, o)
        self.linear_2 = ctx.linear(o, o)

    def forward(self, x):
        return _call(self.linear_2, _call(self.linear_1, x, epilogue="silu"))


class TimeTextEmbed(nn.Module):
    def __init__(self, ctx, cfg: FluxConfig):
        super().__init__()
        self.timestep_embedder = MLPEmbedder(ctx, 256, cfg.hidden)
        self.text_embedder = MLPEmbedder(ctx, cfg.pooled_dim, cfg.hidden)
        self.guidance_embedder = MLPEmbedder(ctx, 256, cfg.hidden) if cfg.supports_guidance else None


class AdaNorm(nn.Module):
    """AdaLayerNormZero / ...ZeroSingle / ...Continuous: only the `linear` has parameters."""

    def __init__(self, ctx, d, chunks, bias=True):
        super().__init__()
        self.linear = ctx.linear(d, chunks * d, bias=bias)


class FeedForward(nn.Module):
    def __init__(self, ctx, d, ratio):
        super().__init__()
        self.linear1 = ctx.linear(d, ratio * d)
        self.linear2 = ctx.linear(ratio * d, d)


class JointAttention(nn.Module):
    def __init__(self, ctx, d):
        super().__init__()
        self.to_q, self.to_k, self.to_v = ctx.linear(d, d), ctx.linear(d, d), ctx.linear(d, d)
        self.to_out = torch.nn.ModuleList([ctx.linear(d, d)])
        self.add_q_proj, self.add_k_proj, self.add_v_proj = ctx.linear(d, d), ctx.linear(d, d), ctx.linear(d, d)
        self.to_add_out = ctx.linear(d, d)
        self.norm_q, self.norm_k = RMSNorm(128, device=ctx.device), RMSNorm(128, device=ctx.device)
        self.norm_added_q, self.norm_added_k = RMSNorm(128, device=ctx.device), RMSNorm(128, device=ctx.device)


class JointTransformerBlock(nn.Module):
    def __init__(self, ctx, cfg):
        super().__init__()
        d = cfg.hidden
        self.norm1 = AdaNorm(ctx, d, 6)
        self.norm1_context = AdaNorm(ctx, d, 6)
        self.attn = JointAttention(ctx, d)
        self.ff = FeedForward(ctx, d, cfg.mlp_ratio)
        self.ff_context = FeedForward(ctx, d, cfg.mlp_ratio)


class SingleBlockAttention(nn.Module):
    def __init__(self, ctx, d):
        super().__init__()
        self.to_q, self.to_k, self.to_v = ctx.linear(d, d), ctx.linear(d, d), ctx.linear(d, d)
        self.norm_q, self.norm_k = RMSNorm(128, device=ctx.device), RMSNorm(128, device=ctx.device)


class SingleTransformerBlock(nn.Module):
    def __init__(self, ctx, cfg):
        super().__init__()
        d = cfg.hidden
        self.norm = AdaNorm(ctx, d, 3)
        self.attn = SingleBlockAttention(ctx, d)
        self.proj_mlp = ctx.linear(d, cfg.mlp_ratio * d)
        self.proj_out = ctx.linear(d + cfg.mlp_ratio * d, d)


class FusedRows:
    """Row-concatenation of several QuantizedLinear layers run as one matmul (same K, bits). Layers wrapped with
    LoRA adapters keep them: the adapters of all layers become one low-rank term of that matmul, each adapter
    acting on its own layer's block of output rows."""

    def __init__(self, layers):
        from .lora import _FusedTerms, split_wrapped

        parts = [split_wrapped(l) for l in layers]
        if any(p is None for p in parts):
            raise ValueError("FusedRows needs quantized layers (bare or LoRA-wrapped)")
        self.layers = [p[0] for p in parts]
        self.groups, row = [], 0
        for base, adapters in parts:
            if adapters:
                self.groups.append((row, 1, adapters))
            row += base.weight.shape[0]
        self.rows = row
        self.terms = _FusedTerms() if self.groups else None
        self.blob = None

    @staticmethod
    def accepts(layers) -> bool:
        from .lora import MAX_FUSED_COLUMNS, split_wrapped

        parts = [split_wrapped(l) for l in layers]
        return (all(p is not None for p in parts)
                and sum(a.lora_A.shape[1] for _, ads in parts for a in ads) <= MAX_FUSED_COLUMNS)

    def __call__(self, x, out):
        l0 = self.layers[0]
        if self.blob is None:
            w = torch.cat([l.weight.data for l in self.layers])
            s = torch.cat([l.scales.data for l in self.layers])
            b = torch.cat([l.biases.data for l in self.layers])
            self.bias = torch.cat([l.bias.data for l in self.layers]) if l0.bias is not None else None
            self.wshape = w.shape
            self.blob = ops.prepare_qlinear(w, s, b, l0.bits, l0.group_size)
            self.wq_stub = torch.empty((w.shape[0], w.shape[1]), dtype=torch.uint32, device="meta")
        if self.terms is None:
            return ops.qlinear(x, self.wq_stub, None, None, self.bias, bits=l0.bits, group_size=l0.group_size,
                               out=out, prepared=self.blob)
        a_cat, b_rows, rank = self.terms.get(None, self.groups, self.rows)   # rows of bare layers stay zero
        xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        return ops.qlinear(xb, self.wq_stub, None, None, self.bias, bits=l0.bits, group_size=l0.group_size, out=out,
                           prepared=self.blob, lora_t=torch.matmul(xb, a_cat), lora_b=b_rows, lora_r=rank)


def _call(layer, x, **kw):
    """Run a Linear or QuantizedLinear (or a LoRA wrapper over one); epilogues of dense layers fall back to
    separate torch ops."""
    if isinstance(layer, nn.QuantizedLinear) or getattr(layer, "fuses_epilogue", False):
        return layer(x, **kw)
    y = layer(x)
    epi = kw.get("epilogue")
    if epi == "silu":
        y = torch.nn.functional.silu(y)
    elif epi in ("gelu", "gelu_approx"):
        y = torch.nn.functional.gelu(y, approximate="tanh" if epi == "gelu_approx" else "none")
    elif epi == "gate_residual":
        y = kw["residual"] + kw["gate"].reshape(y.shape[0], 1, -1).float() * y.float()
    out = kw.get("out")
    if out is not None:
        out.copy_(y)
        return out
    if kw.get("out_dtype") is not None:
        y = y.to(kw["out_dtype"])
    return y


class Transformer(nn.Module):
    """FLUX.1 MMDiT: transformer.py:15-80 of the reference."""

    def __init__(self, cfg: FluxConfig = FluxConfig(), bits: int | None = 4, device="cuda", std: float = 0.02,
                 seed: int = 0, mode: str = "mlx"):
        super().__init__()
        self.cfg, self.bits = cfg, bits
        ctx = _Ctx(device, bits, std, seed, mode)
        d = cfg.hidden
        self.x_embedder = ctx.linear(cfg.in_channels, d)
        self.time_text_embed = TimeTextEmbed(ctx, cfg)
        self.context_embedder = ctx.linear(cfg.context_dim, d)
        self.transformer_blocks = torch.nn.ModuleList([JointTransformerBlock(ctx, cfg) for _ in range(cfg.num_joint)])
        self.single_transformer_blocks = torch.nn.ModuleList(
            [SingleTransformerBlock(ctx, cfg) for _ in range(cfg.num_single)])
        self.norm_out = AdaNorm(ctx, d, 2, bias=False)
        self.proj_out = ctx.linear(d, cfg.in_channels)
        self._fused = {}
        self._text_stream = {}
        self._buffers_for = None
        self._rope = {}
        self.trace = None   # a dict here receives a copy of the residual stream after every block (parity tests)

    # ------------------------------------------------------------------ helpers
    def _fuse(self, key, layers):
        fused = nn.fused_cache(self)
        f = fused.get(key)
        if f is None:
            if FusedRows.accepts(layers):
                f = FusedRows(layers)
            else:
                f = lambda x, out, ls=layers: out.copy_(torch.cat([l(x) for l in ls], dim=-1))  # noqa: E731
            fused[key] = f
        return f

    def _workspace(self, b, s, device):
        key = (b, s, str(device))
        if self._buffers_for != key:
            d = self.cfg.hidden
            r = self.cfg.mlp_ratio
            self.xs = torch.empty(b, s, d, dtype=torch.float32, device=device)       # residual stream
            self.nbuf = torch.empty(b, s, d, dtype=torch.bfloat16, device=device)    # normalised activations
            self.qkv = torch.empty(b, s, 3 * d, dtype=torch.bfloat16, device=device)
            self.cat = torch.empty(b, s, (1 + r) * d, dtype=torch.bfloat16, device=device)  # [attn | mlp]
            self._buffers_for = key
        return self.xs, self.nbuf, self.qkv, self.cat

    def rope_table(self, height, width, txt_len, device):
        key = (height, width, txt_len, str(device))
        t = self._rope.get(key)
        if t is None:
            lh, lw = height // 16, width // 16
            ids = torch.zeros(txt_len + lh * lw, 3, dtype=torch.float32)
            ids[txt_len:, 1] = torch.arange(lh, dtype=torch.float32).repeat_interleave(lw)
            ids[txt_len:, 2] = torch.arange(lw, dtype=torch.float32).repeat(lh)
            outs = []
            for i, dim in enumerate((16, 56, 56)):  # EmbedND axes (embed_nd.py:8-31)
                omega = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
                ang = ids[:, i:i + 1] * omega[None, :]
                outs.append(torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1))
            t = torch.cat(outs, dim=1).contiguous().to(device)
            self._rope[key] = t
        return t

    @staticmethod
    def time_proj(t: torch.Tensor) -> torch.Tensor:
        """TimeTextEmbed._time_proj (time_text_embed.py:33-43)."""
        half = 128
        freqs = torch.exp(-math.log(10000) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
        emb = t.float()[:, None] * freqs[None, :]
        return torch.cat([torch.cos(emb), torch.sin(emb)], dim=-1)

    def conditioning(self, timestep: torch.Tensor, pooled: torch.Tensor, guidance: torch.Tensor | None):
        """silu(time + guidance + pooled-text embedding) as bf16 [B, D] (time_text_embed.py:19-31)."""
        tte = self.time_text_embed
        # the reference casts the scaled timestep and guidance to bf16 before the sinusoid (transformer.py:153-155)
        timestep = timestep.to(torch.bfloat16).float()
        guidance = None if guidance is None else guidance.to(torch.bfloat16).float()
        t = tte.timestep_embedder(self.time_proj(timestep).to(torch.bfloat16))
        p = tte.text_embedder(pooled.to(torch.bfloat16))
        g = None
        if tte.guidance_embedder is not None:
            g = tte.guidance_embedder(self.time_proj(guidance).to(torch.bfloat16))
        return ops.vec_sum_act(t, p, g, act="silu", out_dtype=torch.bfloat16)

    # ------------------------------------------------------------------ forward
    def forward(self, hidden_states: torch.Tensor, prompt_embeds: torch.Tensor, pooled_prompt_embeds: torch.Tensor,
                timestep: torch.Tensor, guidance: torch.Tensor | None, height: int, width: int) -> torch.Tensor:
        """One denoiser evaluation: latents [B, Si, C] + conditioning -> predicted noise [B, Si, C] (bf16)."""
        cfg = self.cfg
        d, heads = cfg.hidden, cfg.heads
        b, si, _ = hidden_states.shape
        st = prompt_embeds.shape[1]
        s = st + si
        dev = hidden_states.device
        xs, nbuf, qkv, cat = self._workspace(b, s, dev)
        x_img, x_txt = xs[:, st:], xs[:, :st]
        n_img, n_txt = nbuf[:, st:], nbuf[:, :st]
        attn = cat[..., :d]
        ffb = cat[..., d:]
        cos_sin = self.rope_table(height, width, st, dev)

        _call(self.x_embedder, hidden_states.to(torch.bfloat16), out=x_img)
        _call(self.context_embedder, prompt_embeds.to(torch.bfloat16), out=x_txt)
        sv = self.conditioning(timestep, pooled_prompt_embeds, guidance)

        # With few text rows (a handful of 256 x 256 tiles for 74 CTA pairs) the text stream's kernels run on a second
        # CUDA stream beside the image stream's: between the two points where the streams meet (attention, block
        # end) they share no data, and the text launches start on the SMs the image kernels leave idle. With many
        # rows (the 16-image batch) both streams fill the GPU by themselves and stay on one CUDA stream.
        main = torch.cuda.current_stream(dev)
        side = None
        if b * st <= 2048 and dev.type == "cuda" and ops.TRACE is None:   # per-launch timing: one stream
            side = self._text_stream.get(str(dev))
            if side is None:
                side = self._text_stream[str(dev)] = torch.cuda.Stream(device=dev)

        def pair(img_fn, txt_fn):
            if side is None:
                img_fn()
                txt_fn()
                return
            side.wait_stream(main)
            img_fn()
            with torch.cuda.stream(side):
                txt_fn()
            main.wait_stream(side)

        for i, blk in enumerate(self.transformer_blocks):
            a = blk.attn
            mod_i = _call(blk.norm1.linear, sv)            # [B, 6D]: shift, scale, gate (msa) | shift, scale, gate (mlp)
            mod_t = _call(blk.norm1_context.linear, sv)

            def img_in():
                ops.norm_modulate(x_img, mod_i[:, 0:d], mod_i[:, d:2 * d], out=n_img)
                self._fuse(("jq", i), [a.to_q, a.to_k, a.to_v])(n_img, qkv[:, st:])

            def txt_in():
                ops.norm_modulate(x_txt, mod_t[:, 0:d], mod_t[:, d:2 * d], out=n_txt)
                self._fuse(("ja", i), [a.add_q_proj, a.add_k_proj, a.add_v_proj])(n_txt, qkv[:, :st])

            def img_out():
                _call(a.to_out[0], attn[:, st:], epilogue="gate_residual", gate=mod_i[:, 2 * d:3 * d], residual=x_img,
                      out=x_img)
                ops.norm_modulate(x_img, mod_i[:, 3 * d:4 * d], mod_i[:, 4 * d:5 * d], out=n_img)
                _call(blk.ff.linear1, n_img, epilogue="gelu", out=ffb[:, st:])
                _call(blk.ff.linear2, ffb[:, st:], epilogue="gate_residual", gate=mod_i[:, 5 * d:6 * d],
                      residual=x_img, out=x_img)

            def txt_out():
                _call(a.to_add_out, attn[:, :st], epilogue="gate_residual", gate=mod_t[:, 2 * d:3 * d], residual=x_txt,
                      out=x_txt)
                ops.norm_modulate(x_txt, mod_t[:, 3 * d:4 * d], mod_t[:, 4 * d:5 * d], out=n_txt)
                _call(blk.ff_context.linear1, n_txt, epilogue="gelu_approx", out=ffb[:, :st])
                _call(blk.ff_context.linear2, ffb[:, :st], epilogue="gate_residual", gate=mod_t[:, 5 * d:6 * d],
                      residual=x_txt, out=x_txt)

            pair(img_in, txt_in)
            ops.qknorm_rope(qkv, heads, a.norm_added_q.weight.data, a.norm_added_k.weight.data, a.norm_q.weight.data,
                            a.norm_k.weight.data, st, cos_sin, a.norm_q.eps)
            ops.fmha(qkv, heads, out=attn)
            pair(img_out, txt_out)
            if self.trace is not None:
                self.trace[f"joint{i}"] = xs.clone()

        for i, blk in enumerate(self.single_transformer_blocks):
            a = blk.attn
            mod = _call(blk.norm.linear, sv)                # [B, 3D]: shift, scale, gate
            ops.norm_modulate(xs, mod[:, 0:d], mod[:, d:2 * d], out=nbuf)
            self._fuse(("sq", i), [a.to_q, a.to_k, a.to_v])(nbuf, qkv)
            ops.qknorm_rope(qkv, heads, a.norm_q.weight.data, a.norm_k.weight.data, a.norm_q.weight.data,
                            a.norm_k.weight.data, 0, cos_sin, a.norm_q.eps)
            ops.fmha(qkv, heads, out=attn)
            _call(blk.proj_mlp, nbuf, epilogue="gelu_approx", out=ffb)
            _call(blk.proj_out, cat, epilogue="gate_residual", gate=mod[:, 2 * d:3 * d], residual=xs, out=xs)
            if self.trace is not None:
                self.trace[f"single{i}"] = xs.clone()

        mod = _call(self.norm_out.linear, sv)               # [B, 2D]: scale, shift
        ops.norm_modulate(x_img, mod[:, d:2 * d], mod[:, 0:d], out=n_img)
        return _call(self.proj_out, n_img)


class Flux1:
    """Counterpart of the reference's Flux1 variant (src/mflux/models/flux/variants/txt2img/flux.py:30-147)
    restricted to the denoise loop: random-init or caller-loaded transformer, LinearScheduler, Euler steps."""

    def __init__(self, quantize: int | None = None, model_config: FluxConfig | None = None, device="cuda",
                 seed: int = 0, stored_quantization: int | None = None, cuda_graph: bool = False):
        bits, warning = resolution.resolve(stored_quantization, quantize)
        if warning:
            print(f"Warning: {warning}")
        resolution.check_supported(bits)
        self.bits = bits
        self.model_config = model_config or FluxConfig()
        self.transformer = Transformer(self.model_config, bits=bits, device=device, seed=seed)
        # cuda_graph: one denoiser evaluation is recorded per (shapes, image size) and replayed; worth it for single
        # images, where a step is some 600 short launches (the reference gets the same from MLX's lazy graph)
        self.cuda_graph, self._captured, self._captured_epoch = cuda_graph, {}, nn.weights_epoch()

    def predict_noise(self, latents, prompt_embeds, pooled_prompt_embeds, timestep, guidance, height, width):
        """One denoiser evaluation; `timestep` and `guidance` are [B] tensors on the device."""
        if not self.cuda_graph:
            return self.transformer(latents, prompt_embeds, pooled_prompt_embeds, timestep, guidance, height, width)
        from .graphs import CapturedStep

        if self._captured and self._captured_epoch != nn.weights_epoch():
            self.release_graphs()
        self._captured_epoch = nn.weights_epoch()
        key = (height, width, guidance is None)
        step = self._captured.get(key)
        if step is None:
            if guidance is None:
                fn = lambda lat, ctx, pool, ts: self.transformer(lat, ctx, pool, ts, None, height, width)  # noqa: E731
            else:
                fn = lambda lat, ctx, pool, ts, gd: self.transformer(lat, ctx, pool, ts, gd, height, width)  # noqa: E731
            step = self._captured[key] = CapturedStep(fn)
        args = (latents, prompt_embeds, pooled_prompt_embeds, timestep) + (() if guidance is None else (guidance,))
        return step(*args)

    def release_graphs(self) -> None:
        for step in self._captured.values():
            step.release()
        self._captured = {}

    def save_model(self, base_path: str) -> None:
        """ModelSaver.save_model for the component this class owns: `<base_path>/transformer/{i}.safetensors` plus
        the index file, in the reference's format (the other components stay with the caller)."""
        from . import checkpoint

        checkpoint.save_weights(base_path, self.bits, self.transformer, "transformer")

    def load_model(self, base_path: str) -> None:
        """Loads `<base_path>/transformer` as saved by `save_model` or by the reference's ModelSaver."""
        from . import checkpoint

        checkpoint.load_into(self.transformer, base_path, "transformer", self.bits)
        if hasattr(self.transformer, "_fused"):
            self.transformer._fused = {}

    def generate_image(self, seed: int, prompt_embeds: torch.Tensor, pooled_prompt_embeds: torch.Tensor,
                       num_inference_steps: int = 4, height: int = 1024, width: int = 1024, guidance: float = 3.5,
                       latents: torch.Tensor | None = None) -> torch.Tensor:
        """Runs the denoise loop (flux.py:101-122) and returns the final latents [B, (H/16)(W/16), C] (f32).

        `prompt_embeds` [B, St, ctx] and `pooled_prompt_embeds` [B, pooled] stand in for the reference's
        text encoders; decoding the latents with a VAE is left to the caller.
        """
        cfg = self.model_config
        dev = prompt_embeds.device
        b = prompt_embeds.shape[0]
        sched = LinearScheduler(num_inference_steps, width, height, cfg.requires_sigma_shift)
        if latents is None:
            g = torch.Generator(device=dev).manual_seed(seed)
            latents = torch.randn(b, (height // 16) * (width // 16), cfg.in_channels, device=dev, generator=g)
        latents = latents.float()
        gvec = torch.full((b,), guidance * cfg.num_train_steps, device=dev) if cfg.supports_guidance else None
        for t in range(num_inference_steps):
            ts = torch.full((b,), float(sched.sigmas[t]) * cfg.num_train_steps, device=dev)
            noise = self.predict_noise(latents, prompt_embeds, pooled_prompt_embeds, ts, gvec, height, width)
            latents = ops.euler_step(latents, noise, sched.dt(t))
        return latents
