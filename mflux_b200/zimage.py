"""Z-Image-shaped single-stream DiT denoising step on the B200 kernels.

Module tree, attribute names and arithmetic follow the reference's ZImageTransformer
(src/mflux/models/z_image/model/z_image_transformer/transformer.py:11-143, transformer_block.py:7-38,
context_block.py:7-24, attention.py:7-98, feed_forward.py:5-14, final_layer.py:5-17, rope_embedder.py:4-41,
timestep_embedder.py:7-38), so parameter paths such as `layers.7.attention.to_q.weight` or
`noise_refiner.0.feed_forward.w1.scales` match an mflux checkpoint. What differs is the execution:
  * image and caption tokens live in one float32 residual buffer [B, Si + Sc, D] from the start (image first,
    the order of transformer.py:121); the refiners run on strided views of it, so the concatenation is free;
  * to_q/to_k/to_v run as one matmul over row-concatenated packed weights, and w1/w3 as one matmul over
    row-interleaved packed weights whose epilogue writes silu(w1 x) * (w3 x) directly;
  * the post-norms (attention_norm2 / ffn_norm2), the tanh gate, the residual add and the pre-norm (with its
    modulation) of the sub-layer that follows are one pass over the stream;
  * the reference evaluates one image at a time; here B images of one shape (and one caption length) run as
    a batch, every sample with its own timestep.
The text encoder and the VAE of the reference are outside this path: callers pass caption features and
receive latents.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch

from . import nn, ops, resolution
from .flux import FusedRows, RMSNorm, _call, _Ctx
from .schedulers import FlowMatchEulerDiscreteScheduler, LinearScheduler


@dataclass
class ZImageConfig:
    dim: int = 3840
    n_layers: int = 30
    n_refiner_layers: int = 2
    n_heads: int = 30
    norm_eps: float = 1e-5
    in_channels: int = 16
    patch_size: int = 2
    f_patch_size: int = 1
    cap_feat_dim: int = 2560
    rope_theta: float = 256.0
    t_scale: float = 1000.0
    axes_dims: tuple = (32, 48, 48)
    axes_lens: tuple = (1024, 512, 512)
    ffn_hidden: int = field(default=0)
    # False = the Turbo checkpoint (guidance forced to 0, linear schedule); True = the base model, which runs with
    # a negative prompt on the flow-match schedule (models/common/config/model_config.py:580-603)
    supports_guidance: bool = False
    requires_sigma_shift: bool = True

    def __post_init__(self):
        if self.dim != self.n_heads * 128:
            raise ValueError("dim must equal n_heads * 128 (head dimension 128)")
        if sum(self.axes_dims) != 128:
            raise ValueError("the rotary axes must add up to the head dimension 128")
        if self.ffn_hidden == 0:
            self.ffn_hidden = int(self.dim / 3 * 8)   # transformer_block.py:11

    @property
    def key(self) -> str:
        return f"{self.patch_size}-{self.f_patch_size}"

    @property
    def embed_dim(self) -> int:
        return self.f_patch_size * self.patch_size * self.patch_size * self.in_channels


class FusedSwiGLU:
    """w1 and w3 of a FeedForward as one quantized matmul: row 2j of the fused weight is w1's row j, row 2j+1
    is w3's row j, and the matmul epilogue reduces each (gate, up) column pair to silu(gate) * up. Interleaving
    whole rows keeps every packed code, scale and bias of the two layers unchanged. LoRA-wrapped layers keep
    their adapters: w1's act on the even rows of the fused product, w3's on the odd rows, as one low-rank term of
    the same matmul (added before the epilogue)."""

    def __init__(self, w1, w3):
        from .lora import _FusedTerms, split_wrapped

        (self.w1, ad1), (self.w3, ad3) = split_wrapped(w1), split_wrapped(w3)
        self.groups = [(r0, 2, ads) for r0, ads in ((0, ad1), (1, ad3)) if ads]
        self.terms = _FusedTerms() if self.groups else None
        self.blob = None

    @staticmethod
    def accepts(w1, w3) -> bool:
        from .lora import MAX_FUSED_COLUMNS, split_wrapped

        parts = [split_wrapped(w1), split_wrapped(w3)]
        return (all(p is not None for p in parts)
                and sum(a.lora_A.shape[1] for _, ads in parts for a in ads) <= MAX_FUSED_COLUMNS)

    def __call__(self, x, out):
        w1 = self.w1
        if self.blob is None:
            def inter(a, b):
                return torch.stack([a, b], dim=1).reshape(2 * a.shape[0], *a.shape[1:]).contiguous()
            w = inter(w1.weight.data.view(torch.int32), self.w3.weight.data.view(torch.int32)).view(torch.uint32)
            s = inter(w1.scales.data, self.w3.scales.data)
            b = inter(w1.biases.data, self.w3.biases.data)
            self.bias = inter(w1.bias.data, self.w3.bias.data) if w1.bias is not None else None
            self.blob = ops.prepare_qlinear(w, s, b, w1.bits, w1.group_size)
            self.wq_stub = torch.empty((w.shape[0], w.shape[1]), dtype=torch.uint32, device="meta")
        if self.terms is None:
            return ops.qlinear(x, self.wq_stub, None, None, self.bias, bits=w1.bits, group_size=w1.group_size,
                               epilogue="swiglu", out=out, prepared=self.blob)
        a_cat, b_rows, rank = self.terms.get(None, self.groups, self.wq_stub.shape[0])
        xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        return ops.qlinear(xb, self.wq_stub, None, None, self.bias, bits=w1.bits, group_size=w1.group_size,
                           epilogue="swiglu", out=out, prepared=self.blob, lora_t=torch.matmul(xb, a_cat),
                           lora_b=b_rows, lora_r=rank)


class ZImageAttention(nn.Module):
    def __init__(self, ctx, dim):
        super().__init__()
        self.to_q, self.to_k, self.to_v = (ctx.linear(dim, dim, bias=False) for _ in range(3))
        self.to_out = torch.nn.ModuleList([ctx.linear(dim, dim, bias=False)])
        self.norm_q, self.norm_k = RMSNorm(128, 1e-5, ctx.device), RMSNorm(128, 1e-5, ctx.device)


class FeedForward(nn.Module):
    def __init__(self, ctx, dim, hidden):
        super().__init__()
        self.w1 = ctx.linear(dim, hidden, bias=False)
        self.w2 = ctx.linear(hidden, dim, bias=False)
        self.w3 = ctx.linear(dim, hidden, bias=False)


class ZImageContextBlock(nn.Module):
    """Unmodulated block of the caption refiner (context_block.py)."""
    modulated = False

    def __init__(self, ctx, cfg: ZImageConfig):
        super().__init__()
        d = cfg.dim
        self.attention = ZImageAttention(ctx, d)
        self.feed_forward = FeedForward(ctx, d, cfg.ffn_hidden)
        self.attention_norm1, self.attention_norm2 = RMSNorm(d, cfg.norm_eps, ctx.device), RMSNorm(d, cfg.norm_eps, ctx.device)
        self.ffn_norm1, self.ffn_norm2 = RMSNorm(d, cfg.norm_eps, ctx.device), RMSNorm(d, cfg.norm_eps, ctx.device)


class ZImageTransformerBlock(ZImageContextBlock):
    """Timestep-modulated block (transformer_block.py): scale and tanh gate for attention and for the FFN."""
    modulated = True

    def __init__(self, ctx, cfg: ZImageConfig):
        super().__init__(ctx, cfg)
        self.adaLN_modulation = torch.nn.ModuleList([ctx.linear(min(cfg.dim, 256), 4 * cfg.dim)])


class TimestepEmbedder(nn.Module):
    def __init__(self, ctx, out_size, mid_size):
        super().__init__()
        self.linear1 = ctx.linear(256, mid_size)
        self.linear2 = ctx.linear(mid_size, out_size)

    @staticmethod
    def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: float = 10000.0) -> torch.Tensor:
        """timestep_embedder.py:29-38: [cos, sin] halves, float32."""
        half = dim // 2
        freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
        args = t.float()[:, None] * freqs[None]
        return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)

    def forward(self, t):
        f = self.timestep_embedding(t).to(torch.bfloat16)
        return _call(self.linear2, _call(self.linear1, f, epilogue="silu"))


class FinalLayer(nn.Module):
    def __init__(self, ctx, hidden, out_channels):
        super().__init__()
        self.linear = ctx.linear(hidden, out_channels)
        self.adaLN_modulation = torch.nn.ModuleList([ctx.linear(min(hidden, 256), hidden)])


class ZImageTransformer(nn.Module):
    def __init__(self, cfg: ZImageConfig = ZImageConfig(), bits: int | None = 8, device="cuda", std: float = 0.02,
                 seed: int = 0, mode: str = "mlx"):
        super().__init__()
        self.cfg, self.bits = cfg, bits
        ctx = _Ctx(device, bits, std, seed, mode)
        d = cfg.dim
        self.all_x_embedder = torch.nn.ModuleDict({cfg.key: ctx.linear(cfg.embed_dim, d)})
        self.all_final_layer = torch.nn.ModuleDict({cfg.key: FinalLayer(ctx, d, cfg.embed_dim)})
        self.t_embedder = TimestepEmbedder(ctx, min(d, 256), 1024)
        self.cap_embedder = torch.nn.ModuleList([RMSNorm(cfg.cap_feat_dim, cfg.norm_eps, device),
                                                 ctx.linear(cfg.cap_feat_dim, d)])
        self.x_pad_token = torch.nn.Parameter(torch.zeros(1, d, device=device, dtype=torch.bfloat16), requires_grad=False)
        self.cap_pad_token = torch.nn.Parameter(torch.zeros(1, d, device=device, dtype=torch.bfloat16), requires_grad=False)
        self.noise_refiner = torch.nn.ModuleList([ZImageTransformerBlock(ctx, cfg) for _ in range(cfg.n_refiner_layers)])
        self.context_refiner = torch.nn.ModuleList([ZImageContextBlock(ctx, cfg) for _ in range(cfg.n_refiner_layers)])
        self.layers = torch.nn.ModuleList([ZImageTransformerBlock(ctx, cfg) for _ in range(cfg.n_layers)])
        self._fused, self._rope, self._buffers_for = {}, {}, None
        self.trace = None   # a dict here receives a copy of the unified stream after every main layer (parity tests)

    # ------------------------------------------------------------------ helpers
    def _qkv(self, blk):
        fused = nn.fused_cache(self)
        f = fused.get(("qkv", id(blk)))
        if f is None:
            a = blk.attention
            layers = [a.to_q, a.to_k, a.to_v]
            if FusedRows.accepts(layers):
                f = FusedRows(layers)
            else:
                f = lambda x, out, ls=layers: out.copy_(torch.cat([l(x) for l in ls], dim=-1))  # noqa: E731
            fused[("qkv", id(blk))] = f
        return f

    def _swiglu(self, blk):
        fused = nn.fused_cache(self)
        f = fused.get(("ffn", id(blk)))
        if f is None:
            ff = blk.feed_forward
            if FusedSwiGLU.accepts(ff.w1, ff.w3):
                f = FusedSwiGLU(ff.w1, ff.w3)
            else:
                f = lambda x, out, ff=ff: out.copy_(torch.nn.functional.silu(ff.w1(x).float()) * ff.w3(x).float())  # noqa: E731
            fused[("ffn", id(blk))] = f
        return f

    def _workspace(self, b, s, device):
        key = (b, s, str(device))
        if self._buffers_for != key:
            d, h = self.cfg.dim, self.cfg.ffn_hidden
            self.xs = torch.empty(b, s, d, dtype=torch.float32, device=device)      # residual stream
            self.nbuf = torch.empty(b, s, d, dtype=torch.bfloat16, device=device)   # normalised activations
            self.qkv = torch.empty(b, s, 3 * d, dtype=torch.bfloat16, device=device)
            self.attn = torch.empty(b, s, d, dtype=torch.bfloat16, device=device)
            self.ybuf = torch.empty(b, s, d, dtype=torch.bfloat16, device=device)   # projection outputs before the post-norm
            self.ffb = torch.empty(b, s, h, dtype=torch.bfloat16, device=device)
            self._buffers_for = key
        return self.xs, self.nbuf, self.qkv, self.attn, self.ybuf, self.ffb

    @staticmethod
    def padded(n: int) -> int:
        return n + (-n) % 32

    def position_ids(self, grid: tuple[int, int, int], cap_len: int) -> tuple[np.ndarray, np.ndarray]:
        """transformer.py:160-181: caption ids (1 + i, 0, 0) over the padded caption; image ids
        (padded caption length + 1 + f, row, col); padded image tokens sit at (0, 0, 0)."""
        cap_p = self.padded(cap_len)
        cap_ids = np.zeros((cap_p, 3), dtype=np.int64)
        cap_ids[:, 0] = 1 + np.arange(cap_p)
        ft, ht, wt = grid
        f, r, c = np.meshgrid(np.arange(ft), np.arange(ht), np.arange(wt), indexing="ij")
        img = np.stack([cap_p + 1 + f, r, c], axis=-1).reshape(-1, 3)
        img = np.concatenate([img, np.zeros((self.padded(len(img)) - len(img), 3), dtype=np.int64)], axis=0)
        return img, cap_ids

    def rope_table(self, grid, cap_len, device):
        """RopeEmbedder (rope_embedder.py:20-41): per axis cos/sin of position * theta^(-2i/d), concatenated to the
        64 rotated pairs of a head; rows ordered image first, caption second."""
        key = (grid, cap_len, str(device))
        t = self._rope.get(key)
        if t is None:
            cfg = self.cfg
            parts = []
            for ids in self.position_ids(grid, cap_len):
                cols = []
                for i, (dim, length) in enumerate(zip(cfg.axes_dims, cfg.axes_lens)):
                    if ids[:, i].max() >= length:
                        raise ValueError(f"position {ids[:, i].max()} exceeds the rotary table of axis {i} ({length})")
                    freqs = 1.0 / (cfg.rope_theta ** (np.arange(0, dim, 2, dtype=np.float32) / np.float32(dim)))
                    ang = np.outer(ids[:, i].astype(np.float32), freqs.astype(np.float32)).astype(np.float32)
                    cols.append(np.stack([np.cos(ang), np.sin(ang)], axis=-1))
                parts.append(np.concatenate(cols, axis=1))
            full = torch.from_numpy(np.concatenate(parts, axis=0).astype(np.float32)).contiguous().to(device)
            si = parts[0].shape[0]
            t = (full, full[:si].contiguous(), full[si:].contiguous())
            self._rope[key] = t
        return t

    def patchify(self, x: torch.Tensor) -> torch.Tensor:
        """[B, C, F, H, W] -> [B, tokens, pF*pH*pW*C], channel fastest (transformer.py:167-171)."""
        b, c, f, h, w = x.shape
        p, pf = self.cfg.patch_size, self.cfg.f_patch_size
        x = x.reshape(b, c, f // pf, pf, h // p, p, w // p, p).permute(0, 2, 4, 6, 3, 5, 7, 1)
        return x.reshape(b, (f // pf) * (h // p) * (w // p), pf * p * p * c)

    def unpatchify(self, t: torch.Tensor, size: tuple[int, int, int]) -> torch.Tensor:
        """Inverse of patchify on the first F*H*W/(pF*pH*pW) tokens (transformer.py:184-199)."""
        f, h, w = size
        p, pf, c = self.cfg.patch_size, self.cfg.f_patch_size, self.cfg.in_channels
        b = t.shape[0]
        n = (f // pf) * (h // p) * (w // p)
        t = t[:, :n].reshape(b, f // pf, h // p, w // p, pf, p, p, c).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return t.reshape(b, c, f, h, w)

    # ------------------------------------------------------------------ one block on a view of the stream
    def _modulation(self, blk, t_emb):
        """(scale_msa, gate_msa, scale_mlp, gate_mlp) of a block, or four Nones for an unmodulated one: the scales
        as views of the adaLN output (the kernels add the 1), the gates through tanh."""
        if not blk.modulated:
            return None, None, None, None
        d = self.cfg.dim
        mod = _call(blk.adaLN_modulation[0], t_emb)          # [B, 4D]: scale_msa, gate_msa, scale_mlp, gate_mlp
        return (mod[:, 0:d], ops.vec_sum_act(mod[:, d:2 * d], act="tanh"), mod[:, 2 * d:3 * d],
                ops.vec_sum_act(mod[:, 3 * d:4 * d], act="tanh"))

    def _run_blocks(self, blocks, lo, hi, cos_sin, t_emb, tag=None):
        """A run of blocks on rows lo:hi of the stream. Every post-norm + gated residual also writes the pre-norm
        of whatever comes next on the same rows (this block's FFN, or the next block's attention), so the stream is
        read once per sub-layer instead of twice."""
        xs, nbuf, qkv, attn, ybuf, ffb = (t[:, lo:hi] for t in (self.xs, self.nbuf, self.qkv, self.attn, self.ybuf,
                                                                self.ffb))
        heads, eps = self.cfg.n_heads, self.cfg.norm_eps
        mods = [self._modulation(blk, t_emb) for blk in blocks]
        for i, blk in enumerate(blocks):
            a, ff = blk.attention, blk.feed_forward
            scale_msa, gate_msa, scale_mlp, gate_mlp = mods[i]
            if i == 0:
                ops.norm_modulate(xs, None, scale_msa, weight=blk.attention_norm1.weight.data, eps=eps, rms=True,
                                  out=nbuf)
            self._qkv(blk)(nbuf, qkv)
            ops.qknorm_rope(qkv, heads, a.norm_q.weight.data, a.norm_k.weight.data, a.norm_q.weight.data,
                            a.norm_k.weight.data, 0, cos_sin, a.norm_q.eps)
            ops.fmha(qkv, heads, out=attn)
            _call(a.to_out[0], attn, out=ybuf)
            ops.norm_gate_residual(ybuf, blk.attention_norm2.weight.data, xs, gate_msa, eps,
                                   next_weight=blk.ffn_norm1.weight.data, next_scale=scale_mlp, next_out=nbuf)
            self._swiglu(blk)(nbuf, ffb)
            _call(ff.w2, ffb, out=ybuf)
            if i + 1 < len(blocks):
                nxt = blocks[i + 1]
                ops.norm_gate_residual(ybuf, blk.ffn_norm2.weight.data, xs, gate_mlp, eps,
                                       next_weight=nxt.attention_norm1.weight.data, next_scale=mods[i + 1][0],
                                       next_out=nbuf)
            else:
                ops.norm_gate_residual(ybuf, blk.ffn_norm2.weight.data, xs, gate_mlp, eps)
            if tag is not None and self.trace is not None:
                self.trace[f"{tag}{i}"] = xs.clone()   # rows lo:hi of the stream

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, timestep: torch.Tensor, cap_feats: torch.Tensor) -> torch.Tensor:
        """latents [B, C, F, H, W], timestep [B] (= 1 - sigma, transformer.py:66-67), caption features
        [B, L, cap_feat_dim] -> predicted noise [B, C, F, H, W] (float32, already negated as transformer.py:143)."""
        cfg = self.cfg
        d = cfg.dim
        b, _, f, h, w = x.shape
        dev = x.device
        grid = (f // cfg.f_patch_size, h // cfg.patch_size, w // cfg.patch_size)
        tokens = self.patchify(x.to(torch.bfloat16))
        n_img, n_cap = tokens.shape[1], cap_feats.shape[1]
        si, sc = self.padded(n_img), self.padded(n_cap)
        if si > n_img:   # padding repeats the last token (transformer.py:178)
            tokens = torch.cat([tokens, tokens[:, -1:].expand(b, si - n_img, -1)], dim=1)
        cap = cap_feats.to(torch.bfloat16)
        if sc > n_cap:
            cap = torch.cat([cap, cap[:, -1:].expand(b, sc - n_cap, -1)], dim=1)
        xs, nbuf, *_ = self._workspace(b, si + sc, dev)
        cs_all, cs_img, cs_cap = self.rope_table(grid, n_cap, dev)

        t_emb = self.t_embedder(timestep.float() * cfg.t_scale)

        _call(self.all_x_embedder[cfg.key], tokens.contiguous(), out=xs[:, :si])
        if si > n_img:
            xs[:, n_img:si] = self.x_pad_token.data.float()
        self._run_blocks(list(self.noise_refiner), 0, si, cs_img, t_emb, tag="noise")

        cn = ops.norm_modulate(cap.contiguous(), weight=self.cap_embedder[0].weight.data, eps=self.cap_embedder[0].eps,
                               rms=True)
        _call(self.cap_embedder[1], cn, out=xs[:, si:])
        if sc > n_cap:
            xs[:, si + n_cap:] = self.cap_pad_token.data.float()
        self._run_blocks(list(self.context_refiner), si, si + sc, cs_cap, None, tag="context")

        self._run_blocks(list(self.layers), 0, si + sc, cs_all, t_emb, tag="layer")

        fl = self.all_final_layer[cfg.key]
        scale = _call(fl.adaLN_modulation[0], ops.vec_sum_act(t_emb, act="silu"))
        ops.norm_modulate(xs[:, :si], None, scale, eps=1e-6, out=nbuf[:, :si])
        out = _call(fl.linear, nbuf[:, :si], out_dtype=torch.float32)
        return -self.unpatchify(out.float(), (f, h, w))


class ZImage:
    """Denoise loop of the reference's ZImage variant (variants/z_image.py:101-118,185-209): one denoiser
    evaluation per step, or two (prompt and negative prompt, run as one batch) with the plain guidance
    combine noise + g * (noise - negative) when guidance > 1 and negative features are given."""

    def __init__(self, quantize: int | None = None, model_config: ZImageConfig | None = None, device="cuda",
                 seed: int = 0, stored_quantization: int | None = None, cuda_graph: bool = False):
        bits, warning = resolution.resolve(stored_quantization, quantize)
        if warning:
            print(f"Warning: {warning}")
        resolution.check_supported(bits)
        self.bits = bits
        self.model_config = model_config or ZImageConfig()
        self.transformer = ZImageTransformer(self.model_config, bits=bits, device=device, seed=seed)
        self.cuda_graph, self._captured, self._captured_epoch = cuda_graph, None, nn.weights_epoch()

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

    def make_scheduler(self, num_inference_steps: int, width: int, height: int, scheduler: str | None = None):
        """The schedule Config.scheduler builds for this model (models/common/config/config.py:146-164): by name,
        defaulting to "flow_match_euler_discrete" with guidance support and "linear" without; a scheduler that
        has set_image_seq_len gets the image sequence length when the model wants its sigmas shifted."""
        cfg = self.model_config
        if scheduler is None:
            scheduler = "flow_match_euler_discrete" if cfg.supports_guidance else "linear"
        if scheduler == "linear":
            return LinearScheduler(num_inference_steps, width, height, cfg.requires_sigma_shift)
        if scheduler == "flow_match_euler_discrete":
            sched = FlowMatchEulerDiscreteScheduler(num_inference_steps)
            if cfg.requires_sigma_shift:
                sched.set_image_seq_len((height // 16) * (width // 16))
            return sched
        raise NotImplementedError(f"The scheduler {scheduler!r} is not implemented.")

    def _evaluate(self, latents, t, cap_feats):
        """The transformer call, replayed from a recorded CUDA graph when the model was built with cuda_graph=True
        (one graph per set of input shapes; a single image is a few hundred short launches per step)."""
        if not self.cuda_graph:
            return self.transformer(latents, t, cap_feats)
        from .graphs import CapturedStep

        if self._captured is not None and self._captured_epoch != nn.weights_epoch():
            self.release_graphs()
        self._captured_epoch = nn.weights_epoch()
        if self._captured is None:
            self._captured = CapturedStep(lambda lat, tt, cap: self.transformer(lat, tt, cap))
        return self._captured(latents, t, cap_feats)

    def release_graphs(self) -> None:
        if self._captured is not None:
            self._captured.release()
        self._captured = None

    def denoise_step(self, latents, cap_feats, negative_cap_feats, sigma, dt, guidance):
        b = latents.shape[0]
        t = torch.full((b,), 1.0 - sigma, device=latents.device)
        if negative_cap_feats is None:
            noise = self._evaluate(latents, t, cap_feats)
        else:
            both = self._evaluate(torch.cat([latents, latents]), torch.cat([t, t]),
                                  torch.cat([cap_feats, negative_cap_feats]))
            noise = ops.cfg_combine(both[:b], both[b:], guidance, mode="plain")
        return ops.euler_step(latents, noise, dt)

    def generate_image(self, seed: int, cap_feats: torch.Tensor, negative_cap_feats: torch.Tensor | None = None,
                       num_inference_steps: int = 9, height: int = 1024, width: int = 1024, guidance: float = 0.0,
                       latents: torch.Tensor | None = None, scheduler: str | None = None) -> torch.Tensor:
        """Returns the final latents [B, C, 1, H/8, W/8] (f32); caption features stand in for the text encoder.

        As in the reference (variants/z_image.py:60-66) a model without guidance support runs with guidance 0 on
        the linear schedule, one with it on the flow-match schedule unless `scheduler` names the other."""
        dev = cap_feats.device
        b = cap_feats.shape[0]
        if not self.model_config.supports_guidance:
            guidance = 0.0
        sched = self.make_scheduler(num_inference_steps, width, height, scheduler)
        if latents is None:
            g = torch.Generator(device=dev).manual_seed(seed)
            latents = torch.randn(b, self.model_config.in_channels, 1, height // 8, width // 8, device=dev, generator=g)
        latents = latents.float()
        if guidance <= 1.0:
            negative_cap_feats = None
        for t in range(num_inference_steps):
            latents = self.denoise_step(latents, cap_feats, negative_cap_feats, float(sched.sigmas[t]), sched.dt(t),
                                        guidance)
        return latents
