"""Qwen-Image-shaped dual-stream MMDiT denoising step on the B200 kernels, optionally tensor-parallel.

Module tree, attribute names and arithmetic follow the reference's QwenTransformer
(src/mflux/models/qwen/model/qwen_transformer/qwen_transformer.py:15-72, qwen_transformer_block.py:10-76,
qwen_attention.py:8-158, qwen_feed_forward.py, qwen_rope.py, qwen_timesteps.py, qwen_transformer_rms_norm.py).
As in flux.py, text and image tokens share one sequence buffer (text first, qwen_attention.py:67-69), q/k/v run
as one matmul and gate*y+residual / GELU are matmul epilogues.

Tensor parallelism (no counterpart in the single-device reference): to_q/k/v, add_*_proj and mlp_in are split by
output rows (whole heads per rank), attn_to_out / to_add_out / mlp_out by input columns; their partial sums are
all-reduced with NCCL in row chunks, each chunk's all-reduce running beside the next chunk's matmul, and the gated
residual is applied chunk by chunk afterwards. Every rank quantizes its own shard; because
quantization groups run along the input dimension and K / tp stays a multiple of 64, the shards' packed codes,
scales and biases are slices of what quantizing the full weight would give. LayerNorm, modulation and the residual
stream are replicated.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from . import nn, ops, resolution
from .flux import AdaNorm, FusedRows, MLPEmbedder, RMSNorm, _call, _linear
from .schedulers import LinearScheduler


@dataclass
class QwenConfig:
    hidden: int = 3072
    heads: int = 24
    num_layers: int = 60
    in_channels: int = 64
    joint_attention_dim: int = 3584
    mlp_ratio: int = 4
    # sigma schedule of the reference's "qwen-image" ModelConfig (models/common/config/model_config.py:505-520):
    # a flatter resolution shift than FLUX and a last sigma stretched to 0.02
    sigma_base_shift: float = 0.5
    sigma_max_shift: float = 0.9
    sigma_base_seq_len: int = 256
    sigma_max_seq_len: int = 8192
    sigma_shift_terminal: float | None = 0.02

    def scheduler(self, num_inference_steps: int, width: int, height: int) -> LinearScheduler:
        return LinearScheduler(num_inference_steps, width, height, True, base_shift=self.sigma_base_shift,
                               max_shift=self.sigma_max_shift, base_seq_len=self.sigma_base_seq_len,
                               max_seq_len=self.sigma_max_seq_len, shift_terminal=self.sigma_shift_terminal)

    def __post_init__(self):
        if self.hidden != self.heads * 128:
            raise ValueError("hidden must equal heads * 128 (head dimension 128)")


class _Ctx:
    """Creates every linear from the same seeded stream on all ranks, keeps this rank's shard, quantizes it."""

    def __init__(self, device, bits, std, seed, mode, tp_rank, tp_world):
        self.device, self.bits, self.std, self.mode = device, bits, std, mode
        self.rank, self.world = tp_rank, tp_world
        self.gen = torch.Generator(device=device).manual_seed(seed)

    def _finish(self, lin):
        if self.bits is not None and lin.weight.shape[1] % 64 == 0:
            return lin.to_quantized(group_size=64, bits=self.bits, mode=self.mode)
        return lin

    def linear(self, i, o, bias=True, split=None):
        lin = _linear(i, o, bias, self.device, self.std, self.gen)
        if split is not None and self.world > 1:
            if split == "col":  # output rows
                n = o // self.world
                sl = slice(self.rank * n, (self.rank + 1) * n)
                lin.weight = torch.nn.Parameter(lin.weight.data[sl].contiguous(), requires_grad=False)
                if bias:
                    lin.bias = torch.nn.Parameter(lin.bias.data[sl].contiguous(), requires_grad=False)
            else:  # "row": input columns; the bias is added once, after the all-reduce
                k = i // self.world
                if k % 64 != 0:
                    raise ValueError("K / tp must stay a multiple of the quantization group size 64")
                sl = slice(self.rank * k, (self.rank + 1) * k)
                lin.weight = torch.nn.Parameter(lin.weight.data[:, sl].contiguous(), requires_grad=False)
        return self._finish(lin)


class QwenFeedForward(nn.Module):
    def __init__(self, ctx, d, ratio):
        super().__init__()
        self.mlp_in = ctx.linear(d, ratio * d, split="col")
        self.mlp_out = ctx.linear(ratio * d, d, split="row")


class QwenAttention(nn.Module):
    def __init__(self, ctx, d):
        super().__init__()
        self.to_q, self.to_k, self.to_v = (ctx.linear(d, d, split="col") for _ in range(3))
        self.add_q_proj, self.add_k_proj, self.add_v_proj = (ctx.linear(d, d, split="col") for _ in range(3))
        self.norm_q, self.norm_k = RMSNorm(128, 1e-6, ctx.device), RMSNorm(128, 1e-6, ctx.device)
        self.norm_added_q, self.norm_added_k = RMSNorm(128, 1e-6, ctx.device), RMSNorm(128, 1e-6, ctx.device)
        self.attn_to_out = torch.nn.ModuleList([ctx.linear(d, d, split="row")])
        self.to_add_out = ctx.linear(d, d, split="row")


class QwenTransformerBlock(nn.Module):
    def __init__(self, ctx, cfg):
        super().__init__()
        d = cfg.hidden
        # tensor parallel: every rank holds 1/tp of the modulation linears' output rows (QwenTransformer._modulations)
        self.img_mod_linear = ctx.linear(d, 6 * d, split="col")
        self.attn = QwenAttention(ctx, d)
        self.img_ff = QwenFeedForward(ctx, d, cfg.mlp_ratio)
        self.txt_mod_linear = ctx.linear(d, 6 * d, split="col")
        self.txt_ff = QwenFeedForward(ctx, d, cfg.mlp_ratio)


class QwenTimeTextEmbed(nn.Module):
    def __init__(self, ctx, d):
        super().__init__()
        self.timestep_embedder = MLPEmbedder(ctx, 256, d)


class QwenTransformer(nn.Module):
    def __init__(self, cfg: QwenConfig = QwenConfig(), bits: int | None = 4, device="cuda", std: float = 0.02,
                 seed: int = 0, mode: str = "mlx", tp_rank: int = 0, tp_world: int = 1, tp_group=None,
                 tp_mode: str = "peer"):
        super().__init__()
        if cfg.heads % tp_world != 0:
            raise ValueError("the number of heads must be divisible by the tensor-parallel size")
        if tp_mode not in ("peer", "nccl"):
            raise ValueError("tp_mode is 'peer' (fused exchange over peer-mapped memory) or 'nccl' (all-reduce)")
        self.cfg, self.bits = cfg, bits
        self.tp_rank, self.tp_world, self.tp_group, self.tp_mode = tp_rank, tp_world, tp_group, tp_mode
        self._exchange = {}
        self._text_stream = {}
        ctx = _Ctx(device, bits, std, seed, mode, tp_rank, tp_world)
        d = cfg.hidden
        self.img_in = ctx.linear(cfg.in_channels, d)
        self.txt_norm = RMSNorm(cfg.joint_attention_dim, 1e-6, device)
        self.txt_in = ctx.linear(cfg.joint_attention_dim, d)
        self.time_text_embed = QwenTimeTextEmbed(ctx, d)
        self.transformer_blocks = torch.nn.ModuleList([QwenTransformerBlock(ctx, cfg) for _ in range(cfg.num_layers)])
        self.norm_out = AdaNorm(ctx, d, 2, bias=False)
        self.proj_out = ctx.linear(d, cfg.in_channels)
        self._fused, self._rope, self._buffers_for = {}, {}, None
        self._partials, self.tp_chunks, self.tp_chunk_min_rows = {}, 4, 512
        self.trace = None   # a dict here receives copies of the two residual streams after every block (parity tests)

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
            d, r, tp = self.cfg.hidden, self.cfg.mlp_ratio, self.tp_world
            self.nbuf = torch.empty(b, s, d, dtype=torch.bfloat16, device=device)
            self.qkv = torch.empty(b, s, 3 * d // tp, dtype=torch.bfloat16, device=device)
            self.attn = torch.empty(b, s, d // tp, dtype=torch.bfloat16, device=device)
            self.ffb = torch.empty(b, s, r * d // tp, dtype=torch.bfloat16, device=device)
            self._buffers_for = key
        return self.nbuf, self.qkv, self.attn, self.ffb

    @staticmethod
    def _rope_params(index: np.ndarray, dim: int, theta: float = 10000.0) -> np.ndarray:
        omega = 1.0 / (theta ** (np.arange(0, dim, 2, dtype=np.float32) / dim))
        f = np.outer(index.astype(np.float32), omega)
        return np.stack([np.cos(f), np.sin(f)], axis=-1)

    def rope_table(self, height, width, txt_len, device):
        """QwenEmbedRopeMLX with scale_rope=True (qwen_rope.py:35-113): image rows/cols are centred
        (-(h - h//2) .. h//2 - 1), the frame index is 0, text positions continue after max(h//2, w//2)."""
        key = (height, width, txt_len, str(device))
        t = self._rope.get(key)
        if t is None:
            lh, lw = height // 16, width // 16
            rows = np.concatenate([np.arange(-(lh - lh // 2), 0), np.arange(0, lh // 2)])
            cols = np.concatenate([np.arange(-(lw - lw // 2), 0), np.arange(0, lw // 2)])
            fr = np.broadcast_to(self._rope_params(np.zeros(1), 16)[None], (lh, lw, 8, 2))
            fh = np.broadcast_to(self._rope_params(rows, 56)[:, None], (lh, lw, 28, 2))
            fw = np.broadcast_to(self._rope_params(cols, 56)[None, :], (lh, lw, 28, 2))
            img = np.concatenate([fr, fh, fw], axis=2).reshape(lh * lw, 64, 2)
            start = max(lh // 2, lw // 2)
            tpos = np.arange(start, start + txt_len)
            txt = np.concatenate([self._rope_params(tpos, 16), self._rope_params(tpos, 56),
                                  self._rope_params(tpos, 56)], axis=1)
            t = torch.from_numpy(np.concatenate([txt, img], axis=0).astype(np.float32)).contiguous().to(device)
            self._rope[key] = t
        return t

    @staticmethod
    def time_proj(timestep: torch.Tensor) -> torch.Tensor:
        """QwenTimesteps (qwen_timesteps.py:15-34): the reference holds the timestep and the frequency table
        in the activation dtype (bf16); scale 1000; [cos, sin] order."""
        half = 128
        freqs = torch.exp(-math.log(10000) * torch.arange(half, dtype=torch.float32, device=timestep.device) / half)
        freqs = freqs.to(torch.bfloat16).float()
        emb = 1000.0 * (timestep.to(torch.bfloat16).float()[:, None] * freqs[None, :])
        return torch.cat([torch.cos(emb), torch.sin(emb)], dim=-1)

    def _row_parallel(self, layer, x, gate, residual):
        """residual += gate * (x . W^T + bias) for a layer split by input columns.

        With several ranks the rows go in chunks: the matmul of a chunk is followed by an asynchronous all-reduce of
        its partial sums, which NCCL runs beside the next chunk's matmul; the gated residual is applied chunk by
        chunk once the sums have arrived."""
        if self.tp_world == 1:
            return _call(layer, x, epilogue="gate_residual", gate=gate, residual=residual, out=residual)
        b, rows, _ = x.shape
        d = residual.shape[-1]
        n_chunks = self.tp_chunks if rows >= self.tp_chunk_min_rows * self.tp_chunks else 1
        bounds = [rows * c // n_chunks for c in range(n_chunks + 1)]
        bias = layer.bias
        pending = []
        for c in range(n_chunks):
            r0, r1 = bounds[c], bounds[c + 1]
            part = self._partial(rows, c, b, r1 - r0, d, x.device)
            if isinstance(layer, nn.QuantizedLinear):
                ops.qlinear(x[:, r0:r1], layer.weight.data, layer.scales.data, layer.biases.data, None, bits=layer.bits,
                            out=part, prepared=layer.prepared())
            else:
                part.copy_(torch.nn.functional.linear(x[:, r0:r1], layer.weight))
            work = dist.all_reduce(part, group=self.tp_group, async_op=True)
            pending.append((work, part, r0, r1))
        for work, part, r0, r1 in pending:
            work.wait()
            ops.gate_residual(part, gate, residual[:, r0:r1], None if bias is None else bias.data)
        return residual

    def _partial(self, rows, chunk, b, n, d, device):
        """Dense bf16 buffers for the partial sums (NCCL wants contiguous operands), one per (stream length, chunk)."""
        key = (rows, chunk, b, n, d, str(device))
        t = self._partials.get(key)
        if t is None:
            t = torch.empty(b, n, d, dtype=torch.bfloat16, device=device)
            self._partials[key] = t
        return t

    # ------------------------------------------------------------------ forward
    def forward(self, hidden_states: torch.Tensor, encoder_hidden_states: torch.Tensor, timestep: torch.Tensor,
                height: int, width: int, encoder_hidden_states_mask: torch.Tensor | None = None) -> torch.Tensor:
        """latents [B, Si, C] + text states [B, St, joint_dim] + sigma [B] -> predicted noise [B, Si, C] (bf16).

        `encoder_hidden_states_mask` [B, St] (1 = real token, 0 = padding) is the reference's text mask
        (qwen_transformer.py:37-72 passes it down to qwen_attention.py:117-135): padded text keys get an additive
        -1e9 in every block's attention, image keys 0. None means all ones, which the reference drops as well
        (:131-132); a caller that knows its mask is all ones should pass None, the masked kernel does more work."""
        cfg = self.cfg
        if self.tp_world > 1 and self.tp_mode == "peer":
            return self._forward_peer(hidden_states, encoder_hidden_states, timestep, height, width,
                                      encoder_hidden_states_mask)
        d, heads = cfg.hidden, cfg.heads // self.tp_world
        b, si, _ = hidden_states.shape
        st = encoder_hidden_states.shape[1]
        dev = hidden_states.device
        # two dense stream buffers (the all-reduced partial sums want dense operands)
        nbuf, qkv, attn, ffb = self._workspace(b, st + si, dev)
        if getattr(self, "_streams_for", None) != (b, si, st, str(dev)):
            self.x_img = torch.empty(b, si, d, dtype=torch.float32, device=dev)   # residual streams
            self.x_txt = torch.empty(b, st, d, dtype=torch.float32, device=dev)
            self._streams_for = (b, si, st, str(dev))
        x_img, x_txt = self.x_img, self.x_txt
        n_img, n_txt = nbuf[:, st:], nbuf[:, :st]
        cos_sin = self.rope_table(height, width, st, dev)
        key_bias = None
        if encoder_hidden_states_mask is not None:
            key_bias = torch.zeros(b, st + si, dtype=torch.float32, device=dev)
            key_bias[:, :st] = (1.0 - encoder_hidden_states_mask.to(dev, torch.float32)) * -1e9

        _call(self.img_in, hidden_states.to(torch.bfloat16), out=x_img)
        tn = ops.norm_modulate(encoder_hidden_states.to(torch.bfloat16), weight=self.txt_norm.weight.data,
                               eps=self.txt_norm.eps, rms=True)
        _call(self.txt_in, tn, out=x_txt)
        temb = self.time_text_embed.timestep_embedder(self.time_proj(timestep).to(torch.bfloat16))
        sv = ops.vec_sum_act(temb, act="silu", out_dtype=torch.bfloat16)

        all_mods = self._modulations(sv) if self.tp_world > 1 else None
        # One rank: the text stream's linears (a few hundred rows: a dozen tiles for 74 CTA pairs) run on a second
        # stream beside the image stream's and start on the SMs the image matmul's last wave leaves idle. The
        # all-reduce path keeps everything on one stream (its chunked collectives have their own).
        main = torch.cuda.current_stream(dev)
        side = None
        if self.tp_world == 1 and ops.TRACE is None:   # per-launch timing wants the launches one after the other
            side = self._text_stream.get(str(dev))
            if side is None:
                side = self._text_stream[str(dev)] = torch.cuda.Stream(device=dev)

        def pair(img_fn, txt_fn):
            """image-stream launch on the main stream, text-stream launch beside it"""
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
            if all_mods is None:
                mi = _call(blk.img_mod_linear, sv)   # [B, 6D]: (shift, scale, gate) x 2
                mt = _call(blk.txt_mod_linear, sv)
            else:
                mt, mi = all_mods[2 * i], all_mods[2 * i + 1]
            ops.norm_modulate(x_img, mi[:, 0:d], mi[:, d:2 * d], out=n_img)
            ops.norm_modulate(x_txt, mt[:, 0:d], mt[:, d:2 * d], out=n_txt)
            pair(lambda: self._fuse(("q", i), [a.to_q, a.to_k, a.to_v])(n_img, qkv[:, st:]),
                 lambda: self._fuse(("a", i), [a.add_q_proj, a.add_k_proj, a.add_v_proj])(n_txt, qkv[:, :st]))
            ops.qknorm_rope(qkv, heads, a.norm_added_q.weight.data, a.norm_added_k.weight.data, a.norm_q.weight.data,
                            a.norm_k.weight.data, st, cos_sin, a.norm_q.eps)
            ops.fmha(qkv, heads, out=attn, key_bias=key_bias)
            pair(lambda: self._row_parallel(a.attn_to_out[0], attn[:, st:], mi[:, 2 * d:3 * d], x_img),
                 lambda: self._row_parallel(a.to_add_out, attn[:, :st], mt[:, 2 * d:3 * d], x_txt))
            ops.norm_modulate(x_img, mi[:, 3 * d:4 * d], mi[:, 4 * d:5 * d], out=n_img)
            ops.norm_modulate(x_txt, mt[:, 3 * d:4 * d], mt[:, 4 * d:5 * d], out=n_txt)
            pair(lambda: _call(blk.img_ff.mlp_in, n_img, epilogue="gelu_approx", out=ffb[:, st:]),
                 lambda: _call(blk.txt_ff.mlp_in, n_txt, epilogue="gelu_approx", out=ffb[:, :st]))
            pair(lambda: self._row_parallel(blk.img_ff.mlp_out, ffb[:, st:], mi[:, 5 * d:6 * d], x_img),
                 lambda: self._row_parallel(blk.txt_ff.mlp_out, ffb[:, :st], mt[:, 5 * d:6 * d], x_txt))
            if self.trace is not None:
                self.trace[f"block{i}"] = (x_txt.clone(), x_img.clone())

        mod = _call(self.norm_out.linear, sv)   # [B, 2D]: scale, shift (ada_layer_norm_continuous.py:16-19)
        ops.norm_modulate(x_img, mod[:, d:2 * d], mod[:, 0:d], out=n_img)
        return _call(self.proj_out, n_img)


def _forward_peer(self, hidden_states, encoder_hidden_states, timestep, height, width, encoder_hidden_states_mask):
    """The tensor-parallel forward with the exchange fused into this library's kernels (see tp.py).

    Every rank keeps the residual stream of the joint-sequence rows it owns only. Per block:
      all ranks hold n1 (normalised rows of the whole sequence: every rank's own rows, copied to its peers by the
      copy engines) -> q/k/v (column split) -> attention over this rank's heads -> attn_to_out / to_add_out (row
      split): the matmul epilogue scatters every partial row to its owner -> tp_fuse on the owned rows: sum of the
      partials + bias, gated residual, second modulated LayerNorm into this rank's copy of the sequence, from where
      the copy engines carry the rows to the peers -> mlp_in (column split, GELU) -> mlp_out (row split, scattered)
      -> tp_fuse with the next block's first norm. The text stream's linears run on a second stream beside the image
      stream's; all modulation vectors are computed before the first block (_modulations).
    Linears, attention and the arithmetic per row are those of the one-GPU path; only the order of the bf16
    partial sums differs (they are rounded to bf16 per rank before they are added, as in the all-reduce path)."""
    from .tp import PeerExchange

    cfg = self.cfg
    d, heads = cfg.hidden, cfg.heads // self.tp_world
    b, si, _ = hidden_states.shape
    st = encoder_hidden_states.shape[1]
    s = st + si
    dev = hidden_states.device
    key = (b, st, si, str(dev))
    ex = self._exchange.get(key)
    if ex is None:
        ex = self._exchange[key] = PeerExchange(self.tp_group, self.tp_rank, self.tp_world, b, s, st, d, dev)
    sp = ex.seq_pad
    if getattr(self, "_peer_buffers_for", None) != key:
        tp, r = self.tp_world, cfg.mlp_ratio
        self.joint = torch.zeros(b, sp, d, dtype=torch.float32, device=dev)       # embeddings before the split
        self.qkv = torch.zeros(b, sp, 3 * d // tp, dtype=torch.bfloat16, device=dev)
        self.attn = torch.zeros(b, sp, d // tp, dtype=torch.bfloat16, device=dev)
        self.ffb = torch.zeros(b, sp, r * d // tp, dtype=torch.bfloat16, device=dev)
        self._peer_buffers_for = key
    joint, qkv, attn, ffb, nbuf = self.joint, self.qkv, self.attn, self.ffb, ex.nbuf
    cos_sin = self.rope_table(height, width, st, dev)
    key_bias = None
    if encoder_hidden_states_mask is not None:
        key_bias = torch.zeros(b, s, dtype=torch.float32, device=dev)
        key_bias[:, :st] = (1.0 - encoder_hidden_states_mask.to(dev, torch.float32)) * -1e9

    # embeddings (small, replicated), then every rank keeps its own rows
    _call(self.img_in, hidden_states.to(torch.bfloat16), out=joint[:, st:s])
    tn = ops.norm_modulate(encoder_hidden_states.to(torch.bfloat16), weight=self.txt_norm.weight.data,
                           eps=self.txt_norm.eps, rms=True)
    _call(self.txt_in, tn, out=joint[:, :st])
    ex.x.copy_(joint[:, ex.lo:ex.lo + ex.rows])
    temb = self.time_text_embed.timestep_embedder(self.time_proj(timestep).to(torch.bfloat16))
    sv = ops.vec_sum_act(temb, act="silu", out_dtype=torch.bfloat16)

    all_mods = self._modulations(sv)

    def mods(i):
        return all_mods[2 * i], all_mods[2 * i + 1]   # [B, 6D] each: (shift, scale, gate) x 2 of the text / image stream

    def ch(m, j):
        return m[:, j * d:(j + 1) * d]

    # The text stream's linears (256 rows: a dozen tiles for 74 CTA pairs, 35-50 us each whatever their size) run on
    # a second stream beside the image stream's: their CTAs start on the SMs the image matmul's last wave leaves
    # idle. The main stream joins the second one before anything reads their output, in particular before tp_fuse,
    # which waits for the arrival counts this rank's own text scatter contributes to.
    main = torch.cuda.current_stream(dev)
    side = self._text_stream.get(str(dev))
    if side is None:
        side = self._text_stream[str(dev)] = torch.cuda.Stream(device=dev)

    two_streams = ops.TRACE is None   # per-launch timing wants the launches one after the other

    def fork():
        """The second stream continues from what the main stream has queued so far. Called BEFORE the image
        matmul is launched, so that the text matmul launched after it does not wait for its end."""
        if two_streams:
            side.wait_stream(main)

    def on_side(fn):
        if not two_streams:
            fn()
            return
        with torch.cuda.stream(side):
            fn()

    def join():
        if two_streams:
            main.wait_stream(side)

    def scattered(layer, x, row_offset, lane=0):
        ops.qlinear(x, layer.weight.data, None, None, None, bits=layer.bits, prepared=layer.prepared(),
                    scatter=ex.scatter(row_offset, lane))

    own_lo, own_hi = ex.lo, min(s, ex.lo + ex.rows)

    def gathered(jobs):
        """Column-split matmuls over the gathered activations. `jobs` are (fn(x_rows, out_rows), a, b, x, out, text)
        over joint rows [a, b); text-stream jobs go to the second stream. The rows this rank normalised itself are
        in place already: their share of every matmul runs first and hides the flight time of the peers' rows; the
        rest follows the wait for their arrival."""
        def run(pieces):
            fork()
            for text_pass in (False, True):     # image matmuls first: the text tiles fill the SMs they leave
                for fn, x, out, lo_, hi_, text in pieces:
                    if text == text_pass:
                        if text:
                            on_side(lambda: fn(x[:, lo_:hi_], out[:, lo_:hi_]))
                        else:
                            fn(x[:, lo_:hi_], out[:, lo_:hi_])

        own = [(fn, x, out, max(a_, own_lo), min(b_, own_hi), text) for fn, a_, b_, x, out, text in jobs
               if max(a_, own_lo) < min(b_, own_hi)]
        run(own)
        ex.wait_gathered()
        rest = [(fn, x, out, lo_, hi_, text) for fn, a_, b_, x, out, text in jobs
                for lo_, hi_ in ((a_, min(b_, own_lo)), (max(a_, own_hi), b_)) if lo_ < hi_]
        run(rest)
        join()

    ex.begin()
    blocks = list(self.transformer_blocks)
    mt, mi = mods(0)
    ex.fuse(reduce=False, shift=(ch(mt, 0), ch(mi, 0)), scale=(ch(mt, 1), ch(mi, 1)))
    for i, blk in enumerate(blocks):
        a = blk.attn
        gathered([(self._fuse(("q", i), [a.to_q, a.to_k, a.to_v]), st, s, nbuf, qkv, False),
                  (self._fuse(("a", i), [a.add_q_proj, a.add_k_proj, a.add_v_proj]), 0, st, nbuf, qkv, True)])
        ops.qknorm_rope(qkv[:, :s], heads, a.norm_added_q.weight.data, a.norm_added_k.weight.data,
                        a.norm_q.weight.data, a.norm_k.weight.data, st, cos_sin, a.norm_q.eps)
        ops.fmha(qkv[:, :s], heads, out=attn[:, :s], key_bias=key_bias)
        fork()
        scattered(a.attn_to_out[0], attn[:, st:s], st)
        on_side(lambda: scattered(a.to_add_out, attn[:, :st], 0, 1))
        join()
        ex.fuse(reduce=True, bias=(a.to_add_out.bias, a.attn_to_out[0].bias), gate=(ch(mt, 2), ch(mi, 2)),
                shift=(ch(mt, 3), ch(mi, 3)), scale=(ch(mt, 4), ch(mi, 4)))
        gathered([(lambda x, o, l=blk.img_ff.mlp_in: _call(l, x, epilogue="gelu_approx", out=o), st, s, nbuf, ffb, False),
                  (lambda x, o, l=blk.txt_ff.mlp_in: _call(l, x, epilogue="gelu_approx", out=o), 0, st, nbuf, ffb, True)])
        fork()
        scattered(blk.img_ff.mlp_out, ffb[:, st:s], st)
        on_side(lambda: scattered(blk.txt_ff.mlp_out, ffb[:, :st], 0, 1))
        join()
        gate = (ch(mt, 5), ch(mi, 5))
        bias = (blk.txt_ff.mlp_out.bias, blk.img_ff.mlp_out.bias)
        if i + 1 < len(blocks):
            mt, mi = mods(i + 1)       # the next block's first norm rides on this exchange
            ex.fuse(reduce=True, bias=bias, gate=gate, shift=(ch(mt, 0), ch(mi, 0)), scale=(ch(mt, 1), ch(mi, 1)))
        else:
            ex.fuse(reduce=True, bias=bias, gate=gate)
        if self.trace is not None:
            self.trace[f"block{i}"] = ex.x.clone()    # this rank's rows of the joint stream
    ex.end()

    # output head on the owned rows, then the ranks' pieces are put together (a few hundred kilobytes)
    mod = _call(self.norm_out.linear, sv)   # [B, 2D]: scale, shift
    own = torch.zeros(b, ex.rows, cfg.in_channels, dtype=torch.bfloat16, device=dev)
    n_live = max(0, ex.hi - ex.lo)
    if n_live > 0:
        nrm = ops.norm_modulate(ex.x[:, :n_live], mod[:, d:2 * d], mod[:, 0:d])
        _call(self.proj_out, nrm, out=own[:, :n_live])
    parts = torch.empty(self.tp_world, b, ex.rows, cfg.in_channels, dtype=torch.bfloat16, device=dev)
    dist.all_gather_into_tensor(parts, own, group=self.tp_group)
    return parts.permute(1, 0, 2, 3).reshape(b, sp, cfg.in_channels)[:, st:s].contiguous()


def _modulations(self, sv):
    """Modulation vectors of every block on a tensor-parallel group: [2 * blocks, B, 6D], text stream at 2i, image
    stream at 2i + 1. The 2 x 60 AdaLN linears (qwen_transformer_block.py:27-34) all read the same conditioning
    vector and stream 28 MB of weights each; replicated, they were 9 % of the 8-GPU step. Every rank computes its
    1/tp of each linear's output rows before the first block, one all-gather of a few megabytes puts the rows
    together."""
    blocks = list(self.transformer_blocks)
    tp, b = self.tp_world, sv.shape[0]
    n = 6 * self.cfg.hidden // tp
    part = torch.empty(2 * len(blocks), b, n, dtype=torch.bfloat16, device=sv.device)
    for i, blk in enumerate(blocks):
        _call(blk.txt_mod_linear, sv, out=part[2 * i])
        _call(blk.img_mod_linear, sv, out=part[2 * i + 1])
    gathered = torch.empty(tp, 2 * len(blocks), b, n, dtype=torch.bfloat16, device=sv.device)
    dist.all_gather_into_tensor(gathered, part, group=self.tp_group)
    return gathered.permute(1, 2, 0, 3).reshape(2 * len(blocks), b, tp * n)


QwenTransformer._forward_peer = _forward_peer
QwenTransformer._modulations = _modulations


class QwenImage:
    """Denoise loop of the reference's QwenImage variant (variants/txt2img/qwen_image.py:99-128,165-174):
    two denoiser evaluations per step (prompt and negative prompt) and the norm-preserving guidance combine.

    On one rank the two evaluations run as one batch of 2. With `cfg_group` (a process group of two ranks, or of
    two tensor-parallel groups' matching ranks) every rank evaluates only the branch `cfg_rank` (0 = prompt,
    1 = negative prompt) and the two predictions are exchanged with one small all-gather before the combine, so
    the pair needs no other communication; this composes with tensor parallelism inside each branch."""

    def __init__(self, quantize: int | None = None, model_config: QwenConfig | None = None, device="cuda",
                 seed: int = 0, stored_quantization: int | None = None, tp_rank: int = 0, tp_world: int = 1,
                 tp_group=None, cfg_rank: int | None = None, cfg_group=None, cuda_graph: bool = False,
                 tp_mode: str = "peer"):
        bits, warning = resolution.resolve(stored_quantization, quantize)
        if warning:
            print(f"Warning: {warning}")
        resolution.check_supported(bits)
        self.bits = bits
        self.model_config = model_config or QwenConfig()
        self.cfg_rank, self.cfg_group = cfg_rank, cfg_group
        self.cuda_graph, self._captured, self._captured_epoch = cuda_graph, {}, nn.weights_epoch()
        self.transformer = QwenTransformer(self.model_config, bits=bits, device=device, seed=seed, tp_rank=tp_rank,
                                           tp_world=tp_world, tp_group=tp_group, tp_mode=tp_mode)

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
        self.release_graphs()   # recorded graphs hold the prepared weights of the old parameters

    @staticmethod
    def _pad_pair(pos, neg, pos_mask, neg_mask):
        """Text states of the two guidance branches as one batch. The reference evaluates the branches one after
        the other, each at its own token count (qwen_image.py:105-118); batched, the shorter one is padded with
        zero rows that the key mask removes from every attention, which leaves its real rows unchanged."""
        lp, ln = pos.shape[1], neg.shape[1]
        if lp == ln and pos_mask is None and neg_mask is None:
            return torch.cat([pos, neg]), None
        lt = max(lp, ln)

        def grow(t, m):
            if m is None:
                m = torch.ones(t.shape[0], t.shape[1], dtype=torch.float32, device=t.device)
            m = m.to(t.device, torch.float32)
            if t.shape[1] < lt:
                t = torch.cat([t, t.new_zeros(t.shape[0], lt - t.shape[1], t.shape[2])], dim=1)
                m = torch.cat([m, m.new_zeros(m.shape[0], lt - m.shape[1])], dim=1)
            return t, m

        (pos, pm), (neg, nm) = grow(pos, pos_mask), grow(neg, neg_mask)
        return torch.cat([pos, neg]), torch.cat([pm, nm])

    def predict_noise(self, latents, prompt_embeds, negative_prompt_embeds, sigma, height, width,
                      prompt_mask=None, negative_prompt_mask=None):
        """(noise for the prompt, noise for the negative prompt), each [B, Si, C]. `sigma` is a number or a
        one-element tensor on the device. The two prompts may differ in token count; `prompt_mask` /
        `negative_prompt_mask` [B, St] (1 = real token) are the reference's text masks."""
        b = latents.shape[0]
        if not torch.is_tensor(sigma):
            sigma = torch.full((1,), sigma, device=latents.device)
        sigma = sigma.reshape(1).float()
        if self.cfg_group is None:
            embeds, mask = self._pad_pair(prompt_embeds, negative_prompt_embeds, prompt_mask, negative_prompt_mask)
            both = self.transformer(torch.cat([latents, latents]), embeds, sigma.expand(2 * b), height, width,
                                    encoder_hidden_states_mask=mask)
            return both[:b], both[b:]
        mine = self.transformer(latents, prompt_embeds if self.cfg_rank == 0 else negative_prompt_embeds,
                                sigma.expand(b), height, width,
                                encoder_hidden_states_mask=prompt_mask if self.cfg_rank == 0 else negative_prompt_mask
                                ).contiguous()
        parts = torch.empty(2, *mine.shape, dtype=mine.dtype, device=mine.device)
        dist.all_gather_into_tensor(parts, mine, group=self.cfg_group)
        return parts[0], parts[1]

    def guided_noise(self, latents, prompt_embeds, negative_prompt_embeds, sigma, guidance, height, width):
        """The guidance-combined prediction of one step. With `cuda_graph=True` the two evaluations, their
        collectives and the combine replay as one CUDA graph (one graph per shape, guidance scale and image size);
        the result is then the graph's output buffer, valid until the next call."""
        def run(lat, pos, neg, sig):
            noise, noise_negative = self.predict_noise(lat, pos, neg, sig, height, width)
            return ops.cfg_combine(noise, noise_negative, guidance, mode="qwen")

        if not torch.is_tensor(sigma):
            sigma = torch.full((1,), sigma, device=latents.device)
        if not self.cuda_graph:
            return run(latents, prompt_embeds, negative_prompt_embeds, sigma)
        from .graphs import CapturedStep

        if self._captured and self._captured_epoch != nn.weights_epoch():
            self.release_graphs()   # recorded launches point at the prepared blobs of replaced weights
        self._captured_epoch = nn.weights_epoch()

        key = (float(guidance), height, width)
        step = self._captured.get(key)
        if step is None:
            step = self._captured[key] = CapturedStep(run)
        return step(latents, prompt_embeds, negative_prompt_embeds, sigma.reshape(1).float())

    def release_graphs(self) -> None:
        """Drops every recorded CUDA graph (call before `torch.distributed.destroy_process_group`: a live graph
        with recorded collectives keeps the communicator from shutting down)."""
        for step in self._captured.values():
            step.release()
        self._captured = {}

    def denoise_step(self, latents, prompt_embeds, negative_prompt_embeds, sigma, dt, guidance, height, width):
        guided = self.guided_noise(latents, prompt_embeds, negative_prompt_embeds, sigma, guidance, height, width)
        return ops.euler_step(latents, guided, dt)

    def generate_image(self, seed: int, prompt_embeds: torch.Tensor, negative_prompt_embeds: torch.Tensor,
                       num_inference_steps: int = 20, height: int = 1328, width: int = 1328, guidance: float = 4.0,
                       latents: torch.Tensor | None = None) -> torch.Tensor:
        """Returns the final latents [B, (H/16)(W/16), C] (f32); prompt embeddings stand in for the text encoder."""
        dev = prompt_embeds.device
        b = prompt_embeds.shape[0]
        sched = self.model_config.scheduler(num_inference_steps, width, height)
        if latents is None:
            g = torch.Generator(device=dev).manual_seed(seed)
            latents = torch.randn(b, (height // 16) * (width // 16), self.model_config.in_channels, device=dev,
                                  generator=g)
        latents = latents.float()
        for t in range(num_inference_steps):
            latents = self.denoise_step(latents, prompt_embeds, negative_prompt_embeds, float(sched.sigmas[t]),
                                        sched.dt(t), guidance, height, width)
        return latents
