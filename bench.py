"""Benchmark of the quantized DiT denoising step: FLUX.1-shaped 12B MMDiT, W4 group 64, 1024x1024.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--small] [--workload NAME]

One process per GPU (torchrun for N > 1). A step is one denoiser evaluation plus the Euler update for a
batch of 16 images (4096 image + 512 text tokens each) on synthetic inputs with random-init weights.
The batch is the unit that shards: every rank runs its own 16-image batch with replicated weights and no
collective on the data path (weak scaling); `value` = steps all ranks completed / max-over-ranks device
time. Rank 0 prints one JSON line.

`--workload` selects another configuration of the same path (the default, `flux`, is the headline):
`zimage` (Z-Image-shaped 6B single-stream DiT, W8, 8 images, batch-sharded like flux), `qwen` (Qwen-Image-shaped
20B dual-stream DiT, W4, prompt/negative-prompt pair at 1328x1328; with N > 1 the weights are tensor-parallel
over the N ranks with an NCCL all-reduce per row-split linear, strong scaling) and `sweep` (single quantized
linears over bits x (N, K) x M, reporting TFLOP/s per shape).

`--impl reference` times the CPU oracle (the restatement of the reference's MLX arithmetic; MLX itself is
not installable offline) on the host cores on a bounded sample of the same workload and prints the same
line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

TRAFFIC_RECORD = ROOT / "profiles" / "qmm_flux_step_dram_traffic.json"


def recorded_traffic():
    """Mean DRAM bytes (read + write) per quantized-matmul launch of the full flux step, from the committed record
    of an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum on the reduced-depth model at the same per-GPU
    batch, weighted by the block counts of the full model). The record names the command that made it and the
    SHA-256 of the kernel source it was taken on; it is reported only while that source is unchanged."""
    import hashlib

    if not TRAFFIC_RECORD.exists():
        return None
    rec = json.loads(TRAFFIC_RECORD.read_text())
    src = ROOT / "mflux_b200" / "csrc" / "qmm.cu"
    if hashlib.sha256(src.read_bytes()).hexdigest() != rec.get("qmm_cu_sha256"):
        return None
    return rec.get("dram_bytes_per_launch")


def step_flops(cfg, batch, si, st):
    """Algorithmic flops of one denoiser evaluation: 2*M*N*K per linear, 4*H*S^2*128 per attention."""
    d, r = cfg.hidden, cfg.mlp_ratio
    s = si + st
    lin = 0
    lin += 2 * batch * si * cfg.in_channels * d + 2 * batch * st * cfg.context_dim * d
    per_stream = lambda rows: 2 * batch * rows * (3 * d * d + d * d + 2 * r * d * d)  # noqa: E731
    lin += cfg.num_joint * (per_stream(si) + per_stream(st) + 2 * 2 * batch * d * 6 * d)
    lin += cfg.num_single * (2 * batch * s * (3 * d * d + r * d * d + (1 + r) * d * d) + 2 * batch * d * 3 * d)
    lin += 2 * batch * d * 2 * d + 2 * batch * si * d * cfg.in_channels
    attn = (cfg.num_joint + cfg.num_single) * 4 * batch * cfg.heads * s * s * 128
    return lin, attn


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = max((int(s[1]) for s in self.samples if s[1].isdigit()), default=None)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples for i in range(4) if s[2 + i].lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": reasons,
                "samples": len(self.samples)}


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return d.get("bf16_tflops_sustained") or d.get("bf16_tflops"), "measured (sustained)", d.get("bf16_tflops")
    return 1400.0, "fallback (sustained)", 1590.0


def blas_threads(cores: int) -> int:
    """Gives the BLAS behind NumPy `cores` threads (a launcher may have exported OMP_NUM_THREADS=1) and returns
    the number it reports afterwards."""
    try:
        from threadpoolctl import threadpool_info, threadpool_limits

        threadpool_limits(limits=cores)
        return max((int(p.get("num_threads", 1)) for p in threadpool_info()), default=1)
    except Exception:
        return int(os.environ.get("OMP_NUM_THREADS", "1") or 1)


def measured_hbm():
    f = ROOT / "MEASURED_PEAKS.json"
    return json.loads(f.read_text()).get("hbm_gbs", 6650.0) if f.exists() else 6650.0


def cpu_sample(seconds_target: float = 12.0):
    """Times the CPU oracle (dequantize + float32 matmul on all host cores) on a bounded sample: quantized
    linears of the step's dominant shape. Returns (TFLOP/s, description, cores, BLAS threads)."""
    import numpy as np

    from oracle import quant

    cores = os.cpu_count() or 1
    threads = blas_threads(cores)
    m, n, k = 2048, 3072, 3072
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    pq, ps, pb = quant.quantize_affine(w, 64, 4)
    quant.qlinear(x, pq, ps, pb, None, 64, 4)  # warm-up
    t0, reps = time.perf_counter(), 0
    while True:
        quant.qlinear(x, pq, ps, pb, None, 64, 4)
        reps += 1
        if time.perf_counter() - t0 > seconds_target or reps >= 200:
            break
    dt = (time.perf_counter() - t0) / reps
    desc = (f"{reps} x quantized linear M={m} N={n} K={k} W4 g64 (dequantize + float32 GEMM, numpy/OpenBLAS), "
            f"scaled to a step by algorithmic flops")
    return 2.0 * m * n * k / dt / 1e12, desc, cores, threads


def run_reference(args, spec):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    flops = spec["lin"] + spec["attn"]
    vals = []
    desc, cores, threads = "", 1, 1
    for i in range(args.warmup + args.steps):
        tf, desc, cores, threads = cpu_sample(seconds_target=max(2.0, 20.0 / max(1, args.steps + args.warmup)))
        if i >= args.warmup:
            vals.append(tf)
    tflops = sum(vals) / len(vals)
    value = tflops * 1e12 / flops
    line = {
        "impl": "reference", "metric": spec["metric"], "value": value, "unit": spec["unit"], "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / value, "higher_is_better": True,
        "scaling": spec["scaling"], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": spec["workload"], "note": "CPU oracle port of the MLX arithmetic (MLX itself is not "
                   "installable offline); every step times the bounded sample below, value and ms_per_step are "
                   "that sample's rate extrapolated to a whole step by algorithmic flops, not a step that ran"},
        "cpu_baseline": {"value": value, "unit": spec["unit"], "cores": cores, "threads": threads, "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": spec["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- workloads
# A spec is plain data (no GPU needed): names, algorithmic flops of one step, how the step scales over ranks.
# build(dev, rank, world, steps) returns (pinned host inputs, pinned host output, step(i, *device inputs)).

def flux_spec(args):
    from mflux_b200.flux import FluxConfig

    cfg = FluxConfig(num_joint=1, num_single=1) if args.small else FluxConfig()
    batch = args.batch or (2 if args.small else 16)
    height = width = 1024
    si, st = (height // 16) * (width // 16), 512
    lin, attn = step_flops(cfg, batch, si, st)

    def build(dev, rank, world, steps):
        import torch

        from mflux_b200 import ops
        from mflux_b200.flux import Transformer
        from mflux_b200.schedulers import LinearScheduler

        model = Transformer(cfg, bits=4, device=dev, seed=1234)  # same weights on every rank (replicated)
        if args.lora_rank:
            # one adapter on every attention projection and feed-forward linear of every block (the modulation
            # linears stay bare), random A and B: the usual target set of a LoRA file for this model
            from mflux_b200 import nn as mnn
            from mflux_b200.lora import apply_lora

            ga = torch.Generator(device=dev).manual_seed(77)
            adapters = {}
            for name, mod in list(model.named_modules()):
                if (not isinstance(mod, mnn.QuantizedLinear) or "blocks." not in name
                        or ".norm" in name):   # norm*.linear are the modulation linears
                    continue
                n_out, k_in = mod.output_dims, mod.input_dims
                a = (torch.randn(k_in, args.lora_rank, device=dev, generator=ga) * k_in ** -0.5).to(torch.bfloat16)
                b = (torch.randn(args.lora_rank, n_out, device=dev, generator=ga) * 0.02).to(torch.bfloat16)
                adapters[name] = [(a, b, 1.0)]
            apply_lora(model, adapters)
            if args.lora_library:   # the same adapters through two library GEMMs per layer, for comparison
                import mflux_b200.lora as mlora

                mlora.MAX_FUSED_COLUMNS = 0
            flux_spec.adapters = len(adapters)
        g = torch.Generator(device="cpu").manual_seed(100 + rank)  # every rank has its own batch of images
        lat_h = torch.randn(batch, si, cfg.in_channels, generator=g).pin_memory()
        ctx_h = torch.randn(batch, st, cfg.context_dim, generator=g).to(torch.bfloat16).pin_memory()
        pool_h = torch.randn(batch, cfg.pooled_dim, generator=g).to(torch.bfloat16).pin_memory()
        out_h = torch.empty(batch, si, cfg.in_channels).pin_memory()
        sched = LinearScheduler(max(steps, 2), width, height, True)
        gvec = torch.full((batch,), 3.5 * cfg.num_train_steps, device=dev)

        def step(i, lat_d, ctx_d, pool_d):
            j = i % len(sched.timesteps)
            nb = lat_d.shape[0]
            ts = torch.full((nb,), float(sched.sigmas[j]) * cfg.num_train_steps, device=dev)
            noise = model(lat_d, ctx_d, pool_d, ts, gvec[:nb], height, width)
            return ops.euler_step(lat_d, noise, sched.dt(j))

        def shard(images):
            """Device inputs of this rank's share of one batch of `images` images split evenly over the ranks
            (strong scaling: the same model, fewer images per GPU)."""
            nb = images // world
            gs = torch.Generator(device="cpu").manual_seed(500 + rank)
            return [torch.randn(nb, si, cfg.in_channels, generator=gs).to(dev),
                    torch.randn(nb, st, cfg.context_dim, generator=gs).to(torch.bfloat16).to(dev),
                    torch.randn(nb, cfg.pooled_dim, generator=gs).to(torch.bfloat16).to(dev)]

        step.shard = shard
        return [lat_h, ctx_h, pool_h], out_h, step

    return {
        "metric": "flux1_w4_dit_steps_per_sec_1024px_batch16",
        "unit": "steps/s (one step = 16 images x 4608 tokens through 19+38 blocks)",
        "workload": (f"FLUX.1-shaped MMDiT {cfg.num_joint}+{cfg.num_single} blocks, hidden {cfg.hidden}, "
                     f"{cfg.heads}x128 heads, W4 g64, batch {batch}, {si} image + {st} text tokens, "
                     f"guidance-embedded, CFG-free"
                     + (f", rank-{args.lora_rank} LoRA adapter on every attention and feed-forward linear ("
                        + ("library GEMMs" if args.lora_library else "inside the quantized matmul") + ")"
                        if args.lora_rank else "")),
        "scaling": "weak", "lin": lin, "attn": attn, "per_gpu_batch": batch, "build": build,
        "l2_policy": "inputs larger than L2 (6.7 GB of packed weights stream every step)",
    }


def zimage_spec(args):
    from mflux_b200.zimage import ZImageConfig

    cfg = ZImageConfig()
    batch = args.batch or 8
    height = width = 1024
    si, sc = (height // 16) * (width // 16), 512
    d, h, s = cfg.dim, cfg.ffn_hidden, si + sc
    per_row = 2 * (4 * d * d + 3 * d * h)
    rows = cfg.n_layers * s + cfg.n_refiner_layers * (si + sc)
    lin = batch * rows * per_row + 2 * batch * (si * cfg.embed_dim * d * 2 + sc * cfg.cap_feat_dim * d)
    lin += 2 * batch * 256 * 4 * d * (cfg.n_layers + cfg.n_refiner_layers)
    attn = 4 * batch * cfg.n_heads * 128 * (cfg.n_layers * s * s + cfg.n_refiner_layers * (si * si + sc * sc))

    def build(dev, rank, world, steps):
        import torch

        from mflux_b200 import ops
        from mflux_b200.schedulers import LinearScheduler
        from mflux_b200.zimage import ZImageTransformer

        model = ZImageTransformer(cfg, bits=8, device=dev, seed=1234)
        g = torch.Generator(device="cpu").manual_seed(100 + rank)
        lat_h = torch.randn(batch, cfg.in_channels, 1, height // 8, width // 8, generator=g).pin_memory()
        cap_h = torch.randn(batch, sc, cfg.cap_feat_dim, generator=g).to(torch.bfloat16).pin_memory()
        out_h = torch.empty_like(lat_h).pin_memory()
        sched = LinearScheduler(max(steps, 2), width, height, True)

        def step(i, lat_d, cap_d):
            j = i % len(sched.timesteps)
            t = torch.full((batch,), 1.0 - float(sched.sigmas[j]), device=dev)
            return ops.euler_step(lat_d, model(lat_d, t, cap_d), sched.dt(j))

        return [lat_h, cap_h], out_h, step

    return {
        "metric": "zimage_w8_dit_steps_per_sec_1024px_batch8",
        "unit": "steps/s (one step = 8 images x 4608 tokens through 2+2 refiner and 30 main blocks)",
        "workload": (f"Z-Image-shaped single-stream DiT {cfg.n_layers} blocks + 2x{cfg.n_refiner_layers} refiners, hidden "
                     f"{d}, {cfg.n_heads}x128 heads, SwiGLU {h}, W8 g64, batch {batch}, {si} image + {sc} caption tokens"),
        "scaling": "weak", "lin": lin, "attn": attn, "per_gpu_batch": batch, "build": build,
        "l2_policy": "inputs larger than L2 (6.2 GB of packed weights stream every step)",
    }


def qwen_spec(args):
    from mflux_b200.qwen import QwenConfig

    cfg = QwenConfig()
    height = width = 1328
    si, st = (height // 16) * (width // 16), 256
    b, d = 2, cfg.hidden   # the prompt / negative-prompt pair of one image
    s = si + st
    lin = cfg.num_layers * (2 * b * s * 12 * d * d + 2 * 2 * b * d * 6 * d)
    lin += 2 * b * (si * cfg.in_channels * d * 2 + st * cfg.joint_attention_dim * d)
    attn = cfg.num_layers * 4 * b * cfg.heads * s * s * 128

    def build(dev, rank, world, steps):
        import torch
        import torch.distributed as dist

        from mflux_b200.qwen import QwenImage
        from mflux_b200.schedulers import LinearScheduler

        graph = not args.no_cuda_graph
        # 1 rank: both branches as a batch of 2. Even rank counts: the prompt branch on the first half of the
        # ranks, the negative-prompt branch on the second half, tensor parallelism inside each half.
        if world > 1 and args.qwen_parallel == "cfg+tp":
            tp = world // 2
            branch, tp_rank = rank // tp, rank % tp
            tp_groups = [dist.new_group(list(range(g * tp, (g + 1) * tp))) for g in range(2)]
            cfg_groups = [dist.new_group([r, r + tp]) for r in range(tp)]
            pipe = QwenImage(quantize=4, model_config=cfg, device=dev, seed=1234, tp_rank=tp_rank, tp_world=tp,
                             tp_group=tp_groups[branch] if tp > 1 else None, cfg_rank=branch,
                             cfg_group=cfg_groups[tp_rank], cuda_graph=graph, tp_mode=args.qwen_tp_mode)
        else:
            pipe = QwenImage(quantize=4, model_config=cfg, device=dev, seed=1234, tp_rank=rank, tp_world=world,
                             cuda_graph=graph, tp_mode=args.qwen_tp_mode)
        g = torch.Generator(device="cpu").manual_seed(100)   # every rank sees the same image and prompts
        lat_h = torch.randn(1, si, cfg.in_channels, generator=g).pin_memory()
        emb_h = torch.randn(b, st, cfg.joint_attention_dim, generator=g).to(torch.bfloat16).pin_memory()
        out_h = torch.empty_like(lat_h).pin_memory()
        sched = LinearScheduler(max(steps, 2), width, height, True)

        def step(i, lat_d, emb_d):
            j = i % len(sched.timesteps)
            return pipe.denoise_step(lat_d, emb_d[:1], emb_d[1:], float(sched.sigmas[j]), sched.dt(j), 4.0, height,
                                     width)

        def eager(i, lat_d, emb_d):   # the same step launch by launch (the per-launch event pairs need it)
            pipe.cuda_graph = False
            try:
                return step(i, lat_d, emb_d)
            finally:
                pipe.cuda_graph = graph

        step.eager = eager
        step.release = pipe.release_graphs   # recorded collectives must go before the process group does
        return [lat_h, emb_h], out_h, step

    par = "1 GPU" if args.gpus == 1 else (f"prompt / negative-prompt branch x tensor-parallel {args.gpus // 2}"
                                          if args.qwen_parallel == "cfg+tp" else f"tensor-parallel {args.gpus}")
    return {
        "metric": "qwen_image_w4_dit_steps_per_sec_1328px_cfg2",
        "unit": "steps/s (one step = prompt + negative prompt of one image, 2 x 7145 tokens through 60 blocks)",
        "workload": (f"Qwen-Image-shaped dual-stream MMDiT {cfg.num_layers} blocks, hidden {d}, {cfg.heads}x128 heads, "
                     f"W4 g64, CFG batch 2, {si} image + {st} text tokens, {par}"
                     f"{'' if args.gpus == 1 else ' (' + args.qwen_tp_mode + ' exchange)'}, "
                     f"{'launches issued one by one' if args.no_cuda_graph else 'step replayed as a CUDA graph'}"),
        "scaling": "strong", "lin": lin, "attn": attn, "per_gpu_batch": b, "build": build,
        "l2_policy": "inputs larger than L2 (10 GB of packed weights, split over the ranks, stream every step)",
    }


SPECS = {"flux": flux_spec, "zimage": zimage_spec, "qwen": qwen_spec}


def run_lora(args, dev):
    """Adapters over the single-linear configuration (M 4096, N 12288, K 3072, group 64): per call the frozen layer
    alone, the wrapper with the low-rank product inside the quantized-matmul kernel, and the wrapper with both
    thin products as library GEMMs accumulating into the output. Operand copies rotate past the L2."""
    import torch

    from mflux_b200 import nn
    from mflux_b200.lora import FusedLoRALinear, LoRALinear, _low_rank_add

    m, n, k = 4096, 12288, 3072
    rows = []
    g = torch.Generator(device=dev).manual_seed(0)
    copies = 4
    # --small: one width, one rank, a handful of launches (the case a profiler capture runs)
    all_bits = (4,) if args.small else (4, 8)
    all_ranks = ((64,),) if args.small else ((16,), (64,), (128,), (16, 16, 32))
    for bits in all_bits:
        layers = []
        for _ in range(copies):
            lin = nn.Linear(k, n, bias=True, device=dev)
            with torch.no_grad():
                lin.weight.copy_(torch.randn(n, k, device=dev, generator=g) * 0.02)
            layers.append(lin.to_quantized(bits=bits))
            del lin
        xs = [torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16) for _ in range(copies)]
        ys = [torch.empty(m, n, device=dev, dtype=torch.bfloat16) for _ in range(copies)]

        def timed_together(fns, reps=4 if args.small else 40, chunks=1 if args.small else 7):
            """Per function (median, worst) microseconds per call. The functions take turns, one run of `reps`
            calls each per round, so that clock drift under the power cap falls on all of them alike."""
            for fn in fns:
                for i in range(max(3, args.warmup, copies)):
                    fn(i % copies)
            per = [[] for _ in fns]
            for _ in range(chunks):
                for j, fn in enumerate(fns):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    e0.record()
                    for i in range(reps):
                        fn(i % copies)
                    e1.record()
                    torch.cuda.synchronize()
                    per[j].append(e0.elapsed_time(e1) * 1e3 / reps)
            return [(sorted(v)[len(v) // 2], max(v)) for v in per]

        for ranks in all_ranks:
            wrapped = []
            for q in layers:
                adapters = [LoRALinear.from_linear(q, r=r, scale=0.8) for r in ranks]
                wrapped.append(adapters[0] if len(adapters) == 1 else FusedLoRALinear(q, adapters))

            def library(i):
                y = layers[i](xs[i], out=ys[i])
                w = wrapped[i]
                for l in ([w] if isinstance(w, LoRALinear) else w.loras):
                    _low_rank_add(y, xs[i], l.lora_A.data, l.lora_B.data, l.scale)

            (base_us, base_w), (fused_us, fused_w), (library_us, library_w) = timed_together(
                [lambda i: layers[i](xs[i], out=ys[i]), lambda i: wrapped[i](xs[i], out=ys[i]), library])
            rows.append({"bits": bits, "M": m, "N": n, "K": k, "ranks": list(ranks), "base_us": round(base_us, 1),
                         "fused_us": round(fused_us, 1), "library_us": round(library_us, 1),
                         "worst_chunk_us": [round(base_w, 1), round(fused_w, 1), round(library_w, 1)],
                         "fused_over_base": round(fused_us / base_us, 3),
                         "library_over_base": round(library_us / base_us, 3)})
        del layers, xs, ys
    return rows


def run_sweep(args, dev):
    """Single quantized linears: bits x (N, K) x M. Every shape cycles through enough weight/activation copies
    that consecutive launches never find their operands in L2."""
    import torch

    from mflux_b200 import ops

    peak, _, burst = measured_peaks()
    f = ROOT / "MEASURED_PEAKS.json"
    hbm = json.loads(f.read_text()).get("hbm_gbs") if f.exists() else 6650.0
    rows = []
    g = torch.Generator(device=dev).manual_seed(0)
    for bits in (4, 8):
        for n, k in ((3072, 3072), (9216, 3072), (12288, 3072), (3072, 12288)):
            w = torch.randn(n, k, device=dev, generator=g) * 0.02
            wq, sc, bi = ops.quantize_affine(w, 64, bits)
            bias = (torch.randn(n, device=dev, generator=g) * 0.02).to(torch.bfloat16)
            del w
            for m in (1, 16, 256, 1024, 4096, 4608, 16384):
                per = n * k * bits // 8 + 2 * m * k + 2 * m * n
                copies = max(2, min(64, -(-400_000_000 // per)))
                preps = [ops.prepare_qlinear(wq, sc, bi, bits, 64) for _ in range(copies)]
                xs = [torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16) for _ in range(copies)]
                ys = [torch.empty(m, n, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
                reps = max(copies, 20)
                def launch_all():
                    for i in range(reps):
                        ops.qlinear(xs[i % copies], wq, None, None, bias, bits=bits, out=ys[i % copies],
                                    prepared=preps[i % copies])
                for i in range(max(3, args.warmup)):
                    ops.qlinear(xs[i % copies], wq, None, None, bias, bits=bits, out=ys[i % copies], prepared=preps[i % copies])
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                if m <= 1024:
                    # launches of a few (tens of) microseconds: replay them from a CUDA graph so that the host's
                    # launch rate (the Python wrapper and three tensor-map encodings per call) is not what gets timed
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        launch_all()
                    graph.replay()
                    torch.cuda.synchronize()
                    e0.record()
                    graph.replay()
                    e1.record()
                else:
                    e0.record()
                    launch_all()
                    e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / reps
                tf = 2.0 * m * n * k / us / 1e6
                row = {"bits": bits, "N": n, "K": k, "M": m, "us": round(us, 1), "tflops": round(tf, 1),
                       "frac_burst_peak": round(tf / burst, 3) if burst else None, "copies": copies}
                if m <= 16:   # weight-streaming kernel: HBM-bound, report bytes per second as well
                    gbs = (n * k * bits // 8 + n * (k // 64) * 4 + 2 * m * k + 2 * m * n) / us / 1e3
                    row.update({"gbs": round(gbs, 1), "frac_hbm_peak": round(gbs / hbm, 3) if hbm else None})
                rows.append(row)
                del preps, xs, ys
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="flux", choices=["flux", "zimage", "qwen", "sweep", "lora"])
    ap.add_argument("--small", action="store_true", help="flux at reduced depth, lora with one case and few launches: for profiler captures (not a bench value)")
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (default: the workload's own)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--qwen-parallel", default="cfg+tp", choices=["cfg+tp", "tp"],
                    help="qwen on N > 1 GPUs: split the two guidance branches over the halves of the ranks and use "
                         "tensor parallelism inside each half (default), or tensor parallelism over all ranks")
    ap.add_argument("--qwen-tp-mode", default="peer", choices=["peer", "nccl"],
                    help="qwen tensor parallelism: reduce-scatter / all-gather fused into this library's kernels over "
                         "peer-mapped memory (default), or NCCL all-reduces beside the matmuls")
    ap.add_argument("--lora-rank", type=int, default=0,
                    help="flux: wrap every attention / feed-forward linear with one LoRA adapter of this rank")
    ap.add_argument("--lora-library", action="store_true",
                    help="with --lora-rank: run the adapters as library GEMMs instead of inside the quantized matmul")
    ap.add_argument("--breakdown", action="store_true",
                    help="add per-shape kernel times (from the per-launch event pairs) to the JSON line")
    ap.add_argument("--no-extra", action="store_true",
                    help="flux: skip the two extra records (the 16-image batch split over the ranks, and the "
                         "Qwen-Image-shaped tensor-parallel step)")
    ap.add_argument("--no-cuda-graph", action="store_true",
                    help="qwen: issue the step's launches one by one instead of replaying them as a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use every core,
        # at every N, so say so before NumPy's BLAS is loaded
        for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
            os.environ[var] = str(os.cpu_count() or 1)

    if args.workload in ("sweep", "lora"):
        spec = None
    else:
        spec = SPECS[args.workload](args)
        if args.impl == "reference":
            run_reference(args, spec)
            return

    import math

    # The few NCCL collectives of a step (one all-gather per pass) do not need the in-switch reduction, and every
    # number of the tensor-parallel path was measured with it off; a caller's own setting wins.
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

    import torch
    import torch.distributed as dist

    from mflux_b200 import ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)

    if args.workload == "lora":
        if rank == 0:
            sampler = ClockSampler(local)
            sampler.start()
            rows = run_lora(args, dev)
            clocks = sampler.stop()
            print(json.dumps({
                "metric": "lora_over_qlinear_time_ratio", "value": rows[0]["fused_over_base"],
                "unit": "time of the first wrapped case (4 bits, rank 16; rank 64 with --small) / time of the frozen layer", "n_gpus": 1, "steps": 1,
                "warmup": max(3, args.warmup), "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "LoRA adapters over one quantized linear, M 4096 N 12288 K 3072, group 64",
                           "l2_policy": "four operand sets rotated (0.6 GB between reuses)",
                           "device_status": ops.poll_device_status()},
                "clocks": clocks, "lora": rows}), flush=True)
        return

    if spec is None:   # single-GPU table of quantized linears
        if rank == 0:
            sampler = ClockSampler(local)
            sampler.start()
            rows = run_sweep(args, dev)
            clocks = sampler.stop()
            peak, _, burst = measured_peaks()
            big = [r for r in rows if r["M"] > 16]
            geo = math.exp(sum(math.log(r["tflops"]) for r in big) / len(big))
            print(json.dumps({
                "metric": "qlinear_sweep_geomean_tflops", "value": geo, "unit": "TFLOP/s", "n_gpus": 1, "steps": 1,
                "warmup": max(3, args.warmup), "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "quantized-linear sweep, bits {4,8} x (N,K) x M, group 64, bias, bf16 out",
                           "l2_policy": "operand copies rotated so that more than 400 MB pass between reuses",
                           "burst_peak_tflops": burst, "device_status": ops.poll_device_status()},
                "clocks": clocks, "sweep": rows}), flush=True)
        return

    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    host_in, out_h, step = spec["build"](dev, rank, world, args.steps + args.warmup)
    dev_in = [t.to(dev) for t in host_in]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i, *dev_in)
    barrier()

    sampler = ClockSampler(local)
    sampler.start()
    ops.TRACE = {}
    launches0 = ops.LAUNCHES[0]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    cur = dev_in[0]
    for i in range(args.steps):
        cur = step(i, cur, *dev_in[1:])
    e1.record()
    barrier()
    launches = ops.LAUNCHES[0] - launches0
    trace, ops.TRACE = ops.TRACE, None
    ms = e0.elapsed_time(e1)

    # end to end through the public call with host buffers: pinned H2D of the step's inputs, D2H of its result
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(args.steps):
        res = step(i, *[t.to(dev, non_blocking=True) for t in host_in])
        out_h.copy_(res, non_blocking=True)
    t1.record()
    barrier()
    ms_e2e = t0.elapsed_time(t1)
    clocks = sampler.stop()
    trace_steps = args.steps
    if not trace and hasattr(step, "eager"):
        # a replayed graph has no per-launch events: time the kernels on launch-by-launch passes
        trace_steps = min(2, args.steps)
        ops.TRACE = {}
        for i in range(trace_steps):
            step.eager(i, *dev_in)
        barrier()
        trace, ops.TRACE = ops.TRACE, None
    status = ops.poll_device_status()

    def timed(fn, steps, warm):
        """max-over-ranks device milliseconds per step of fn(i), after `warm` untimed steps."""
        for i in range(warm):
            fn(i)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            fn(i)
        b.record()
        barrier()
        t = torch.tensor([a.elapsed_time(b) / steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    extras = {}
    if args.workload == "flux" and not args.small and not args.no_extra and not args.lora_rank and not args.batch \
            and 16 % world == 0:
        # (1) strong scaling of the headline step: the SAME 16 images split over the ranks, no collective
        shard_in = step.shard(16)
        ms_strong = timed(lambda i: step(i, *shard_in), 3, 2)
        extras["strong"] = {"metric": "flux1_w4_dit_16_image_steps_per_sec_1024px_split_over_gpus",
                            "value": 1e3 / ms_strong, "unit": "steps/s (one step = the same 16 images, 16 / N per GPU)",
                            "ms_per_step": ms_strong, "n_gpus": world, "per_gpu_batch": 16 // world,
                            "scaling": "strong"}
        del shard_in
        # (2) the part of the path that communicates: the Qwen-Image-shaped 20B step, its two guidance branches on
        # the two halves of the ranks and tensor parallelism inside each half (one rank: both branches as a batch)
        if world in (1, 2, 4, 8):
            import gc

            host_in_main, step_main = host_in, step
            del dev_in, cur, res
            step = None
            gc.collect()
            torch.cuda.empty_cache()
            qspec = qwen_spec(args)
            q_host, _, q_step = qspec["build"](dev, rank, world, 8)
            q_dev = [t.to(dev) for t in q_host]
            ms_tp = timed(lambda i: q_step(i, *q_dev), 4, 3)
            q_status = ops.poll_device_status()
            extras["tp"] = {"metric": qspec["metric"], "value": 1e3 / ms_tp, "unit": qspec["unit"],
                            "ms_per_step": ms_tp, "n_gpus": world, "scaling": "strong",
                            "workload": qspec["workload"], "exchange": args.qwen_tp_mode if world > 2 else None,
                            "algorithmic_tflop_per_step": (qspec["lin"] + qspec["attn"]) / 1e12,
                            "device_status": q_status}
            getattr(q_step, "release", lambda: None)()
            del q_step, q_dev
            host_in, step = host_in_main, step_main

    times = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(times[0]), float(times[1])

    if rank == 0:
        units = world if spec["scaling"] == "weak" else 1   # weak: every rank finishes its own steps
        value = units * args.steps / (ms / 1e3)
        e2e_value = units * args.steps / (ms_e2e / 1e3)
        def totals(kind):
            rows = trace.get(kind, [])
            return (sum(t[0] for t in rows), sum(t[1] for t in rows), sum(t[2].elapsed_time(t[3]) for t in rows),
                    len(rows))

        q_flops, _, q_ms, q_n = totals("qlinear")
        a_flops, _, a_ms, a_n = totals("fmha")
        _, g_bytes, g_ms, g_n = totals("glue")
        peak, peak_kind, burst = measured_peaks()
        achieved = q_flops / (q_ms / 1e3) / 1e12 if q_ms > 0 else 0.0
        a_achieved = a_flops / (a_ms / 1e3) / 1e12 if a_ms > 0 else 0.0
        g_achieved = g_bytes / (g_ms / 1e3) / 1e9 if g_ms > 0 else 0.0
        hbm = measured_hbm()
        sm_mhz = clocks.get("sm_mhz")
        step_ms = ms / args.steps
        flops = spec["lin"] + spec["attn"]
        traffic = recorded_traffic() if (args.workload == "flux" and not args.small and
                                         spec["per_gpu_batch"] == 16) else None
        line = {
            "metric": spec["metric"], "value": value, "unit": spec["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": spec["scaling"], "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": spec["workload"], "per_gpu_batch": spec["per_gpu_batch"],
                       "l2_policy": spec["l2_policy"], "algorithmic_tflop_per_step": flops / 1e12,
                       "device_status": status, "small": bool(args.small)},
            "e2e": {"value": e2e_value, "unit": spec["unit"],
                    "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host_in),
                    "d2h_bytes_per_step": out_h.numel() * out_h.element_size()},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "qmm_kernel (quantized linear)", "achieved": achieved,
                         "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if peak else None,
                         "peak_kind": peak_kind, "burst_peak": burst,
                         "frac_of_burst": achieved / burst if burst else None,
                         "tflops_per_sm_mhz": achieved / sm_mhz if sm_mhz else None, "launches": q_n,
                         "share_of_step_time": (q_ms / trace_steps) / step_ms if ms > 0 else None, "traffic": traffic,
                         "traffic_unit": "DRAM bytes per launch, mean over the step's launches (ncu record under "
                                         "profiles/, null when the kernel source changed since the capture)"},
            "roofline_attention": {"bound": "tensor", "kernel": "attn::sdpa_pingpong_kernel / attn::sdpa_pair_kernel (flash attention, head dim 128)",
                                   "achieved": a_achieved, "peak": peak, "unit": "TFLOP/s",
                                   "frac": a_achieved / peak if peak else None, "peak_kind": peak_kind,
                                   "burst_peak": burst, "frac_of_burst": a_achieved / burst if burst else None,
                                   "launches": a_n,
                                   "share_of_step_time": (a_ms / trace_steps) / step_ms if ms > 0 else None},
            "roofline_glue": {"bound": "hbm", "kernel": "norm / modulate / qk-norm + RoPE / gated-residual kernels",
                              "achieved": g_achieved, "peak": hbm, "unit": "GB/s",
                              "frac": g_achieved / hbm if hbm else None, "peak_kind": "measured copy bandwidth",
                              "launches": g_n,
                              "share_of_step_time": (g_ms / trace_steps) / step_ms if ms > 0 else None},
            "step_tflops": flops / 1e12 * args.steps / (ms / 1e3) / (world if spec["scaling"] == "strong" else 1),
        }
        line.update(extras)
        if args.breakdown:
            groups = {}
            for kind, rows_ in trace.items():
                for t in rows_:
                    g_ = groups.setdefault((kind, round(t[0]), round(t[1])), [0, 0.0])
                    g_[0] += 1
                    g_[1] += t[2].elapsed_time(t[3])
            line["breakdown"] = sorted(
                ({"kind": k[0], "flop": k[1], "bytes": k[2], "launches": v[0], "ms_total": round(v[1], 3),
                  "us_avg": round(1e3 * v[1] / v[0], 1)} for k, v in groups.items()), key=lambda r: -r["ms_total"])
        if not args.no_cpu_baseline and world == 1:
            tf, desc, cores, threads = cpu_sample()
            line["cpu_baseline"] = {"value": tf * 1e12 / flops, "unit": spec["unit"], "cores": cores,
                                    "threads": threads, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    getattr(step, "release", lambda: None)()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
