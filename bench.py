"""Benchmark of the quantized DiT denoising step: FLUX.1-shaped 12B MMDiT, W4 group 64, 1024x1024.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--small]

One process per GPU (torchrun for N > 1). A step is one denoiser evaluation plus the Euler update for a
batch of 16 images (4096 image + 512 text tokens each) on synthetic inputs with random-init weights.
The batch is the unit that shards: every rank runs its own 16-image batch with replicated weights and no
collective on the data path (weak scaling); `value` = steps all ranks completed / max-over-ranks device
time. Rank 0 prints one JSON line.

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

METRIC = "flux1_w4_dit_steps_per_sec_1024px_batch16"
UNIT = "steps/s (one step = 16 images x 4608 tokens through 19+38 blocks)"


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


def cpu_sample(seconds_target: float = 12.0):
    """Times the CPU oracle (dequantize + float32 matmul on all host cores) on a bounded sample: quantized
    linears of the step's dominant shape. Returns (TFLOP/s, description, cores)."""
    import numpy as np

    from oracle import quant

    cores = os.cpu_count() or 1
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
    return 2.0 * m * n * k / dt / 1e12, desc, cores


def run_reference(args, cfg, batch, si, st):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    lin, attn = step_flops(cfg, batch, si, st)
    vals = []
    desc, cores = "", 1
    for i in range(args.warmup + args.steps):
        tf, desc, cores = cpu_sample(seconds_target=max(2.0, 20.0 / max(1, args.steps + args.warmup)))
        if i >= args.warmup:
            vals.append(tf)
    tflops = sum(vals) / len(vals)
    value = tflops * 1e12 / (lin + attn)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / value, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(cfg, batch, si, st), "note": "CPU oracle port of the MLX arithmetic; "
                   "MLX itself is not installable offline"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_name(cfg, batch, si, st):
    return (f"FLUX.1-shaped MMDiT {cfg.num_joint}+{cfg.num_single} blocks, hidden {cfg.hidden}, {cfg.heads}x128 heads, "
            f"W4 g64, batch {batch}, {si} image + {st} text tokens, guidance-embedded, CFG-free")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--small", action="store_true", help="reduced model for profiler captures (not a bench value)")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    from mflux_b200.flux import FluxConfig

    if args.small:
        cfg = FluxConfig(num_joint=1, num_single=1)
        batch = min(args.batch, 2)
    else:
        cfg = FluxConfig()
        batch = args.batch
    height = width = 1024
    si, st = (height // 16) * (width // 16), 512

    if args.impl == "reference":
        run_reference(args, cfg, batch, si, st)
        return

    import torch
    import torch.distributed as dist

    from mflux_b200 import ops
    from mflux_b200.flux import Transformer
    from mflux_b200.schedulers import LinearScheduler

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    model = Transformer(cfg, bits=4, device=dev, seed=1234)  # same weights on every rank (replicated)
    g = torch.Generator(device="cpu").manual_seed(100 + rank)  # every rank has its own batch of images
    lat_h = torch.randn(batch, si, cfg.in_channels, generator=g).pin_memory()
    ctx_h = torch.randn(batch, st, cfg.context_dim, generator=g).to(torch.bfloat16).pin_memory()
    pool_h = torch.randn(batch, cfg.pooled_dim, generator=g).to(torch.bfloat16).pin_memory()
    out_h = torch.empty(batch, si, cfg.in_channels).pin_memory()
    sched = LinearScheduler(max(args.steps + args.warmup, 2), width, height, True)
    gvec = torch.full((batch,), 3.5 * cfg.num_train_steps, device=dev)
    lat, ctx, pool = lat_h.to(dev), ctx_h.to(dev), pool_h.to(dev)

    def step(i, lat_d, ctx_d, pool_d):
        ts = torch.full((batch,), float(sched.sigmas[i % len(sched.timesteps)]) * cfg.num_train_steps, device=dev)
        noise = model(lat_d, ctx_d, pool_d, ts, gvec, height, width)
        return ops.euler_step(lat_d, noise, sched.dt(i % len(sched.timesteps)))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i, lat, ctx, pool)
    barrier()

    sampler = ClockSampler(local)
    sampler.start()
    ops.QLINEAR_TRACE = []
    launches0 = ops.LAUNCHES[0]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    cur = lat
    for i in range(args.steps):
        cur = step(i, cur, ctx, pool)
    e1.record()
    barrier()
    launches = ops.LAUNCHES[0] - launches0
    trace, ops.QLINEAR_TRACE = ops.QLINEAR_TRACE, None
    ms = e0.elapsed_time(e1)

    # end to end through the public call with host buffers: pinned H2D of the step's inputs, D2H of its result
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(args.steps):
        lat_d = lat_h.to(dev, non_blocking=True)
        ctx_d = ctx_h.to(dev, non_blocking=True)
        pool_d = pool_h.to(dev, non_blocking=True)
        res = step(i, lat_d, ctx_d, pool_d)
        out_h.copy_(res, non_blocking=True)
    t1.record()
    barrier()
    ms_e2e = t0.elapsed_time(t1)
    clocks = sampler.stop()
    status = ops.poll_device_status()

    times = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(times[0]), float(times[1])

    if rank == 0:
        value = world * args.steps / (ms / 1e3)
        e2e_value = world * args.steps / (ms_e2e / 1e3)
        q_flops = sum(t[0] for t in trace)
        q_ms = sum(t[1].elapsed_time(t[2]) for t in trace)
        peak, peak_kind, burst = measured_peaks()
        achieved = q_flops / (q_ms / 1e3) / 1e12 if q_ms > 0 else 0.0
        lin, attn = step_flops(cfg, batch, si, st)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(cfg, batch, si, st), "per_gpu_batch": batch,
                       "l2_policy": "inputs larger than L2 (6.7 GB of packed weights stream every step)",
                       "algorithmic_tflop_per_step": (lin + attn) / 1e12, "device_status": status,
                       "small": bool(args.small)},
            "e2e": {"value": e2e_value, "unit": UNIT,
                    "h2d_bytes_per_step": lat_h.numel() * 4 + ctx_h.numel() * 2 + pool_h.numel() * 2,
                    "d2h_bytes_per_step": out_h.numel() * 4},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "qmm_kernel (quantized linear)", "achieved": achieved,
                         "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if peak else None,
                         "peak_kind": peak_kind, "burst_peak": burst, "launches": len(trace),
                         "share_of_step_time": q_ms / ms if ms > 0 else None, "traffic": None},
            "step_tflops": (lin + attn) / 1e12 * args.steps / (ms / 1e3),
        }
        if not args.no_cpu_baseline:
            tf, desc, cores = cpu_sample()
            line["cpu_baseline"] = {"value": tf * 1e12 / (lin + attn), "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
