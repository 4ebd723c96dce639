"""World-size-2 gloo test (CPU) of the host-side multi-GPU logic: shard plan, max-over-ranks timing,
latent gather, and the reference arm printing on rank 0 only."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mflux_b200 import sharding

ROOT = Path(__file__).resolve().parent.parent


def test_shard_ranges_cover_batch():
    for total in (0, 1, 2, 15, 16, 17):
        for world in (1, 2, 4, 8):
            spans = [sharding.shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    a, b = sharding.shard_range(5, world, rank)
    local = torch.arange(a, b, dtype=torch.float32)[:, None].repeat(1, 3)
    t = sharding.max_over_ranks(10.0 + rank)
    full = sharding.gather_latents(local, 5)
    q.put((rank, t, None if full is None else full[:, 0].tolist()))
    dist.destroy_process_group()


def test_two_rank_gloo_timing_and_gather():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29731, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert got[0] == (0, 11.0, [0.0, 1.0, 2.0, 3.0, 4.0])
    assert got[1] == (1, 11.0, None)


def test_reference_arm_prints_on_rank0_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                        "--warmup", "0"], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""
