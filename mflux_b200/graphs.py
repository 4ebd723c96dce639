"""CUDA-graph replay of a denoiser evaluation.

A tensor-parallel step is a few thousand short launches and collectives. `CapturedStep` records the launches of
one call (this library's kernels, torch's own and NCCL's collectives alike -- all of them are stream work) into a
CUDA graph and replays it with new inputs copied into the recorded input buffers, which takes the per-launch host
work out of the step. Measured on the Qwen-Image-shaped step the gain is small, 2.5 % on two and 1.5 % on four
tensor-parallel B200s: those steps are bound by the GPUs, not by the host; eight ranks were not measured. Everything that changes between denoising steps therefore has to arrive
as a tensor (the noise level is a one-element tensor, not a Python float); shapes, guidance scale and image size
are part of the recorded graph, one graph per distinct set of input shapes.

The reference gets the same effect from MLX's lazy evaluation, which builds the step's graph before running it.
"""
from __future__ import annotations

from typing import Callable

import torch

from . import ops


class CapturedStep:
    """`step = CapturedStep(fn)`; `step(*tensors)` returns what `fn(*tensors)` returns (a tensor or a tuple of
    tensors). The returned tensors are the graph's own output buffers: the next call overwrites them.

    `fn` must be free of host synchronisation and of data-dependent control flow, and every process of a
    process group used inside `fn` has to call the step the same number of times (the warm-up calls and the
    capture run the collectives for real / record them on every rank alike)."""

    def __init__(self, fn: Callable, warmup: int = 2):
        self.fn, self.warmup = fn, warmup
        self._entries: dict = {}

    def __call__(self, *tensors: torch.Tensor):
        key = tuple((tuple(t.shape), t.dtype, str(t.device)) for t in tensors)
        entry = self._entries.get(key)
        if entry is None:
            entry = self._entries[key] = self._capture(tensors)
        static_in, graph, out, launches = entry
        for s, t in zip(static_in, tensors):
            s.copy_(t, non_blocking=True)
        graph.replay()
        ops.LAUNCHES[0] += launches   # the replay runs every recorded kernel of this library again
        return out

    def _capture(self, tensors):
        if not tensors or not all(t.is_cuda for t in tensors):
            raise ValueError("CapturedStep needs CUDA tensors as inputs")
        static_in = [t.clone() for t in tensors]
        current = torch.cuda.current_stream()
        side = torch.cuda.Stream(device=tensors[0].device)
        side.wait_stream(current)
        with torch.cuda.stream(side):   # lazy initialisation (prepared weights, workspaces, communicators)
            for _ in range(self.warmup):
                self.fn(*static_in)
        current.wait_stream(side)
        torch.cuda.synchronize(tensors[0].device)
        graph = torch.cuda.CUDAGraph()
        # thread-local: another thread of the process (NCCL's watchdog polling its events) must not end the capture
        before = ops.LAUNCHES[0]
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            out = self.fn(*static_in)
        launches = ops.LAUNCHES[0] - before
        ops.LAUNCHES[0] = before        # recording launched nothing
        return static_in, graph, out, launches

    def release(self) -> None:
        """Destroys the recorded graphs. A graph that holds NCCL collectives keeps its communicator busy:
        `destroy_process_group` waits for ever while one is alive, so release before tearing the group down."""
        import gc

        devices = {e[0][0].device for e in self._entries.values()}
        for dev in devices:
            torch.cuda.synchronize(dev)
        self._entries.clear()
        gc.collect()

    @property
    def captured_shapes(self):
        return list(self._entries)
