"""Sigma schedule and Euler step of the denoise loop (host arithmetic, float32).

LinearScheduler follows src/mflux/models/common/schedulers/linear_scheduler.py:25-58: sigmas =
linspace(1, 1/steps, steps) + [0]; with `requires_sigma_shift` they are shifted by
exp(mu) / (exp(mu) + (1/sigma - 1)) with mu linear in the image sequence length
(width * height / 256) between (base_seq_len, base_shift) and (max_seq_len, max_shift).
step(): latents + noise * (sigma[t+1] - sigma[t]).
"""
from __future__ import annotations

import math

import numpy as np


class LinearScheduler:
    def __init__(self, num_inference_steps: int, width: int = 1024, height: int = 1024,
                 requires_sigma_shift: bool = True, base_shift: float = 0.5, max_shift: float = 1.15,
                 base_seq_len: int = 256, max_seq_len: int = 4096, shift_terminal: float | None = None):
        n = num_inference_steps
        sig = np.linspace(1.0, 1.0 / n, n).astype(np.float32)
        if requires_sigma_shift:
            m = (max_shift - base_shift) / (max_seq_len - base_seq_len)
            b = base_shift - m * base_seq_len
            mu = np.float32(m * width * height / 256 + b)
            e = np.exp(mu, dtype=np.float32)
            sig = (e / (e + (np.float32(1.0) / sig - np.float32(1.0)))).astype(np.float32)
            if shift_terminal is not None:
                one_minus = np.float32(1.0) - sig
                scale = one_minus[-1] / np.float32(1.0 - shift_terminal)
                sig = (np.float32(1.0) - one_minus / scale).astype(np.float32)
        self.sigmas = np.concatenate([sig, np.zeros(1, np.float32)]).astype(np.float32)
        self.timesteps = np.arange(n, dtype=np.float32)

    def dt(self, t: int) -> float:
        return float(self.sigmas[t + 1] - self.sigmas[t])

    def step(self, noise, t: int, latents):
        """Euler step on torch tensors: latents + noise * (sigma[t+1] - sigma[t]) in the latents' dtype."""
        return latents + noise.to(latents.dtype) * self.dt(t)
