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


class FlowMatchEulerDiscreteScheduler:
    """Host arithmetic of src/mflux/models/common/schedulers/flow_match_euler_discrete_scheduler.py.

    Default schedule (:99-120): `steps` timesteps spaced linearly from 1000 down to 1, sigma = t / 1000 shifted by
    e / (e + (1/sigma - 1)) (mu = 1), then stretched so that the last sigma equals shift_terminal = 0.02; a final 0
    is appended. `set_image_seq_len` (:37-41,63-76) replaces it by linspace(1, 1/steps) shifted with the empirical
    mu of the image sequence length (:78-88); `set_mu` (:43-49) does the same with a given mu. step() is the same
    Euler update as the linear scheduler (:13-17,122-124).
    """

    def __init__(self, num_inference_steps: int, num_train_timesteps: int = 1000, shift_terminal: float = 0.02):
        self.num_inference_steps = num_inference_steps
        self.num_train_timesteps = num_train_timesteps
        self.shift_terminal = shift_terminal
        n, nt = num_inference_steps, num_train_timesteps
        sigma_min, sigma_max = 1.0 / nt, 1.0
        t_lin = [sigma_max * nt - i * (sigma_max - sigma_min) * nt / max(n - 1, 1) for i in range(n)]
        shifted = [self._time_shift(1.0, 1.0, t / nt) for t in t_lin]
        one_minus = [1.0 - s for s in shifted]
        scale = one_minus[-1] / (1.0 - shift_terminal)
        final = [1.0 - om / scale for om in one_minus]
        self.sigmas = np.asarray(final + [0.0], dtype=np.float32)
        self.timesteps = np.asarray([s * nt for s in final], dtype=np.float32)

    @staticmethod
    def _time_shift(mu: float, sigma_power: float, t: float) -> float:
        return math.exp(mu) / (math.exp(mu) + ((1.0 / t - 1.0) ** sigma_power))

    @staticmethod
    def compute_linear_mu(image_seq_len: int, base_seq_len: int = 256, max_seq_len: int = 4096,
                          base_shift: float = 0.5, max_shift: float = 1.15) -> float:
        m = (max_shift - base_shift) / (max_seq_len - base_seq_len)
        return float(m * image_seq_len + (base_shift - m * base_seq_len))

    @staticmethod
    def compute_empirical_mu(image_seq_len: int, num_steps: int) -> float:
        a1, b1 = 8.73809524e-05, 1.89833333
        a2, b2 = 0.00016927, 0.45666666
        if image_seq_len > 4300:
            return float(a2 * image_seq_len + b2)
        m_200 = a2 * image_seq_len + b2
        m_10 = a1 * image_seq_len + b1
        a = (m_200 - m_10) / 190.0
        b = m_200 - 200.0 * a
        return float(a * num_steps + b)

    def set_mu(self, mu: float) -> None:
        n = self.num_inference_steps
        sig = np.linspace(1.0, 1.0 / n, n).astype(np.float32)
        e = np.exp(np.float32(mu), dtype=np.float32)
        sig = (e / (e + (np.float32(1.0) / sig - np.float32(1.0)))).astype(np.float32)
        self.timesteps = (sig * np.float32(self.num_train_timesteps)).astype(np.float32)
        self.sigmas = np.concatenate([sig, np.zeros(1, np.float32)]).astype(np.float32)

    def set_image_seq_len(self, image_seq_len: int) -> None:
        self.set_mu(self.compute_empirical_mu(image_seq_len, self.num_inference_steps))

    def dt(self, t: int) -> float:
        return float(self.sigmas[t + 1] - self.sigmas[t])

    def step(self, noise, t: int, latents):
        return latents + noise.to(latents.dtype) * self.dt(t)

    def scale_model_input(self, latents, t: int):
        return latents
