"""Discrete flow-matching Euler scheduler with stateful step index (HunyuanVideo super-resolution, Z-Image).

Sigmas run from 1 to 0 over `num_inference_steps + 1` points and are warped either by the token-count
dependent exponential shift (mu linear in the number of tokens between two anchor points) or by the
constant shift s*t / (1 + (s-1)*t). `step` advances an internal index, so one scheduler serves one
trajectory at a time; `set_timesteps` resets it. `set_timesteps_mu` builds the N-point variant used by
Z-Image (linspace(1, sigma_min, N), exponential shift with a given mu, terminal 0 appended).
Role parity: telefuser/schedulers/flow_match_discrete.py:50-325.
"""

from __future__ import annotations

import math
from types import SimpleNamespace

import torch


def linear_mu(n_tokens: float, x1: float = 256, y1: float = 0.5, x2: float = 4096, y2: float = 1.15) -> float:
    m = (y2 - y1) / (x2 - x1)
    return m * n_tokens + (y1 - m * x1)


def exponential_shift(mu: float, t: torch.Tensor, power: float = 1.0) -> torch.Tensor:
    return math.exp(mu) / (math.exp(mu) + (1 / t - 1) ** power)


def constant_shift(t: torch.Tensor, shift: float) -> torch.Tensor:
    return (shift * t) / (1 + (shift - 1) * t)


class FlowMatchDiscreteScheduler:
    def __init__(self, num_train_timesteps: int = 1000, shift: float = 1.0, reverse: bool = True, solver: str = "euler",
                 use_flux_shift: bool = False, flux_base_shift: float = 0.5, flux_max_shift: float = 1.15,
                 n_tokens: int | None = None, flux_base_token: float = 256.0, flux_max_token: float = 4096.0,
                 flux_shift_factor: float = 1.0) -> None:  # fmt: skip
        if solver != "euler":
            raise ValueError(f"Solver {solver} not supported. Supported solvers: ['euler']")
        self.config = SimpleNamespace(num_train_timesteps=num_train_timesteps, shift=shift, reverse=reverse, solver=solver,
                                      use_flux_shift=use_flux_shift, flux_base_shift=flux_base_shift,
                                      flux_max_shift=flux_max_shift, flux_base_token=flux_base_token,
                                      flux_max_token=flux_max_token, flux_shift_factor=flux_shift_factor)  # fmt: skip
        sigmas = torch.linspace(1, 0, num_train_timesteps + 1)
        self.sigmas = sigmas if reverse else sigmas.flip(0)
        self.timesteps = (self.sigmas[:-1] * num_train_timesteps).float()
        self.sigma_min = 0.0
        self._step_index = None
        self._begin_index = None

    @classmethod
    def from_config(cls, config: dict) -> "FlowMatchDiscreteScheduler":
        import inspect

        known = set(inspect.signature(cls.__init__).parameters) - {"self"}
        return cls(**{k: v for k, v in config.items() if k in known})

    @property
    def step_index(self):
        return self._step_index

    @property
    def begin_index(self):
        return self._begin_index

    def set_begin_index(self, begin_index: int = 0) -> None:
        self._begin_index = begin_index

    def set_timesteps(self, num_inference_steps: int, device=None, n_tokens: int | None = None, shift: float | None = None):
        c = self.config
        self.num_inference_steps = num_inference_steps
        sigmas = torch.linspace(1, 0, num_inference_steps + 1)
        if c.use_flux_shift and n_tokens is not None:
            mu = linear_mu(n_tokens, c.flux_base_token, c.flux_base_shift * c.flux_shift_factor, c.flux_max_token,
                           c.flux_max_shift * c.flux_shift_factor)  # fmt: skip
            sigmas = exponential_shift(mu, sigmas)
        elif shift is not None and shift != 1.0:
            sigmas = constant_shift(sigmas, shift)
        elif c.shift != 1.0:
            sigmas = constant_shift(sigmas, c.shift)
        if not c.reverse:
            sigmas = 1 - sigmas
        self.sigmas = sigmas
        self.timesteps = (sigmas[:-1] * c.num_train_timesteps).to(dtype=torch.float32, device=device)
        self._step_index = None

    def set_timesteps_mu(self, num_inference_steps: int, mu: float, device=None) -> None:
        """N sigmas from 1 to `sigma_min`, exponentially shifted by mu, plus the terminal 0."""
        s = torch.linspace(1.0, float(self.sigma_min), num_inference_steps, dtype=torch.float64)
        shifted = torch.where(s > 0, exponential_shift(mu, s.clamp_min(1e-12)), torch.zeros_like(s)).float()
        self.num_inference_steps = num_inference_steps
        self.sigmas = torch.cat([shifted, shifted.new_zeros(1)])
        self.timesteps = (shifted * self.config.num_train_timesteps).to(device=device)
        self._step_index = None

    def index_for_timestep(self, timestep, schedule_timesteps=None) -> int:
        ts = self.timesteps if schedule_timesteps is None else schedule_timesteps
        idx = (ts == timestep).nonzero()
        if len(idx) == 0:
            return int(torch.argmin((ts - timestep).abs()))
        return int(idx[1 if len(idx) > 1 else 0])

    def scale_model_input(self, sample, timestep=None):
        return sample

    def step(self, model_output, timestep, sample, generator=None, n_tokens=None, return_dict: bool = True):
        if isinstance(timestep, int) or (isinstance(timestep, torch.Tensor) and not timestep.is_floating_point()):
            raise ValueError("pass one of scheduler.timesteps, not an integer index")
        if self._step_index is None:
            if self._begin_index is not None:
                self._step_index = self._begin_index
            else:
                t = timestep.to(self.timesteps.device) if isinstance(timestep, torch.Tensor) else timestep
                self._step_index = self.index_for_timestep(t)
        dt = float(self.sigmas[self._step_index + 1] - self.sigmas[self._step_index])
        prev = sample.float() + model_output.float() * dt
        self._step_index += 1
        return SimpleNamespace(prev_sample=prev) if return_dict else (prev,)

    def __len__(self) -> int:
        return self.config.num_train_timesteps
