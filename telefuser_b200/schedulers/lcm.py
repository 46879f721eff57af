"""Consistency-style few-step sampler: predict x0 from the velocity, then re-noise to the next sigma.

The N sampling points are taken every `T // N` entries of the shifted T-point sigma table
(sigma' = s*sigma / (1 + (s-1)*sigma)). A step computes x0 = x - sigma * v and, except at the last step,
returns (1 - sigma_next) * x0 + sigma_next * noise with noise drawn from the scheduler's own seeded generator.
Role parity: telefuser/schedulers/lcm.py:13-81.
"""

from __future__ import annotations

import torch


class LCMScheduler:
    def __init__(self, num_train_timesteps: int = 1000, shift: float = 1.0) -> None:
        self.num_train_timesteps, self.shift = num_train_timesteps, shift
        self.sigma_max, self.sigma_min = 1.0, 0.0

    def set_timesteps(self, num_inference_steps: int, device="cpu", shift: float | None = None, seed: int | None = None):
        shift = self.shift if shift is None else shift
        self.generator = torch.Generator(device=device)
        if seed is not None:
            self.generator.manual_seed(seed)
        T = self.num_train_timesteps
        stride = T // num_inference_steps
        self.denoising_step_list = [T - i * stride for i in range(num_inference_steps)]
        self.num_inference_steps, self.device = num_inference_steps, device
        table = torch.linspace(self.sigma_max, self.sigma_min, T + 1)[:-1]
        table = shift * table / (1 + (shift - 1) * table)
        index = [T - x for x in self.denoising_step_list]
        self.sigmas = table[index]
        self.timesteps = (table * T)[index].to(device)

    @staticmethod
    def add_noise(original_samples, noise, sigma):
        return ((1 - sigma) * original_samples + sigma * noise).type_as(noise)

    def step(self, model_output, timestep, sample):
        t = timestep.cpu() if isinstance(timestep, torch.Tensor) else timestep
        i = int(torch.argmin((self.timesteps.cpu() - t).abs()))
        x0 = sample - float(self.sigmas[i]) * model_output
        if i < self.num_inference_steps - 1:
            noise = torch.randn(x0.shape, dtype=torch.float32, device=self.device, generator=self.generator)
            x0 = self.add_noise(x0, noise, float(self.sigmas[i + 1]))
        return x0
