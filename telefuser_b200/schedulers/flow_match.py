"""Flow-matching (rectified-flow) schedulers.

Sigma schedules for the model families the framework serves, an Euler step,
noising and the training target. Behaviour matches the reference's
``telefuser/schedulers/flow_match.py:22-377``; the structure differs: schedules
are plain functions in a registry (`SIGMA_SCHEDULES`) returning
``(sigmas, timesteps)``, and the Euler update can run fused with classifier-free
guidance through ``ops.functional.cfg_euler_step`` (see ``step_with_guidance``).
"""

from __future__ import annotations

import math
from typing import Callable

import torch

NUM_TRAIN_TIMESTEPS = 1000


def _time_shift(sigmas: torch.Tensor, shift: float) -> torch.Tensor:
    return shift * sigmas / (1 + (shift - 1) * sigmas)


def _exp_shift(sigmas: torch.Tensor, mu: float) -> torch.Tensor:
    e = math.exp(mu)
    return e / (e + (1 / sigmas - 1))


def _descending(start: float, end: float, n: int, drop_last: bool) -> torch.Tensor:
    return torch.linspace(start, end, n + 1)[:-1] if drop_last else torch.linspace(start, end, n)


def schedule_flux(num_inference_steps=100, denoising_strength=1.0, shift=None):
    lo = 0.003 / 1.002
    s = _descending(lo + (1.0 - lo) * denoising_strength, lo, num_inference_steps, drop_last=False)
    s = _time_shift(s, 3 if shift is None else shift)
    return s, s * NUM_TRAIN_TIMESTEPS


def schedule_wan(num_inference_steps=100, denoising_strength=1.0, shift=None):
    """sigma = linspace(1, 0, N+1)[:-1], shifted by s*sigma / (1 + (s-1)*sigma); t = 1000*sigma."""
    s = _descending(denoising_strength, 0.0, num_inference_steps, drop_last=True)
    s = _time_shift(s, 5 if shift is None else shift)
    return s, s * NUM_TRAIN_TIMESTEPS


def merge_by_threshold(a: torch.Tensor, b: torch.Tensor, threshold: float) -> torch.Tensor:
    """Entries of `a` at or above the threshold followed by entries of `b` below it."""
    return torch.cat((a[a >= threshold], b[b < threshold]))


def schedule_wan_mix(num_inference_steps, shift=None, boundary=0.9, denoising_strength=1.0,
                     num_train_timesteps=NUM_TRAIN_TIMESTEPS):  # fmt: skip
    """Two Wan schedules (high-noise / low-noise expert) joined at `boundary`."""
    s1, t1 = schedule_wan(num_inference_steps[0], denoising_strength, shift[0])
    s2, t2 = schedule_wan(num_inference_steps[1], denoising_strength, shift[1])
    return merge_by_threshold(s1, s2, boundary), merge_by_threshold(t1, t2, boundary * num_train_timesteps)


def qwen_image_mu(image_seq_len, base_seq_len=256, max_seq_len=8192, base_shift=0.5, max_shift=0.9):
    m = (max_shift - base_shift) / (max_seq_len - base_seq_len)
    return image_seq_len * m + (base_shift - m * base_seq_len)


def schedule_qwen_image(num_inference_steps=100, denoising_strength=1.0, exponential_shift_mu=None,
                        dynamic_shift_len=None, shift_terminal=0.02, base_shift=0.5, max_shift=0.9):  # fmt: skip
    s = _descending(denoising_strength, 0.0, num_inference_steps, drop_last=True)
    if exponential_shift_mu is not None:
        mu = exponential_shift_mu
    elif dynamic_shift_len is not None:
        mu = qwen_image_mu(dynamic_shift_len, base_shift=base_shift, max_shift=max_shift)
    else:
        mu = 0.8
    s = _exp_shift(s, mu)
    if shift_terminal is not None:
        one_minus = 1 - s
        s = 1 - one_minus / (one_minus[-1] / (1 - shift_terminal))
    return s, s * NUM_TRAIN_TIMESTEPS


def flux2_empirical_mu(image_seq_len: int, num_steps: int) -> float:
    a1, b1 = 8.73809524e-05, 1.89833333
    a2, b2 = 0.00016927, 0.45666666
    if image_seq_len > 4300:
        return float(a2 * image_seq_len + b2)
    m_200 = a2 * image_seq_len + b2
    m_10 = a1 * image_seq_len + b1
    a = (m_200 - m_10) / 190.0
    return float(a * num_steps + (m_200 - 200.0 * a))


def schedule_flux2(num_inference_steps=100, denoising_strength=1.0, dynamic_shift_len=1024 // 16 * 1024 // 16):
    lo = 1 / num_inference_steps
    s = _descending(lo + (1.0 - lo) * denoising_strength, lo, num_inference_steps, drop_last=False)
    s = _exp_shift(s, flux2_empirical_mu(dynamic_shift_len, num_inference_steps))
    return s, s * NUM_TRAIN_TIMESTEPS


def schedule_z_image(num_inference_steps=100, denoising_strength=1.0, shift=None, target_timesteps=None):
    s = _descending(denoising_strength, 0.0, num_inference_steps, drop_last=True)
    s = _time_shift(s, 3 if shift is None else shift)
    t = s * NUM_TRAIN_TIMESTEPS
    if target_timesteps is not None:
        for ts in target_timesteps.to(dtype=t.dtype, device=t.device):
            t[torch.argmin((t - ts).abs())] = ts
    return s, t


def schedule_ltx2(num_inference_steps=100, denoising_strength=1.0, latent=None, max_shift=2.05, base_shift=0.95,
                  stretch=True, terminal=0.1, default_number_of_tokens=4096):  # fmt: skip
    tokens = math.prod(latent.shape[2:]) if latent is not None else default_number_of_tokens
    s = torch.linspace(denoising_strength, 0.0, num_inference_steps + 1)
    m = (max_shift - base_shift) / (4096 - 1024)
    mu = tokens * m + (base_shift - m * 1024)
    nz = s != 0
    shifted = torch.zeros_like(s)
    shifted[nz] = _exp_shift(s[nz], mu)
    s = shifted
    if stretch:
        one_minus = 1.0 - s[nz]
        s[nz] = 1.0 - one_minus / (one_minus[-1] / (1.0 - terminal))
    s[0] = float(denoising_strength)
    s[-1] = 0.0
    return s.float(), (s[:-1] * NUM_TRAIN_TIMESTEPS).float()


SIGMA_SCHEDULES: dict[str, Callable] = {
    "FLUX.1": schedule_flux,
    "Wan": schedule_wan,
    "Qwen-Image": schedule_qwen_image,
    "FLUX.2": schedule_flux2,
    "Z-Image": schedule_z_image,
    "Wan-Mix": schedule_wan_mix,
    "LTX.2": schedule_ltx2,
}


class FlowMatchScheduler:
    """Flow-matching scheduler; ``template`` picks the sigma schedule."""

    def __init__(self, template: str = "FLUX.1") -> None:
        self.template = template
        self.set_timesteps_fn = SIGMA_SCHEDULES.get(template, schedule_flux)
        self.num_train_timesteps = NUM_TRAIN_TIMESTEPS
        self.sigmas = torch.zeros(0)
        self.timesteps = torch.zeros(0)
        self.training = False
        self.linear_timesteps_weights = None

    # static aliases kept for callers that use the schedule functions through the class
    set_timesteps_flux = staticmethod(schedule_flux)
    set_timesteps_wan = staticmethod(schedule_wan)
    set_mix_timesteps_wan = staticmethod(schedule_wan_mix)
    set_timesteps_qwen_image = staticmethod(schedule_qwen_image)
    set_timesteps_flux2 = staticmethod(schedule_flux2)
    set_timesteps_z_image = staticmethod(schedule_z_image)
    set_timesteps_ltx2 = staticmethod(schedule_ltx2)
    compute_empirical_mu = staticmethod(flux2_empirical_mu)
    _calculate_shift_qwen_image = staticmethod(qwen_image_mu)

    def set_timesteps(self, num_inference_steps=100, denoising_strength=1.0, training=False, **kwargs) -> None:
        self.sigmas, self.timesteps = self.set_timesteps_fn(
            num_inference_steps=num_inference_steps, denoising_strength=denoising_strength, **kwargs
        )
        self.training = bool(training)
        if training:
            self.set_training_weight()

    def set_timesteps_with_mu(self, sigmas=None, mu=None, num_inference_steps=None) -> None:
        if sigmas is not None:
            s = torch.as_tensor(sigmas, dtype=torch.float32)
            num_inference_steps = num_inference_steps or len(s)
        else:
            num_inference_steps = num_inference_steps or 50
            s = torch.linspace(1.0, 1 / num_inference_steps, num_inference_steps, dtype=torch.float32)
        if mu is not None:
            s = _exp_shift(s, mu)
        self.sigmas = s
        self.timesteps = s * self.num_train_timesteps
        self.num_inference_steps = num_inference_steps

    def set_training_weight(self) -> None:
        steps = 1000
        x = self.timesteps
        y = torch.exp(-2 * ((x - steps / 2) / steps) ** 2)
        y = y - y.min()
        w = y * (steps / y.sum())
        if len(self.timesteps) != 1000:
            w = w * (len(self.timesteps) / steps)
            w = w + w[1]
        self.linear_timesteps_weights = w

    # ---- index helpers -------------------------------------------------
    def _index(self, timestep) -> int:
        if isinstance(timestep, torch.Tensor):
            timestep = timestep.detach().cpu()
        return int(torch.argmin((self.timesteps - timestep).abs()))

    def sigma_pair(self, timestep, to_final: bool = False) -> tuple[float, float]:
        """(sigma at `timestep`, sigma of the following step or 0 at the end)."""
        i = self._index(timestep)
        sigma = float(self.sigmas[i])
        if self.template == "LTX.2":
            nxt = 0.0 if to_final else float(self.sigmas[i + 1])
        else:
            nxt = 0.0 if (to_final or i + 1 >= len(self.timesteps)) else float(self.sigmas[i + 1])
        return sigma, nxt

    # ---- sampling ------------------------------------------------------
    def step(self, model_output, timestep, sample, to_final: bool = False, **kwargs):
        sigma, nxt = self.sigma_pair(timestep, to_final)
        if self.template == "LTX.2":
            velocity = (sample - model_output) / sigma
            return (sample.float() + velocity.float() * (nxt - sigma)).to(sample.dtype)
        return sample + model_output * (nxt - sigma)

    def step_with_guidance(self, cond, uncond, cfg_scale, timestep, sample, to_final: bool = False):
        """``v = uncond + s (cond - uncond); sample + v * dsigma`` in one fused pass."""
        from telefuser_b200.ops.functional import cfg_euler_step

        sigma, nxt = self.sigma_pair(timestep, to_final)
        return cfg_euler_step(sample, cond, uncond, cfg_scale, nxt - sigma)

    def return_to_timestep(self, timestep, sample, sample_stablized):
        sigma = float(self.sigmas[self._index(timestep)])
        return (sample - sample_stablized) / sigma

    def add_noise(self, original_samples, noise, timestep):
        sigma = float(self.sigmas[self._index(timestep)])
        return (1 - sigma) * original_samples + sigma * noise

    def training_target(self, sample, noise, timestep):
        return noise - sample

    def training_weight(self, timestep):
        i = int(torch.argmin((self.timesteps - timestep.to(self.timesteps.device)).abs()))
        return self.linear_timesteps_weights[i]
