"""UniPC multistep predictor-corrector for flow-matching models (data prediction, B(h) = e^h - 1).

Flow parameterisation: x_t = (1 - sigma) x0 + sigma * noise, the model predicts the velocity
v = noise - x0, hence x0 = x_t - sigma * v. With alpha = 1 - sigma and lambda = log(alpha / sigma)
each step applies the UniC corrector (using the new model output at the current point) and then
the UniP predictor of order <= `solver_order` (lower order for the first and, optionally, last
steps). Interface parity: FlowUniPCMultistepScheduler, telefuser/schedulers/unipc.py
(set_timesteps with `shift`, step, add_noise, sigmas / timesteps tensors); self-contained, no
diffusers dependency.
"""

from __future__ import annotations

import math

import numpy as np
import torch


class FlowUniPCMultistepScheduler:
    order = 1

    def __init__(self, num_train_timesteps: int = 1000, solver_order: int = 2, prediction_type: str = "flow_prediction",
                 shift: float = 1.0, use_dynamic_shifting: bool = False, predict_x0: bool = True,
                 solver_type: str = "bh2", lower_order_final: bool = True, disable_corrector: tuple = (),
                 final_sigmas_type: str = "zero"):  # fmt: skip
        if solver_type not in ("bh1", "bh2"):
            raise NotImplementedError(f"{solver_type} is not implemented")
        self.num_train_timesteps = num_train_timesteps
        self.solver_order = solver_order
        self.prediction_type = prediction_type
        self.shift = shift
        self.use_dynamic_shifting = use_dynamic_shifting
        self.predict_x0 = predict_x0
        self.solver_type = solver_type
        self.lower_order_final = lower_order_final
        self.disable_corrector = list(disable_corrector)
        self.final_sigmas_type = final_sigmas_type
        alphas = np.linspace(1, 1 / num_train_timesteps, num_train_timesteps)[::-1].copy()
        sigmas = 1.0 - alphas
        if not use_dynamic_shifting:
            sigmas = shift * sigmas / (1 + (shift - 1) * sigmas)
        self.sigmas = torch.from_numpy(sigmas).float()
        self.timesteps = self.sigmas * num_train_timesteps
        self.sigma_min = float(self.sigmas[-1])
        self.sigma_max = float(self.sigmas[0])
        self.num_inference_steps = None
        self._reset()

    def _reset(self) -> None:
        self.model_outputs = [None] * self.solver_order
        self.timestep_list = [None] * self.solver_order
        self.lower_order_nums = 0
        self.last_sample = None
        self.this_order = 1
        self._step_index = None
        self._begin_index = None

    @property
    def step_index(self):
        return self._step_index

    def set_begin_index(self, begin_index: int = 0) -> None:
        self._begin_index = begin_index

    # ---- schedule ---------------------------------------------------------------
    def set_timesteps(self, num_inference_steps: int | None = None, device=None, sigmas=None, mu: float | None = None,
                      shift: float | None = None) -> None:  # fmt: skip
        if self.use_dynamic_shifting and mu is None:
            raise ValueError("mu is required with use_dynamic_shifting")
        if sigmas is None:
            sigmas = np.linspace(self.sigma_max, self.sigma_min, num_inference_steps + 1)[:-1]
        sigmas = np.asarray(sigmas, dtype=np.float64)
        if self.use_dynamic_shifting:
            sigmas = math.exp(mu) / (math.exp(mu) + (1 / sigmas - 1))
        else:
            s = self.shift if shift is None else shift
            sigmas = s * sigmas / (1 + (s - 1) * sigmas)
        last = 0.0 if self.final_sigmas_type == "zero" else (1 - 1 / self.num_train_timesteps)
        timesteps = sigmas * self.num_train_timesteps
        self.sigmas = torch.from_numpy(np.concatenate([sigmas, [last]]).astype(np.float32))
        self.timesteps = torch.from_numpy(timesteps).to(device=device, dtype=torch.int64)
        self.num_inference_steps = len(timesteps)
        self._reset()

    @staticmethod
    def _alpha_sigma(sigma):
        return 1 - sigma, sigma

    def index_for_timestep(self, timestep, schedule=None) -> int:
        schedule = self.timesteps if schedule is None else schedule
        idx = (schedule == timestep).nonzero()
        if len(idx) == 0:
            return int(torch.argmin((schedule.double() - float(timestep)).abs()))
        return int(idx[1 if len(idx) > 1 else 0])

    def _init_step_index(self, timestep) -> None:
        if self._begin_index is None:
            if isinstance(timestep, torch.Tensor):
                timestep = timestep.to(self.timesteps.device)
            self._step_index = self.index_for_timestep(timestep)
        else:
            self._step_index = self._begin_index

    # ---- model output ---------------------------------------------------------------
    def convert_model_output(self, model_output, sample):
        sigma = self.sigmas[self._step_index]
        if self.prediction_type != "flow_prediction":
            raise ValueError("only flow_prediction is supported")
        if self.predict_x0:
            return sample - sigma * model_output
        return sample - (1 - sigma) * model_output  # noise prediction form

    def _uni_update(self, this_output, x, order: int, corrector: bool):
        """Shared UniP / UniC body. For the corrector `this_output` is the model output at the new point."""
        outs, dev = self.model_outputs, x.device
        if corrector:
            s0_idx, t_idx = self._step_index - 1, self._step_index
            m0 = outs[-1]
        else:
            s0_idx, t_idx = self._step_index, self._step_index + 1
            m0 = outs[-1]
        sigma_t, sigma_s0 = self.sigmas[t_idx], self.sigmas[s0_idx]
        alpha_t, alpha_s0 = 1 - sigma_t, 1 - sigma_s0
        lam = lambda a, s: torch.log(a) - torch.log(s)  # noqa: E731
        lambda_t, lambda_s0 = lam(alpha_t, sigma_t), lam(alpha_s0, sigma_s0)
        h = lambda_t - lambda_s0
        rks, D1s = [], []
        for i in range(1, order):
            si = s0_idx - i
            mi = outs[-(i + 1)]
            sig_i = self.sigmas[si]
            rk = (lam(1 - sig_i, sig_i) - lambda_s0) / h
            rks.append(rk)
            D1s.append((mi - m0) / rk)
        rks.append(torch.tensor(1.0))
        rks = torch.stack([r.to(torch.float64) if isinstance(r, torch.Tensor) else torch.tensor(r) for r in rks]).to(dev)
        hh = (-h if self.predict_x0 else h).to(torch.float64)
        h_phi_1 = torch.expm1(hh)
        h_phi_k = h_phi_1 / hh - 1
        B_h = hh if self.solver_type == "bh1" else torch.expm1(hh)
        R, b, fact = [], [], 1
        for i in range(1, order + 1):
            R.append(torch.pow(rks, i - 1))
            b.append(h_phi_k * fact / B_h)
            fact *= i + 1
            h_phi_k = h_phi_k / hh - 1 / fact
        R = torch.stack(R)
        b = torch.stack(b).to(dev)
        D1s_t = torch.stack(D1s, dim=1) if D1s else None
        if corrector:
            rhos = torch.tensor([0.5], dtype=torch.float64, device=dev) if order == 1 else torch.linalg.solve(R, b)
        else:
            if order == 2:
                rhos = torch.tensor([0.5], dtype=torch.float64, device=dev)
            elif order > 2:
                rhos = torch.linalg.solve(R[:-1, :-1], b[:-1])
            else:
                rhos = None
        rhos = None if rhos is None else rhos.to(x.dtype)
        h_phi_1, B_h = h_phi_1.to(x.dtype), B_h.to(x.dtype)
        if self.predict_x0:
            x_t_ = (sigma_t / sigma_s0) * x - alpha_t * h_phi_1 * m0
        else:
            x_t_ = (alpha_t / alpha_s0) * x - sigma_t * h_phi_1 * m0
        scale = alpha_t if self.predict_x0 else sigma_t
        res = 0
        if D1s_t is not None:
            k = D1s_t.shape[1]
            coef = rhos[:k] if corrector else rhos
            res = torch.einsum("k,bk...->b...", coef, D1s_t)
        if corrector:
            res = res + rhos[-1] * (this_output - m0)
        return (x_t_ - scale * B_h * res).to(x.dtype)

    # ---- public step -------------------------------------------------------------------
    def step(self, model_output, timestep, sample, return_dict: bool = False, generator=None):
        if self.num_inference_steps is None:
            raise ValueError("call set_timesteps first")
        if self._step_index is None:
            self._init_step_index(timestep)
        use_corrector = (self._step_index > 0 and self._step_index - 1 not in self.disable_corrector
                         and self.last_sample is not None)  # fmt: skip
        converted = self.convert_model_output(model_output, sample)
        if use_corrector:
            sample = self._uni_update(converted, self.last_sample, self.this_order, corrector=True)
        for i in range(self.solver_order - 1):
            self.model_outputs[i] = self.model_outputs[i + 1]
            self.timestep_list[i] = self.timestep_list[i + 1]
        self.model_outputs[-1] = converted
        self.timestep_list[-1] = timestep
        if self.lower_order_final:
            this_order = min(self.solver_order, len(self.timesteps) - self._step_index)
        else:
            this_order = self.solver_order
        self.this_order = min(this_order, self.lower_order_nums + 1)
        self.last_sample = sample
        prev = self._uni_update(None, sample, self.this_order, corrector=False)
        if self.lower_order_nums < self.solver_order:
            self.lower_order_nums += 1
        self._step_index += 1
        return {"prev_sample": prev} if return_dict else (prev,)

    def scale_model_input(self, sample, *args, **kwargs):
        return sample

    def add_noise(self, original_samples, noise, timesteps):
        sigmas = self.sigmas.to(device=original_samples.device, dtype=original_samples.dtype)
        schedule = self.timesteps.to(original_samples.device)
        ts = timesteps.to(original_samples.device).reshape(-1)
        idx = [self.index_for_timestep(t, schedule) for t in ts]
        sigma = sigmas[idx].flatten()
        while sigma.ndim < original_samples.ndim:
            sigma = sigma.unsqueeze(-1)
        return (1 - sigma) * original_samples + sigma * noise

    def __len__(self) -> int:
        return self.num_train_timesteps
