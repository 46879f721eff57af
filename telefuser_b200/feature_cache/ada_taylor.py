"""AdaTaylor feature cache: skip the DiT block stack on planned steps and rebuild its
residual from finite-difference Taylor terms (or plain reuse when too far from the
last computed step).

Algorithm parity with the reference's
``telefuser/feature_cache/ada_taylor_cache/ada_taylor_cache.py:100-656``:
the compute-step plan is derived once from calibrated per-step magnitude ratios,
an error threshold, a maximum run of skipped steps ``K`` and a retention ratio;
cond and uncond branches keep separate state. Calibrated parameter files are
JSON ``{K, retention_ratio, thresh, cond_mag_ratios, uncond_mag_ratios}`` looked
up in ``TFB_TAYLOR_PARAMS_DIR`` (or ``<package>/feature_cache/params``); when a
model has no file a neutral default plan is used and the calibrator can write one.
"""

from __future__ import annotations

import json
import math
import os
from pathlib import Path

import numpy as np
import torch

from .base import BaseFeatureCache


def safe_model_name(model_name: str) -> str:
    return model_name.replace(".", "_").replace("/", "_")


def params_dir() -> Path:
    env = os.environ.get("TFB_TAYLOR_PARAMS_DIR")
    return Path(env) if env else Path(__file__).parent / "params"


def default_cache_params(num_steps: int = 50) -> dict:
    """Neutral plan for uncalibrated models: ratios drift slowly from 1, so runs of <= K steps are skipped."""
    idx = np.arange(num_steps)
    ratios = 1.0 + 0.02 * np.exp(-idx / max(num_steps / 6.0, 1.0))
    ratios[0] = 1.0
    r = [round(float(v), 5) for v in ratios]
    return {"K": min(4, max(1, num_steps // 10)), "retention_ratio": 0.2, "thresh": 0.12,
            "num_inference_steps": num_steps, "cond_mag_ratios": r, "uncond_mag_ratios": list(r)}  # fmt: skip


def load_cache_params(model_name: str, num_steps: int = 50, strict: bool = False) -> dict:
    f = params_dir() / f"{safe_model_name(model_name)}.json"
    if f.exists():
        return json.loads(f.read_text())
    if strict:
        raise FileNotFoundError(f"Parameters not found for model '{model_name}'. Expected file: {f}")
    return default_cache_params(num_steps)


def nearest_interp(src, target_length: int) -> np.ndarray:
    src = np.asarray(src)
    if target_length == 1:
        return np.array([src[-1]])
    idx = np.round(np.arange(target_length) * (len(src) - 1) / (target_length - 1)).astype(int)
    return src[idx]


def plan_compute_steps(num_steps, mag_ratios, thresh, K, start_step, init_step=0) -> set[int]:
    """Steps that must run the real block stack.

    Always: steps up to `start_step`, the last step and `init_step`. Otherwise a
    step is skipped while the accumulated |1 - prod(ratios)| stays under `thresh`
    and at most `K` steps have been skipped in a row.
    """
    steps: set[int] = set()
    err, run, ratio = 0.0, 0, 1.0
    for s in range(num_steps):
        forced = s <= start_step or s == num_steps - 1 or s == init_step
        if not forced:
            ratio *= float(mag_ratios[s])
            run += 1
            err += abs(1.0 - ratio)
            if err < thresh and run <= K:
                continue
        steps.add(s)
        err, run, ratio = 0.0, 0, 1.0
    return steps


class TaylorBranchState:
    """Residual history of one guidance branch."""

    def __init__(self, num_inference_steps, thresh, K, mag_ratios, retention_ratio, n_derivatives=1,
                 taylor_threshold=2, init_step=0):  # fmt: skip
        self.num_inference_steps = num_inference_steps
        self.init_step = init_step
        self.thresh, self.K = thresh, K
        self.start_step = int(num_inference_steps * retention_ratio)
        self.n_derivatives = n_derivatives
        self.order = n_derivatives + 1
        self.mag_ratios = mag_ratios
        self.taylor_threshold = taylor_threshold
        self.compute_steps = plan_compute_steps(num_inference_steps, mag_ratios, thresh, K, self.start_step,
                                                init_step)  # fmt: skip
        self.reset()

    def reset(self) -> None:
        self.prev_terms: list = [None] * self.order
        self.terms: list = [None] * self.order
        self.last_residual = None
        self.step = self.init_step - 1
        self.last_compute_step = self.init_step - 1

    @property
    def current_step(self) -> int:
        return self.step

    def advance(self) -> int:
        self.step += 1
        return self.step

    def should_compute(self) -> bool:
        return self.step in self.compute_steps

    def _finite_differences(self, residual):
        terms = [None] * self.order
        terms[0] = residual
        window = max(self.step - self.last_compute_step, 1)
        if self.terms[0] is not None and self.terms[0].shape != residual.shape:
            self.reset_history()
            return terms
        for i in range(self.n_derivatives):
            if self.terms[i] is None or terms[i] is None or self.step <= 0:
                break
            terms[i + 1] = (terms[i] - self.terms[i]) / window
        return terms

    def reset_history(self) -> None:
        self.prev_terms = [None] * self.order
        self.terms = [None] * self.order
        self.last_residual = None

    @staticmethod
    def _fused_ok(t) -> bool:
        return t.is_cuda and t.dtype == torch.bfloat16 and t.numel() % 8 == 0

    def _update_fused(self, output, ori_input) -> None:
        """One pass over persistent term buffers (residual and finite differences formed in registers)."""
        from telefuser_b200.ops import functional as TF

        bufs = getattr(self, "_bufs", None)
        if bufs is None or bufs[0].shape != output.shape or bufs[0].device != output.device:
            self._bufs = bufs = [torch.empty_like(output, memory_format=torch.contiguous_format) for _ in range(self.order)]
            self.terms = [None] * self.order
        n_old = sum(t is not None for t in self.terms) if self.step > 0 else 0
        n_new = min(self.order, n_old + 1) if n_old > 0 else 1
        window = max(self.step - self.last_compute_step, 1)
        TF.taylor_update_(output.contiguous(), ori_input.contiguous(), bufs, n_old, n_new, window)
        self.prev_terms = [None] * self.order
        self.terms = bufs[:n_new] + [None] * (self.order - n_new)
        self.last_residual = bufs[0]
        self.last_compute_step = self.step

    def update(self, output, ori_input) -> None:
        if self._fused_ok(output) and self.order <= 4:
            return self._update_fused(output, ori_input)
        residual = (output - ori_input).detach()
        new_terms = self._finite_differences(residual)
        self.prev_terms = self.terms
        self.terms = new_terms
        self.last_residual = residual
        self.last_compute_step = self.step

    def approximate_residual(self):
        elapsed = self.step - self.last_compute_step
        if elapsed > self.taylor_threshold:
            return self.last_residual if self.last_residual is not None else self.terms[0]
        out = None
        for i, term in enumerate(self.terms):
            if term is None:
                break
            contrib = term * (float(elapsed**i) / math.factorial(i))
            out = contrib if out is None else out + contrib
        return out

    def approximate(self, current_input):
        valid = [t for t in self.terms if t is not None]
        if valid and self._fused_ok(current_input) and current_input.is_contiguous() and len(valid) <= 4:
            from telefuser_b200.ops import functional as TF

            elapsed = self.step - self.last_compute_step
            if elapsed > self.taylor_threshold:
                return TF.taylor_apply(current_input, [self.last_residual], [1.0])
            return TF.taylor_apply(current_input, valid, [float(elapsed**i) / math.factorial(i) for i in range(len(valid))])
        r = self.approximate_residual()
        return current_input if r is None else current_input + r


class AdaTaylorCache(BaseFeatureCache):
    def __init__(self, model_type: str, num_inference_steps: int, n_derivatives: int = 1, taylor_threshold: int = 2,
                 init_step: int = 0, params: dict | None = None):  # fmt: skip
        params = params or load_cache_params(model_type, num_inference_steps)
        self.model_type = model_type
        self.num_inference_steps = num_inference_steps
        self.n_derivatives = n_derivatives
        self.taylor_threshold = taylor_threshold
        self.init_step = init_step

        def branch(key):
            r = params[key]
            if len(r) != num_inference_steps:
                r = nearest_interp(r, num_inference_steps)
            return TaylorBranchState(num_inference_steps, params["thresh"], params["K"], np.asarray(r),
                                     params["retention_ratio"], n_derivatives, taylor_threshold, init_step)  # fmt: skip

        self.cond_state = branch("cond_mag_ratios")
        self.uncond_state = branch("uncond_mag_ratios")

    def _state(self, is_cond: bool) -> TaylorBranchState:
        return self.cond_state if is_cond else self.uncond_state

    def reset(self) -> None:
        self.cond_state.reset()
        self.uncond_state.reset()

    def should_compute(self, is_cond: bool) -> bool:
        st = self._state(is_cond)
        st.advance()
        return st.should_compute()

    def update(self, output, ori_input, is_cond: bool) -> None:
        self._state(is_cond).update(output, ori_input)

    def approximate(self, input, is_cond: bool):  # noqa: A002
        return self._state(is_cond).approximate(input)

    def last_step_was_compute(self, is_cond: bool = True) -> bool:
        st = self._state(is_cond)
        return st.current_step in st.compute_steps

    def get_compute_steps(self) -> list[int]:
        return sorted(self.cond_state.compute_steps)

    def __repr__(self) -> str:
        return (f"AdaTaylorCache(n_derivatives={self.n_derivatives}, taylor_threshold={self.taylor_threshold}, "
                f"steps={self.num_inference_steps})")  # fmt: skip


class _RatioRecorder:
    def __init__(self, num_steps: int):
        self.num_steps = num_steps
        self.reset()

    def reset(self) -> None:
        self.count, self.ratios, self.prev = 0, [], None

    def store(self, x, ori_x) -> None:
        residual = x - ori_x
        if self.count >= 1:
            self.ratios.append(round((residual.norm(dim=-1) / self.prev.norm(dim=-1)).mean().item(), 5))
        self.prev = residual
        self.count += 1

    def finished(self) -> bool:
        return self.count >= self.num_steps


class AdaTaylorCacheCalibrator(BaseFeatureCache):
    """Runs every step for real and records residual-magnitude ratios; writes the JSON plan file."""

    def __init__(self, num_inference_steps: int, sigma_shift: float, model_name: str, output_path: str | None = None):
        self.num_inference_steps = num_inference_steps
        self.sigma_shift = sigma_shift
        self.model_name = model_name
        self.output_path = output_path or str(params_dir() / f"{safe_model_name(model_name)}.json")
        self.cond = _RatioRecorder(num_inference_steps)
        self.uncond = _RatioRecorder(num_inference_steps)
        self._finished = False

    def reset(self) -> None:
        self.cond.reset()
        self.uncond.reset()
        self._finished = False

    def should_compute(self, is_cond: bool) -> bool:
        return True

    def update(self, x, ori_x, is_cond: bool) -> None:
        (self.cond if is_cond else self.uncond).store(x, ori_x)
        if not self._finished and self.cond.finished() and self.uncond.finished():
            self.save()
            self._finished = True

    def approximate(self, input, is_cond: bool):  # noqa: A002
        return input

    def result(self) -> dict:
        return {
            "K": min(4, max(1, self.num_inference_steps // 10)),
            "retention_ratio": 0.2,
            "thresh": 0.12,
            "sigma_shift": self.sigma_shift,
            "num_inference_steps": self.num_inference_steps,
            "cond_mag_ratios": [1.0] + self.cond.ratios,
            "uncond_mag_ratios": [1.0] + self.uncond.ratios,
        }

    def save(self) -> str:
        os.makedirs(os.path.dirname(self.output_path) or ".", exist_ok=True)
        with open(self.output_path, "w") as f:
            json.dump(self.result(), f, indent=4)
        return self.output_path
