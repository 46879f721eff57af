"""Stage = the unit that owns models and exposes ``process``; runs in-process or
inside every rank of a ``ParallelWorker``.

Covers the reference's ``telefuser/core/base_stage.py:22-169``: the
``with_model_offload`` decorator (load named models before a call and move them
back according to the offload policy), ``parallel_models`` (hook executed in
each worker rank after the process group exists), metrics hooks and
feature-cache set-up.
"""

from __future__ import annotations

import functools
from abc import ABC
from typing import Any, Callable

import torch

from .config import FeatureCacheConfig, ModelRuntimeConfig, WeightOffloadType


def with_model_offload(model_names: list[str]) -> Callable:
    def decorator(func):
        @functools.wraps(func)
        def wrapper(self: "BaseStage", *args, **kwargs):
            policy = self.model_runtime_config.offload_config.offload_type
            if self.onload_models_flag and policy == WeightOffloadType.NO_CPU_OFFLOAD:
                return func(self, *args, **kwargs)
            if not self.onload_models_flag:
                for name in model_names:
                    model = getattr(self, name, None)
                    if model is not None:
                        self._move(model, self.device)
                self.onload_models_flag = True
            try:
                return func(self, *args, **kwargs)
            finally:
                if policy != WeightOffloadType.NO_CPU_OFFLOAD:
                    pin = self.model_runtime_config.offload_config.pin_cpu_memory
                    for name in model_names:
                        model = getattr(self, name, None)
                        if model is None:
                            continue
                        if hasattr(model, "offload_device"):
                            model.offload_device(pin)
                        else:
                            model.cpu()
                    if torch.cuda.is_available():
                        torch.cuda.empty_cache()
                    self.onload_models_flag = False

        return wrapper

    return decorator


class BaseStage(ABC):
    def __init__(self, name: str, model_runtime_config: ModelRuntimeConfig) -> None:
        self.name = name
        self.model_runtime_config = model_runtime_config
        self.torch_dtype = model_runtime_config.torch_dtype
        self.device_type = model_runtime_config.device_type or ("cuda" if torch.cuda.is_available() else "cpu")
        self.device = (torch.device("cpu") if self.device_type == "cpu"
                       else torch.device(self.device_type, model_runtime_config.device_id))  # fmt: skip
        self.model_names: list[str] = []
        self.onload_models_flag = False
        self._metrics_hook = None

    # ---- metrics ---------------------------------------------------------
    def enable_metrics(self, registry: Any | None = None) -> None:
        from telefuser_b200.metrics import get_metrics_registry

        self._metrics_hook = (registry or get_metrics_registry()).register_stage(self.name)

    def disable_metrics(self) -> None:
        self._metrics_hook = None

    @property
    def metrics_hook(self):
        return self._metrics_hook

    # ---- model placement -----------------------------------------------------
    @staticmethod
    def _move(model, device) -> None:
        if hasattr(model, "onload_device"):
            model.onload_device(device)
        else:
            model.to(device)

    def onload_models(self) -> None:
        for name in self.model_names:
            model = getattr(self, name, None)
            if model is not None:
                self._move(model, self.device)
        self.onload_models_flag = True

    def offload_models(self) -> None:
        pin = self.model_runtime_config.offload_config.pin_cpu_memory
        for name in self.model_names:
            model = getattr(self, name, None)
            if model is None:
                continue
            if hasattr(model, "offload_device"):
                model.offload_device(pin)
            else:
                model.cpu()
        self.onload_models_flag = False

    def parallel_models(self) -> None:
        """Called once in every worker rank after the process group is up. Override."""

    # ---- device health ---------------------------------------------------------
    def configure_device_waits(self) -> None:
        """Bounds every wait of a kernel on another rank by the parallel configuration's timeout."""
        if self.device.type != "cuda":
            return
        from telefuser_b200.ops import native

        cfg = self.model_runtime_config.parallel_config
        limit_s = min(float(getattr(cfg, "device_wait_timeout", 30.0)), float(cfg.timeout))
        native.set_peer_wait_ms(int(max(0.1, min(600.0, limit_s)) * 1000))

    def check_device_waits(self, final: bool = False) -> None:
        """Surfaces an expired bounded wait of a device kernel (a peer that stopped answering, a lost copy) as
        `DeviceWaitTimeout`, so that the worker rank reports a failure instead of returning data computed from
        stale buffers. Inside a loop (`final=False`) nothing blocks: the word posted after the previous step is
        read and a new copy is enqueued behind the work issued so far. `final=True` synchronises; it belongs
        where the caller reads the result anyway."""
        if self.device.type != "cuda":
            return
        from telefuser_b200.ops import native

        what = f"stage {self.name!r}"
        if final:
            native.finish_status(what)
        else:
            native.poll_status(what)
            native.post_status()

    def setup_feature_cache(self, model, cache_config: FeatureCacheConfig, num_inference_steps: int,
                            init_step: int = 0) -> None:  # fmt: skip
        from telefuser_b200.feature_cache import create_feature_cache

        if cache_config.enabled:
            model.set_feature_cache(create_feature_cache(
                "ada_taylor", model_type=cache_config.model_type, num_inference_steps=num_inference_steps,
                n_derivatives=cache_config.n_derivatives, taylor_threshold=cache_config.taylor_threshold,
                init_step=init_step))  # fmt: skip
        else:
            model.set_feature_cache(create_feature_cache("none"))

    def process(self, *args, **kwargs):
        raise NotImplementedError
