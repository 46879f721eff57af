"""Stage execution inside a Ray actor (optional: needs the `ray` package at run time).

`create_ray_worker(stage, enable_parallel)` starts one actor with the stage's `RayConfig` resources; the actor
pins its visible GPUs, optionally caps its share of device memory, wraps the stage in a `ParallelWorker` when
asked and serves `process(...)`. `RayStageHandle` gives the actor the same call surface as a local stage
(`handle.process(...)` returns the result; `handle.process_async(...)` returns a waiter), so pipelines do not
care where a stage runs.
Role parity: telefuser/worker/ray_worker.py:28-107.
"""

from __future__ import annotations

import os
from typing import Any

import torch

from telefuser_b200.utils.logging import logger

try:  # optional dependency
    import ray
except ImportError:  # pragma: no cover - exercised through the stub in the tests
    ray = None


class RayWorker:
    def __init__(self, stage, enable_parallel: bool = False) -> None:
        self.ray_config = stage.model_runtime_config.ray_config
        self.worker_id = stage.name
        self._setup_resources()
        if enable_parallel:
            from telefuser_b200.worker.parallel_worker import ParallelWorker

            self._worker: Any = ParallelWorker(stage)
        else:
            self._worker = stage

    def _setup_resources(self) -> None:
        gpu = self.ray_config.gpu_config
        if gpu.num_gpus > 0:
            os.environ["CUDA_VISIBLE_DEVICES"] = ",".join(str(i) for i in range(int(gpu.num_gpus)))
            if gpu.memory_limit > 0 and torch.cuda.is_available():
                torch.cuda.set_per_process_memory_fraction(gpu.memory_limit)
        logger.info(f"RayWorker {self.worker_id}: gpus={gpu.num_gpus} memory_limit={gpu.memory_limit} host_memory_gb={self.ray_config.memory_gb}")

    def process(self, *args: Any, **kwargs: Any) -> Any:
        try:
            out = self._worker.process(*args, **kwargs)
            return out() if callable(out) and getattr(out, "__name__", "") == "_wait_result" else out
        except Exception as exc:
            logger.error(f"RayWorker {self.worker_id} failed: {exc}")
            raise

    def get_status(self) -> dict:
        cuda = torch.cuda.is_available()
        return {"worker_id": self.worker_id, "worker_type": type(self._worker).__name__, "ray_config": self.ray_config,
                "gpu_memory_used": torch.cuda.max_memory_allocated() if cuda else 0,
                "gpu_memory_total": torch.cuda.get_device_properties(0).total_memory if cuda else 0}  # fmt: skip

    def close(self) -> None:
        if hasattr(self._worker, "close"):
            self._worker.close()


class RayStageHandle:
    """Local face of a `RayWorker` actor."""

    def __init__(self, actor, name: str) -> None:
        self.actor, self.name = actor, name

    def process_async(self, *args: Any, **kwargs: Any):
        ref = self.actor.process.remote(*args, **kwargs)
        return lambda: ray.get(ref)

    def process(self, *args: Any, **kwargs: Any) -> Any:
        return ray.get(self.actor.process.remote(*args, **kwargs))

    def get_status(self) -> dict:
        return ray.get(self.actor.get_status.remote())

    def close(self) -> None:
        try:
            ray.get(self.actor.close.remote())
        finally:
            ray.kill(self.actor)


def create_ray_worker(stage, enable_parallel: bool = False) -> RayStageHandle:
    if ray is None:
        raise ImportError("Ray workers need the optional 'ray' package")
    cfg = stage.model_runtime_config.ray_config
    ray.init(ignore_reinit_error=True, address=cfg.ray_address)
    resources = {"num_cpus": cfg.num_cpus, "memory": cfg.memory_gb * 1024**3, "num_gpus": cfg.gpu_config.num_gpus}
    logger.info(f"starting Ray actor for stage {stage.name} with {resources}")
    actor = ray.remote(RayWorker).options(**resources).remote(stage, enable_parallel=enable_parallel)
    return RayStageHandle(actor, stage.name)
