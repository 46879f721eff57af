"""Small CPU stages used by the worker / orchestrator self-tests (picklable, importable from ranks)."""

from __future__ import annotations

import os
import time

import torch
import torch.distributed as dist

from telefuser_b200.core.base_stage import BaseStage
from telefuser_b200.core.config import ModelRuntimeConfig, ParallelConfig


def cpu_runtime_config(world_size: int = 1, timeout: int = 60, **degrees) -> ModelRuntimeConfig:
    pc = ParallelConfig(device_ids=list(range(world_size)) if world_size > 1 else None, timeout=timeout, **degrees)
    return ModelRuntimeConfig(device_type="cpu", torch_dtype=torch.float32, parallel_config=pc)


class AllReduceStage(BaseStage):
    """`process(x)` returns the sum over ranks of `x * (rank + 1)`; other methods inject host-side faults."""

    def __init__(self, config: ModelRuntimeConfig):
        super().__init__("allreduce", config)
        self.parallel_called = False

    def parallel_models(self) -> None:
        self.parallel_called = True

    def process(self, x: torch.Tensor) -> torch.Tensor:
        rank = dist.get_rank() if dist.is_initialized() else 0
        y = x * (rank + 1)
        if dist.is_initialized():
            dist.all_reduce(y)
        return y

    def info(self) -> dict:
        return {"rank": dist.get_rank() if dist.is_initialized() else 0, "pid": os.getpid(),
                "parallel_called": self.parallel_called, "device": str(self.device)}  # fmt: skip

    def fail_on_rank(self, rank: int) -> str:
        me = dist.get_rank() if dist.is_initialized() else 0
        if me == rank:
            raise ValueError(f"injected failure on rank {rank}")
        return "ok"

    def sleep(self, seconds: float) -> str:
        time.sleep(seconds)
        return "slept"

    def exit_on_rank(self, rank: int) -> str:
        me = dist.get_rank() if dist.is_initialized() else 0
        if me == rank:
            os._exit(3)
        time.sleep(0.5)
        return "ok"
