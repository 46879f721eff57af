"""Request-level asyncio orchestrator.

A request walks an ordered list of `StageConfig`s. Consecutive stages that share a
`parallel_group` run concurrently (e.g. text and image encoders); stages that share a
`shared_lock_group` never run at the same time even across requests (e.g. VAE encode
and decode on one model instance). Every stage call runs in a worker thread so CUDA
work does not block the event loop. `generate()` is an async generator of per-stage
events. Role parity: telefuser/orchestrator/pipeline_orchestrator.py:21-358 and
telefuser/orchestrator/stage_wrapper.py:27-276.
"""

from __future__ import annotations

import asyncio
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Callable


@dataclass
class StageConfig:
    stage_id: int
    stage_name: str
    pipeline_attr: str
    param_builder: Callable[[dict, Any], tuple[list, dict]] | None = None
    result_processor: Callable[[Any], Any] | None = None
    shared_lock_group: str | None = None
    parallel_group: str | None = None
    metadata: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.stage_id < 0:
            raise ValueError(f"stage_id must be non-negative, got {self.stage_id}")
        if not self.stage_name:
            raise ValueError("stage_name cannot be empty")
        if not self.pipeline_attr:
            raise ValueError("pipeline_attr cannot be empty")


@dataclass
class StageResult:
    request_id: str
    stage_id: int
    outputs: Any
    finished: bool = False
    error: str | None = None
    metrics: dict = field(default_factory=dict)


class FlexiblePipelineOrchestrator:
    def __init__(self, pipeline: Any, stage_configs: list[StageConfig]) -> None:
        ids = [c.stage_id for c in stage_configs]
        if len(set(ids)) != len(ids):
            raise ValueError("duplicate stage ids")
        self.pipeline = pipeline
        self.stage_configs = sorted(stage_configs, key=lambda c: c.stage_id)
        self._locks: dict[str, threading.Lock] = {}
        for c in self.stage_configs:
            if c.shared_lock_group and c.shared_lock_group not in self._locks:
                self._locks[c.shared_lock_group] = threading.Lock()
            if not hasattr(pipeline, c.pipeline_attr):
                raise AttributeError(f"pipeline has no attribute {c.pipeline_attr}")
        self._running = False

    async def start(self) -> None:
        self._running = True

    async def stop(self) -> None:
        self._running = False

    def _group_stages(self) -> list[list[StageConfig]]:
        groups: list[list[StageConfig]] = []
        for c in self.stage_configs:
            if groups and c.parallel_group is not None and groups[-1][0].parallel_group == c.parallel_group:
                groups[-1].append(c)
            else:
                groups.append([c])
        return groups

    def _call_stage(self, cfg: StageConfig, context: dict, prev: Any):
        target = getattr(self.pipeline, cfg.pipeline_attr)
        fn = target.process if hasattr(target, "process") and not callable(target) else target
        args, kwargs = cfg.param_builder(context, prev) if cfg.param_builder else ([prev] if prev is not None else [], {})
        lock = self._locks.get(cfg.shared_lock_group) if cfg.shared_lock_group else None
        t0 = time.perf_counter()
        if lock is not None:
            with lock:
                out = fn(*args, **kwargs)
        else:
            out = fn(*args, **kwargs)
        if callable(out) and getattr(out, "__name__", "") in ("wait", "_wait_result"):
            out = out()
        if cfg.result_processor is not None:
            out = cfg.result_processor(out)
        return out, time.perf_counter() - t0

    async def _execute_single_stage(self, cfg: StageConfig, request_id: str, context: dict, prev: Any) -> StageResult:
        loop = asyncio.get_running_loop()
        try:
            out, dt = await loop.run_in_executor(None, self._call_stage, cfg, context, prev)
            return StageResult(request_id, cfg.stage_id, out, metrics={"seconds": dt})
        except Exception as e:  # noqa: BLE001 - reported as a stage event
            return StageResult(request_id, cfg.stage_id, None, error=f"{type(e).__name__}: {e}")

    async def generate(self, inputs: dict, request_id: str | None = None) -> AsyncIterator[dict]:
        """Yields one event per finished stage and a final `finished` event with all outputs."""
        request_id = request_id or uuid.uuid4().hex
        context = dict(inputs)
        context.setdefault("results", {})
        prev: Any = None
        for group in self._group_stages():
            results = await asyncio.gather(*[self._execute_single_stage(c, request_id, context, prev) for c in group])
            for cfg, res in zip(group, results):
                if res.error is not None:
                    yield {"request_id": request_id, "stage_id": cfg.stage_id, "stage_name": cfg.stage_name,
                           "status": "error", "error": res.error, "finished": True}  # fmt: skip
                    return
                context["results"][cfg.stage_name] = res.outputs
                yield {"request_id": request_id, "stage_id": cfg.stage_id, "stage_name": cfg.stage_name,
                       "status": "ok", "outputs": res.outputs, "metrics": res.metrics, "finished": False}  # fmt: skip
            prev = results[0].outputs if len(results) == 1 else {c.stage_name: r.outputs for c, r in zip(group, results)}
        yield {"request_id": request_id, "status": "ok", "outputs": prev, "results": context["results"],
               "finished": True}  # fmt: skip

    async def run(self, inputs: dict, request_id: str | None = None) -> Any:
        last = None
        async for ev in self.generate(inputs, request_id):
            last = ev
        if last is None or last.get("status") != "ok":
            raise RuntimeError(last.get("error") if last else "no stages")
        return last["outputs"]
