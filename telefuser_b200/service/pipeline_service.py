"""Server configuration, pipeline loading / running, and the data-parallel replica pool.

* `ServerConfig`: pydantic-settings, environment prefix `TELEFUSER_`.
* `PipelineService`: security check -> import the pipeline file -> contract -> `get_pipeline(parallelism)`
  -> `PipelineRunner` (filters kwargs by signature, sync or async `run_with_file`, measures time and
  peak memory, honours a stop event).
* `PipelinePool`: N replica processes, each with its own `CUDA_VISIBLE_DEVICES` slice and a full
  pipeline; tasks go to an idle replica over a `Pipe`; a dead replica is evicted and the task
  manager's capacity shrinks; when none is left all pending tasks fail.
Role parity: telefuser/service/core/{config,pipeline_loader,pipeline_runner,pipeline_service,
pipeline_pool,replica_worker}.py.
"""

from __future__ import annotations

import asyncio
import importlib.util
import inspect
import multiprocessing as mp
import os
import sys
import threading
import time
import traceback
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch
from pydantic_settings import BaseSettings, SettingsConfigDict

from telefuser_b200.utils.logging import logger

from .contract import PipelineContract, load_contract
from .security import PipelineSecurityValidator, SecurityLevel


class ServerConfig(BaseSettings):
    model_config = SettingsConfigDict(env_prefix="TELEFUSER_", extra="ignore")

    host: str = "0.0.0.0"
    port: int = 8000
    cache_dir: str = "./server_cache"
    max_queue_size: int = 100
    task_timeout: float = 3600.0
    cleanup_keep_count: int = 1000
    security_level: str = "strict"
    rate_limit_enabled: bool = False
    rate_limit_requests: int = 120
    rate_limit_window_s: float = 60.0
    metrics_enabled: bool = True
    max_upload_mb: int = 512
    artifact_retention_hours: float = 24.0
    artifact_max_gb: float = 50.0
    num_replicas: int = 1
    replica_start_timeout: float = 1800.0
    webrtc_disconnect_grace_s: float = 10.0
    webrtc_datachannel_timeout_s: float = 30.0
    stream_fps: int = 16
    stream_max_sessions: int = 0  # 0: no limit; else further session requests are refused (HTTP 503) while this many are open
    enable_latent_cache: bool = False
    latent_cache_mode: str = "readwrite"
    latent_cache_dir: str | None = None  # default: <cache_dir>/latent_cache
    latent_cache_min_similarity: float = 0.85


def resolve_replica_device_ids(num_replicas: int, parallelism: int, available: list[int] | None = None) -> list[list[int]]:
    """Contiguous GPU slices, one per replica."""
    if available is None:
        env = os.environ.get("CUDA_VISIBLE_DEVICES")
        if env:
            available = [int(x) for x in env.split(",") if x.strip() != ""]
        else:
            available = list(range(torch.cuda.device_count() if torch.cuda.is_available() else num_replicas * parallelism))
    need = num_replicas * parallelism
    if len(available) < need:
        raise ValueError(f"{num_replicas} replicas x {parallelism} GPUs need {need} devices, {len(available)} available")
    return [available[i * parallelism : (i + 1) * parallelism] for i in range(num_replicas)]


def load_pipeline_module(path: str, validator: PipelineSecurityValidator | None = None):
    p = Path(path).resolve()
    if not p.is_file():
        raise FileNotFoundError(path)
    if validator is not None:
        validator.check_file(str(p))
        if validator.level == SecurityLevel.SANDBOX:
            return validator.loader.load_module(p.read_text(), str(p))
    name = f"tfb_pipeline_{p.stem}_{abs(hash(str(p))) % 10**8}"
    spec = importlib.util.spec_from_file_location(name, p)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    sys.path.insert(0, str(p.parent))
    try:
        spec.loader.exec_module(mod)
    finally:
        sys.path.remove(str(p.parent))
    return mod


@dataclass
class TaskResponse:
    output_path: str | None
    peak_memory_mb: float | None
    inference_time_s: float
    extra: dict | None = None


class PipelineRunner:
    def __init__(self, module, pipeline, contract: PipelineContract) -> None:
        self.module, self.pipeline, self.contract = module, pipeline, contract
        self.fn = getattr(module, contract.run_with_file)
        self.sig = inspect.signature(self.fn)
        self.accepts_kwargs = any(p.kind == p.VAR_KEYWORD for p in self.sig.parameters.values())

    def filter_kwargs(self, data: dict) -> dict:
        if self.accepts_kwargs:
            return dict(data)
        return {k: v for k, v in data.items() if k in self.sig.parameters}

    def run(self, data: dict, stop_event: threading.Event | None = None) -> Any:
        kw = self.filter_kwargs(data)
        names = list(self.sig.parameters)
        if names and names[0] in ("pipeline", "pipe"):
            kw[names[0]] = self.pipeline
        if "stop_event" in self.sig.parameters:
            kw["stop_event"] = stop_event
        out = self.fn(**kw)
        if inspect.iscoroutine(out):
            out = asyncio.run(out)
        return out


class PipelineService:
    def __init__(self, config: ServerConfig | None = None) -> None:
        self.config = config or ServerConfig()
        self.validator = PipelineSecurityValidator(self.config.security_level)
        self.module = None
        self.pipeline = None
        self.contract: PipelineContract | None = None
        self.runner: PipelineRunner | None = None
        self.task: str | None = None
        self.ppl_file: str | None = None
        self.parallelism = 1

    @property
    def ready(self) -> bool:
        return self.runner is not None

    def validate_only(self, ppl_file: str) -> dict:
        res = self.validator.validate_file(ppl_file)
        return {"passed": res.passed, "violations": [v.to_dict() for v in res.violations],
                "warnings": [v.to_dict() for v in res.warnings]}  # fmt: skip

    def start_pipeline(self, ppl_file: str, task: str | None = None, parallelism: int = 1, skip_validation=False) -> dict:
        self.ppl_file, self.task, self.parallelism = ppl_file, task, parallelism
        self.module = load_pipeline_module(ppl_file, None if skip_validation else self.validator)
        self.contract = load_contract(self.module, task, Path(ppl_file).stem)
        get = getattr(self.module, self.contract.get_pipeline)
        kw = {"parallelism": parallelism} if "parallelism" in inspect.signature(get).parameters else {}
        self.pipeline = get(**kw)
        self.runner = PipelineRunner(self.module, self.pipeline, self.contract)
        logger.info(f"pipeline {self.contract.pipeline_name} ready (tasks {list(self.contract.supported_tasks)})")
        return self.metadata()

    def metadata(self) -> dict:
        """The running pipeline as front ends and gateways should see it: the file, how it was started, and its
        contract (tasks, required inputs, typed parameters with defaults)."""
        if self.contract is None:
            return {}
        from .contract import declares_contract

        return {"pipeline_file": self.ppl_file, "parallelism": self.parallelism, "task": self.task,
                "security_level": str(self.config.security_level).upper(), "runner": type(self.runner).__name__,
                "declared_pipeline_contract": declares_contract(self.module), **self.contract.to_metadata()}  # fmt: skip

    def run_task_with_stop_event(self, data: dict, stop_event: threading.Event | None = None) -> TaskResponse:
        if self.runner is None:
            raise RuntimeError("pipeline is not started")
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
        t0 = time.perf_counter()
        out = self.runner.run(data, stop_event)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        peak = torch.cuda.max_memory_allocated() / 2**20 if torch.cuda.is_available() else None
        path, extra = out, None
        if isinstance(out, dict):
            path, extra = out.get("output_path"), out
        elif out is None:
            path = data.get("output_path")
        return TaskResponse(str(path) if path is not None else None, peak, dt, extra)

    def stop(self) -> None:
        p = self.pipeline
        if p is not None and hasattr(p, "close"):
            try:
                p.close()
            except Exception:  # noqa: BLE001
                logger.exception("pipeline close failed")
        self.pipeline = self.runner = None


# ---------------------------------------------------------------------------
# Replica pool
# ---------------------------------------------------------------------------
class ReplicaDeadError(RuntimeError):
    pass


def _replica_main(conn, ppl_file: str, task: str | None, parallelism: int, device_ids: list[int], security_level: str,
                  skip_validation: bool) -> None:  # fmt: skip
    os.environ["CUDA_VISIBLE_DEVICES"] = ",".join(str(d) for d in device_ids)
    try:
        svc = PipelineService(ServerConfig(security_level=security_level))
        meta = svc.start_pipeline(ppl_file, task, parallelism, skip_validation)
        conn.send(("ready", meta))
    except BaseException as e:  # noqa: BLE001
        conn.send(("error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
        return
    while True:
        try:
            msg = conn.recv()
        except (EOFError, OSError):
            break
        kind = msg[0]
        if kind == "shutdown":
            break
        if kind == "task":
            _, task_id, data = msg
            stop = threading.Event()
            result: dict = {}

            def work():
                try:
                    r = svc.run_task_with_stop_event(data, stop)
                    result["ok"] = (r.output_path, r.peak_memory_mb, r.inference_time_s)
                except BaseException as e:  # noqa: BLE001
                    result["error"] = f"{type(e).__name__}: {e}"

            th = threading.Thread(target=work, daemon=True)
            th.start()
            while th.is_alive():
                if conn.poll(0.05):
                    m = conn.recv()
                    if m[0] == "cancel":
                        stop.set()
                    elif m[0] == "shutdown":
                        stop.set()
                        th.join(5)
                        svc.stop()
                        return
            conn.send(("ok", task_id, result["ok"]) if "ok" in result else ("error", task_id, result["error"]))
    svc.stop()


class ReplicaHandle:
    def __init__(self, index: int, device_ids: list[int], ctx, target=_replica_main, args: tuple = ()) -> None:
        self.index, self.device_ids = index, device_ids
        self.conn, child = ctx.Pipe()
        self.process = ctx.Process(target=target, args=(child, *args), daemon=True)
        self.process.start()
        self.busy = False
        self.metadata: dict = {}
        self.lock = threading.Lock()

    def _recv(self, timeout: float):
        deadline = time.monotonic() + timeout
        while time.monotonic() < deadline:
            if self.conn.poll(0.1):
                try:
                    return self.conn.recv()
                except (EOFError, OSError) as e:
                    raise ReplicaDeadError(f"replica {self.index} pipe closed") from e
            if not self.process.is_alive():
                if self.conn.poll(0.1):
                    continue
                raise ReplicaDeadError(f"replica {self.index} exited with code {self.process.exitcode}")
        raise TimeoutError(f"replica {self.index} did not answer within {timeout} s")

    def wait_ready(self, timeout: float) -> dict:
        kind, payload = self._recv(timeout)
        if kind != "ready":
            raise ReplicaDeadError(f"replica {self.index} failed to start: {payload}")
        self.metadata = payload
        return payload

    def run_task(self, task_id: str, data: dict, stop_event: threading.Event | None, timeout: float) -> TaskResponse:
        self.conn.send(("task", task_id, data))
        deadline = time.monotonic() + timeout
        cancelled = False
        while True:
            if stop_event is not None and stop_event.is_set() and not cancelled:
                self.conn.send(("cancel", task_id))
                cancelled = True
            try:
                msg = self._recv(0.2)
            except TimeoutError:
                if time.monotonic() > deadline:
                    raise
                continue
            if msg[0] == "ok":
                path, peak, dt = msg[2]
                return TaskResponse(path, peak, dt)
            raise RuntimeError(msg[2])

    def shutdown(self) -> None:
        try:
            self.conn.send(("shutdown",))
        except (OSError, BrokenPipeError):
            pass
        self.process.join(10)
        if self.process.is_alive():
            self.process.kill()


class PipelinePool:
    def __init__(self, config: ServerConfig, task_manager=None, replica_target=_replica_main) -> None:
        self.config = config
        self.task_manager = task_manager
        self.replicas: list[ReplicaHandle] = []
        self._cv = threading.Condition()
        self._target = replica_target
        self.metadata_cache: dict = {}

    def start_all(self, ppl_file: str, task: str | None, parallelism: int, num_replicas: int, device_slices=None,
                  skip_validation: bool = False) -> None:  # fmt: skip
        slices = device_slices or resolve_replica_device_ids(num_replicas, parallelism)
        ctx = mp.get_context("spawn")
        for i, devs in enumerate(slices):
            args = (ppl_file, task, parallelism, devs, self.config.security_level, skip_validation)
            self.replicas.append(ReplicaHandle(i, devs, ctx, self._target, args))
        for r in list(self.replicas):
            try:
                self.metadata_cache = r.wait_ready(self.config.replica_start_timeout)
            except (ReplicaDeadError, TimeoutError) as e:
                logger.error(str(e))
                self._evict(r)
        if not self.replicas:
            raise RuntimeError("no pipeline replica could be started")
        if self.task_manager is not None:
            self.task_manager.set_max_concurrent_processing(len(self.replicas))

    @property
    def ready(self) -> bool:
        return bool(self.replicas)

    def metadata(self) -> dict:
        return self.metadata_cache

    def status(self) -> dict:
        return {"replicas": [{"index": r.index, "devices": r.device_ids, "busy": r.busy,
                              "alive": r.process.is_alive()} for r in self.replicas]}  # fmt: skip

    def _evict(self, r: ReplicaHandle) -> None:
        with self._cv:
            if r in self.replicas:
                self.replicas.remove(r)
            self._cv.notify_all()
        try:
            r.process.kill()
        except Exception:  # noqa: BLE001
            pass
        if self.task_manager is not None:
            self.task_manager.set_max_concurrent_processing(len(self.replicas))
            if not self.replicas:
                self.task_manager.fail_all_pending("all pipeline replicas are dead")

    def _acquire(self, timeout: float) -> ReplicaHandle:
        deadline = time.monotonic() + timeout
        with self._cv:
            while True:
                if not self.replicas:
                    raise ReplicaDeadError("all pipeline replicas are dead")
                for r in self.replicas:
                    if not r.busy:
                        r.busy = True
                        return r
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutError("no idle replica")
                self._cv.wait(min(left, 0.5))

    def run_task_with_stop_event(self, data: dict, stop_event: threading.Event | None = None) -> TaskResponse:
        r = self._acquire(self.config.task_timeout)
        try:
            return r.run_task(str(data.get("task_id", "")), data, stop_event, self.config.task_timeout)
        except ReplicaDeadError:
            self._evict(r)
            raise
        finally:
            with self._cv:
                r.busy = False
                self._cv.notify_all()

    def stop(self) -> None:
        for r in self.replicas:
            r.shutdown()
        self.replicas = []
