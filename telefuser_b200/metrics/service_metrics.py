"""Service-level metrics: requests, queue depth, task durations and GPU utilisation / memory via NVML.

Role parity: telefuser/metrics/service_metrics.py:19-436 and metrics/runtime.py:58-95
(`start/finish_runtime_measurement`, `collect_runtime_environment`).
"""

from __future__ import annotations

import platform
import subprocess
import threading
import time

import torch

from .core import MetricRegistry, get_metrics_registry


class GPUCollector:
    """Polls NVML (read-only) for utilisation and memory of the visible GPUs."""

    def __init__(self, nvml=None):
        self._nvml = nvml
        self._ok = False
        try:
            if self._nvml is None:
                import pynvml

                self._nvml = pynvml
            self._nvml.nvmlInit()
            self._ok = True
        except Exception:  # noqa: BLE001 - no NVML on this machine
            self._ok = False

    def sample(self) -> list[dict]:
        if not self._ok:
            return []
        out = []
        n = self._nvml.nvmlDeviceGetCount()
        for i in range(n):
            h = self._nvml.nvmlDeviceGetHandleByIndex(i)
            util = self._nvml.nvmlDeviceGetUtilizationRates(h)
            mem = self._nvml.nvmlDeviceGetMemoryInfo(h)
            out.append({"index": i, "util": float(util.gpu), "mem_used_mb": mem.used / 2**20,
                        "mem_total_mb": mem.total / 2**20})  # fmt: skip
        return out


class ServiceMetrics:
    def __init__(self, registry: MetricRegistry | None = None, gpu_collector: GPUCollector | None = None):
        r = registry or get_metrics_registry()
        self.registry = r
        self.requests = r.counter("http_requests_total", "HTTP requests")
        self.request_latency = r.histogram("http_request_seconds", "HTTP request latency")
        self.tasks = r.counter("tasks_total", "Tasks by final status")
        self.task_seconds = r.histogram("task_seconds", "Task processing time")
        self.queue_depth = r.gauge("task_queue_depth", "Pending tasks")
        self.processing = r.gauge("tasks_processing", "Tasks being processed")
        self.gpu_util = r.gauge("gpu_utilization_percent", "GPU utilisation")
        self.gpu_mem = r.gauge("gpu_memory_used_mb", "GPU memory in use")
        self.stream_sessions = r.gauge("stream_sessions", "Open streaming sessions")
        self.chunk_period = r.summary("stream_chunk_period_seconds", "Time between emitted chunks")
        self._gpu = gpu_collector
        self._thread = None
        self._stop = threading.Event()

    def record_request(self, method: str, path: str, status: int, seconds: float) -> None:
        lab = {"method": method, "path": path, "status": str(status)}
        self.requests.inc(labels=lab)
        self.request_latency.observe(seconds, {"method": method, "path": path})

    def record_task(self, task_type: str, status: str, seconds: float | None = None) -> None:
        self.tasks.inc(labels={"type": task_type, "status": status})
        if seconds is not None:
            self.task_seconds.observe(seconds, {"type": task_type})

    def set_queue(self, pending: int, processing: int) -> None:
        self.queue_depth.set(pending)
        self.processing.set(processing)

    def collect_gpu_once(self) -> None:
        if self._gpu is None:
            self._gpu = GPUCollector()
        for s in self._gpu.sample():
            lab = {"gpu": str(s["index"])}
            self.gpu_util.set(s["util"], lab)
            self.gpu_mem.set(s["mem_used_mb"], lab)

    def start_gpu_polling(self, interval_s: float = 5.0) -> None:
        if self._thread is not None:
            return

        def loop():
            while not self._stop.wait(interval_s):
                try:
                    self.collect_gpu_once()
                except Exception:  # noqa: BLE001
                    pass

        self._thread = threading.Thread(target=loop, name="gpu-metrics", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()


def start_runtime_measurement(devices=()) -> dict:
    for d in devices:
        if torch.cuda.is_available():
            torch.cuda.synchronize(d)
    return {"t0": time.perf_counter(), "devices": list(devices)}


def finish_runtime_measurement(handle: dict) -> dict:
    for d in handle["devices"]:
        if torch.cuda.is_available():
            torch.cuda.synchronize(d)
    return {"wall_seconds": time.perf_counter() - handle["t0"]}


def collect_runtime_environment() -> dict:
    """Facts for `/v1/service/metadata`: versions, devices, git commit."""
    env = {"python": platform.python_version(), "torch": torch.__version__, "cuda": torch.version.cuda,
           "platform": platform.platform(), "devices": []}  # fmt: skip
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            env["devices"].append({"index": i, "name": p.name, "memory_gb": round(p.total_memory / 2**30, 1),
                                   "sm_count": p.multi_processor_count, "capability": f"{p.major}.{p.minor}"})  # fmt: skip
    try:
        env["git_commit"] = subprocess.run(["git", "rev-parse", "--short", "HEAD"], capture_output=True, text=True,
                                           timeout=2).stdout.strip() or None  # fmt: skip
    except Exception:  # noqa: BLE001
        env["git_commit"] = None
    return env
