"""Three-layer profiling support.

1. Stage timing + memory (`TELEFUSER_PROFILE_DEBUG=true`): `ProfilingContext4Debug(name)` is a
   decorator / context manager (sync and async). Timing uses CUDA events on the current stream
   (no device-wide synchronise in steady state; the events are resolved when a report is built),
   host wall time as a fallback on CPU, and a memory snapshot (allocated / reserved / peak).
   Records go to the process-global `GlobalTimingRegistry`; worker ranks dump theirs as JSON into
   `_TELEFUSER_WORKER_TIMING_DIR` and the parent merges them, taking the max over ranks.
2. Kernel traces (`ENABLE_PROFILER_NAMES=denoise,vae`): the named stages run under
   `torch.profiler` and export a chrome trace plus a per-kernel table.
3. `ncu`: run externally; `summarize_ncu_csv` condenses `ncu --page raw --csv` output to the
   roofline figures (duration, DRAM bytes, tensor-pipe activity, stalls).

Role parity: telefuser/utils/profiler.py (stage timing :288-551, context :661-840, torch.profiler
:173-244, ncu helpers :967-1079) and telefuser/utils/memory_snapshot.py.
"""

from __future__ import annotations

import atexit
import csv
import functools
import glob
import inspect
import json
import os
import threading
import time
from dataclasses import asdict, dataclass, field

import torch

_IS_WORKER = False


def mark_as_worker_process() -> None:
    global _IS_WORKER
    _IS_WORKER = True


def is_worker_process() -> bool:
    return _IS_WORKER


def profiling_enabled() -> bool:
    return os.environ.get("TELEFUSER_PROFILE_DEBUG", "false").lower() in ("1", "true", "yes")


def profiler_names() -> set[str]:
    return {n.strip() for n in os.environ.get("ENABLE_PROFILER_NAMES", "").split(",") if n.strip()}


@dataclass
class MemorySnapshot:
    allocated_mb: float = 0.0
    reserved_mb: float = 0.0
    peak_allocated_mb: float = 0.0
    fragmentation: float = 0.0

    @classmethod
    def capture(cls, device=None) -> "MemorySnapshot":
        if not torch.cuda.is_available():
            return cls()
        a = torch.cuda.memory_allocated(device) / 2**20
        r = torch.cuda.memory_reserved(device) / 2**20
        p = torch.cuda.max_memory_allocated(device) / 2**20
        return cls(a, r, p, 0.0 if r == 0 else 1.0 - a / r)


@dataclass
class TimingRecord:
    name: str
    wall_ms: float
    device_ms: float | None = None
    mem_before: MemorySnapshot | None = None
    mem_after: MemorySnapshot | None = None
    io_signature: dict = field(default_factory=dict)
    rank: int = 0


def describe_value(v):
    """Shape/dtype signature of an argument (used to replay one stage call with random tensors)."""
    if isinstance(v, torch.Tensor):
        return {"tensor": list(v.shape), "dtype": str(v.dtype), "device": v.device.type}
    if isinstance(v, (int, float, bool, str)) or v is None:
        return v
    if isinstance(v, (list, tuple)):
        return [describe_value(x) for x in v[:16]]
    if isinstance(v, dict):
        return {str(k): describe_value(x) for k, x in list(v.items())[:32]}
    return type(v).__name__


class GlobalTimingRegistry:
    _instance: "GlobalTimingRegistry | None" = None

    def __init__(self) -> None:
        self._lock = threading.Lock()
        self._records: list[TimingRecord] = []
        self._pending: list[tuple[TimingRecord, torch.cuda.Event, torch.cuda.Event]] = []

    @classmethod
    def instance(cls) -> "GlobalTimingRegistry":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def reset(self) -> None:
        with self._lock:
            self._records.clear()
            self._pending.clear()

    def add(self, rec: TimingRecord, events=None) -> None:
        with self._lock:
            if events is not None:
                self._pending.append((rec, *events))
            self._records.append(rec)

    def resolve(self) -> None:
        """Turns recorded CUDA event pairs into device milliseconds (waits for the events only)."""
        with self._lock:
            pending, self._pending = self._pending, []
        for rec, e0, e1 in pending:
            e1.synchronize()
            rec.device_ms = e0.elapsed_time(e1)

    def records(self) -> list[TimingRecord]:
        self.resolve()
        with self._lock:
            return list(self._records)

    def summary(self) -> dict:
        out: dict[str, dict] = {}
        for r in self.records():
            s = out.setdefault(r.name, {"count": 0, "wall_ms": 0.0, "device_ms": 0.0, "peak_mb": 0.0})
            s["count"] += 1
            s["wall_ms"] += r.wall_ms
            s["device_ms"] += r.device_ms or 0.0
            if r.mem_after is not None:
                s["peak_mb"] = max(s["peak_mb"], r.mem_after.peak_allocated_mb)
        return out

    def export(self, path: str) -> str:
        data = {"summary": self.summary(), "records": [asdict(r) for r in self.records()]}
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            json.dump(data, f, indent=2, default=str)
        return path

    def dump_worker_file(self) -> str | None:
        d = os.environ.get("_TELEFUSER_WORKER_TIMING_DIR")
        if not d:
            return None
        rank = int(os.environ.get("RANK", "0"))
        return self.export(os.path.join(d, f"timing_rank{rank}_{os.getpid()}.json"))


def merge_worker_timing(directory: str) -> dict:
    """Merges per-rank timing files: per stage, the max over ranks of the summed device time."""
    merged: dict[str, dict] = {}
    for f in sorted(glob.glob(os.path.join(directory, "timing_rank*.json"))):
        with open(f) as fh:
            for name, s in json.load(fh)["summary"].items():
                m = merged.setdefault(name, {"count": 0, "wall_ms": 0.0, "device_ms": 0.0, "peak_mb": 0.0})
                m["count"] = max(m["count"], s["count"])
                for k in ("wall_ms", "device_ms", "peak_mb"):
                    m[k] = max(m[k], s[k])
    return merged


class _NullContext:
    def __init__(self, *a, **k):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def __call__(self, fn):
        return fn


class ProfilingContext4Debug:
    """`with ProfilingContext4Debug("vae"):` or `@ProfilingContext4Debug("dit_denoise")` (sync or async def)."""

    def __new__(cls, name: str = "", *args, **kwargs):
        if not profiling_enabled() and not (profiler_names() and any(n in name for n in profiler_names())):
            return _NullContext()
        return super().__new__(cls)

    def __init__(self, name: str, capture_io: bool = True):
        self.name = name
        self.capture_io = capture_io
        self._io: dict = {}
        self._prof = None

    def __enter__(self):
        self._mem0 = MemorySnapshot.capture()
        self._events = None
        if torch.cuda.is_available():
            torch.cuda.reset_peak_memory_stats()
            self._events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._events[0].record()
        if any(n in self.name for n in profiler_names()):
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(
                activities=acts,
                record_shapes=os.environ.get("TELEFUSER_TORCH_PROFILER_RECORD_SHAPES", "0") == "1",
                profile_memory=os.environ.get("TELEFUSER_TORCH_PROFILER_PROFILE_MEMORY", "0") == "1",
                with_stack=os.environ.get("TELEFUSER_TORCH_PROFILER_WITH_STACK", "0") == "1")  # fmt: skip
            self._prof.__enter__()
        self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        wall = (time.perf_counter() - self._t0) * 1e3
        if self._events is not None:
            self._events[1].record()
        if self._prof is not None:
            self._prof.__exit__(*exc)
            self._export_trace()
        rec = TimingRecord(self.name, wall, None, self._mem0, MemorySnapshot.capture(), self._io,
                           int(os.environ.get("RANK", "0")))  # fmt: skip
        GlobalTimingRegistry.instance().add(rec, self._events)
        return False

    def _export_trace(self) -> None:
        out = os.path.join("work_dirs", "profiler_output", os.environ.get("TELEFUSER_PIPELINE_NAME", "pipeline"),
                           time.strftime("%Y%m%d_%H%M"))  # fmt: skip
        os.makedirs(out, exist_ok=True)
        self._prof.export_chrome_trace(os.path.join(out, f"{self.name}_rank{os.environ.get('RANK', '0')}.json"))
        with open(os.path.join(out, f"{self.name}_kernels.txt"), "w") as f:
            f.write(self._prof.key_averages().table(sort_by="cuda_time_total" if torch.cuda.is_available()
                                                    else "cpu_time_total", row_limit=50))  # fmt: skip

    def __call__(self, fn):
        if inspect.iscoroutinefunction(fn):
            @functools.wraps(fn)
            async def awrapper(*args, **kwargs):
                with self._fresh(args, kwargs):
                    return await fn(*args, **kwargs)

            return awrapper

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            with self._fresh(args, kwargs):
                return fn(*args, **kwargs)

        return wrapper

    def _fresh(self, args, kwargs):
        ctx = ProfilingContext4Debug(self.name, self.capture_io)
        if isinstance(ctx, ProfilingContext4Debug) and self.capture_io:
            ctx._io = {"args": [describe_value(a) for a in args[1:]],
                       "kwargs": {k: describe_value(v) for k, v in kwargs.items()}}  # fmt: skip
        return ctx


def compare_timing_reports(path_a: str, path_b: str) -> dict:
    """Per-stage ratio b/a of device (or wall) time between two exported reports."""
    with open(path_a) as fa, open(path_b) as fb:
        a, b = json.load(fa)["summary"], json.load(fb)["summary"]
    out = {}
    for name in sorted(set(a) & set(b)):
        ta = a[name]["device_ms"] or a[name]["wall_ms"]
        tb = b[name]["device_ms"] or b[name]["wall_ms"]
        out[name] = {"a_ms": ta, "b_ms": tb, "ratio": (tb / ta) if ta else None}
    return out


NCU_KEYS = (
    "gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum", "gpu__dram_throughput",
    "sm__pipe_tensor_cycles_active", "sm__warps_active", "launch__registers_per_thread",
    "sm__cycles_elapsed.avg.per_second", "smsp__issue_active", "sm__inst_executed_pipe_xu",
)  # fmt: skip


def summarize_ncu_csv(path: str, keys=NCU_KEYS) -> list[dict]:
    """Condenses `ncu -i report --page raw --csv` output: one dict per captured launch."""
    with open(path, newline="") as f:
        rows = list(csv.reader(f))
    if len(rows) < 3:
        return []
    header, units = rows[0], rows[1]
    out = []
    for row in rows[2:]:
        d = {}
        for h, u, v in zip(header, units, row):
            if h in ("Kernel Name", "ID") or any(h.startswith(k) for k in keys):
                d[h] = f"{v} {u}".strip()
        out.append(d)
    return out


def _auto_export() -> None:
    target = os.environ.get("TELEFUSER_TIMING_REPORT")
    reg = GlobalTimingRegistry.instance()
    if _IS_WORKER:
        reg.dump_worker_file()
    elif target and reg._records:
        reg.export(target)


atexit.register(_auto_export)
