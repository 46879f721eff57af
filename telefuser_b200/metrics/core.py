"""In-house Prometheus-compatible metric primitives and registry.

Counter / Gauge / Histogram / Summary with label sets, a namespaced `MetricRegistry` with text
exposition, per-stage contexts (`StageMetricContext`: calls, latency histogram, errors, peak
memory) and the `with_metrics` decorator for stage `process` methods.
Role parity: telefuser/metrics/collector.py:89-407, registry.py:35-485, stage_metrics.py:18-207.
"""

from __future__ import annotations

import functools
import math
import threading
import time
from bisect import bisect_left
from collections import deque

import torch

DEFAULT_BUCKETS = (0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10, 30, 60, 120, 300, 600)


def _label_key(labels: dict | None) -> tuple:
    return tuple(sorted((labels or {}).items()))


def _fmt_labels(key: tuple, extra: tuple = ()) -> str:
    items = [*key, *extra]
    if not items:
        return ""
    return "{" + ",".join(f'{k}="{v}"' for k, v in items) + "}"


class _Metric:
    kind = "untyped"

    def __init__(self, name: str, description: str = ""):
        self.name, self.description = name, description
        self._lock = threading.Lock()

    def header(self) -> list[str]:
        return [f"# HELP {self.name} {self.description}", f"# TYPE {self.name} {self.kind}"]


class Counter(_Metric):
    kind = "counter"

    def __init__(self, name, description=""):
        super().__init__(name, description)
        self._values: dict[tuple, float] = {}

    def inc(self, amount: float = 1.0, labels: dict | None = None) -> None:
        if amount < 0:
            raise ValueError("counters only go up")
        with self._lock:
            k = _label_key(labels)
            self._values[k] = self._values.get(k, 0.0) + amount

    def value(self, labels: dict | None = None) -> float:
        return self._values.get(_label_key(labels), 0.0)

    def samples(self):
        return [(self.name, k, v) for k, v in self._values.items()] or [(self.name, (), 0.0)]


class Gauge(_Metric):
    kind = "gauge"

    def __init__(self, name, description=""):
        super().__init__(name, description)
        self._values: dict[tuple, float] = {}

    def set(self, value: float, labels: dict | None = None) -> None:
        with self._lock:
            self._values[_label_key(labels)] = float(value)

    def inc(self, amount: float = 1.0, labels: dict | None = None) -> None:
        with self._lock:
            k = _label_key(labels)
            self._values[k] = self._values.get(k, 0.0) + amount

    def dec(self, amount: float = 1.0, labels: dict | None = None) -> None:
        self.inc(-amount, labels)

    def value(self, labels: dict | None = None) -> float:
        return self._values.get(_label_key(labels), 0.0)

    def samples(self):
        return [(self.name, k, v) for k, v in self._values.items()] or [(self.name, (), 0.0)]


class Histogram(_Metric):
    kind = "histogram"

    def __init__(self, name, description="", buckets=DEFAULT_BUCKETS):
        super().__init__(name, description)
        self.buckets = tuple(sorted(buckets))
        self._data: dict[tuple, list] = {}

    def observe(self, value: float, labels: dict | None = None) -> None:
        with self._lock:
            d = self._data.setdefault(_label_key(labels), [[0] * (len(self.buckets) + 1), 0.0, 0])
            d[0][bisect_left(self.buckets, value)] += 1
            d[1] += value
            d[2] += 1

    def count(self, labels: dict | None = None) -> int:
        d = self._data.get(_label_key(labels))
        return 0 if d is None else d[2]

    def sum(self, labels: dict | None = None) -> float:
        d = self._data.get(_label_key(labels))
        return 0.0 if d is None else d[1]

    def samples(self):
        out = []
        for k, (counts, total, n) in self._data.items():
            acc = 0
            for b, c in zip(self.buckets, counts):
                acc += c
                out.append((self.name + "_bucket", (*k, ("le", repr(float(b)))), acc))
            out.append((self.name + "_bucket", (*k, ("le", "+Inf")), n))
            out.append((self.name + "_sum", k, total))
            out.append((self.name + "_count", k, n))
        return out


class Summary(_Metric):
    kind = "summary"

    def __init__(self, name, description="", window: int = 1024, quantiles=(0.5, 0.9, 0.95, 0.99)):
        super().__init__(name, description)
        self.quantiles = quantiles
        self._window = window
        self._data: dict[tuple, list] = {}

    def observe(self, value: float, labels: dict | None = None) -> None:
        with self._lock:
            d = self._data.setdefault(_label_key(labels), [deque(maxlen=self._window), 0.0, 0])
            d[0].append(value)
            d[1] += value
            d[2] += 1

    def quantile(self, q: float, labels: dict | None = None) -> float:
        d = self._data.get(_label_key(labels))
        if d is None or not d[0]:
            return math.nan
        vals = sorted(d[0])
        return vals[min(len(vals) - 1, int(q * (len(vals) - 1) + 0.5))]

    def samples(self):
        out = []
        for k, (_, total, n) in self._data.items():
            for q in self.quantiles:
                out.append((self.name, (*k, ("quantile", str(q))), self.quantile(q, dict(k))))
            out.append((self.name + "_sum", k, total))
            out.append((self.name + "_count", k, n))
        return out


class StageMetricContext:
    """Metrics of one pipeline stage; use `with ctx.measure():` or the `with_metrics` decorator."""

    def __init__(self, registry: "MetricRegistry", stage: str):
        self.stage = stage
        lab = {"stage": stage}
        self._labels = lab
        self.calls = registry.counter("stage_calls_total", "Stage invocations")
        self.errors = registry.counter("stage_errors_total", "Stage invocations that raised")
        self.latency = registry.histogram("stage_latency_seconds", "Stage wall time")
        self.peak_memory = registry.gauge("stage_peak_memory_mb", "Peak device memory during the last call")

    class _Measure:
        def __init__(self, ctx):
            self.ctx = ctx

        def __enter__(self):
            if torch.cuda.is_available():
                torch.cuda.reset_peak_memory_stats()
            self.t0 = time.perf_counter()
            return self

        def __exit__(self, et, ev, tb):
            c = self.ctx
            c.calls.inc(labels=c._labels)
            c.latency.observe(time.perf_counter() - self.t0, c._labels)
            if et is not None:
                c.errors.inc(labels=c._labels)
            if torch.cuda.is_available():
                c.peak_memory.set(torch.cuda.max_memory_allocated() / 2**20, c._labels)
            return False

    def measure(self):
        return self._Measure(self)


class MetricRegistry:
    def __init__(self, namespace: str = "telefuser"):
        self.namespace = namespace
        self._metrics: dict[str, _Metric] = {}
        self._stages: dict[str, StageMetricContext] = {}
        self._lock = threading.Lock()

    def _get(self, cls, name, description, **kw):
        full = f"{self.namespace}_{name}" if self.namespace else name
        with self._lock:
            m = self._metrics.get(full)
            if m is None:
                m = self._metrics[full] = cls(full, description, **kw)
            elif not isinstance(m, cls):
                raise TypeError(f"{full} already registered as {type(m).__name__}")
            return m

    def counter(self, name, description="") -> Counter:
        return self._get(Counter, name, description)

    def gauge(self, name, description="") -> Gauge:
        return self._get(Gauge, name, description)

    def histogram(self, name, description="", buckets=DEFAULT_BUCKETS) -> Histogram:
        return self._get(Histogram, name, description, buckets=buckets)

    def summary(self, name, description="") -> Summary:
        return self._get(Summary, name, description)

    def register_stage(self, stage: str) -> StageMetricContext:
        if stage not in self._stages:
            self._stages[stage] = StageMetricContext(self, stage)
        return self._stages[stage]

    def to_prometheus(self) -> str:
        lines = []
        for m in self._metrics.values():
            lines.extend(m.header())
            for name, key, value in m.samples():
                lines.append(f"{name}{_fmt_labels(key)} {value}")
        return "\n".join(lines) + "\n"

    def to_dict(self) -> dict:
        out = {}
        for m in self._metrics.values():
            out[m.name] = {"type": m.kind, "samples": [{"name": n, "labels": dict(k), "value": v}
                                                      for n, k, v in m.samples()]}  # fmt: skip
        return out

    def reset(self) -> None:
        with self._lock:
            self._metrics.clear()
            self._stages.clear()


_GLOBAL = MetricRegistry()


def get_metrics_registry() -> MetricRegistry:
    return _GLOBAL


def with_metrics(fn):
    """Decorator for stage methods: records into the stage's metric context when metrics are enabled."""

    @functools.wraps(fn)
    def wrapper(self, *a, **k):
        hook = getattr(self, "metrics_hook", None)
        if hook is None:
            return fn(self, *a, **k)
        with hook.measure():
            return fn(self, *a, **k)

    return wrapper
