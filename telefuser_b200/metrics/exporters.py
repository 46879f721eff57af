"""Metric exporters and the metrics configuration record.

Three wire formats over one `MetricRegistry`:
  * Prometheus text exposition (what `GET /metrics` serves);
  * OpenTelemetry: the OTLP/JSON `resourceMetrics` document (sum / gauge / histogram / summary data points), ready
    to POST to a collector's `/v1/metrics` or to write to a file;
  * StatsD / DogStatsD lines (`name:value|type|#tag:value`), optionally sent as UDP datagrams.
Role parity: telefuser/metrics/exporters.py:17-113 (there the OpenTelemetry and StatsD exporters only format
placeholders), telefuser/metrics/config.py:14-111.
"""

from __future__ import annotations

import json
import socket
import time
from dataclasses import dataclass, field

from .core import Counter, Gauge, Histogram, MetricRegistry, Summary

DEFAULT_HISTOGRAM_BUCKETS = (0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0)


@dataclass
class MetricsConfig:
    """Which metric families are collected and how they are exposed."""

    enabled: bool = True
    enable_stage_metrics: bool = True
    enable_gpu_metrics: bool = True
    enable_http_metrics: bool = True
    enable_queue_metrics: bool = True
    gpu_metrics_interval: float = 5.0  # seconds between NVML samples
    histogram_buckets: tuple = field(default_factory=lambda: DEFAULT_HISTOGRAM_BUCKETS)
    metrics_path: str = "/metrics"
    namespace: str = "telefuser"

    def __post_init__(self) -> None:
        self.histogram_buckets = tuple(float(b) for b in self.histogram_buckets)
        if self.gpu_metrics_interval <= 0:
            raise ValueError(f"gpu_metrics_interval is a period in seconds, got {self.gpu_metrics_interval}")
        if not self.histogram_buckets or list(self.histogram_buckets) != sorted(set(self.histogram_buckets)):
            raise ValueError("histogram_buckets must be a non-empty, strictly increasing sequence")
        if not self.metrics_path.startswith("/"):
            raise ValueError(f"metrics_path is a URL path and starts with '/', got {self.metrics_path!r}")
        if not self.enabled:  # the master switch wins over the per-family ones
            self.enable_stage_metrics = self.enable_gpu_metrics = self.enable_http_metrics = self.enable_queue_metrics = False


def create_metrics_config(**overrides) -> MetricsConfig:
    return MetricsConfig(**overrides)


class MetricsExporter:
    """Turns the registry's current state into one payload (a string) in the exporter's wire format."""

    content_type = "text/plain"

    def export(self, registry: MetricRegistry) -> str:
        raise NotImplementedError


class PrometheusExporter(MetricsExporter):
    content_type = "text/plain; version=0.0.4; charset=utf-8"

    def export(self, registry: MetricRegistry) -> str:
        return registry.to_prometheus()


def _attributes(key: tuple) -> list[dict]:
    return [{"key": k, "value": {"stringValue": str(v)}} for k, v in key]


class OpenTelemetryExporter(MetricsExporter):
    """OTLP/JSON. Counters become monotonic cumulative sums, histograms keep their explicit bounds, summaries their
    quantiles."""

    content_type = "application/json"

    def __init__(self, service_name: str = "telefuser", resource: dict | None = None) -> None:
        self.resource = {"service.name": service_name, **(resource or {})}

    def to_document(self, registry: MetricRegistry) -> dict:
        now = str(time.time_ns())
        metrics = []
        for m in registry._metrics.values():
            entry = {"name": m.name, "description": m.description}
            if isinstance(m, Counter):
                entry["sum"] = {"aggregationTemporality": 2, "isMonotonic": True,
                                "dataPoints": [{"attributes": _attributes(k), "timeUnixNano": now, "asDouble": v}
                                               for _, k, v in m.samples()]}  # fmt: skip
            elif isinstance(m, Gauge):
                entry["gauge"] = {"dataPoints": [{"attributes": _attributes(k), "timeUnixNano": now, "asDouble": v}
                                                 for _, k, v in m.samples()]}  # fmt: skip
            elif isinstance(m, Histogram):
                entry["histogram"] = {"aggregationTemporality": 2, "dataPoints": [
                    {"attributes": _attributes(k), "timeUnixNano": now, "count": str(n), "sum": total,
                     "bucketCounts": [str(c) for c in counts], "explicitBounds": list(m.buckets)}
                    for k, (counts, total, n) in m._data.items()]}  # fmt: skip
            elif isinstance(m, Summary):
                entry["summary"] = {"dataPoints": [
                    {"attributes": _attributes(k), "timeUnixNano": now, "count": str(n), "sum": total,
                     "quantileValues": [{"quantile": q, "value": m.quantile(q, dict(k))} for q in m.quantiles]}
                    for k, (_, total, n) in m._data.items()]}  # fmt: skip
            else:
                continue
            metrics.append(entry)
        return {"resourceMetrics": [{"resource": {"attributes": _attributes(tuple(self.resource.items()))},
                                     "scopeMetrics": [{"scope": {"name": "telefuser_b200.metrics"}, "metrics": metrics}]}]}  # fmt: skip

    def export(self, registry: MetricRegistry) -> str:
        return json.dumps(self.to_document(registry))


class StatsDExporter(MetricsExporter):
    """One line per sample: counters as `|c`, gauges as `|g`, histogram and summary sums / counts as gauges and their
    buckets / quantiles as tagged gauges. `send()` ships the lines as UDP datagrams of at most `max_datagram` bytes."""

    def __init__(self, host: str = "127.0.0.1", port: int = 8125, max_datagram: int = 1400) -> None:
        self.host, self.port, self.max_datagram = host, port, max_datagram

    @staticmethod
    def _line(name: str, key: tuple, value, kind: str) -> str:
        tags = ",".join(f"{k}:{v}" for k, v in key)
        return f"{name.replace(' ', '_')}:{value}|{kind}" + (f"|#{tags}" if tags else "")

    def lines(self, registry: MetricRegistry) -> list[str]:
        out = []
        for m in registry._metrics.values():
            kind = "c" if isinstance(m, Counter) else "g"
            out.extend(self._line(name, key, value, kind) for name, key, value in m.samples())
        return out

    def export(self, registry: MetricRegistry) -> str:
        return "\n".join(self.lines(registry))

    def send(self, registry: MetricRegistry, sock: socket.socket | None = None) -> int:
        """Sends the current samples; returns the number of datagrams."""
        own = sock is None
        sock = sock or socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        sent, batch, size = 0, [], 0
        try:
            for line in self.lines(registry) + [None]:
                if line is None or (batch and size + len(line) + 1 > self.max_datagram):
                    if batch:
                        sock.sendto("\n".join(batch).encode(), (self.host, self.port))
                        sent += 1
                    batch, size = [], 0
                if line is not None:
                    batch.append(line)
                    size += len(line) + 1
        finally:
            if own:
                sock.close()
        return sent


_EXPORTERS = {"prometheus": PrometheusExporter, "opentelemetry": OpenTelemetryExporter, "otel": OpenTelemetryExporter,
              "statsd": StatsDExporter}  # fmt: skip


def get_exporter(exporter_type: str = "prometheus", **kwargs) -> MetricsExporter:
    try:
        return _EXPORTERS[exporter_type.lower()](**kwargs)
    except KeyError:
        raise ValueError(f"unknown exporter {exporter_type!r}; known: {sorted(set(_EXPORTERS))}") from None


__all__ = ["MetricsConfig", "create_metrics_config", "MetricsExporter", "PrometheusExporter", "OpenTelemetryExporter",
           "StatsDExporter", "get_exporter", "DEFAULT_HISTOGRAM_BUCKETS"]  # fmt: skip
