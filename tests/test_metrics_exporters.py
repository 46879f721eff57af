"""Metric exporters: Prometheus text, OTLP/JSON document, StatsD lines and datagrams; the configuration record."""

import json
import socket

import pytest

from telefuser_b200.metrics import (MetricRegistry, MetricsConfig, OpenTelemetryExporter, PrometheusExporter, StatsDExporter,
                                    create_metrics_config, get_exporter)  # fmt: skip


def filled_registry() -> MetricRegistry:
    reg = MetricRegistry("tfb")
    reg.counter("requests_total", "requests served").inc(3, {"route": "/v1/tasks", "code": "200"})
    reg.counter("requests_total").inc(1, {"route": "/v1/tasks", "code": "500"})
    reg.gauge("queue_depth", "tasks waiting").set(7)
    h = reg.histogram("latency_seconds", "request latency", buckets=(0.1, 1.0))
    for v in (0.05, 0.5, 0.7, 3.0):
        h.observe(v, {"stage": "dit"})
    s = reg.summary("chunk_seconds", "chunk period")
    for v in (1.0, 2.0, 3.0):
        s.observe(v)
    return reg


def test_prometheus_text_and_factory():
    reg = filled_registry()
    text = get_exporter("prometheus").export(reg)
    assert isinstance(get_exporter(), PrometheusExporter) and text == reg.to_prometheus()
    assert 'tfb_requests_total{code="200",route="/v1/tasks"} 3.0' in text and "# TYPE tfb_latency_seconds histogram" in text
    assert 'tfb_latency_seconds_bucket{stage="dit",le="+Inf"} 4' in text
    with pytest.raises(ValueError, match="unknown exporter"):
        get_exporter("graphite")


def test_opentelemetry_document_carries_every_kind():
    reg = filled_registry()
    exp = get_exporter("otel", service_name="video-service", resource={"host.name": "node-1"})
    assert isinstance(exp, OpenTelemetryExporter) and exp.content_type == "application/json"
    doc = json.loads(exp.export(reg))
    (rm,) = doc["resourceMetrics"]
    res = {a["key"]: a["value"]["stringValue"] for a in rm["resource"]["attributes"]}
    assert res == {"service.name": "video-service", "host.name": "node-1"}
    by_name = {m["name"]: m for m in rm["scopeMetrics"][0]["metrics"]}
    assert set(by_name) == {"tfb_requests_total", "tfb_queue_depth", "tfb_latency_seconds", "tfb_chunk_seconds"}
    total = by_name["tfb_requests_total"]["sum"]
    assert total["isMonotonic"] and total["aggregationTemporality"] == 2
    values = {tuple(sorted((a["key"], a["value"]["stringValue"]) for a in p["attributes"])): p["asDouble"] for p in total["dataPoints"]}
    assert values[(("code", "200"), ("route", "/v1/tasks"))] == 3.0 and values[(("code", "500"), ("route", "/v1/tasks"))] == 1.0
    assert by_name["tfb_queue_depth"]["gauge"]["dataPoints"][0]["asDouble"] == 7.0
    (hp,) = by_name["tfb_latency_seconds"]["histogram"]["dataPoints"]
    assert hp["explicitBounds"] == [0.1, 1.0] and hp["bucketCounts"] == ["1", "2", "1"] and hp["count"] == "4" and hp["sum"] == pytest.approx(4.25)
    (sp,) = by_name["tfb_chunk_seconds"]["summary"]["dataPoints"]
    assert sp["count"] == "3" and {q["quantile"]: q["value"] for q in sp["quantileValues"]}[0.5] == 2.0


def test_statsd_lines_and_datagrams_reach_a_udp_listener():
    reg = filled_registry()
    server = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
    server.bind(("127.0.0.1", 0))
    server.settimeout(5)
    exp = StatsDExporter("127.0.0.1", server.getsockname()[1], max_datagram=160)
    lines = exp.lines(reg)
    assert "tfb_requests_total:3.0|c|#code:200,route:/v1/tasks" in lines and "tfb_queue_depth:7.0|g" in lines
    assert "tfb_latency_seconds_bucket:3|g|#stage:dit,le:1.0" in lines and exp.export(reg).split("\n") == lines
    n = exp.send(reg)
    assert n > 1  # the small datagram limit forces several packets
    got = []
    for _ in range(n):
        data = server.recv(4096)
        assert len(data) <= 160
        got.extend(data.decode().split("\n"))
    server.close()
    assert got == lines


def test_metrics_config_validation_and_master_switch():
    cfg = create_metrics_config(namespace="svc", histogram_buckets=[0.1, 1, 10])
    assert isinstance(cfg, MetricsConfig) and cfg.histogram_buckets == (0.1, 1.0, 10.0) and cfg.metrics_path == "/metrics"
    off = MetricsConfig(enabled=False)
    assert not (off.enable_stage_metrics or off.enable_gpu_metrics or off.enable_http_metrics or off.enable_queue_metrics)
    for bad in (dict(gpu_metrics_interval=0), dict(histogram_buckets=[1, 1]), dict(histogram_buckets=[]), dict(metrics_path="metrics")):
        with pytest.raises(ValueError):
            MetricsConfig(**bad)
