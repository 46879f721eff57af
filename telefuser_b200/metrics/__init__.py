from .core import (Counter, Gauge, Histogram, MetricRegistry, StageMetricContext, Summary, get_metrics_registry,
                   with_metrics)  # fmt: skip
from .service_metrics import (GPUCollector, ServiceMetrics, collect_runtime_environment, finish_runtime_measurement,
                              start_runtime_measurement)  # fmt: skip
from .exporters import (MetricsConfig, MetricsExporter, OpenTelemetryExporter, PrometheusExporter, StatsDExporter,
                        create_metrics_config, get_exporter)  # fmt: skip
