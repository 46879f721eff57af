"""Types of the chunk-level streaming scheduler: pipeline spec, task keys, actor protocol, metrics.

Names and fields follow the reference's public surface
(telefuser/orchestrator/streaming_pipeline_orchestrator.py:18-257) so pipeline
code written against it ports directly.
"""

from __future__ import annotations

from concurrent.futures import Future
from dataclasses import dataclass
from enum import Enum
from typing import Mapping, Protocol


class StageOrdering(str, Enum):
    NONE = "none"
    PER_SESSION_STRICT = "per_session_strict"


class StreamingActorState(str, Enum):
    RUNNING = "running"
    FAILED = "failed"
    CLOSED = "closed"


class StreamingSessionStatus(str, Enum):
    RUNNING = "running"
    CANCELLED = "cancelled"
    FAILED = "failed"
    CLOSED = "closed"


class StreamingSessionCloseReason(str, Enum):
    CANCELLED = "cancelled"
    FAILED = "failed"
    CLOSED = "closed"
    SHUTDOWN = "shutdown"


class StreamingActorBusyError(RuntimeError):
    """The actor's mailbox is full; the scheduler puts the inputs back and retries later."""


class StreamingActorFailedError(RuntimeError):
    """The actor stopped for good; every session that uses it fails."""


@dataclass(frozen=True)
class StreamingTaskKey:
    session_id: str
    session_epoch: int
    sequence_id: int
    stage_id: str
    request_id: str


@dataclass(frozen=True)
class StreamingSessionContext:
    session_id: str
    session_epoch: int


@dataclass(frozen=True)
class StreamingStageSpec:
    stage_id: str
    consumes: frozenset
    produces: frozenset
    ordering: StageOrdering = StageOrdering.PER_SESSION_STRICT
    max_in_flight_per_session: int = 1
    max_in_flight_global: int = 1
    resource_group: str | None = None

    def __post_init__(self) -> None:
        object.__setattr__(self, "consumes", frozenset(self.consumes))
        object.__setattr__(self, "produces", frozenset(self.produces))
        if not self.stage_id or not self.consumes or not self.produces:
            raise ValueError("A stage requires a non-empty ID, at least one input, and at least one output")
        if self.resource_group == "":
            raise ValueError("resource_group must be non-empty when provided")
        if self.max_in_flight_per_session < 1:
            raise ValueError("max_in_flight_per_session must be at least one")
        if self.max_in_flight_global < 1:
            raise ValueError("max_in_flight_global must be at least one")
        if self.max_in_flight_per_session > self.max_in_flight_global:
            raise ValueError("max_in_flight_per_session cannot exceed max_in_flight_global")
        if self.ordering == StageOrdering.PER_SESSION_STRICT and self.max_in_flight_per_session != 1:
            raise ValueError("PER_SESSION_STRICT stages require max_in_flight_per_session=1")


@dataclass(frozen=True)
class StreamingResourceGroupSpec:
    name: str
    max_concurrency: int = 1

    def __post_init__(self) -> None:
        if not self.name:
            raise ValueError("A resource group requires a non-empty name")
        if self.max_concurrency < 1:
            raise ValueError("max_concurrency must be at least one")


@dataclass(frozen=True)
class StreamingEdgeSpec:
    artifact: str
    target_stage: str
    source_stage: str | None = None  # None: the artifact is pushed from outside (ingress)
    capacity_per_session: int = 1

    def __post_init__(self) -> None:
        if not self.artifact or not self.target_stage:
            raise ValueError("An edge requires artifact and target_stage")
        if self.capacity_per_session < 1:
            raise ValueError("capacity_per_session must be at least one")


@dataclass(frozen=True)
class StreamingPipelineSpec:
    stages: tuple
    edges: tuple
    output_artifacts: frozenset = frozenset()
    output_capacity_per_session: int = 1
    resource_groups: tuple = ()

    def __post_init__(self) -> None:
        object.__setattr__(self, "stages", tuple(self.stages))
        object.__setattr__(self, "edges", tuple(self.edges))
        object.__setattr__(self, "output_artifacts", frozenset(self.output_artifacts))
        object.__setattr__(self, "resource_groups", tuple(self.resource_groups))
        if self.output_capacity_per_session < 1:
            raise ValueError("output_capacity_per_session must be at least one")


@dataclass(frozen=True)
class StreamingStageInvocation:
    key: StreamingTaskKey
    inputs: Mapping[str, object]
    is_first: bool
    is_last: bool


@dataclass(frozen=True)
class StreamingStageTiming:
    stage_id: str
    sequence_id: int
    inputs_ready_at: float | None
    admitted_at: float | None
    completed_at: float | None


@dataclass(frozen=True)
class StreamingLatencySummary:
    count: int
    minimum_seconds: float | None
    p50_seconds: float | None
    p95_seconds: float | None
    maximum_seconds: float | None
    mean_seconds: float | None


@dataclass(frozen=True)
class StreamingSessionMetrics:
    ingress_accepted_at: tuple
    output_emitted_at: tuple
    first_output_latency_seconds: float | None
    control_to_output_latency: StreamingLatencySummary
    chunk_period: StreamingLatencySummary


@dataclass(frozen=True)
class StreamingActorHealth:
    state: StreamingActorState
    pending_invocations: int
    failure_reason: str | None = None


@dataclass(frozen=True)
class StreamingArtifactStats:
    slot_count: int
    reference_count: int


@dataclass(frozen=True)
class StreamingSchedulerDiagnostics:
    stale_epoch_results: int
    orphaned_results: int
    duplicate_results: int
    cleanup_failures: int
    slot_leaks: int


@dataclass(frozen=True)
class StreamingStageIdleInterval:
    stage_id: str
    previous_sequence_id: int
    sequence_id: int
    idle_seconds: float
    reason: str
    missing_inputs: tuple


class StreamingStageActor(Protocol):
    def submit(self, invocation: StreamingStageInvocation) -> Future: ...

    def health(self) -> StreamingActorHealth: ...

    def barrier(self, timeout: float = 5.0) -> None: ...

    def close_session(self, context: StreamingSessionContext, reason: StreamingSessionCloseReason,
                      timeout: float = 5.0) -> None: ...  # fmt: skip

    def close(self) -> None: ...


def summarize_latencies(values) -> StreamingLatencySummary:
    vals = sorted(float(v) for v in values)
    if not vals:
        return StreamingLatencySummary(0, None, None, None, None, None)

    def pct(fraction: float) -> float:
        if len(vals) == 1:
            return vals[0]
        pos = fraction * (len(vals) - 1)
        lo = int(pos)
        hi = min(lo + 1, len(vals) - 1)
        return vals[lo] + (vals[hi] - vals[lo]) * (pos - lo)

    return StreamingLatencySummary(len(vals), vals[0], pct(0.5), pct(0.95), vals[-1], sum(vals) / len(vals))
