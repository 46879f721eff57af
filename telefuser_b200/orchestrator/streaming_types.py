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


# ---- failures the scheduler distinguishes ----

class StreamingActorBusyError(RuntimeError):
    """The actor's mailbox is full; the scheduler puts the inputs back and retries later."""


class StreamingActorFailedError(RuntimeError):
    """The actor stopped for good; every session that uses it fails."""


# ---- states ----

class StreamingSessionStatus(str, Enum):
    """Where a session is; anything but RUNNING is final."""

    RUNNING = "running"
    CANCELLED = "cancelled"
    FAILED = "failed"
    CLOSED = "closed"


class StreamingSessionCloseReason(str, Enum):
    """Why `close_session` is being called on an actor (it decides what the actor may drop)."""

    CANCELLED = "cancelled"
    FAILED = "failed"
    CLOSED = "closed"
    SHUTDOWN = "shutdown"


class StreamingActorState(str, Enum):
    """Life cycle of a stage actor as reported by `health()`."""

    RUNNING = "running"
    FAILED = "failed"
    CLOSED = "closed"


class StageOrdering(str, Enum):
    """How the chunks of ONE session may overlap inside a stage."""

    NONE = "none"
    PER_SESSION_STRICT = "per_session_strict"


# ---- identities ----

@dataclass(frozen=True)
class StreamingSessionContext:
    """A session and its epoch; results that carry an older epoch are stale and are discarded."""

    session_id: str
    session_epoch: int


@dataclass(frozen=True)
class StreamingTaskKey:
    """Identity of one stage run: which session (and which incarnation of it), which chunk, which stage, plus a
    unique request id that makes duplicates detectable."""

    session_id: str
    session_epoch: int
    sequence_id: int
    stage_id: str
    request_id: str


@dataclass(frozen=True)
class StreamingStageInvocation:
    """What an actor receives: the key, the input artifacts by name, and whether this is the session's first / last
    chunk."""

    key: StreamingTaskKey
    inputs: Mapping[str, object]
    is_first: bool
    is_last: bool


# ---- measurements ----

@dataclass(frozen=True)
class StreamingLatencySummary:
    """Order statistics of a list of durations; every field is None when the list was empty."""

    count: int
    minimum_seconds: float | None
    p50_seconds: float | None
    p95_seconds: float | None
    maximum_seconds: float | None
    mean_seconds: float | None


def summarize_latencies(values) -> StreamingLatencySummary:
    """Count, min, median, p95 (linear interpolation), max and mean of `values`."""
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


@dataclass(frozen=True)
class StreamingStageTiming:
    """Three timestamps of one stage run (monotonic seconds): inputs complete, admitted to the actor, result back."""

    stage_id: str
    sequence_id: int
    inputs_ready_at: float | None
    admitted_at: float | None
    completed_at: float | None


@dataclass(frozen=True)
class StreamingStageIdleInterval:
    """A gap between two consecutive runs of a stage, with the reason (e.g. which inputs it was waiting for)."""

    stage_id: str
    previous_sequence_id: int
    sequence_id: int
    idle_seconds: float
    reason: str
    missing_inputs: tuple


@dataclass(frozen=True)
class StreamingSessionMetrics:
    """Per-session measurements the scheduler keeps: when each chunk entered and left, and the two latency
    summaries built from them."""

    ingress_accepted_at: tuple
    output_emitted_at: tuple
    first_output_latency_seconds: float | None
    control_to_output_latency: StreamingLatencySummary
    chunk_period: StreamingLatencySummary


@dataclass(frozen=True)
class StreamingArtifactStats:
    """Slots currently allocated for a session and the references still held on them (both zero after a clean
    close)."""

    slot_count: int
    reference_count: int


@dataclass(frozen=True)
class StreamingSchedulerDiagnostics:
    """Counters of everything the scheduler had to drop or could not clean up; all zero in a healthy run."""

    stale_epoch_results: int
    orphaned_results: int
    duplicate_results: int
    cleanup_failures: int
    slot_leaks: int


@dataclass(frozen=True)
class StreamingActorHealth:
    """Snapshot an actor returns: state, mailbox depth and, once failed, why."""

    state: StreamingActorState
    pending_invocations: int
    failure_reason: str | None = None


# ---- the graph ----

def _positive(owner: str, **limits: int) -> None:
    """Every keyword is a capacity / concurrency limit of `owner` and has to be 1 or more."""
    for field_name, value in limits.items():
        if int(value) < 1:
            raise ValueError(f"{owner}: {field_name}={value!r} is not a positive count")


def _freeze(obj, **collections) -> None:
    """Stores normalised immutable collections on a frozen dataclass instance."""
    for field_name, value in collections.items():
        object.__setattr__(obj, field_name, value)


@dataclass(frozen=True)
class StreamingResourceGroupSpec:
    """A named pool that several stages draw from, e.g. stages that share one GPU."""

    name: str
    max_concurrency: int = 1

    def __post_init__(self) -> None:
        if not self.name:
            raise ValueError("a resource group is looked up by name; it cannot be empty")
        _positive(f"resource group {self.name!r}", max_concurrency=self.max_concurrency)


@dataclass(frozen=True)
class StreamingEdgeSpec:
    """Routing of one artifact to one consuming stage, with the number of slots a session may hold on that edge."""

    artifact: str
    target_stage: str
    source_stage: str | None = None  # None: the artifact is pushed from outside (ingress)
    capacity_per_session: int = 1

    def __post_init__(self) -> None:
        if not (self.artifact and self.target_stage):
            raise ValueError(f"edge {self.artifact!r} -> {self.target_stage!r}: both the artifact and the consuming stage must be named")
        _positive(f"edge {self.artifact!r} -> {self.target_stage!r}", capacity_per_session=self.capacity_per_session)


@dataclass(frozen=True)
class StreamingStageSpec:
    """One node of the graph: the artifacts it waits for and makes, how many of its runs may be in flight, and the
    resource group (shared device, shared lock) it competes in."""

    stage_id: str
    consumes: frozenset
    produces: frozenset
    ordering: StageOrdering = StageOrdering.PER_SESSION_STRICT
    max_in_flight_per_session: int = 1
    max_in_flight_global: int = 1
    resource_group: str | None = None

    def __post_init__(self) -> None:
        _freeze(self, consumes=frozenset(self.consumes), produces=frozenset(self.produces))
        label = f"stage {self.stage_id!r}"
        missing = [what for what, have in (("an id", self.stage_id), ("an input artifact", self.consumes),
                                           ("an output artifact", self.produces)) if not have]  # fmt: skip
        if missing:
            raise ValueError(f"{label} lacks {' and '.join(missing)}")
        if self.resource_group is not None and not self.resource_group:
            raise ValueError(f"{label}: an empty string does not name a resource group (use None for no group)")
        _positive(label, max_in_flight_per_session=self.max_in_flight_per_session,
                  max_in_flight_global=self.max_in_flight_global)  # fmt: skip
        per_session, overall = self.max_in_flight_per_session, self.max_in_flight_global
        if per_session > overall:
            raise ValueError(f"{label}: {per_session} chunks in flight per session cannot fit the overall limit {overall}")
        if self.ordering is StageOrdering.PER_SESSION_STRICT and per_session > 1:
            raise ValueError(f"{label}: strict per-session ordering runs one chunk of a session at a time, not {per_session}")


@dataclass(frozen=True)
class StreamingPipelineSpec:
    """The whole graph: stages, edges, which artifacts leave the pipeline and how many finished outputs may wait
    per session."""

    stages: tuple
    edges: tuple
    output_artifacts: frozenset = frozenset()
    output_capacity_per_session: int = 1
    resource_groups: tuple = ()

    def __post_init__(self) -> None:
        _freeze(self, stages=tuple(self.stages), edges=tuple(self.edges),
                output_artifacts=frozenset(self.output_artifacts), resource_groups=tuple(self.resource_groups))  # fmt: skip
        _positive("pipeline", output_capacity_per_session=self.output_capacity_per_session)


# ---- the actor side ----

class StreamingStageActor(Protocol):
    """What the scheduler needs from an actor, whether it is a thread in this process or a group of worker ranks."""

    def submit(self, invocation: StreamingStageInvocation) -> Future: ...

    def health(self) -> StreamingActorHealth: ...

    def barrier(self, timeout: float = 5.0) -> None: ...

    def close_session(self, context: StreamingSessionContext, reason: StreamingSessionCloseReason,
                      timeout: float = 5.0) -> None: ...  # fmt: skip

    def close(self) -> None: ...
