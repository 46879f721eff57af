"""Chunk-level streaming scheduler over stage actors.

A pipeline is a DAG of stages joined by named artifacts. Every (session, sequence id)
pair flows through the DAG; an invocation of stage X for sequence n is admitted when

  * all artifacts X consumes for n are present,
  * X (and its resource group, if any) has a free execution slot,
  * every edge X produces into, and the output buffer for egress artifacts, has room,
    counting results already reserved by invocations in flight,
  * for strictly ordered stages, n is the next sequence id of that session.

Inputs are reference counted per consumer and released when the last consumer takes
them. Results are classified before use: a result whose session is unknown is an
orphan, one from an earlier incarnation of the session id (epoch) is stale, one for an
already finished task is a duplicate; none of them touches live state. A stage failure
fails the session (an actor failure fails every session); clean-up closes the session on
each actor in reverse topological order, retries failed clean-ups on a background thread
and reports artifact slots that were still referenced as leaks.

Role parity: StreamingPipelineOrchestrator,
telefuser/orchestrator/streaming_pipeline_orchestrator.py:475-1455.
"""

from __future__ import annotations

import itertools
import threading
import time
from collections import deque
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Collection, Mapping

from .streaming_types import (
    StreamingActorBusyError,
    StreamingActorFailedError,
    StreamingActorHealth,
    StreamingActorState,
    StreamingArtifactStats,
    StreamingEdgeSpec,
    StreamingPipelineSpec,
    StreamingSchedulerDiagnostics,
    StreamingSessionCloseReason,
    StreamingSessionContext,
    StreamingSessionMetrics,
    StreamingSessionStatus,
    StreamingStageActor,
    StreamingStageIdleInterval,
    StreamingStageInvocation,
    StreamingStageSpec,
    StreamingStageTiming,
    StreamingTaskKey,
    summarize_latencies,
)


@dataclass
class _Slot:
    value: object
    waiting: set  # stage ids that still have to take this value

    @property
    def reference_count(self) -> int:
        return len(self.waiting)


@dataclass
class _Timing:
    inputs_ready_at: float | None = None
    admitted_at: float | None = None
    completed_at: float | None = None
    block_reason: str = ""
    missing_inputs: tuple = ()


@dataclass
class _Session:
    session_id: str
    epoch: int
    final_sequence_id: int | None = None
    status: StreamingSessionStatus = StreamingSessionStatus.RUNNING
    error: BaseException | None = None
    cleanup_error: BaseException | None = None
    cleanup_pending: bool = False
    cleaned: bool = False
    slots: dict = field(default_factory=dict)  # artifact -> {sequence_id: _Slot}
    next_seq: dict = field(default_factory=dict)  # stage_id -> next sequence id to admit
    in_flight: dict = field(default_factory=dict)  # stage_id -> {sequence_id: StreamingTaskKey}
    done_keys: set = field(default_factory=set)  # (stage_id, sequence_id) finished
    egress: dict = field(default_factory=dict)  # sequence_id -> {artifact: value} waiting for ordered emission
    next_emit: int = 0
    emitted: deque = field(default_factory=deque)  # (sequence_id, artifact, value) not yet polled
    timings: dict = field(default_factory=dict)  # (stage_id, sequence_id) -> _Timing
    ingress_at: dict = field(default_factory=dict)
    emitted_at: dict = field(default_factory=dict)
    first_sequence_id: int | None = None


class StreamingPipelineOrchestrator:
    def __init__(self, spec: StreamingPipelineSpec, actors: Mapping[str, StreamingStageActor]) -> None:
        self.spec = spec
        self.actors = dict(actors)
        self._lock = threading.RLock()
        self._idle = threading.Condition(self._lock)
        self._sessions: dict[str, _Session] = {}
        self._epochs: dict[str, int] = {}
        self._request_ids = itertools.count()
        self._stages: dict[str, StreamingStageSpec] = {s.stage_id: s for s in spec.stages}
        self._groups = {g.name: g for g in spec.resource_groups}
        self._diag = dict(stale=0, orphan=0, duplicate=0, cleanup_failures=0, slot_leaks=0)
        self._closed = False
        self._failed_cleanups: deque = deque()
        self._cleanup_thread: threading.Thread | None = None
        self._cleanup_wakeup = threading.Event()
        self._validate()
        self._topo = self._topological_order()
        # artifact -> list of edges; artifact -> producing stage (None = ingress)
        self._edges_by_artifact: dict[str, list[StreamingEdgeSpec]] = {}
        for e in spec.edges:
            self._edges_by_artifact.setdefault(e.artifact, []).append(e)

    # ------------------------------------------------------------------ validation
    def _validate(self) -> None:
        spec = self.spec
        ids = [s.stage_id for s in spec.stages]
        if len(set(ids)) != len(ids):
            raise ValueError("duplicate stage ids")
        missing = [i for i in ids if i not in self.actors]
        if missing:
            raise ValueError(f"no actor for stage(s) {missing}")
        producer: dict[str, str] = {}
        for s in spec.stages:
            if s.resource_group is not None and s.resource_group not in self._groups:
                raise ValueError(f"stage {s.stage_id} names unknown resource group {s.resource_group}")
            for a in s.produces:
                if a in producer:
                    raise ValueError(f"artifact {a} has more than one producer")
                producer[a] = s.stage_id
        seen_edges = set()
        for e in spec.edges:
            if e.target_stage not in self._stages:
                raise ValueError(f"edge {e.artifact} targets unknown stage {e.target_stage}")
            if e.artifact not in self._stages[e.target_stage].consumes:
                raise ValueError(f"stage {e.target_stage} does not consume {e.artifact}")
            if e.source_stage is not None:
                if e.source_stage not in self._stages:
                    raise ValueError(f"edge {e.artifact} has unknown source stage {e.source_stage}")
                if producer.get(e.artifact) != e.source_stage:
                    raise ValueError(f"stage {e.source_stage} does not produce {e.artifact}")
            elif e.artifact in producer:
                raise ValueError(f"artifact {e.artifact} is produced by {producer[e.artifact]} but its edge has no source")
            if (e.artifact, e.target_stage) in seen_edges:
                raise ValueError(f"duplicate edge {e.artifact} -> {e.target_stage}")
            seen_edges.add((e.artifact, e.target_stage))
        for s in spec.stages:
            for a in s.consumes:
                if (a, s.stage_id) not in seen_edges:
                    raise ValueError(f"stage {s.stage_id} consumes {a} but no edge delivers it")
            for a in s.produces:
                consumed = any(e.artifact == a for e in spec.edges)
                if not consumed and a not in spec.output_artifacts:
                    raise ValueError(f"artifact {a} is produced but neither consumed nor an output")
        for a in spec.output_artifacts:
            if a not in producer:
                raise ValueError(f"output artifact {a} has no producer")
        self._producer = producer
        # reachability from ingress + acyclicity
        order = self._topological_order()
        reachable: set[str] = set()
        for sid in order:
            st = self._stages[sid]
            ok = True
            for a in st.consumes:
                src = producer.get(a)
                if src is not None and src not in reachable:
                    ok = False
            if ok:
                reachable.add(sid)
        if reachable != set(ids):
            raise ValueError(f"stages not reachable from external inputs: {sorted(set(ids) - reachable)}")

    def _topological_order(self) -> list[str]:
        deps = {s.stage_id: set() for s in self.spec.stages}
        for e in self.spec.edges:
            if e.source_stage is not None:
                deps[e.target_stage].add(e.source_stage)
        order, ready = [], [s for s, d in deps.items() if not d]
        deps = {s: set(d) for s, d in deps.items()}
        while ready:
            n = ready.pop(0)
            order.append(n)
            for s, d in deps.items():
                if n in d:
                    d.remove(n)
                    if not d and s not in order and s not in ready:
                        ready.append(s)
        if len(order) != len(deps):
            raise ValueError("the stage graph has a cycle")
        return order

    def _external_input_edges(self, artifact: str) -> tuple:
        return tuple(e for e in self._edges_by_artifact.get(artifact, ()) if e.source_stage is None)

    # ------------------------------------------------------------------ sessions
    def create_session(self, session_id: str, final_sequence_id: int | None = None) -> int:
        with self._lock:
            if self._closed:
                raise RuntimeError("orchestrator is closed")
            old = self._sessions.get(session_id)
            if old is not None and (old.status == StreamingSessionStatus.RUNNING or old.cleanup_pending):
                raise ValueError(f"session {session_id} is still active")
            epoch = self._epochs.get(session_id, 0) + 1
            self._epochs[session_id] = epoch
            rt = _Session(session_id, epoch, final_sequence_id)
            rt.next_seq = {s: None for s in self._stages}
            rt.in_flight = {s: {} for s in self._stages}
            self._sessions[session_id] = rt
            return epoch

    def _runtime(self, session_id: str) -> _Session:
        rt = self._sessions.get(session_id)
        if rt is None:
            raise KeyError(f"unknown session {session_id}")
        return rt

    def _active_runtime(self, session_id: str) -> _Session:
        rt = self._runtime(session_id)
        if rt.status != StreamingSessionStatus.RUNNING:
            if rt.error is not None:
                raise RuntimeError(f"session {session_id} is {rt.status.value}") from rt.error
            raise RuntimeError(f"session {session_id} is {rt.status.value}")
        return rt

    def push_input(self, session_id: str, sequence_id: int, artifact: str, value: object) -> None:
        if not self.try_push_inputs(session_id, sequence_id, {artifact: value}):
            raise StreamingActorBusyError(f"no capacity for {artifact} in session {session_id}")

    def can_push_input(self, session_id: str, artifact: str) -> bool:
        return self.can_push_inputs(session_id, [artifact])

    def can_push_inputs(self, session_id: str, artifacts: Collection[str]) -> bool:
        with self._lock:
            rt = self._active_runtime(session_id)
            return all(self._ingress_has_room(rt, a) for a in artifacts)

    def _ingress_has_room(self, rt: _Session, artifact: str) -> bool:
        edges = self._external_input_edges(artifact)
        if not edges:
            raise ValueError(f"{artifact} is not an external input")
        return all(self._edge_occupancy(rt, e) < e.capacity_per_session for e in edges)

    def try_push_inputs(self, session_id: str, sequence_id: int, inputs: Mapping[str, object]) -> bool:
        """Atomically accepts all `inputs` of one sequence id, or none when any edge is full."""
        with self._lock:
            rt = self._active_runtime(session_id)
            if rt.final_sequence_id is not None and sequence_id > rt.final_sequence_id:
                raise ValueError(f"sequence {sequence_id} is beyond the final sequence {rt.final_sequence_id}")
            for a in inputs:
                if sequence_id in rt.slots.get(a, {}):
                    raise ValueError(f"{a} for sequence {sequence_id} was already pushed")
            if not all(self._ingress_has_room(rt, a) for a in inputs):
                return False
            now = time.monotonic()
            for a, v in inputs.items():
                targets = {e.target_stage for e in self._external_input_edges(a)}
                rt.slots.setdefault(a, {})[sequence_id] = _Slot(v, targets)
            rt.ingress_at.setdefault(sequence_id, now)
            if rt.first_sequence_id is None or sequence_id < rt.first_sequence_id:
                rt.first_sequence_id = sequence_id
            self._pump_all()
            return True

    def finish_inputs(self, session_id: str, final_sequence_id: int) -> None:
        with self._lock:
            rt = self._active_runtime(session_id)
            rt.final_sequence_id = final_sequence_id
            self._pump_all()

    def poll_outputs(self, session_id: str) -> list:
        """Returns (sequence_id, artifact, value) triples in sequence order and frees their output slots."""
        with self._lock:
            rt = self._runtime(session_id)
            out = list(rt.emitted)
            rt.emitted.clear()
            if out and rt.status == StreamingSessionStatus.RUNNING:
                self._pump_all()
            return out

    def status(self, session_id: str) -> StreamingSessionStatus:
        with self._lock:
            return self._runtime(session_id).status

    def error(self, session_id: str) -> BaseException | None:
        with self._lock:
            return self._runtime(session_id).error

    def cleanup_error(self, session_id: str) -> BaseException | None:
        with self._lock:
            return self._runtime(session_id).cleanup_error

    # ------------------------------------------------------------------ observability
    def artifact_stats(self, session_id: str) -> StreamingArtifactStats:
        with self._lock:
            rt = self._runtime(session_id)
            slots = [s for per in rt.slots.values() for s in per.values()]
            return StreamingArtifactStats(len(slots), sum(s.reference_count for s in slots))

    def resource_group_usage(self, name: str) -> int:
        with self._lock:
            if name not in self._groups:
                raise KeyError(name)
            return self._resource_group_in_flight(name)

    def diagnostics(self) -> StreamingSchedulerDiagnostics:
        with self._lock:
            d = self._diag
            return StreamingSchedulerDiagnostics(d["stale"], d["orphan"], d["duplicate"], d["cleanup_failures"],
                                                 d["slot_leaks"])  # fmt: skip

    def stage_timings(self, session_id: str, stage_id: str) -> tuple:
        with self._lock:
            rt = self._runtime(session_id)
            rows = sorted((seq, t) for (sid, seq), t in rt.timings.items() if sid == stage_id)
            return tuple(StreamingStageTiming(stage_id, seq, t.inputs_ready_at, t.admitted_at, t.completed_at)
                         for seq, t in rows)  # fmt: skip

    def session_metrics(self, session_id: str) -> StreamingSessionMetrics:
        with self._lock:
            rt = self._runtime(session_id)
            ingress = tuple(sorted(rt.ingress_at.items()))
            emitted = tuple(sorted(rt.emitted_at.items()))
            first = None
            if ingress and emitted:
                first = emitted[0][1] - ingress[0][1]
            c2o = [t - rt.ingress_at[s] for s, t in emitted if s in rt.ingress_at]
            times = [t for _, t in emitted]
            periods = [b - a for a, b in zip(times, times[1:])]
            return StreamingSessionMetrics(ingress, emitted, first, summarize_latencies(c2o),
                                           summarize_latencies(periods))  # fmt: skip

    def stage_idle_intervals(self, session_id: str, stage_id: str) -> tuple:
        """Gaps between the end of one invocation of a stage and the admission of the next, with the cause."""
        with self._lock:
            rt = self._runtime(session_id)
            rows = sorted((seq, t) for (sid, seq), t in rt.timings.items() if sid == stage_id)
            out = []
            for (pseq, pt), (seq, t) in zip(rows, rows[1:]):
                if pt.completed_at is None or t.admitted_at is None:
                    continue
                idle = max(0.0, t.admitted_at - pt.completed_at)
                if t.inputs_ready_at is not None and t.inputs_ready_at > pt.completed_at:
                    reason = "waiting_for_inputs"
                else:
                    reason = t.block_reason or "scheduler"
                out.append(StreamingStageIdleInterval(stage_id, pseq, seq, idle, reason, tuple(t.missing_inputs)))
            return tuple(out)

    def actor_health(self, stage_id: str) -> StreamingActorHealth:
        return self.actors[stage_id].health()

    def barrier(self, timeout: float = 5.0) -> None:
        """Waits until nothing is in flight and every actor has drained its mailbox."""
        deadline = time.monotonic() + timeout
        with self._idle:
            while any(any(f for f in rt.in_flight.values()) for rt in self._sessions.values()):
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutError("barrier timed out with invocations in flight")
                self._idle.wait(left)
        for actor in self.actors.values():
            actor.barrier(max(0.0, deadline - time.monotonic()))

    def wait_until_idle(self, session_id: str, timeout: float = 5.0) -> bool:
        """True once the session has nothing in flight and nothing admissible."""
        deadline = time.monotonic() + timeout
        with self._idle:
            while True:
                rt = self._runtime(session_id)
                busy = any(rt.in_flight[s] for s in rt.in_flight)
                if not busy and (rt.status != StreamingSessionStatus.RUNNING or not self._has_admissible_task(rt)):
                    return True
                left = deadline - time.monotonic()
                if left <= 0:
                    return False
                self._idle.wait(min(left, 0.05))
                if rt.status == StreamingSessionStatus.RUNNING:
                    self._pump_all()

    # ------------------------------------------------------------------ termination
    def cancel_session(self, session_id: str, timeout: float = 5.0) -> None:
        self._end_session(session_id, StreamingSessionStatus.CANCELLED, StreamingSessionCloseReason.CANCELLED, timeout)

    def close_session(self, session_id: str, timeout: float = 5.0) -> None:
        self._end_session(session_id, StreamingSessionStatus.CLOSED, StreamingSessionCloseReason.CLOSED, timeout)

    def _end_session(self, session_id, status, reason, timeout) -> None:
        with self._lock:
            rt = self._runtime(session_id)
            if rt.status == StreamingSessionStatus.RUNNING:
                rt.status = status
            elif rt.status == StreamingSessionStatus.FAILED:
                reason = StreamingSessionCloseReason.FAILED
            if not rt.cleanup_pending and rt.status != StreamingSessionStatus.RUNNING and rt.cleaned:
                return
        self._cleanup_session(rt, reason, timeout)

    def close(self, timeout: float = 300.0) -> None:
        with self._lock:
            if self._closed:
                return
            self._closed = True
            sessions = list(self._sessions.values())
        deadline = time.monotonic() + timeout
        for rt in sessions:
            with self._lock:
                if rt.status == StreamingSessionStatus.RUNNING:
                    rt.status = StreamingSessionStatus.CLOSED
                cleaned = rt.cleaned and not rt.cleanup_pending
            if not cleaned:
                self._cleanup_session(rt, StreamingSessionCloseReason.SHUTDOWN, max(0.1, deadline - time.monotonic()))
        self._cleanup_wakeup.set()
        for sid in reversed(self._topo):
            try:
                self.actors[sid].close()
            except Exception:  # noqa: BLE001 - shutting down regardless
                with self._lock:
                    self._diag["cleanup_failures"] += 1

    @staticmethod
    def _discard_buffered_state(rt: _Session) -> int:
        """Drops buffered artifacts and outputs; returns how many slots were still referenced."""
        leaked = sum(1 for per in rt.slots.values() for s in per.values() if s.reference_count > 0)
        rt.slots.clear()
        rt.egress.clear()
        return leaked

    def _cleanup_session(self, rt: _Session, reason: StreamingSessionCloseReason, timeout: float) -> None:
        """Drains in-flight work, drops buffers and closes the session on every actor, sinks first."""
        deadline = time.monotonic() + timeout
        with self._idle:
            while any(rt.in_flight[s] for s in rt.in_flight):
                left = deadline - time.monotonic()
                if left <= 0:
                    break
                self._idle.wait(min(left, 0.05))
            finished_all = (rt.final_sequence_id is not None and rt.error is None and
                            all(n is not None and n > rt.final_sequence_id for n in rt.next_seq.values()))  # fmt: skip
            leaked = self._discard_buffered_state(rt)
            if reason == StreamingSessionCloseReason.CLOSED and finished_all and leaked:
                self._diag["slot_leaks"] += leaked
            stuck = {s: dict(f) for s, f in rt.in_flight.items() if f}
            if stuck:
                # results that arrive later are classified stale through the epoch bump below
                self._epochs[rt.session_id] = self._epochs.get(rt.session_id, rt.epoch) + 1
                for f in rt.in_flight.values():
                    f.clear()
        ctx = StreamingSessionContext(rt.session_id, rt.epoch)
        failure: BaseException | None = None
        for sid in reversed(self._topo):
            try:
                self.actors[sid].close_session(ctx, reason, max(0.05, deadline - time.monotonic()))
            except BaseException as e:  # noqa: BLE001 - keep closing the remaining stages
                failure = failure or e
        with self._lock:
            rt.cleaned = True
            if failure is not None:
                rt.cleanup_error = failure
                self._diag["cleanup_failures"] += 1
                if not rt.cleanup_pending:
                    rt.cleanup_pending = True
                    self._schedule_failed_cleanup(rt, reason)
            else:
                rt.cleanup_error = None
                rt.cleanup_pending = False
            self._idle.notify_all()

    def _schedule_failed_cleanup(self, rt: _Session, reason: StreamingSessionCloseReason) -> None:
        self._failed_cleanups.append((rt, reason, 0))
        if self._cleanup_thread is None or not self._cleanup_thread.is_alive():
            self._cleanup_thread = threading.Thread(target=self._run_failed_cleanups, name="stream-cleanup",
                                                    daemon=True)  # fmt: skip
            self._cleanup_thread.start()
        self._cleanup_wakeup.set()

    def _run_failed_cleanups(self, max_attempts: int = 5, backoff_s: float = 0.05) -> None:
        while True:
            with self._lock:
                if not self._failed_cleanups:
                    return
                rt, reason, attempt = self._failed_cleanups.popleft()
            time.sleep(backoff_s * (attempt + 1))
            ctx = StreamingSessionContext(rt.session_id, rt.epoch)
            failure = None
            for sid in reversed(self._topo):
                try:
                    self.actors[sid].close_session(ctx, reason, 1.0)
                except BaseException as e:  # noqa: BLE001
                    failure = failure or e
            with self._lock:
                if failure is None:
                    rt.cleanup_error, rt.cleanup_pending = None, False
                elif attempt + 1 < max_attempts and not self._closed:
                    self._failed_cleanups.append((rt, reason, attempt + 1))
                else:
                    rt.cleanup_error, rt.cleanup_pending = failure, False
                self._idle.notify_all()

    # ------------------------------------------------------------------ scheduling
    def _pump_all(self) -> None:
        """Admits every admissible invocation, visiting sessions round-robin until nothing moves."""
        with self._lock:
            progressed = True
            while progressed:
                progressed = False
                for rt in list(self._sessions.values()):
                    if rt.status == StreamingSessionStatus.RUNNING and self._pump_once(rt):
                        progressed = True
            self._idle.notify_all()

    def _pump_once(self, rt: _Session) -> bool:
        """Tries each stage once for this session; returns True when something was admitted or emitted."""
        moved = self._emit_ready_outputs(rt)
        self._observe_input_readiness(rt)
        for sid in self._topo:
            stage = self._stages[sid]
            seq = self._runnable_sequence(rt, stage)
            if seq is None:
                continue
            timing = rt.timings.setdefault((sid, seq), _Timing())
            failure = self._actor_failure(sid)
            if failure is not None:
                self._fail_all_sessions_for_actor(sid, failure)
                return True
            if not self._has_execution_capacity(stage):
                timing.block_reason = "resource_group" if self._resource_group_is_full(stage) else "execution_slots"
                continue
            if not self._has_output_capacity(rt, stage):
                timing.block_reason = "output_backpressure"
                continue
            inputs = self._take_inputs(rt, stage, seq)
            key = StreamingTaskKey(rt.session_id, rt.epoch, seq, sid, f"req-{next(self._request_ids)}")
            inv = StreamingStageInvocation(key, inputs, is_first=(seq == rt.first_sequence_id),
                                           is_last=(rt.final_sequence_id is not None and seq == rt.final_sequence_id))  # fmt: skip
            rt.in_flight[sid][seq] = key
            try:
                fut = self.actors[sid].submit(inv)
            except StreamingActorBusyError:
                del rt.in_flight[sid][seq]
                self._restore_inputs(rt, stage, seq, inputs)
                timing.block_reason = "actor_busy"
                continue
            except BaseException as e:  # noqa: BLE001 - submit refused for good
                del rt.in_flight[sid][seq]
                self._restore_inputs(rt, stage, seq, inputs)
                err = e if isinstance(e, StreamingActorFailedError) else StreamingActorFailedError(repr(e))
                self._fail_all_sessions_for_actor(sid, err)
                return True
            timing.admitted_at = time.monotonic()
            rt.next_seq[sid] = seq + 1
            fut.add_done_callback(lambda f, k=key: self._complete(k.session_id, k, f))
            moved = True
        return moved

    def _has_admissible_task(self, rt: _Session) -> bool:
        for sid in self._topo:
            stage = self._stages[sid]
            if (self._runnable_sequence(rt, stage) is not None and self._has_execution_capacity(stage)
                    and self._has_output_capacity(rt, stage)):  # fmt: skip
                return True
        return False

    def _next_candidate(self, rt: _Session, stage: StreamingStageSpec) -> int | None:
        nxt = rt.next_seq[stage.stage_id]
        if nxt is None:
            nxt = rt.first_sequence_id
        return nxt

    def _runnable_sequence(self, rt: _Session, stage: StreamingStageSpec) -> int | None:
        """The sequence id this stage may run next for the session, or None."""
        seq = self._next_candidate(rt, stage)
        if seq is None:
            return None
        if rt.final_sequence_id is not None and seq > rt.final_sequence_id:
            return None
        if len(rt.in_flight[stage.stage_id]) >= stage.max_in_flight_per_session:
            return None
        for a in stage.consumes:
            slot = rt.slots.get(a, {}).get(seq)
            if slot is None or stage.stage_id not in slot.waiting:
                return None
        return seq

    def _stage_in_flight(self, stage_id: str) -> int:
        return sum(len(rt.in_flight[stage_id]) for rt in self._sessions.values())

    def _resource_group_in_flight(self, name: str) -> int:
        return sum(self._stage_in_flight(s.stage_id) for s in self.spec.stages if s.resource_group == name)

    def _resource_group_is_full(self, stage: StreamingStageSpec) -> bool:
        if stage.resource_group is None:
            return False
        return self._resource_group_in_flight(stage.resource_group) >= self._groups[stage.resource_group].max_concurrency

    def _has_execution_capacity(self, stage: StreamingStageSpec) -> bool:
        if self._stage_in_flight(stage.stage_id) >= stage.max_in_flight_global:
            return False
        return not self._resource_group_is_full(stage)

    @staticmethod
    def _edge_occupancy(rt: _Session, edge: StreamingEdgeSpec) -> int:
        return sum(1 for s in rt.slots.get(edge.artifact, {}).values() if edge.target_stage in s.waiting)

    def _reserved(self, rt: _Session, artifact: str) -> int:
        """Results of `artifact` promised by invocations in flight."""
        src = self._producer.get(artifact)
        return 0 if src is None else len(rt.in_flight[src])

    @staticmethod
    def _output_occupancy(rt: _Session, artifact: str) -> int:
        return sum(1 for _, a, _ in rt.emitted if a == artifact) + sum(1 for v in rt.egress.values() if artifact in v)

    def _has_output_capacity(self, rt: _Session, stage: StreamingStageSpec) -> bool:
        for a in stage.produces:
            reserved = self._reserved(rt, a)
            for e in self._edges_by_artifact.get(a, ()):
                if self._edge_occupancy(rt, e) + reserved >= e.capacity_per_session:
                    return False
            if a in self.spec.output_artifacts:
                if self._output_occupancy(rt, a) + reserved >= self.spec.output_capacity_per_session:
                    return False
        return True

    def _take_inputs(self, rt: _Session, stage: StreamingStageSpec, seq: int) -> dict:
        inputs = {}
        for a in stage.consumes:
            slot = rt.slots[a][seq]
            inputs[a] = slot.value
            slot.waiting.discard(stage.stage_id)
            if not slot.waiting:
                del rt.slots[a][seq]
        return inputs

    def _restore_inputs(self, rt: _Session, stage: StreamingStageSpec, seq: int, inputs: Mapping[str, object]) -> None:
        for a, v in inputs.items():
            slot = rt.slots.setdefault(a, {}).get(seq)
            if slot is None:
                rt.slots[a][seq] = _Slot(v, {stage.stage_id})
            else:
                slot.waiting.add(stage.stage_id)

    def _observe_input_readiness(self, rt: _Session) -> None:
        now = time.monotonic()
        for sid, stage in self._stages.items():
            seq = self._next_candidate(rt, stage)
            if seq is None or (rt.final_sequence_id is not None and seq > rt.final_sequence_id):
                continue
            if not any(seq in rt.slots.get(a, {}) for a in stage.consumes) and (sid, seq) not in rt.timings:
                continue  # nothing of this sequence has arrived yet
            timing = rt.timings.setdefault((sid, seq), _Timing())
            if timing.inputs_ready_at is not None:
                continue
            missing = tuple(sorted(a for a in stage.consumes if seq not in rt.slots.get(a, {})))
            if missing:
                timing.missing_inputs = missing
            else:
                timing.inputs_ready_at = now

    # ------------------------------------------------------------------ completion
    def _complete(self, session_id: str, key: StreamingTaskKey, future: Future) -> None:
        with self._lock:
            rt = self._sessions.get(session_id)
            if rt is None:
                self._diag["orphan"] += 1
                return
            if key.session_epoch != rt.epoch or self._epochs.get(session_id) != key.session_epoch:
                self._diag["stale"] += 1
                self._idle.notify_all()
                return
            if (key.stage_id, key.sequence_id) in rt.done_keys or rt.in_flight[key.stage_id].get(key.sequence_id) != key:
                self._diag["duplicate"] += 1
                return
            del rt.in_flight[key.stage_id][key.sequence_id]
            rt.done_keys.add((key.stage_id, key.sequence_id))
            timing = rt.timings.setdefault((key.stage_id, key.sequence_id), _Timing())
            timing.completed_at = time.monotonic()
            if rt.status != StreamingSessionStatus.RUNNING:
                self._idle.notify_all()  # a cancelled / failed session only needs its in-flight count to drop
                return
            exc = future.exception()
            if exc is not None:
                failure = self._actor_failure(key.stage_id)
                if failure is not None:
                    self._fail_all_sessions_for_actor(key.stage_id, failure, cause=exc)
                else:
                    self._fail_runtime(rt, exc)
                self._pump_all()
                return
            stage = self._stages[key.stage_id]
            outputs = future.result()
            if not isinstance(outputs, Mapping) or set(outputs.keys()) != set(stage.produces):
                got = sorted(outputs.keys()) if isinstance(outputs, Mapping) else type(outputs).__name__
                self._fail_runtime(rt, ValueError(
                    f"stage {key.stage_id} returned {got}, expected exactly {sorted(stage.produces)}"))  # fmt: skip
                self._pump_all()
                return
            for a, v in outputs.items():
                targets = {e.target_stage for e in self._edges_by_artifact.get(a, ())}
                if targets:
                    rt.slots.setdefault(a, {})[key.sequence_id] = _Slot(v, set(targets))
                if a in self.spec.output_artifacts:
                    rt.egress.setdefault(key.sequence_id, {})[a] = v
            self._pump_all()

    def _emit_ready_outputs(self, rt: _Session) -> bool:
        """Moves finished egress artifacts to the poll queue in sequence order."""
        if not self.spec.output_artifacts:
            return False
        moved = False
        if rt.next_emit == 0 and rt.first_sequence_id is not None and not rt.emitted_at:
            rt.next_emit = rt.first_sequence_id
        while True:
            ready = rt.egress.get(rt.next_emit)
            if ready is None or set(ready.keys()) != set(self.spec.output_artifacts):
                return moved
            del rt.egress[rt.next_emit]
            for a in sorted(ready):
                rt.emitted.append((rt.next_emit, a, ready[a]))
            rt.emitted_at[rt.next_emit] = time.monotonic()
            rt.next_emit += 1
            moved = True

    # ------------------------------------------------------------------ failures
    def _actor_failure(self, stage_id: str) -> StreamingActorFailedError | None:
        h = self.actors[stage_id].health()
        if h.state == StreamingActorState.FAILED:
            return StreamingActorFailedError(f"actor {stage_id} failed: {h.failure_reason}")
        return None

    def _fail_all_sessions_for_actor(self, stage_id: str, error: BaseException, cause: BaseException | None = None):
        if cause is not None and error.__cause__ is None:
            error.__cause__ = cause
        for rt in self._sessions.values():
            if rt.status == StreamingSessionStatus.RUNNING:
                self._fail_runtime(rt, error)

    def _fail_runtime(self, rt: _Session, error: BaseException) -> None:
        if rt.status != StreamingSessionStatus.RUNNING:
            return
        rt.status = StreamingSessionStatus.FAILED
        rt.error = error
        rt.cleanup_pending = True
        threading.Thread(target=self._failed_session_cleanup, args=(rt,), name="stream-failed-cleanup",
                         daemon=True).start()  # fmt: skip
        self._idle.notify_all()

    def _failed_session_cleanup(self, rt: _Session) -> None:
        with self._lock:
            rt.cleanup_pending = False
        self._cleanup_session(rt, StreamingSessionCloseReason.FAILED, 5.0)
