"""Adapter that lets a `ParallelWorker` (an SPMD rank group) act as one streaming stage actor.

The worker answers calls in order over one response queue, so the adapter owns it
exclusively and keeps at most one call outstanding: submissions go through a
`LocalStageActor` whose handler performs the remote call. Health merges the
adapter's state with the worker's (`failed`, `closed`). Role parity:
telefuser/orchestrator/parallel_worker_stage_actor.py:21-100.
"""

from __future__ import annotations

from concurrent.futures import Future
from typing import Any, Callable, Mapping

from .local_actor import LocalStageActor
from .streaming_types import (
    StreamingActorHealth,
    StreamingActorState,
    StreamingSessionCloseReason,
    StreamingSessionContext,
    StreamingStageInvocation,
)


class ParallelWorkerStageActor:
    def __init__(self, worker, method_name: str,
                 input_builder: Callable[[StreamingStageInvocation], tuple[tuple, dict]],
                 output_builder: Callable[[Any, StreamingStageInvocation], Mapping[str, object]],
                 mailbox_capacity: int = 1, close_worker: bool = True,
                 session_closer: Callable[[StreamingSessionContext, StreamingSessionCloseReason], None] | None = None,
                 ) -> None:  # fmt: skip
        self.worker = worker
        self.method_name = method_name
        self._input_builder = input_builder
        self._output_builder = output_builder
        self._close_worker = close_worker
        self._actor = LocalStageActor(f"worker-{method_name}", self._invoke, mailbox_capacity, session_closer)

    def _invoke(self, invocation: StreamingStageInvocation) -> Mapping[str, object]:
        args, kwargs = self._input_builder(invocation)
        result = getattr(self.worker, self.method_name)(*args, **kwargs)
        if callable(result):  # asynchronous call style: a wait() closure
            result = result()
        return self._output_builder(result, invocation)

    def submit(self, invocation: StreamingStageInvocation) -> Future:
        return self._actor.submit(invocation)

    def health(self) -> StreamingActorHealth:
        h = self._actor.health()
        if getattr(self.worker, "failed", False):
            return StreamingActorHealth(StreamingActorState.FAILED, h.pending_invocations,
                                        getattr(self.worker, "failure_reason", None))  # fmt: skip
        if getattr(self.worker, "closed", False):
            return StreamingActorHealth(StreamingActorState.CLOSED, h.pending_invocations, h.failure_reason)
        return h

    def barrier(self, timeout: float = 5.0) -> None:
        self._actor.barrier(timeout)

    def close_session(self, context: StreamingSessionContext, reason: StreamingSessionCloseReason,
                      timeout: float = 5.0) -> None:  # fmt: skip
        self._actor.close_session(context, reason, timeout)

    def close(self) -> None:
        self._actor.close()
        if self._close_worker:
            self.worker.close()
