"""LocalStageActor: one thread, one bounded mailbox, one stage callable.

`submit` never blocks: a full mailbox raises `StreamingActorBusyError`. Invocations
and session-close requests are served strictly in arrival order on the actor's
thread, so a stage never sees two calls at once and `close_session` cannot
overtake a chunk submitted before it. An exception from the handler fails the
actor for good: queued futures are failed, later submits raise
`StreamingActorFailedError`. Role parity: LocalStageActor,
telefuser/orchestrator/streaming_pipeline_orchestrator.py:271-436.
"""

from __future__ import annotations

import queue
import threading
from concurrent.futures import Future
from dataclasses import dataclass
from typing import Callable, Mapping

from .streaming_types import (
    StreamingActorBusyError,
    StreamingActorFailedError,
    StreamingActorHealth,
    StreamingActorState,
    StreamingSessionCloseReason,
    StreamingSessionContext,
    StreamingStageInvocation,
)


@dataclass
class _Work:
    kind: str  # "invoke" | "close_session" | "barrier" | "stop"
    future: Future
    invocation: StreamingStageInvocation | None = None
    context: StreamingSessionContext | None = None
    reason: StreamingSessionCloseReason | None = None


class LocalStageActor:
    def __init__(self, stage_id: str, handler: Callable[[StreamingStageInvocation], Mapping[str, object]],
                 mailbox_size: int = 1,
                 close_session_handler: Callable[[StreamingSessionContext, StreamingSessionCloseReason], None]
                 | None = None, close_handler: Callable[[], None] | None = None) -> None:  # fmt: skip
        if mailbox_size < 1:
            raise ValueError("mailbox_size must be at least one")
        self.stage_id = stage_id
        self._handler = handler
        self._close_session_handler = close_session_handler
        self._close_handler = close_handler
        self._mailbox: queue.Queue[_Work] = queue.Queue()
        self._mailbox_size = mailbox_size
        self._lock = threading.Lock()
        self._pending = 0  # invocations accepted and not yet finished
        self._state = StreamingActorState.RUNNING
        self._failure: BaseException | None = None
        self._thread = threading.Thread(target=self._run, name=f"stage-actor-{stage_id}", daemon=True)
        self._thread.start()

    # ---- protocol -----------------------------------------------------------
    def submit(self, invocation: StreamingStageInvocation) -> Future:
        fut: Future = Future()
        with self._lock:
            if self._state == StreamingActorState.FAILED:
                raise StreamingActorFailedError(f"actor {self.stage_id} failed: {self._failure!r}")
            if self._state == StreamingActorState.CLOSED:
                raise StreamingActorFailedError(f"actor {self.stage_id} is closed")
            if self._pending >= self._mailbox_size:
                raise StreamingActorBusyError(f"actor {self.stage_id} mailbox is full")
            self._pending += 1
            self._mailbox.put(_Work("invoke", fut, invocation=invocation))
        return fut

    def health(self) -> StreamingActorHealth:
        with self._lock:
            return StreamingActorHealth(self._state, self._pending,
                                        None if self._failure is None else repr(self._failure))  # fmt: skip

    def barrier(self, timeout: float = 5.0) -> None:
        """Returns once everything queued before the call has been served."""
        fut: Future = Future()
        with self._lock:
            if self._state != StreamingActorState.RUNNING:
                return
            self._mailbox.put(_Work("barrier", fut))
        fut.result(timeout=timeout)

    def close_session(self, context: StreamingSessionContext, reason: StreamingSessionCloseReason,
                      timeout: float = 5.0) -> None:  # fmt: skip
        fut: Future = Future()
        with self._lock:
            if self._state == StreamingActorState.CLOSED:
                return
            if self._state == StreamingActorState.FAILED:
                # the thread is gone: release session state on the caller's thread
                run_inline = True
            else:
                run_inline = False
                self._mailbox.put(_Work("close_session", fut, context=context, reason=reason))
        if run_inline:
            if self._close_session_handler is not None:
                self._close_session_handler(context, reason)
            return
        fut.result(timeout=timeout)

    def close(self) -> None:
        with self._lock:
            if self._state == StreamingActorState.CLOSED:
                return
            was_running = self._state == StreamingActorState.RUNNING
            self._state = StreamingActorState.CLOSED
            if was_running:
                self._mailbox.put(_Work("stop", Future()))
        if was_running:
            self._thread.join(timeout=10.0)
        if self._close_handler is not None:
            self._close_handler()

    # ---- actor thread ---------------------------------------------------------
    def _run(self) -> None:
        while True:
            work = self._mailbox.get()
            if work.kind == "stop":
                self._drain(StreamingActorFailedError(f"actor {self.stage_id} is closed"))
                return
            if work.kind == "barrier":
                work.future.set_result(None)
                continue
            if work.kind == "close_session":
                try:
                    if self._close_session_handler is not None:
                        self._close_session_handler(work.context, work.reason)
                    work.future.set_result(None)
                except BaseException as e:  # noqa: BLE001 - reported to the caller of close_session
                    work.future.set_exception(e)
                continue
            try:
                result = self._handler(work.invocation)
            except BaseException as e:  # noqa: BLE001 - a handler failure is terminal for the actor
                self._fail(e, work)
                return
            with self._lock:
                self._pending -= 1
            work.future.set_result(result)

    def _fail(self, exc: BaseException, current: _Work) -> None:
        with self._lock:
            self._state = StreamingActorState.FAILED
            self._failure = exc
            self._pending -= 1
        current.future.set_exception(exc)
        self._drain(StreamingActorFailedError(f"actor {self.stage_id} failed: {exc!r}"))

    def _drain(self, error: BaseException) -> None:
        while True:
            try:
                work = self._mailbox.get_nowait()
            except queue.Empty:
                return
            if work.kind == "invoke":
                with self._lock:
                    self._pending -= 1
                work.future.set_exception(error)
            elif work.kind == "close_session":
                try:
                    if self._close_session_handler is not None:
                        self._close_session_handler(work.context, work.reason)
                    work.future.set_result(None)
                except BaseException as e:  # noqa: BLE001
                    work.future.set_exception(e)
            elif not work.future.done():
                work.future.set_result(None)
