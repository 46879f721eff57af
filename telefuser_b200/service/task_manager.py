"""Task lifecycle: PENDING -> PROCESSING -> COMPLETED | FAILED | CANCELLED.

Thread-safe; bounded queue; N processing slots (one per pipeline replica) that can shrink when a
replica dies; cooperative cancellation through a per-task stop event; old finished tasks are
pruned. Role parity: telefuser/service/core/task_manager.py:21-437.
"""

from __future__ import annotations

import threading
import uuid
from collections import OrderedDict
from dataclasses import dataclass, field
from datetime import datetime
from enum import Enum
from typing import Any


class TaskStatus(str, Enum):
    PENDING = "pending"
    PROCESSING = "processing"
    STREAMING = "streaming"
    COMPLETED = "completed"
    FAILED = "failed"
    CANCELLED = "cancelled"


ACTIVE = frozenset({TaskStatus.PENDING, TaskStatus.PROCESSING, TaskStatus.STREAMING})
VIDEO_TASKS = frozenset({"t2v", "i2v", "fl2v", "vc", "s2v", "vsr"})
IMAGE_TASKS = frozenset({"t2i", "i2i", "edit"})


class QueueFullError(RuntimeError):
    pass


class NoCapacityError(RuntimeError):
    pass


@dataclass
class TaskInfo:
    task_id: str
    status: TaskStatus
    message: Any
    start_time: datetime = field(default_factory=datetime.now)
    end_time: datetime | None = None
    error: str | None = None
    output_path: str | None = None
    peak_memory_mb: float | None = None
    inference_time_s: float | None = None
    stop_event: threading.Event = field(default_factory=threading.Event)

    def to_dict(self) -> dict:
        return {"task_id": self.task_id, "status": self.status.value, "error": self.error,
                "output_path": self.output_path, "peak_memory_mb": self.peak_memory_mb,
                "inference_time_s": self.inference_time_s, "start_time": self.start_time.isoformat(),
                "end_time": self.end_time.isoformat() if self.end_time else None}  # fmt: skip


class TaskManager:
    def __init__(self, max_queue_size: int = 100, cleanup_keep_count: int = 1000,
                 max_concurrent_processing: int = 1) -> None:  # fmt: skip
        self.max_queue_size = max_queue_size
        self.cleanup_keep_count = cleanup_keep_count
        self._max_concurrent = max(1, max_concurrent_processing)
        self._zero_capacity = False
        self._tasks: OrderedDict[str, TaskInfo] = OrderedDict()
        self._processing: set[str] = set()
        self._lock = threading.RLock()
        self.total_tasks = self.completed_tasks = self.failed_tasks = 0

    # ---- creation / lookup ----------------------------------------------------
    def create_task(self, message: Any) -> str:
        with self._lock:
            if self._zero_capacity:
                raise NoCapacityError("No inference capacity: all pipeline replicas are dead")
            tid = getattr(message, "task_id", None) or (message.get("task_id") if isinstance(message, dict) else None)
            tid = tid or uuid.uuid4().hex
            if tid in self._tasks:
                raise RuntimeError(f"Task ID {tid} already exists")
            if sum(1 for t in self._tasks.values() if t.status in ACTIVE) >= self.max_queue_size:
                raise QueueFullError(f"Task queue is full (max {self.max_queue_size} tasks)")
            self._tasks[tid] = TaskInfo(tid, TaskStatus.PENDING, message)
            self.total_tasks += 1
            self._cleanup()
            return tid

    def get_task(self, task_id: str) -> TaskInfo | None:
        with self._lock:
            return self._tasks.get(task_id)

    def get_status(self, task_id: str) -> dict | None:
        t = self.get_task(task_id)
        return None if t is None else t.to_dict()

    def current_task_id(self) -> str | None:
        """The task that has been in a processing slot the longest (None while idle)."""
        with self._lock:
            live = [t for t in self._processing if t in self._tasks]
            return min(live, key=lambda t: self._tasks[t].start_time) if live else None

    def queue_status(self) -> dict:
        with self._lock:
            counts = {s.value: 0 for s in TaskStatus}
            for t in self._tasks.values():
                counts[t.status.value] += 1
            return {"counts": counts, "max_queue_size": self.max_queue_size, "processing_slots": self._max_concurrent,
                    "total": self.total_tasks, "completed": self.completed_tasks, "failed": self.failed_tasks}  # fmt: skip

    # ---- processing slots --------------------------------------------------------
    def claim_next_pending_task(self) -> TaskInfo | None:
        """Atomically moves the oldest pending task to PROCESSING if a slot is free."""
        with self._lock:
            if len(self._processing) >= self._max_concurrent:
                return None
            for t in self._tasks.values():
                if t.status == TaskStatus.PENDING:
                    t.status = TaskStatus.PROCESSING
                    self._processing.add(t.task_id)
                    return t
            return None

    def release_processing_slot(self, task_id: str) -> None:
        with self._lock:
            self._processing.discard(task_id)

    def set_max_concurrent_processing(self, n: int) -> None:
        with self._lock:
            self._zero_capacity = n <= 0
            self._max_concurrent = max(1, n)

    def fail_all_pending(self, reason: str) -> int:
        with self._lock:
            n = 0
            for t in self._tasks.values():
                if t.status == TaskStatus.PENDING:
                    self._finish(t, TaskStatus.FAILED, error=reason)
                    n += 1
            return n

    # ---- completion -----------------------------------------------------------------
    def _finish(self, t: TaskInfo, status: TaskStatus, **fields) -> None:
        t.status = status
        t.end_time = datetime.now()
        for k, v in fields.items():
            setattr(t, k, v)
        self._processing.discard(t.task_id)
        if status == TaskStatus.COMPLETED:
            self.completed_tasks += 1
        elif status == TaskStatus.FAILED:
            self.failed_tasks += 1

    def complete_task(self, task_id: str, output_path=None, peak_memory_mb=None, inference_time_s=None) -> None:
        with self._lock:
            t = self._tasks.get(task_id)
            if t is not None and t.status in ACTIVE:
                self._finish(t, TaskStatus.COMPLETED, output_path=output_path, peak_memory_mb=peak_memory_mb,
                             inference_time_s=inference_time_s)  # fmt: skip

    def fail_task(self, task_id: str, error: str) -> None:
        with self._lock:
            t = self._tasks.get(task_id)
            if t is not None and t.status in ACTIVE:
                self._finish(t, TaskStatus.FAILED, error=error)

    def cancel_task(self, task_id: str) -> bool:
        """Pending tasks are cancelled at once; running ones get their stop event set (cooperative)."""
        with self._lock:
            t = self._tasks.get(task_id)
            if t is None or t.status not in ACTIVE:
                return False
            t.stop_event.set()
            if t.status == TaskStatus.PENDING:
                self._finish(t, TaskStatus.CANCELLED)
            return True

    def mark_cancelled(self, task_id: str) -> None:
        with self._lock:
            t = self._tasks.get(task_id)
            if t is not None and t.status in ACTIVE:
                self._finish(t, TaskStatus.CANCELLED)

    def _cleanup(self) -> None:
        done = [k for k, t in self._tasks.items() if t.status not in ACTIVE]
        for k in done[: max(0, len(done) - self.cleanup_keep_count)]:
            del self._tasks[k]
