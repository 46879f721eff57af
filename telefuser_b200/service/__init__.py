"""Serving layer: task queue, pipeline loading with security validation, replica pool, HTTP API,
streaming sessions. Heavy modules (FastAPI app) are imported on demand."""

from .contract import PipelineContract, TaskContract, load_contract
from .security import PipelineSecurityValidator, SecurityError, SecurityLevel
from .task_manager import TaskManager, TaskStatus

__all__ = ["PipelineContract", "TaskContract", "load_contract", "PipelineSecurityValidator", "SecurityError",
           "SecurityLevel", "TaskManager", "TaskStatus", "run_server", "run_stream_server"]  # fmt: skip


def __getattr__(name: str):
    if name in ("run_server", "run_stream_server", "ServiceContainer"):
        from . import main

        return getattr(main, name)
    if name in ("ServerConfig", "PipelineService", "PipelinePool"):
        from . import pipeline_service

        return getattr(pipeline_service, name)
    raise AttributeError(name)
