from .openai import OpenAICompatibleClient
from .tf_client import TaskCreationError, TaskFailedError, TaskTimeoutError, TeleFuserError, TFClient

__all__ = ["OpenAICompatibleClient", "TFClient", "TeleFuserError", "TaskCreationError", "TaskFailedError",
           "TaskTimeoutError"]  # fmt: skip
