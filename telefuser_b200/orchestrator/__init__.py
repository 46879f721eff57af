from .local_actor import LocalStageActor
from .streaming import StreamingPipelineOrchestrator
from .streaming_types import *  # noqa: F401,F403
