from .pipeline import (TIMESTEPS, AudioEncodingStage, LiveActDenoisingStage, LiveActPipeline, LiveActPipelineConfig,
                       resample_to_16k)  # fmt: skip

__all__ = ["TIMESTEPS", "AudioEncodingStage", "LiveActDenoisingStage", "LiveActPipeline", "LiveActPipelineConfig",
           "resample_to_16k"]  # fmt: skip
