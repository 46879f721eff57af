from .pipeline import QwenImageDenoisingStage, QwenImagePipeline, QwenImagePipelineConfig, norm_preserving_cfg

__all__ = ["QwenImageDenoisingStage", "QwenImagePipeline", "QwenImagePipelineConfig", "norm_preserving_cfg"]
