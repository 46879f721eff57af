from .pipeline import HunyuanVideo15Pipeline, HunyuanVideo15PipelineConfig, HunyuanVideoDenoisingStage, HunyuanVideoSRDenoisingStage

__all__ = ["HunyuanVideo15Pipeline", "HunyuanVideo15PipelineConfig", "HunyuanVideoDenoisingStage",
           "HunyuanVideoSRDenoisingStage"]  # fmt: skip
