from .pipeline import HunyuanTextEncodingStage, HunyuanVideo15Pipeline, HunyuanVideo15PipelineConfig, HunyuanVideoDenoisingStage, HunyuanVideoSRDenoisingStage

__all__ = ["HunyuanTextEncodingStage", "HunyuanVideo15Pipeline", "HunyuanVideo15PipelineConfig", "HunyuanVideoDenoisingStage",
           "HunyuanVideoSRDenoisingStage"]  # fmt: skip
